"""Profiler, timers, loss-spike recorder, meta-init helpers, common utilities (CPU)."""
import torch
import torch.nn as nn

from atorch_b200.common.constants import GPUCapability
from atorch_b200.common.env import EnvSetting
from atorch_b200.common.log_utils import TimeStats, Timer
from atorch_b200.common.util_func import data_float_to_dtype, data_to_device, recursively_getattr
from atorch_b200.utils.loss_spike_utils import TokenLossSpike
from atorch_b200.utils.meta_model_utils import (build_recorded_module, init_empty_weights_with_disk_offload, is_meta,
                                                materialize_modules_to_device, record_module_init)
from atorch_b200.utils.prof import AProfiler
from atorch_b200.utils.timer import ThroughputTimer


def test_profiler_counts_linear_flops():
    m = nn.Sequential(nn.Linear(8, 16), nn.ReLU(), nn.Linear(16, 4))
    p = AProfiler(m)
    p.start_profile()
    m(torch.randn(5, 8))
    p.stop_profile()
    assert p.get_total_flops() == 2 * 5 * (8 * 16 + 16 * 4)
    assert p.get_total_params() == 8 * 16 + 16 + 16 * 4 + 4
    assert "Linear" in p.print_model_profile(output_file=None)
    p.end_profile()
    assert GPUCapability.peak("NVIDIA B200", "bf16") == 2250.0


def test_timers_and_env(monkeypatch):
    st = TimeStats()
    with Timer("a", st):
        pass
    assert "a" in st.summary()
    t = ThroughputTimer(batch_size=4, start_step=1, steps_per_output=2, logging_fn=lambda s: None)
    for _ in range(4):
        t.start()
        t.stop()
    assert t.avg_samples_per_sec() > 0
    monkeypatch.setenv("MOE_FSDP_PREFETCH_NUM", "3")
    assert EnvSetting().MOE_FSDP_PREFETCH_NUM == 3


def test_loss_spike(tmp_path):
    ls = TokenLossSpike(str(tmp_path), min_iter=10, min_loss=2.0)
    assert not ls.save_loss("f.txt", 1.0, 20, "1.0,1.0", "a,b")
    assert not ls.save_loss("f.txt", 5.0, 5, "5.0", "a")
    assert ls.save_loss("f.txt", 5.0, 20, "4.0,6.0", "s1,s2")
    rec = ls.parse("f.txt")
    assert rec[0]["iter"] == 20 and rec[0]["losses"] == [4.0, 6.0] and rec[0]["sample_infos"] == ["s1", "s2"]
    n = ls.decode_loss_spike(str(tmp_path / "out.txt"), fetch_sample=lambda s: [1, 2])
    assert n == 2


def test_meta_init_and_record():
    with init_empty_weights_with_disk_offload():
        m = nn.Sequential(nn.Linear(4, 4), nn.LayerNorm(4))
    assert is_meta(m)
    materialize_modules_to_device(m, "cpu")
    assert not is_meta(m) and m(torch.randn(2, 4)).shape == (2, 4)
    undo = record_module_init()

    class Tiny(nn.Module):
        def __init__(self, d, k=2):
            super().__init__()
            self.l = nn.Linear(d, k)
    t = Tiny(3, k=5)
    undo()
    t2 = build_recorded_module(t)
    assert t2.l.out_features == 5 and t2 is not t


def test_util_funcs():
    b = {"x": torch.ones(2), "y": [torch.ones(1, dtype=torch.int64)]}
    b2 = data_float_to_dtype(data_to_device(b, "cpu"), torch.bfloat16)
    assert b2["x"].dtype == torch.bfloat16 and b2["y"][0].dtype == torch.int64
    m = nn.Sequential(nn.Linear(2, 2))
    assert recursively_getattr(m, "0.weight") is m[0].weight


def test_bench_loss_curve_helpers(tmp_path):
    """bench.py's loss-curve mode: name-seeded weights and the token stream are reproducible, and the
    comparison reports the largest per-step difference."""
    import importlib.util
    import json
    import os

    import torch

    spec = importlib.util.spec_from_file_location("bench", os.path.join(os.path.dirname(os.path.dirname(__file__)),
                                                                        "bench.py"))
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    a, b = torch.empty(4, 6), torch.empty(4, 6)
    bench.name_seeded_init_("model.layers.0.mlp.up_proj.weight", a)
    bench.name_seeded_init_("model.layers.0.mlp.up_proj.weight", b)
    assert torch.equal(a, b) and 0.005 < a.std() < 0.04
    bench.name_seeded_init_("model.layers.0.mlp.down_proj.weight", b)
    assert not torch.equal(a, b)
    n = torch.empty(5)
    bench.name_seeded_init_("model.norm.weight", n)
    assert (n == 1).all()
    s1, s2 = bench.loss_stream(100, 2, 8, 0, 3), bench.loss_stream(100, 2, 8, 0, 3)
    assert all(torch.equal(x, y) for x, y in zip(s1, s2)) and not torch.equal(s1[0], s1[1])
    fa, fb = tmp_path / "a.json", tmp_path / "b.json"
    json.dump({"impl": "ours", "loss_curve": [10.0, 9.5, 9.0]}, open(fa, "w"))
    json.dump({"impl": "reference", "loss_curve": [10.0, 9.4, 9.05]}, open(fb, "w"))
    r = bench.compare_loss(str(fa), str(fb))
    assert abs(r["max_abs_diff"] - 0.1) < 1e-9 and r["steps"] == 3


def test_small_utils_version_import_gc_trace(tmp_path):
    import json
    import pickle

    from atorch_b200.utils import gc as mgc
    from atorch_b200.utils import import_util, parse_memory_pickle, parse_trace_json, version

    assert version.torch_version() >= (2, 0, 0) and version.torch_version("2.4.1+cu121") == (2, 4, 1)
    assert version.package_version_bigger_than("torch", "1.0") and not version.package_version_smaller_than("torch", "1.0")
    assert version.get_version("definitely_not_a_package") is None
    assert import_util.import_module("os.path.join") is __import__("os").path.join
    f = tmp_path / "m_mod.py"
    f.write_text("X = 41 + 1\n")
    assert import_util.import_module_from_py_file(str(f)).X == 42
    assert import_util.is_triton_available() in (True, False) and not import_util.is_xla_device_available()
    g = mgc.ManualGarbageCollection(gc_freq=2)
    try:
        assert [g.run(s) for s in (1, 2, 3, 4)] == [False, True, False, True]
    finally:
        g.restore()
    ev = [{"ph": "X", "cat": "kernel", "name": "gemm_bf16_2cta_kernel", "ts": 0, "dur": 100},
          {"ph": "X", "cat": "kernel", "name": "ncclDevKernel_AllGather", "ts": 50, "dur": 100},
          {"ph": "X", "cat": "kernel", "name": "adamw_kernel", "ts": 200, "dur": 50},
          {"ph": "X", "cat": "user_annotation", "name": "ProfilerStep#1", "ts": 0, "dur": 250}]
    t = tmp_path / "trace.json"
    t.write_text(json.dumps({"traceEvents": ev}))
    r = parse_trace_json.parse_trace_file(str(t))
    assert r["comm_busy_us"] == 100 and r["comm_hidden_us"] == 50 and r["comm_exposed_us"] == 50 and r["idle_us"] == 50
    snap = {"segments": [{"blocks": [
        {"state": "active_allocated", "size": 1 << 20, "frames": [{"filename": "torch/x.py", "line": 1, "name": "a"},
                                                                   {"filename": "/m/model.py", "line": 7, "name": "fwd"}]},
        {"state": "inactive", "size": 1 << 22, "frames": []}]}]}
    p = tmp_path / "snap.pickle"
    p.write_bytes(pickle.dumps(snap))
    c = parse_memory_pickle.parse_memory_pickle_file(str(p), blocklist=["torch/"])
    assert c["/m/model.py:7 fwd"] == 1 << 20 and sum(c.values()) == 1 << 20
