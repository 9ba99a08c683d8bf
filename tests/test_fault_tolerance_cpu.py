"""Failure detection on the host only: a rank that stops reporting, a rank that exits, relaunch loop."""
import os
import sys
import textwrap
import time

from atorch_b200.distributed.launch import launch
from atorch_b200.fault_tolerance.hanging_detector import HangingDetector, RelaunchStatus


class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_detector_reports_hang_and_agent_sees_it():
    store = DictStore()
    agent = RelaunchStatus("agent", world_size=2, store=store)
    fired = []
    d0 = HangingDetector(timeout=0.3, monitor_interval=0.05, rank=0, store=store, on_hang=lambda: fired.append(0))
    d1 = HangingDetector(timeout=0.3, monitor_interval=0.05, rank=1, store=store)
    d0.start()
    d1.start()
    t0 = time.time()
    while time.time() - t0 < 0.25:          # both report: nothing happens
        d0.report_normal()
        d1.report_normal()
        time.sleep(0.02)
    assert not agent.should_relaunch()
    t0 = time.time()
    while time.time() - t0 < 1.0 and not agent.should_relaunch():   # rank 0 goes silent
        d1.report_normal()
        time.sleep(0.02)
    assert agent.should_relaunch() and d0.hang_detected and fired == [0] and not d1.hang_detected
    agent.step_relaunch()
    assert not agent.should_relaunch()
    d1.stop(finalize=True)


def test_launcher_restarts_failed_group(tmp_path):
    marker = tmp_path / "attempt"
    script = tmp_path / "w.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys
        m = r"{marker}" + os.environ["RANK"]
        n = int(open(m).read()) if os.path.exists(m) else 0
        open(m, "w").write(str(n + 1))
        assert os.environ["WORLD_SIZE"] == "2" and os.environ["MASTER_ADDR"] == "127.0.0.1"
        sys.exit(1 if (n == 0 and os.environ["RANK"] == "1") else 0)   # rank 1 fails on the first attempt
    """))
    rc = launch([sys.executable, str(script)], nproc_per_node=2, max_restarts=1, monitor_interval=0.1)
    assert rc == 0
    assert int(open(str(marker) + "1").read()) == 2
    rc = launch([sys.executable, "-c", "import sys; sys.exit(3)"], nproc_per_node=2, max_restarts=0,
                monitor_interval=0.1)
    assert rc == 3


def test_relaunch_on_hanging(tmp_path):
    marker = tmp_path / "n"
    script = tmp_path / "h.py"
    script.write_text(textwrap.dedent(f"""
        import os, sys, time
        sys.path.insert(0, r"{os.path.dirname(os.path.dirname(os.path.abspath(__file__)))}")
        from atorch_b200.fault_tolerance.hanging_detector import HangingDetector
        m = r"{marker}" + os.environ["RANK"]
        n = int(open(m).read()) if os.path.exists(m) else 0
        open(m, "w").write(str(n + 1))
        d = HangingDetector(timeout=0.5, monitor_interval=0.1)
        d.start()
        for step in range(10):
            if n == 0 and os.environ["RANK"] == "0" and step == 3:
                time.sleep(60)              # first attempt: rank 0 never reports again
            d.report_normal()
            time.sleep(0.05)
        d.stop(finalize=True)
    """))
    t0 = time.time()
    rc = launch([sys.executable, str(script)], nproc_per_node=2, max_restarts=2, monitor_interval=0.1,
                relaunch_on_hanging=True)
    assert rc == 0 and time.time() - t0 < 40
    assert int(open(str(marker) + "0").read()) == 2
