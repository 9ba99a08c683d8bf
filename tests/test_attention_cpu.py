"""Host-side parts of the attention operator: mask lowering to key intervals and the dropout-mask restatement."""
import torch

from atorch_b200.ops import attention_reference, flash
from atorch_b200.ops.attention import build_dense_mask


def test_row_intervals_agree_with_the_dense_masks():
    B, S = 2, 48
    dev = torch.device("cpu")
    cases = [
        dict(causal=True),
        dict(causal=True, glm_mask=torch.tensor([7, 30], dtype=torch.int32)),
        dict(causal=True, pack_glm_mask=torch.tensor([[[0, 20, -1], [5, 30, -1]], [[3, 16, 40], [8, 24, 48]]],
                                                      dtype=torch.int32)),
        dict(causal=True, cu_seqlens=torch.tensor([0, 10, 25, 48], dtype=torch.int32)),
        dict(causal=False, cu_seqlens=torch.tensor([0, 10, 25, 48], dtype=torch.int32)),
    ]
    kp = torch.ones(B, S, dtype=torch.bool)
    kp[0, 30:] = False
    kp[1, :5] = False
    cases.append(dict(causal=False, key_padding_mask=kp))
    j = torch.arange(S)
    for kw in cases:
        causal = kw.pop("causal")
        lo, hi = flash.row_intervals(B, S, S, dev, causal, kw.get("glm_mask"), kw.get("pack_glm_mask"),
                                     kw.get("key_padding_mask"), kw.get("cu_seqlens"))
        if lo is None:       # analytic causal form inside the kernel
            lo = torch.zeros(B, S, dtype=torch.int32)
            hi = (torch.arange(S, dtype=torch.int32) + 1)[None].expand(B, S)
        vis = (j[None, None] >= lo[:, :, None]) & (j[None, None] < hi[:, :, None])
        dense = build_dense_mask(B, S, S, dev, causal, kw.get("glm_mask"), kw.get("pack_glm_mask"),
                                 kw.get("key_padding_mask"), kw.get("cu_seqlens"))
        assert torch.equal(vis, dense.expand(B, -1, S, S)[:, 0]), kw


def test_flash_dropout_mask_restatement_statistics():
    """Host restatement of the kernels' dropout hash: keep rate, determinism, independence of rows and heads."""
    drop = flash.dropout_config(0.1, seed=42)
    assert drop[0] == round(0.1 * 65536)
    keep = flash.dropout_keep_mask(2, 3, 64, 257, drop)
    assert keep.shape == (2, 3, 64, 257)
    assert abs(keep.float().mean().item() - 0.9) < 0.01
    assert torch.equal(keep, flash.dropout_keep_mask(2, 3, 64, 257, drop))
    assert not torch.equal(keep[0, 0], keep[0, 1]) and not torch.equal(keep[0, 0, 0], keep[0, 0, 1])
    other = flash.dropout_keep_mask(2, 3, 64, 257, flash.dropout_config(0.1, seed=43))
    assert 0.15 < (keep ^ other).float().mean().item() < 0.21       # 2 p (1 - p) = 0.18 for independent masks
    # without a seed, torch's CPU generator supplies it (so checkpoint recomputation replays it)
    torch.manual_seed(5)
    a = flash.dropout_config(0.1)
    torch.manual_seed(5)
    b = flash.dropout_config(0.1)
    assert a == b


def test_attention_reference_dropout_keeps_expectation():
    torch.manual_seed(0)
    q, k, v = (torch.randn(1, 64, 2, 16) for _ in range(3))
    base = attention_reference(q, k, v, causal=True)
    acc = torch.zeros_like(base)
    n = 200
    for _ in range(n):
        acc += attention_reference(q, k, v, causal=True, dropout_p=0.3)
    assert (acc / n - base).abs().mean().item() < 0.05


def _glm_ltor_mask(B, S, seps):
    m = torch.tril(torch.ones(S, S))[None].repeat(B, 1, 1)
    for b, sep in enumerate(seps):
        m[b, :, :sep] = 1
    return m[:, None]                                  # [B, 1, S, S], 1 = visible


def test_dense_binary_masks_lower_to_intervals():
    B, S = 2, 40
    ltor = _glm_ltor_mask(B, S, [7, 19])
    for mask in (ltor > 0.5, -65504.0 * (1.0 - ltor), torch.where(ltor > 0.5, 0.0, float("-inf"))):
        lo, hi = flash.intervals_from_additive_mask(mask, B, S, S)
        j = torch.arange(S)
        vis = (j[None, None] >= lo[:, :, None]) & (j[None, None] < hi[:, :, None])
        assert torch.equal(vis, ltor[:, 0] > 0.5)
    # with causal=True the upper end is clamped to the diagonal
    lo, hi = flash.intervals_from_additive_mask(ltor > 0.5, B, S, S, causal=True)
    assert torch.equal(hi, (torch.arange(S, dtype=torch.int32) + 1)[None].expand(B, S))
    # a soft bias, a per-head mask and a mask with holes are not intervals
    assert flash.intervals_from_additive_mask(torch.randn(B, 1, S, S), B, S, S) is None
    assert flash.intervals_from_additive_mask(torch.zeros(B, 3, S, S), B, S, S) is None
    holed = (ltor > 0.5).clone()
    holed[0, 0, 20, 3] = False
    assert flash.intervals_from_additive_mask(holed, B, S, S) is None
    # fully hidden rows become empty intervals
    hidden = (ltor > 0.5).clone()
    hidden[1, 0, 5] = False
    lo, hi = flash.intervals_from_additive_mask(hidden, B, S, S)
    assert lo[1, 5] == 0 and hi[1, 5] == 0


def test_glm_self_attention_module_matches_plain_math():
    from types import SimpleNamespace

    from atorch_b200.modules.transformer.layers import HFGLMSelfAttentionFA

    torch.manual_seed(3)
    cfg = SimpleNamespace(hidden_size=64, num_attention_heads=4, attention_dropout_prob=0.0, output_dropout_prob=0.0)
    m = HFGLMSelfAttentionFA(cfg).eval()
    B, S = 2, 24
    x = torch.randn(B, S, 64)
    ltor = _glm_ltor_mask(B, S, [5, 11])
    out = m(x, ltor)
    q, k, v = m.query_key_value(x).chunk(3, -1)
    h = lambda t: t.view(B, S, 4, 16).transpose(1, 2)
    s = h(q) @ h(k).transpose(-1, -2) / 4.0 + (-65504.0) * (1.0 - ltor)
    ref = m.dense((torch.softmax(s, -1) @ h(v)).transpose(1, 2).reshape(B, S, 64))
    assert torch.allclose(out, ref, atol=1e-5)
    # with memory of earlier tokens the keys are longer than the queries
    mem = torch.randn(B, 6, 64)
    ltor2 = torch.cat([torch.ones(B, 1, S, 6), ltor], -1)
    out2 = m(x, ltor2, mem=mem)
    assert out2.shape == (B, S, 64)
    # building from an existing module keeps its parameters
    m2 = HFGLMSelfAttentionFA(src_module=m)
    assert m2.query_key_value is m.query_key_value and torch.equal(m2(x, ltor), out)


def test_bias_config_sums_mask_and_bias_and_reports_broadcast_strides():
    B, H, Sq, Sk = 2, 3, 4, 8
    alibi = torch.randn(1, H, Sq, Sk)
    pad = torch.zeros(B, 1, 1, Sk)
    pad[1, 0, 0, 5:] = float("-inf")
    t, sb, sh, sq = flash.bias_config(B, H, Sq, Sk, pad, alibi)
    assert t.dtype == torch.bfloat16 and t.shape == (B, H, Sq, Sk) and (sb, sh, sq) == (H * Sq * Sk, Sq * Sk, Sk)
    assert torch.allclose(t.float(), (pad + alibi).to(torch.bfloat16).float(), atol=2e-2, equal_nan=True)
    t, sb, sh, sq = flash.bias_config(B, H, Sq, Sk, None, alibi)
    assert (sb, sh, sq) == (0, Sq * Sk, Sk)
    t, sb, sh, sq = flash.bias_config(B, H, Sq, Sk, pad, None)
    assert t.shape == (B, 1, 1, Sk) and (sb, sh, sq) == (Sk, 0, 0)
    t, *_ = flash.bias_config(B, H, Sq, Sk, torch.ones(Sq, Sk, dtype=torch.bool).tril(), None)
    assert t.shape == (1, 1, Sq, Sk) and t[0, 0, 0, 1] == float("-inf") and t[0, 0, 1, 1] == 0
