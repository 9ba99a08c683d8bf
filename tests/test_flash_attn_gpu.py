"""sm_100a flash attention against the dense fp32 reference, for every mask form."""
import math

import pytest
import torch

from atorch_b200 import _lib
from atorch_b200.ops import attention_reference
from atorch_b200.ops import flash

pytestmark = pytest.mark.gpu


def _qkv(B, Sq, Sk, Hq, Hkv, D=128, fused=False):
    if fused and Sq == Sk:
        qkv = torch.randn(B, Sq, Hq + 2 * Hkv, D, device="cuda", dtype=torch.bfloat16)
        return qkv[:, :, :Hq], qkv[:, :, Hq:Hq + Hkv], qkv[:, :, Hq + Hkv:]
    q = torch.randn(B, Sq, Hq, D, device="cuda", dtype=torch.bfloat16)
    k = torch.randn(B, Sk, Hkv, D, device="cuda", dtype=torch.bfloat16)
    v = torch.randn(B, Sk, Hkv, D, device="cuda", dtype=torch.bfloat16)
    return q, k, v


def _fwd(q, k, v, **kw):
    B, Sq, Hq, D = q.shape
    lo, hi = flash.row_intervals(B, Sq, k.shape[1], q.device, kw.get("causal", False), kw.get("glm_mask"),
                                 kw.get("pack_glm_mask"), kw.get("key_padding_mask"), kw.get("cu_seqlens"))
    out, lse = flash.flash_fwd_raw(q, k, v, kw.get("causal", False), 1.0 / math.sqrt(D), lo, hi)
    torch.cuda.synchronize()
    _lib.check_status(q.device)
    return out, lse


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv", [(1, 128, 128, 1, 1), (2, 256, 256, 4, 4), (1, 1024, 1024, 8, 2),
                                            (2, 200, 200, 2, 2), (1, 384, 640, 2, 1), (1, 1, 300, 4, 4)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_fwd_basic(B, Sq, Sk, Hq, Hkv, causal):
    torch.manual_seed(B * 1000 + Sq + Sk)
    q, k, v = _qkv(B, Sq, Sk, Hq, Hkv, fused=(Sq == Sk and Hq == 4))
    if Sq == 1:
        causal = False
    out, lse = _fwd(q, k, v, causal=causal)
    ref = attention_reference(q, k, v, causal=causal)
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2), (out.float() - ref.float()).abs().max().item()
    kf = k.float().repeat_interleave(Hq // Hkv, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q.float(), kf) / math.sqrt(128)
    if causal:
        i = torch.arange(Sq, device="cuda")[:, None] + (Sk - Sq)
        s = s.masked_fill(torch.arange(Sk, device="cuda")[None, :] > i, float("-inf"))
    assert torch.allclose(lse, torch.logsumexp(s, -1), rtol=1e-3, atol=1e-2)


def test_flash_fwd_glm_and_packed_masks():
    torch.manual_seed(7)
    B, S, H = 2, 512, 2
    q, k, v = _qkv(B, S, S, H, H)
    glm = torch.tensor([100, 333], device="cuda", dtype=torch.int32)
    out, _ = _fwd(q, k, v, causal=True, glm_mask=glm)
    ref = attention_reference(q, k, v, causal=True, glm_mask=glm)
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    pack = torch.tensor([[[0, 200, -1], [50, 300, -1]], [[10, 128, 400], [64, 256, 512]]], device="cuda",
                        dtype=torch.int32)
    out, _ = _fwd(q, k, v, causal=True, pack_glm_mask=pack)
    ref = attention_reference(q, k, v, causal=True, pack_glm_mask=pack)
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def test_flash_fwd_padding_and_varlen():
    torch.manual_seed(8)
    B, S, H = 2, 384, 2
    q, k, v = _qkv(B, S, S, H, H)
    kp = torch.ones(B, S, dtype=torch.bool, device="cuda")
    kp[0, 300:] = False
    kp[1, 129:] = False
    out, _ = _fwd(q, k, v, causal=False, key_padding_mask=kp)
    ref = attention_reference(q, k, v, key_padding_mask=kp)
    assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2)
    cu = torch.tensor([0, 100, 228, 384], device="cuda", dtype=torch.int32)
    for causal in (True, False):
        out, _ = _fwd(q, k, v, causal=causal, cu_seqlens=cu)
        ref = attention_reference(q, k, v, causal=causal, cu_seqlens=cu)
        assert torch.allclose(out.float(), ref.float(), rtol=2e-2, atol=2e-2)


def _bwd_check(q, k, v, **kw):
    from atorch_b200.ops import attention
    qs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    out = attention(*qs, **kw)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_status(q.device)
    rs = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = attention_reference(*rs, **kw)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    for name, a, b in zip("qkv", qs, rs):
        err = (a.grad.float() - b.grad).abs().max().item()
        scale = b.grad.abs().max().item() + 1e-6
        assert err / scale < 3e-2, f"d{name}: max err {err} vs scale {scale}"


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv", [(1, 128, 128, 1, 1), (2, 256, 256, 2, 2), (1, 1024, 1024, 4, 2),
                                            (2, 200, 200, 2, 2), (1, 384, 640, 2, 1)])
@pytest.mark.parametrize("causal", [False, True])
def test_flash_bwd_basic(B, Sq, Sk, Hq, Hkv, causal):
    torch.manual_seed(B * 100 + Sq)
    q, k, v = _qkv(B, Sq, Sk, Hq, Hkv)
    _bwd_check(q, k, v, causal=causal)


def test_flash_bwd_masks():
    torch.manual_seed(9)
    B, S, H = 2, 512, 2
    q, k, v = _qkv(B, S, S, H, H)
    _bwd_check(q, k, v, causal=True, glm_mask=torch.tensor([100, 333], device="cuda", dtype=torch.int32))
    pack = torch.tensor([[[0, 200, -1], [50, 300, -1]], [[10, 128, 400], [64, 256, 512]]], device="cuda",
                        dtype=torch.int32)
    _bwd_check(q, k, v, causal=True, pack_glm_mask=pack)
    cu = torch.tensor([0, 100, 228, 512], device="cuda", dtype=torch.int32)
    _bwd_check(q, k, v, causal=True, cu_seqlens=cu)
    kp = torch.ones(B, S, dtype=torch.bool, device="cuda")
    kp[0, 300:] = False
    _bwd_check(q, k, v, causal=False, key_padding_mask=kp)


def test_flash_in_fused_qkv_layout():
    torch.manual_seed(10)
    B, S, H = 1, 512, 4
    qkv = torch.randn(B, S, 3 * H, 128, device="cuda", dtype=torch.bfloat16)
    _bwd_check(qkv[:, :, :H], qkv[:, :, H:2 * H], qkv[:, :, 2 * H:], causal=True)


def test_llama_block_reuses_attention_in_recompute():
    from atorch_b200.models.llama import LlamaConfig, LlamaDecoderLayer
    from atorch_b200.ops import rope_tables
    from atorch_b200.utils.checkpoint import checkpoint_module

    torch.manual_seed(11)
    cfg = LlamaConfig(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256)
    layer = LlamaDecoderLayer(cfg).cuda().bfloat16().train()
    cos, sin = rope_tables(256, 128, device="cuda")
    x = torch.randn(2, 256, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    before = _lib.launch_count
    y = checkpoint_module(layer, x, cos, sin)
    assert len(layer._attn_cache) == 1
    y.float().pow(2).sum().backward()
    with_cache = _lib.launch_count - before
    assert len(layer._attn_cache) == 0
    g1 = x.grad.clone()
    x.grad = None
    cfg.reuse_attention_in_recompute = False
    before = _lib.launch_count
    checkpoint_module(layer, x, cos, sin).float().pow(2).sum().backward()
    assert _lib.launch_count - before == with_cache + 1      # one more flash forward
    assert torch.equal(g1, x.grad)


def test_recompute_cache_ignores_plain_no_grad_forward():
    """A no-grad forward in train() mode (validation without .eval(), reference log-probs) must neither
    fill the recompute cache nor be served to a later checkpointed step."""
    from atorch_b200.models.llama import LlamaConfig, LlamaDecoderLayer
    from atorch_b200.ops.elementwise import rope_tables
    from atorch_b200.utils.checkpoint import checkpoint_module

    cfg = LlamaConfig(vocab_size=64, hidden_size=256, intermediate_size=512, num_hidden_layers=1,
                      num_attention_heads=2, num_key_value_heads=2, max_position_embeddings=256)
    torch.manual_seed(3)
    layer = LlamaDecoderLayer(cfg).cuda().bfloat16().train()
    cos, sin = rope_tables(256, 128, device="cuda")
    other = torch.randn(2, 256, 256, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        layer(other, cos, sin)                      # same shapes, different batch
    assert len(layer._attn_cache) == 0
    x = torch.randn(2, 256, 256, device="cuda", dtype=torch.bfloat16, requires_grad=True)
    checkpoint_module(layer, x, cos, sin).float().pow(2).sum().backward()
    g_cache = x.grad.clone()
    x.grad = None
    cfg.reuse_attention_in_recompute = False
    checkpoint_module(layer, x, cos, sin).float().pow(2).sum().backward()
    assert torch.equal(g_cache, x.grad)
    # a first pass whose backward never runs leaves one entry; it is not handed to another node
    cfg.reuse_attention_in_recompute = True
    y_lost = checkpoint_module(layer, other.clone().requires_grad_(), cos, sin)
    del y_lost
    assert len(layer._attn_cache) == 1
    x.grad = None
    checkpoint_module(layer, x, cos, sin).float().pow(2).sum().backward()
    assert torch.equal(g_cache, x.grad)


def test_flash_left_padded_and_holed_key_masks():
    """Key-padding masks that are not right-padded: left padding (the usual layout for generation) stays an
    interval per row, a mask with holes goes through the unpad path; both match dense attention on the
    valid query rows, forward and backward."""
    torch.manual_seed(21)
    B, S, H = 2, 256, 2
    q, k, v = _qkv(B, S, S, H, H)
    left = torch.ones(B, S, dtype=torch.bool, device="cuda")
    left[0, :70] = False
    left[1, :3] = False
    holes = torch.ones(B, S, dtype=torch.bool, device="cuda")
    holes[0, 10:40] = False
    holes[0, 200:] = False
    holes[1, ::7] = False
    for kp, causal in ((left, False), (left, True), (holes, False), (holes, True)):
        qq, kk, vv = (t.detach().clone().requires_grad_() for t in (q, k, v))
        out = flash.flash_attention(qq, kk, vv, causal=causal, key_padding_mask=kp)
        qr, kr, vr = (t.detach().float().requires_grad_() for t in (q, k, v))
        ref = attention_reference(qr, kr, vr, causal=causal, key_padding_mask=kp)
        rows = kp[:, :, None, None].expand_as(out)          # padded query rows are don't-care
        assert torch.allclose(out.float()[rows], ref.float()[rows], rtol=2e-2, atol=2e-2), (causal, kp is holes)
        g = torch.randn_like(out) * rows
        out.backward(g)
        ref.backward(g.float())
        for a, b, name in ((qq.grad, qr.grad, "dq"), (kk.grad, kr.grad, "dk"), (vv.grad, vr.grad, "dv")):
            tol = 5e-2 * max(1.0, b.abs().max().item())
            assert (a.float() - b).abs().max().item() < tol, (name, causal, kp is holes)
    _lib.check_status(q.device)


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,causal", [(2, 384, 384, 4, 4, True), (1, 200, 330, 4, 2, False)])
def test_flash_dropout_matches_reference_with_the_same_mask(B, Sq, Sk, Hq, Hkv, causal):
    """Forward and backward with dropout inside the kernels against dense fp32 attention that applies the keep
    mask restated on the host (flash.dropout_keep_mask)."""
    torch.manual_seed(21)
    p_drop, seed = 0.2, 0x1234_5678_9ABC
    q, k, v = _qkv(B, Sq, Sk, Hq, Hkv)
    qs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    out = flash.flash_attention(*qs, causal=causal, dropout_p=p_drop, dropout_seed=seed)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_status(q.device)

    drop = flash.dropout_config(p_drop, seed)
    keep = flash.dropout_keep_mask(B, Hq, Sq, Sk, drop, device="cuda")
    frac = keep.float().mean().item()
    assert abs(frac - (1 - p_drop)) < 0.01, frac
    rs = [t.detach().float().requires_grad_() for t in (q, k, v)]
    qf, kf, vf = (t.transpose(1, 2) for t in rs)
    if Hkv != Hq:
        kf, vf = kf.repeat_interleave(Hq // Hkv, dim=1), vf.repeat_interleave(Hq // Hkv, dim=1)
    s = qf @ kf.transpose(-1, -2) / math.sqrt(q.shape[-1])
    if causal:
        i, j = torch.arange(Sq, device="cuda")[:, None], torch.arange(Sk, device="cuda")[None]
        s = s.masked_fill(j > i + (Sk - Sq), float("-inf"))
    pm = torch.softmax(s, -1) * keep * (65536.0 / (65536 - drop[0]))
    ref = (pm @ vf).transpose(1, 2)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    for name, a, b in zip("qkv", qs, rs):
        err = (a.grad.float() - b.grad).abs().max().item()
        scale = b.grad.abs().max().item() + 1e-6
        assert err / scale < 3e-2, f"d{name}: max err {err} vs scale {scale}"
    # a different seed gives a different result, the same seed the same one
    again = flash.flash_attention(q, k, v, causal=causal, dropout_p=p_drop, dropout_seed=seed)
    other = flash.flash_attention(q, k, v, causal=causal, dropout_p=p_drop, dropout_seed=seed + 1)
    assert torch.equal(again, out.detach()) and not torch.equal(other, out.detach())


def test_dense_glm_mask_runs_in_the_flash_kernels():
    """A [B, 1, S, S] left-to-right GLM mask (0 / -65504 additive form) is lowered to key intervals: the result
    equals dense attention with the mask added to the scores, and no library or dense path is taken."""
    from atorch_b200.ops import attention
    import sys

    A = sys.modules["atorch_b200.ops.attention"]      # the module (ops.attention is the function)

    torch.manual_seed(13)
    B, S, H = 2, 384, 4
    q, k, v = _qkv(B, S, S, H, H)
    ltor = torch.tril(torch.ones(S, S, device="cuda"))[None].repeat(B, 1, 1)
    ltor[0, :, :100] = 1
    ltor[1, :, :257] = 1
    add = (-65504.0 * (1.0 - ltor))[:, None].to(torch.bfloat16)
    assert flash.intervals_from_additive_mask(add, B, S, S) is not None
    before = A.library_calls
    qs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    out = attention(*qs, additive_mask=add)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_status(q.device)
    assert A.library_calls == before and type(out.grad_fn).__name__ == "_FlashAttnBackward"
    rs = [t.detach().float().requires_grad_() for t in (q, k, v)]
    ref = attention_reference(*rs, additive_mask=add.float())
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    for name, a, b in zip("qkv", qs, rs):
        err = (a.grad.float() - b.grad).abs().max().item()
        assert err / (b.grad.abs().max().item() + 1e-6) < 3e-2, name


@pytest.mark.parametrize("kind", ["alibi", "soft_padding", "alibi+dropout"])
def test_additive_bias_inside_the_flash_kernels(kind):
    """A soft additive bias (per-head ALiBi slopes, or a per-batch key bias with -inf entries) is added to the
    scores inside the forward and backward kernels; compared with dense fp32 attention."""
    from atorch_b200.ops import attention

    torch.manual_seed(17)
    B, Sq, Sk, H = 2, 320, 320, 4
    q, k, v = _qkv(B, Sq, Sk, H, H)
    i, j = torch.arange(Sq, device="cuda")[:, None], torch.arange(Sk, device="cuda")[None]
    if kind.startswith("alibi"):
        slopes = torch.tensor([0.5, 0.25, 0.125, 0.0625], device="cuda")
        bias = (-(i - j).abs().float())[None, None] * slopes[None, :, None, None]          # [1, H, Sq, Sk]
        kw = dict(additive_bias=bias, causal=True)
    else:
        bias = 0.3 * torch.randn(B, 1, 1, Sk, device="cuda")
        bias[1, 0, 0, 200:] = float("-inf")
        kw = dict(additive_mask=bias)
    p_drop, seed = (0.15, 99) if kind.endswith("dropout") else (0.0, None)
    qs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    if p_drop:
        out = flash.flash_attention(*qs, dropout_p=p_drop, dropout_seed=seed, **kw)
    else:
        out = attention(*qs, **kw)
    assert type(out.grad_fn).__name__ == "_FlashAttnBackward"
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_status(q.device)
    rs = [t.detach().float().requires_grad_() for t in (q, k, v)]
    s = rs[0].transpose(1, 2) @ rs[1].transpose(1, 2).transpose(-1, -2) / math.sqrt(128)
    s = s + bias.to(torch.bfloat16).float()
    if kw.get("causal"):
        s = s.masked_fill(j > i, float("-inf"))
    pm = torch.softmax(s, -1)
    if p_drop:
        drop = flash.dropout_config(p_drop, seed)
        pm = pm * flash.dropout_keep_mask(B, H, Sq, Sk, drop, device="cuda") * (65536.0 / (65536 - drop[0]))
    ref = (pm @ rs[2].transpose(1, 2)).transpose(1, 2)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2), (out.float() - ref).abs().max()
    for name, a, b_ in zip("qkv", qs, rs):
        err = (a.grad.float() - b_.grad).abs().max().item()
        assert err / (b_.grad.abs().max().item() + 1e-6) < 3e-2, (name, err)


@pytest.mark.parametrize("B,Sq,Sk,Hq,Hkv,causal", [(2, 256, 256, 4, 4, True), (1, 200, 200, 12, 12, False),
                                                   (1, 384, 640, 4, 2, True), (2, 1024, 1024, 8, 8, True)])
def test_flash_head_dim_64(B, Sq, Sk, Hq, Hkv, causal):
    """Head dim 64 (GPT-2, BERT, CLIP): the single-tile forward and the one-kernel backward with one 64-column
    panel per tile, against dense fp32 attention; no library path."""
    A = __import__("sys").modules["atorch_b200.ops.attention"]
    torch.manual_seed(B * 10 + Sq)
    q, k, v = _qkv(B, Sq, Sk, Hq, Hkv, D=64)
    assert flash.supported(q, k, v)
    before = A.library_calls
    _bwd_check(q, k, v, causal=causal)
    assert A.library_calls == before


def test_flash_head_dim_64_masks_and_dropout():
    torch.manual_seed(31)
    B, S, H = 2, 512, 4
    q, k, v = _qkv(B, S, S, H, H, D=64)
    _bwd_check(q, k, v, causal=True, glm_mask=torch.tensor([100, 333], device="cuda", dtype=torch.int32))
    kp = torch.ones(B, S, dtype=torch.bool, device="cuda")
    kp[0, 300:] = False
    _bwd_check(q, k, v, causal=False, key_padding_mask=kp)
    # dropout with the host restatement of the mask
    p_drop, seed = 0.1, 4242
    qs = [t.detach().clone().requires_grad_() for t in (q, k, v)]
    out = flash.flash_attention(*qs, causal=True, dropout_p=p_drop, dropout_seed=seed)
    dout = torch.randn_like(out)
    out.backward(dout)
    torch.cuda.synchronize()
    _lib.check_status(q.device)
    drop = flash.dropout_config(p_drop, seed)
    keep = flash.dropout_keep_mask(B, H, S, S, drop, device="cuda")
    rs = [t.detach().float().requires_grad_() for t in (q, k, v)]
    s = rs[0].transpose(1, 2) @ rs[1].transpose(1, 2).transpose(-1, -2) / math.sqrt(64)
    i, j = torch.arange(S, device="cuda")[:, None], torch.arange(S, device="cuda")[None]
    pm = torch.softmax(s.masked_fill(j > i, float("-inf")), -1) * keep * (65536.0 / (65536 - drop[0]))
    ref = (pm @ rs[2].transpose(1, 2)).transpose(1, 2)
    ref.backward(dout.float())
    assert torch.allclose(out.float(), ref, rtol=2e-2, atol=2e-2)
    for name, a, b_ in zip("qkv", qs, rs):
        err = (a.grad.float() - b_.grad).abs().max().item()
        assert err / (b_.grad.abs().max().item() + 1e-6) < 3e-2, (name, err)
