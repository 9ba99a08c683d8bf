"""The Llama model of this package against the Hugging Face implementation with the same weights (CPU, fp32):
logits, loss and gradients; grouped-query attention; activation checkpointing; the carried residual of the norm."""
import pytest
import torch

from atorch_b200 import ops
from atorch_b200.models.llama import LlamaConfig, LlamaModel

transformers = pytest.importorskip("transformers")


def _pair(n_kv):
    from transformers import LlamaConfig as HFConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=120, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=n_kv, max_position_embeddings=64, rms_norm_eps=1e-5)
    torch.manual_seed(0)
    ours = LlamaModel(cfg)
    hf = LlamaForCausalLM(HFConfig(vocab_size=120, hidden_size=64, intermediate_size=176, num_hidden_layers=2,
                                   num_attention_heads=4, num_key_value_heads=n_kv, max_position_embeddings=64,
                                   rms_norm_eps=1e-5, rope_theta=10000.0, attention_bias=False, mlp_bias=False,
                                   tie_word_embeddings=False, attn_implementation="eager"))
    sd = {"model.embed_tokens.weight": ours.embed_tokens.weight, "model.norm.weight": ours.norm.weight,
          "lm_head.weight": ours.lm_head.weight}
    d = cfg.head_dim
    for i, l in enumerate(ours.layers):
        p = f"model.layers.{i}."
        q, k, v = l.qkv_proj.weight.split([4 * d, n_kv * d, n_kv * d], 0)
        g, u = l.gate_up_proj.weight.chunk(2, 0)
        sd.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                   p + "self_attn.o_proj.weight": l.o_proj.weight, p + "mlp.gate_proj.weight": g,
                   p + "mlp.up_proj.weight": u, p + "mlp.down_proj.weight": l.down_proj.weight,
                   p + "input_layernorm.weight": l.input_layernorm.weight,
                   p + "post_attention_layernorm.weight": l.post_attention_layernorm.weight})
    missing, unexpected = hf.load_state_dict({k: v.detach().clone() for k, v in sd.items()}, strict=False)
    assert not [m for m in missing if "rotary" not in m] and not unexpected
    return cfg, ours, hf


@pytest.mark.parametrize("n_kv", [4, 2])
def test_logits_loss_and_gradients_match_hugging_face(n_kv):
    cfg, ours, hf = _pair(n_kv)
    torch.manual_seed(1)
    ids = torch.randint(0, 120, (2, 33))
    loss, logits = ours(ids, labels=ids)
    ref = hf(input_ids=ids, labels=ids)
    assert torch.allclose(logits, ref.logits, atol=2e-4, rtol=1e-4)
    assert abs(loss.item() - ref.loss.item()) < 1e-4
    loss.backward()
    ref.loss.backward()
    l0, h0 = ours.layers[0], hf.model.layers[0]
    d = cfg.head_dim
    gq = l0.qkv_proj.weight.grad[: 4 * d]
    assert torch.allclose(gq, h0.self_attn.q_proj.weight.grad, atol=1e-5, rtol=1e-3)
    assert torch.allclose(l0.gate_up_proj.weight.grad[:176], h0.mlp.gate_proj.weight.grad, atol=1e-5, rtol=1e-3)
    assert torch.allclose(l0.input_layernorm.weight.grad, h0.input_layernorm.weight.grad, atol=1e-5, rtol=1e-3)
    assert torch.allclose(ours.embed_tokens.weight.grad, hf.model.embed_tokens.weight.grad, atol=1e-5, rtol=1e-3)


def test_checkpointed_model_gives_the_same_gradients():
    cfg, ours, _ = _pair(4)
    ids = torch.randint(0, 120, (2, 17))
    ours.train()
    loss, _ = ours(ids, labels=ids)
    loss.backward()
    g = {n: p.grad.clone() for n, p in ours.named_parameters()}
    ours.zero_grad()
    ours.config.gradient_checkpointing = True
    loss2, _ = ours(ids, labels=ids)
    loss2.backward()
    assert torch.equal(loss, loss2)
    for n, p in ours.named_parameters():
        assert torch.allclose(p.grad, g[n], atol=1e-6), n


def test_rms_norm_carry_returns_the_input_for_the_residual_path():
    torch.manual_seed(2)
    x = torch.randn(3, 5, 16, requires_grad=True)
    w = torch.randn(16, requires_grad=True)
    y, carried = ops.rms_norm(x, w, 1e-5, carry=True)
    assert torch.equal(carried, x)
    (y.sum() + (carried * 2).sum()).backward()
    x2 = x.detach().clone().requires_grad_()
    w2 = w.detach().clone().requires_grad_()
    y2 = ops.rms_norm(x2, w2, 1e-5)
    (y2.sum() + (x2 * 2).sum()).backward()
    assert torch.allclose(x.grad, x2.grad) and torch.allclose(w.grad, w2.grad)


def test_linear_swiglu_falls_back_to_the_two_ops_on_cpu():
    torch.manual_seed(3)
    x, w = torch.randn(7, 12), torch.randn(2 * 10, 12)
    out = ops.linear_swiglu(x, w)
    g = x @ w.t()
    assert torch.allclose(out, torch.nn.functional.silu(g[:, :10]) * g[:, 10:], atol=1e-6)


def test_mixtral_logits_match_hugging_face():
    """The sparse-MoE decoder (top-2 router, grouped expert MLPs, grouped-query attention) against the Hugging Face
    Mixtral with the same weights; capacity large enough that no token is dropped."""
    from transformers import MixtralConfig as HFConfig, MixtralForCausalLM

    from atorch_b200.models.mixtral import MixtralConfig, MixtralModel

    torch.manual_seed(0)
    cfg = MixtralConfig.tiny_moe(capacity_factor=8.0, router_aux_loss_coef=0.0, expert_intermediate_size=192)
    ours = MixtralModel(cfg).eval()
    hc = HFConfig(vocab_size=256, hidden_size=128, intermediate_size=192, num_hidden_layers=2, num_attention_heads=2,
                  num_key_value_heads=1, max_position_embeddings=64, num_local_experts=4, num_experts_per_tok=2,
                  sliding_window=None, rms_norm_eps=cfg.rms_norm_eps, rope_theta=cfg.rope_theta, attention_dropout=0.0)
    hc._attn_implementation = "eager"
    hf = MixtralForCausalLM(hc).eval()
    sd = {"model.embed_tokens.weight": ours.embed_tokens.weight, "model.norm.weight": ours.norm.weight,
          "lm_head.weight": ours.lm_head.weight}
    d = cfg.head_dim
    for i, l in enumerate(ours.layers):
        p = f"model.layers.{i}."
        q, k, v = l.qkv_proj.weight.split([2 * d, d, d], 0)
        moe = l.block_sparse_moe
        sd.update({p + "self_attn.q_proj.weight": q, p + "self_attn.k_proj.weight": k, p + "self_attn.v_proj.weight": v,
                   p + "self_attn.o_proj.weight": l.o_proj.weight, p + "mlp.gate.weight": moe.router.classifier.weight,
                   p + "mlp.experts.gate_up_proj": moe.experts.w1,                         # [E, 2F, H], gate | up
                   p + "mlp.experts.down_proj": moe.experts.w2.transpose(1, 2),            # ours [E, F, H]
                   p + "input_layernorm.weight": l.input_layernorm.weight,
                   p + "post_attention_layernorm.weight": l.post_attention_layernorm.weight})
    missing, unexpected = hf.load_state_dict({k: v.detach().clone().contiguous() for k, v in sd.items()}, strict=False)
    assert not missing and not unexpected, (missing, unexpected)
    ids = torch.randint(0, 256, (2, 24))
    out = ours(ids)
    logits = out[1] if isinstance(out, tuple) else out
    ref = hf(input_ids=ids).logits
    assert torch.allclose(logits, ref, atol=2e-4, rtol=1e-3), (logits - ref).abs().max()


@pytest.mark.parametrize("n_kv", [4, 2])
def test_hugging_face_state_dict_conversion_round_trip(n_kv):
    """``to_hf_state_dict`` produces a state dict the Hugging Face model loads (and then computes the same logits);
    ``from_hf_state_dict`` brings it back bit-exactly."""
    from atorch_b200.models.llama import from_hf_state_dict, to_hf_state_dict

    cfg, ours, hf = _pair(n_kv)
    with torch.no_grad():
        for p in hf.parameters():
            p.normal_()                                   # forget the weights _pair copied in
    sd = to_hf_state_dict(ours)
    missing, unexpected = hf.load_state_dict(sd, strict=False)
    assert not [m for m in missing if "rotary" not in m] and not unexpected
    ids = torch.randint(0, 120, (2, 19))
    assert torch.allclose(ours(ids)[1], hf(input_ids=ids).logits, atol=2e-4, rtol=1e-4)
    torch.manual_seed(9)
    other = LlamaModel(cfg)
    from_hf_state_dict(other, hf.state_dict())
    for (n, a), (_, b) in zip(ours.named_parameters(), other.named_parameters()):
        assert torch.equal(a, b), n
