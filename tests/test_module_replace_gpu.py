"""Hugging Face attention modules replaced by the flash-kernel versions (auto/opt_lib/module_replace.py) on a GPU:
GPT-2 and BERT with 64-wide heads, Llama with 128-wide heads; same logits and gradients as the stock modules, and
the sm_100a kernels (not the library path) do the work."""
import sys

import pytest
import torch

from atorch_b200 import _lib

pytestmark = pytest.mark.gpu
transformers = pytest.importorskip("transformers")


def _replace(model):
    from atorch_b200.auto.opt_lib.module_replace import REPLACEMENT_PAIRS, _register_defaults, replace_module

    _register_defaults()
    n = 0
    for name, (src, tgt, kw, _) in REPLACEMENT_PAIRS.items():
        if name.startswith("HF_"):
            n += replace_module(model, src, tgt, kw)
    return n


def _library_calls():
    return sys.modules["atorch_b200.ops.attention"].library_calls


def _compare(model_fn, inputs, out_key="logits", tol=4e-2):
    torch.manual_seed(0)
    ref = model_fn().cuda().bfloat16().eval()
    new = model_fn().cuda().bfloat16().eval()
    new.load_state_dict(ref.state_dict())
    assert _replace(new) > 0
    before = _library_calls()
    a = getattr(ref(**inputs), out_key)
    b = getattr(new(**inputs), out_key)
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    assert _library_calls() == before, "the replacement fell back to the library attention"
    scale = a.float().abs().max().item()
    assert (a.float() - b.float()).abs().max().item() < tol * scale, ((a.float() - b.float()).abs().max().item(), scale)
    # gradients flow through the kernels' backward
    b.float().square().mean().backward()
    a.float().square().mean().backward()
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    ga = next(p.grad for p in ref.parameters() if p.grad is not None and p.dim() == 2)
    gb = next(p.grad for p in new.parameters() if p.grad is not None and p.dim() == 2)
    assert (ga.float() - gb.float()).abs().max().item() < 6e-2 * (ga.float().abs().max().item() + 1e-6)


def test_gpt2_attention_replacement_head_dim_64():
    from transformers import GPT2Config, GPT2LMHeadModel

    cfg = GPT2Config(vocab_size=512, n_positions=256, n_embd=256, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                     attn_pdrop=0.0)
    cfg._attn_implementation = "eager"
    ids = torch.randint(0, 512, (2, 192), device="cuda")
    _compare(lambda: GPT2LMHeadModel(cfg), dict(input_ids=ids))


def test_bert_attention_replacement_with_padding():
    from transformers import BertConfig, BertModel

    cfg = BertConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512,
                     max_position_embeddings=256, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    cfg._attn_implementation = "eager"
    ids = torch.randint(0, 512, (2, 160), device="cuda")
    mask = torch.ones(2, 160, dtype=torch.long, device="cuda")
    mask[1, 100:] = 0
    torch.manual_seed(0)
    ref = BertModel(cfg).cuda().bfloat16().eval()
    new = BertModel(cfg).cuda().bfloat16().eval()
    new.load_state_dict(ref.state_dict())
    assert _replace(new) > 0
    before = _library_calls()
    a = ref(input_ids=ids, attention_mask=mask).last_hidden_state
    b = new(input_ids=ids, attention_mask=mask).last_hidden_state
    torch.cuda.synchronize()
    _lib.check_status(a.device)
    assert _library_calls() == before
    valid = mask.bool()
    d = (a.float() - b.float())[valid].abs().max().item()
    assert d < 4e-2 * a.float()[valid].abs().max().item(), d


def test_llama_attention_replacement_head_dim_128():
    from transformers import LlamaConfig, LlamaForCausalLM

    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    ids = torch.randint(0, 512, (2, 256), device="cuda")
    _compare(lambda: LlamaForCausalLM(cfg), dict(input_ids=ids))
