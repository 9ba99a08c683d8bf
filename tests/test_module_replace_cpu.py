"""Hugging Face attention modules replaced by this package's versions, on CPU in fp32 (dense reference attention):
the replaced model computes what the stock model computes, with the call signatures of the installed transformers."""
import pytest
import torch

transformers = pytest.importorskip("transformers")


def _replace(model):
    from atorch_b200.auto.opt_lib.module_replace import REPLACEMENT_PAIRS, _register_defaults, replace_module

    _register_defaults()
    return sum(replace_module(model, src, tgt, kw) for name, (src, tgt, kw, _) in REPLACEMENT_PAIRS.items()
               if name.startswith("HF_"))


def _pair(make):
    torch.manual_seed(0)
    ref, new = make().eval(), make().eval()
    new.load_state_dict(ref.state_dict())
    assert _replace(new) == 2
    return ref, new


def test_gpt2_bert_llama_replacements_match_the_stock_modules():
    from transformers import (BertConfig, BertModel, GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM)

    ids = torch.randint(0, 512, (2, 48))
    cfg = GPT2Config(vocab_size=512, n_positions=256, n_embd=256, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                     attn_pdrop=0.0)
    cfg._attn_implementation = "eager"
    ref, new = _pair(lambda: GPT2LMHeadModel(cfg))
    assert torch.allclose(ref(input_ids=ids).logits, new(input_ids=ids).logits, atol=1e-4)

    cfg = BertConfig(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=4, intermediate_size=512,
                     max_position_embeddings=256, hidden_dropout_prob=0.0, attention_probs_dropout_prob=0.0)
    cfg._attn_implementation = "eager"
    ref, new = _pair(lambda: BertModel(cfg))
    mask = torch.ones(2, 48, dtype=torch.long)
    mask[1, 30:] = 0
    a = ref(input_ids=ids, attention_mask=mask).last_hidden_state
    b = new(input_ids=ids, attention_mask=mask).last_hidden_state
    assert torch.allclose(a[mask.bool()], b[mask.bool()], atol=1e-4)

    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=4, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    ref, new = _pair(lambda: LlamaForCausalLM(cfg))
    out = new(input_ids=ids, labels=ids)
    assert torch.allclose(ref(input_ids=ids).logits, out.logits, atol=1e-4)
    out.loss.backward()
    assert all(p.grad is not None for n, p in new.named_parameters() if "self_attn" in n)


def test_clip_text_and_vision_replacements():
    from transformers import CLIPTextConfig, CLIPTextModel, CLIPVisionConfig, CLIPVisionModel

    cfg = CLIPTextConfig(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2,
                         num_attention_heads=4, max_position_embeddings=64)
    cfg._attn_implementation = "eager"
    ref, new = _pair(lambda: CLIPTextModel(cfg))
    ids = torch.randint(0, 512, (2, 32))
    am = torch.ones(2, 32, dtype=torch.long)
    am[1, 20:] = 0
    a = ref(input_ids=ids, attention_mask=am).last_hidden_state      # causal + padding, one [B, 1, S, S] mask
    b = new(input_ids=ids, attention_mask=am).last_hidden_state
    assert torch.allclose(a[am.bool()], b[am.bool()], atol=1e-4)
    vc = CLIPVisionConfig(hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
                          image_size=32, patch_size=8)
    vc._attn_implementation = "eager"
    ref, new = _pair(lambda: CLIPVisionModel(vc))
    x = torch.randn(2, 3, 32, 32)
    assert torch.allclose(ref(pixel_values=x).last_hidden_state, new(pixel_values=x).last_hidden_state, atol=1e-4)


def test_decoder_replacements_honour_padding_in_the_4d_mask():
    """GPT-2 and Llama with a left-padded batch: the model hands every layer one [B, 1, S, S] causal + padding mask."""
    from transformers import GPT2Config, GPT2LMHeadModel, LlamaConfig, LlamaForCausalLM

    ids = torch.randint(0, 512, (2, 40))
    am = torch.ones(2, 40, dtype=torch.long)
    am[1, :13] = 0
    cfg = GPT2Config(vocab_size=512, n_positions=256, n_embd=256, n_layer=2, n_head=4, resid_pdrop=0.0, embd_pdrop=0.0,
                     attn_pdrop=0.0)
    cfg._attn_implementation = "eager"
    ref, new = _pair(lambda: GPT2LMHeadModel(cfg))
    a, b = ref(input_ids=ids, attention_mask=am).logits, new(input_ids=ids, attention_mask=am).logits
    assert torch.allclose(a[am.bool()], b[am.bool()], atol=1e-4)
    cfg = LlamaConfig(vocab_size=512, hidden_size=512, intermediate_size=1024, num_hidden_layers=2,
                      num_attention_heads=4, num_key_value_heads=2, max_position_embeddings=512)
    cfg._attn_implementation = "eager"
    ref, new = _pair(lambda: LlamaForCausalLM(cfg))
    a, b = ref(input_ids=ids, attention_mask=am).logits, new(input_ids=ids, attention_mask=am).logits
    assert torch.allclose(a[am.bool()], b[am.bool()], atol=1e-4)
