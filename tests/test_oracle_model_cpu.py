"""Pins the oracle's layer orchestration (norm placement, fused-QKV split, NeoX rotary convention, causal
mask, SwiGLU, residuals) against an independent implementation: transformers' LlamaForCausalLM run in fp32
on the CPU with its weights replaced by the dequantized int8 weights."""
import pytest
import torch

from model_util import OracleLM, oracle_layers, random_hf_state_dict, tiny_config


def test_decoder_oracle_agrees_with_hf_llama():
    transformers = pytest.importorskip("transformers")
    cfg = tiny_config(layers=2, hidden=256, heads=2, d_ff=512, vocab=320)
    sd = random_hf_state_dict(cfg, seed=0)
    hf_cfg = transformers.LlamaConfig(hidden_size=256, num_attention_heads=2, num_key_value_heads=2,
                                      num_hidden_layers=2, intermediate_size=512, vocab_size=320, rms_norm_eps=1e-6,
                                      hidden_act="silu", max_position_embeddings=64, rope_theta=10000.0,
                                      attention_bias=False, tie_word_embeddings=False)
    hf = transformers.LlamaForCausalLM(hf_cfg).float().eval()
    layers = oracle_layers(sd, cfg)
    new_sd = {k: v.float() for k, v in sd.items()}
    for i, L in enumerate(layers):
        p = f"model.layers.{i}."
        qkv = (L.qkv.float() * L.qkv_s.float()[None]).t()          # [3h, h]
        new_sd[p + "self_attn.q_proj.weight"], new_sd[p + "self_attn.k_proj.weight"], \
            new_sd[p + "self_attn.v_proj.weight"] = qkv.chunk(3, 0)
        new_sd[p + "self_attn.o_proj.weight"] = (L.out.float() * L.out_s.float()[None]).t()
        new_sd[p + "mlp.gate_proj.weight"] = (L.gate.float() * L.gate_s.float()[None]).t()
        new_sd[p + "mlp.up_proj.weight"] = (L.up.float() * L.up_s.float()[None]).t()
        new_sd[p + "mlp.down_proj.weight"] = (L.down.float() * L.down_s.float()[None]).t()
    missing = hf.load_state_dict(new_sd, strict=False)
    assert not [k for k in missing.missing_keys if "rotary" not in k]
    gen = torch.Generator().manual_seed(1)
    ids = torch.randint(0, 320, (2, 9), generator=gen)
    with torch.no_grad():
        want = hf(ids).logits
    lm = OracleLM(sd, cfg, max_len=16, batch=2)
    got = lm(ids[:, :6], True)
    assert torch.allclose(got, want[:, :6], atol=3e-2, rtol=3e-2)
    for t in range(6, 9):                                           # incremental steps against the full pass
        step_logits = lm(ids[:, t:t + 1], False)
        assert torch.allclose(step_logits[:, 0], want[:, t], atol=3e-2, rtol=3e-2)
    assert (got.argmax(-1) == want[:, :6].argmax(-1)).float().mean() > 0.9
