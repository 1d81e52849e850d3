"""Shared by the model-level tests: a tiny random LLaMA / Baichuan-architecture model as (i) an EET weight
dictionary for the library and (ii) un-packed layers for the oracle."""
import types

import numpy as np
import torch

from oracle import ops, w8


def tiny_config(layers=2, hidden=256, heads=2, d_ff=512, vocab=320):
    return types.SimpleNamespace(hidden_size=hidden, num_attention_heads=heads, num_hidden_layers=layers,
                                 intermediate_size=d_ff, vocab_size=vocab, rms_norm_eps=1e-6, hidden_act="silu",
                                 pad_token_id=None)


def random_hf_state_dict(cfg, seed=0, fused_qkv=False):
    """fp16 weights ~ N(0, 0.02^2) under HF parameter names (LLaMA: q/k/v_proj; Baichuan: W_pack)."""
    gen = torch.Generator().manual_seed(seed)
    h, f = cfg.hidden_size, cfg.intermediate_size

    def lin(o, i):
        return (torch.randn(o, i, generator=gen) * 0.02).half()

    sd = {"model.embed_tokens.weight": (torch.randn(cfg.vocab_size, h, generator=gen) * 0.5).half(),
          "model.norm.weight": (1 + 0.1 * torch.randn(h, generator=gen)).half(),
          "lm_head.weight": lin(cfg.vocab_size, h)}
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        if fused_qkv:
            sd[p + "self_attn.W_pack.weight"] = lin(3 * h, h)
        else:
            for n in ("q_proj", "k_proj", "v_proj"):
                sd[p + f"self_attn.{n}.weight"] = lin(h, h)
        sd[p + "self_attn.o_proj.weight"] = lin(h, h)
        sd[p + "mlp.gate_proj.weight"] = lin(f, h)
        sd[p + "mlp.up_proj.weight"] = lin(f, h)
        sd[p + "mlp.down_proj.weight"] = lin(h, f)
        sd[p + "input_layernorm.weight"] = (1 + 0.1 * torch.randn(h, generator=gen)).half()
        sd[p + "post_attention_layernorm.weight"] = (1 + 0.1 * torch.randn(h, generator=gen)).half()
    return sd


def _quant(w_out_in):
    """HF [out, in] fp16 weight -> (q int8 [K=in, N=out], scale fp16 [N]) with the oracle quantizer."""
    q, s = w8.c_symmetric_quantize_int8(w_out_in.t().contiguous().numpy())
    return torch.from_numpy(q), torch.from_numpy(s)


def oracle_layers(sd, cfg, fused_qkv=False, int8=True):
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        if fused_qkv:
            qkv = sd[p + "self_attn.W_pack.weight"]
        else:
            qkv = torch.cat([sd[p + f"self_attn.{n}.weight"] for n in ("q_proj", "k_proj", "v_proj")], 0)
        args = []
        for w in (qkv, sd[p + "self_attn.o_proj.weight"], sd[p + "mlp.gate_proj.weight"],
                  sd[p + "mlp.up_proj.weight"], sd[p + "mlp.down_proj.weight"]):
            args.extend(_quant(w) if int8 else (w.t().contiguous(), None))
        layers.append(ops.LayerWeights(*args, sd[p + "input_layernorm.weight"], sd[p + "post_attention_layernorm.weight"]))
    return layers


class OracleLM:
    """Embedding -> DecoderOracle -> final RMSNorm -> lm_head, all on the CPU, mirroring
    EETLlamaForCausalLM.__call__ (python/eet/transformers/modeling_llama.py:262-297,452-491)."""

    def __init__(self, sd, cfg, max_len, batch, rope=True, fused_qkv=False, exact=True, int8=True, lm_head_int8=False):
        self.sd, self.cfg = sd, cfg
        # with lm_head_int8 the head is quantized like the layer projections (an option of the library that the
        # reference does not have) and the logits are rounded to fp16 as a GEMM epilogue would round them
        self.head = _quant(sd["lm_head.weight"]) if lm_head_int8 else None
        self.dec = ops.DecoderOracle(oracle_layers(sd, cfg, fused_qkv, int8), cfg.num_attention_heads,
                                     cfg.hidden_size // cfg.num_attention_heads, cfg.rms_norm_eps, max_len, batch,
                                     rope=rope, exact=exact)

    def __call__(self, ids, first_pass, pad_len=None, reorder=None):
        if reorder is not None:
            self.dec.reorder(reorder)
        x = self.sd["model.embed_tokens.weight"][ids]
        x = self.dec.forward(x, first_pass, pad_len)
        x = ops.rmsnorm(x, self.sd["model.norm.weight"], self.cfg.rms_norm_eps)
        if self.head is not None:
            B, S, h = x.shape
            return ops.gemm_w8a16(x.reshape(B * S, h), self.head[0], self.head[1]).float().view(B, S, -1)
        return (x.float() @ self.sd["lm_head.weight"].float().t())


def oracle_beam_search(lm, prompt, num_beams, new_tokens):
    """Fixed-length beam search over an OracleLM (sum of log-probabilities, no length penalty, no EOS): the
    algorithm of eet_b200.modeling.beam_search restated on the CPU.  Returns (sequences [B, S+new], scores [B],
    margins): margins[t] is the smallest gap between the last kept and the first dropped candidate at step t,
    so a test can tell a real disagreement from a near tie."""
    B, S = prompt.shape
    nb = num_beams
    ids = prompt.repeat_interleave(nb, 0)
    scores = torch.zeros(B, nb)
    scores[:, 1:] = -1e9
    logits = lm(ids, True)[:, -1]
    margins, reorder = [], None
    for t in range(new_tokens):
        if t > 0:
            logits = lm(ids[:, -1:], False, reorder=reorder)[:, -1]
        logp = torch.log_softmax(logits.float(), -1)
        V = logp.shape[-1]
        cand = (scores.view(B, nb, 1) + logp.view(B, nb, V)).view(B, nb * V)
        top = cand.topk(nb + 1, -1)
        margins.append(float((top.values[:, :-1] - top.values[:, 1:]).min()))
        scores, idx = top.values[:, :nb], top.indices[:, :nb]
        beam, tok = idx // V, idx % V
        reorder = (beam + torch.arange(B).view(B, 1) * nb).view(-1)
        ids = torch.cat([ids[reorder], tok.view(-1, 1)], 1)
    best = scores.argmax(-1)
    return ids.view(B, nb, -1)[torch.arange(B), best], scores[torch.arange(B), best], margins
