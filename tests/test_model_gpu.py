"""Whole-model parity: tiny LLaMA- and Baichuan-architecture models through the library's model wrappers
(prefill, then decode steps; eager and CUDA-graph) against the CPU oracle.

Tolerance: logits are O(1) fp32 values computed from fp16 activations that passed through 2 layers with
different (but equally valid) fp32 summation orders; |err| <= 2e-2 + 2e-2*|ref|, stated here per the
fp16-activation budget, and the greedy tokens must agree wherever the oracle's top-2 margin exceeds it."""
import pytest
import torch

from model_util import OracleLM, random_hf_state_dict, tiny_config

pytestmark = pytest.mark.gpu


def _build(cfg, sd, cls_name, convert_name, B, prompt_cap, full_len):
    from eet_b200 import modeling
    conv = getattr(modeling, convert_name)
    eet_dict = conv({k: v.clone() for k, v in sd.items()}, torch.int8)
    assert eet_dict["layer.0.self_attn.qkv_proj.weight"].dtype == torch.int8
    assert eet_dict["layer.0.self_attn.qkv_proj.weight"].shape == (cfg.hidden_size, 3 * cfg.hidden_size)
    assert "layer.1.ffn.output.scale" in eet_dict and "embed_tokens.weight" in eet_dict
    return getattr(modeling, cls_name).from_eet(eet_dict, cfg, B, prompt_cap, full_len, torch.int8)


def _logits_close(got, want):
    return torch.allclose(got.float().cpu(), want, atol=2e-2, rtol=2e-2)


@pytest.mark.parametrize("padded", [False, True])
def test_llama_prefill_and_decode_match_oracle(padded):
    cfg = tiny_config()
    sd = random_hf_state_dict(cfg, seed=0)
    B, S, T = 2, 7, 16
    model = _build(cfg, sd, "EETLlamaForCausalLM", "convert_llama_weights", B, 8, T)
    lm = OracleLM(sd, cfg, max_len=T, batch=B)
    gen = torch.Generator().manual_seed(2)
    ids = torch.randint(0, cfg.vocab_size, (B, S + 4), generator=gen)
    mask, pad = None, None
    if padded:
        mask = torch.ones(B, S, dtype=torch.long)
        mask[1, :3] = 0
        pad = torch.tensor([0, 3])
    out = model(ids[:, :S].cuda(), first_pass=True, attention_mask=None if mask is None else mask.cuda())
    want = lm(ids[:, :S], True, pad)
    rows = slice(None) if not padded else slice(None)
    got = out.logits
    if padded:   # rows of the padding itself carry no meaning; compare the real tokens
        assert _logits_close(got[0], want[0]) and _logits_close(got[1, 3:], want[1, 3:])
    else:
        assert _logits_close(got, want)
    for t in range(S, S + 4):
        out = model(ids[:, t:t + 1].cuda(), first_pass=False, attention_mask=None if mask is None else mask.cuda())
        want = lm(ids[:, t:t + 1], False, pad)
        assert _logits_close(out.logits, want), f"decode step {t}"


def test_baichuan13b_alibi_path_matches_oracle():
    cfg = tiny_config(layers=2, hidden=1024, heads=8, d_ff=512, vocab=320)   # != 32 layers -> ALiBi op
    sd = random_hf_state_dict(cfg, seed=3, fused_qkv=True)
    B, S, T = 2, 6, 12
    model = _build(cfg, sd, "EETBaichuanForCausalLM", "convert_baichuan_weights", B, 8, T)
    lm = OracleLM(sd, cfg, max_len=T, batch=B, rope=False, fused_qkv=True)
    gen = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg.vocab_size, (B, S + 3), generator=gen)
    assert _logits_close(model(ids[:, :S].cuda(), first_pass=True).logits, lm(ids[:, :S], True))
    for t in range(S, S + 3):
        assert _logits_close(model(ids[:, t:t + 1].cuda(), first_pass=False).logits, lm(ids[:, t:t + 1], False))


def test_generate_graph_equals_eager_and_oracle_tokens():
    cfg = tiny_config()
    sd = random_hf_state_dict(cfg, seed=5)
    B, S, NEW, T = 2, 5, 6, 16
    model = _build(cfg, sd, "EETLlamaForCausalLM", "convert_llama_weights", B, 8, T)
    gen = torch.Generator().manual_seed(6)
    prompt = torch.randint(0, cfg.vocab_size, (B, S), generator=gen)
    eager = model.generate(prompt.cuda(), NEW).cpu()
    model.use_cuda_graph = True
    graphed = model.generate(prompt.cuda(), NEW).cpu()
    again = model.generate(prompt.cuda(), NEW).cpu()
    assert torch.equal(eager, graphed) and torch.equal(graphed, again)
    assert eager.shape == (B, S + NEW) and torch.equal(eager[:, :S], prompt)
    # oracle greedy decoding: tokens agree while the oracle's top-2 margin is clear of the tolerance
    lm = OracleLM(sd, cfg, max_len=T, batch=B)
    logits = lm(prompt, True)[:, -1]
    for t in range(NEW):
        top2 = logits.topk(2, -1).values
        clear = (top2[:, 0] - top2[:, 1]) > 4e-2
        tok = eager[:, S + t]
        assert torch.equal(tok[clear], logits.argmax(-1)[clear])
        logits = lm(tok.view(B, 1), False)[:, -1]   # follow the library's tokens so both see the same history


def test_beam_reorder_state_moves_the_cache():
    cfg = tiny_config()
    sd = random_hf_state_dict(cfg, seed=7)
    B, S, T = 2, 4, 12
    model = _build(cfg, sd, "EETLlamaForCausalLM", "convert_llama_weights", B, 8, T)
    gen = torch.Generator().manual_seed(8)
    ids = torch.randint(0, cfg.vocab_size, (B, S + 1), generator=gen)
    model(ids[:, :S].cuda(), first_pass=True)
    # both beams continue from sequence 1: after reordering, row 0 must behave like row 1
    same_tok = ids[1:2, S:S + 1].expand(B, 1).contiguous()
    out = model(same_tok.cuda(), first_pass=False, reorder_state=torch.tensor([1, 1]).cuda()).logits.cpu()
    assert torch.allclose(out[0].float(), out[1].float(), atol=1e-3, rtol=1e-3)


def test_beam_search_matches_oracle():
    from model_util import oracle_beam_search
    cfg = tiny_config()
    sd = random_hf_state_dict(cfg, seed=9)
    B, S, NB, NEW, T = 2, 4, 3, 5, 12
    model = _build(cfg, sd, "EETLlamaForCausalLM", "convert_llama_weights", B * NB, 8, T)
    gen = torch.Generator().manual_seed(10)
    prompt = torch.randint(0, cfg.vocab_size, (B, S), generator=gen)
    seqs, scores = model.beam_search(prompt.cuda(), NB, NEW)
    assert seqs.shape == (B, S + NEW) and torch.equal(seqs[:, :S].cpu(), prompt)
    want_seqs, want_scores, margins = oracle_beam_search(OracleLM(sd, cfg, max_len=T, batch=B * NB), prompt, NB, NEW)
    # log-probabilities carry the logits' tolerance; the beams themselves must agree unless some step of the
    # oracle was a near tie between a kept and a dropped candidate
    assert torch.allclose(scores.cpu(), want_scores, atol=0.1)
    if min(margins) > 5e-2:
        assert torch.equal(seqs.cpu(), want_seqs)
    # greedy generation afterwards is unaffected by the beam state
    assert model.model.reorder_state.numel() == 0


def test_fp16_twin_ops_match_oracle():
    """data_type=torch.float16: GatedFeedForwardNetwork and the fp16 branch of LlamaMmha
    (python/eet/transformers/modeling_llama.py:118-123,336-337)."""
    from eet_b200 import EET, modeling
    cfg = tiny_config()
    sd = random_hf_state_dict(cfg, seed=11)
    B, S, T = 2, 6, 12
    eet_dict = modeling.convert_llama_weights({k: v.clone() for k, v in sd.items()}, torch.float16)
    assert eet_dict["layer.0.self_attn.qkv_proj.weight"].dtype == torch.float16
    assert "layer.0.self_attn.qkv_proj.scale" not in eet_dict
    model = modeling.EETLlamaForCausalLM.from_eet(eet_dict, cfg, B, 8, T, torch.float16)
    assert isinstance(model.model.layers[0].feedforward, EET.GatedFeedForwardNetwork)
    lm = OracleLM(sd, cfg, max_len=T, batch=B, int8=False)
    gen = torch.Generator().manual_seed(12)
    ids = torch.randint(0, cfg.vocab_size, (B, S + 3), generator=gen)
    assert _logits_close(model(ids[:, :S].cuda(), first_pass=True).logits, lm(ids[:, :S], True))
    for t in range(S, S + 3):
        assert _logits_close(model(ids[:, t:t + 1].cuda(), first_pass=False).logits, lm(ids[:, t:t + 1], False))
    toks = model.generate(ids[:, :S].cuda(), 3)
    assert toks.shape == (B, S + 3)


def test_update_requantizes_in_place_and_keeps_the_graph():
    """EETLlamaForCausalLM.update (python/eet/transformers/modeling_llama.py:518-522): new weights go into
    the tensors the ops already hold."""
    import types
    cfg = tiny_config()
    sd_a, sd_b = random_hf_state_dict(cfg, seed=13), random_hf_state_dict(cfg, seed=14)
    B, S, T = 2, 5, 12
    model = _build(cfg, sd_a, "EETLlamaForCausalLM", "convert_llama_weights", B, 8, T)
    ptr = model.model.layers[0].qkv_w.data_ptr()
    gen = torch.Generator().manual_seed(15)
    ids = torch.randint(0, cfg.vocab_size, (B, S), generator=gen)
    model.use_cuda_graph = True
    model.generate(ids.cuda(), 4)          # captures the decode graph on the old weights
    hf_like = types.SimpleNamespace(state_dict=lambda: sd_b, config=cfg)
    model.update(hf_like)
    assert model.model.layers[0].qkv_w.data_ptr() == ptr
    lm = OracleLM(sd_b, cfg, max_len=T, batch=B)
    assert _logits_close(model(ids.cuda(), first_pass=True).logits, lm(ids, True))
    graphed = model.generate(ids.cuda(), 4).cpu()
    model.use_cuda_graph = False
    assert torch.equal(graphed, model.generate(ids.cuda(), 4).cpu())


def test_embedding_op():
    from eet_b200 import EET
    B, S, h, V = 2, 5, 64, 50
    desc = EET.MetaDesc(torch.float16, B, 2, h, 1, 8, 16, "silu", cuda_device="cuda:0")
    gen = torch.Generator().manual_seed(16)
    word, pos, tok = (torch.randn(n, h, generator=gen).half().cuda() for n in (V, 16, 2))
    emb = EET.Embedding(desc, word, pos, tok, torch.ones(h).half().cuda(), torch.zeros(h).half().cuda(), "emb_cache")
    ids = torch.randint(0, V, (B, S), generator=gen).cuda()
    pid = torch.arange(S).view(1, S).cuda()
    tid = torch.zeros(B, S, dtype=torch.long).cuda()
    got = emb.forward_transformers(ids, pid, tid, False)
    want = ((word[ids] + tok[tid]) + pos[pid]).half()
    assert got.shape == (B, S, h) and torch.equal(got, want)
    normed = emb.forward_transformers(ids, pid, tid, True)
    ref = torch.nn.functional.layer_norm(want.float(), (h,), eps=desc.layernorm_eps).half()
    assert torch.allclose(normed.float(), ref.float(), atol=2e-3)


def test_decode_batch_above_16_uses_the_stream_k_kernel_and_matches_oracle():
    """Batches of 17..64 sequences keep the deferred-epilogue decode chain, with the projections on the
    stream-K tensor-core kernel: eager logits against the oracle, and graph replay equal to eager tokens."""
    cfg = tiny_config()
    sd = random_hf_state_dict(cfg, seed=17)
    B, S, NEW, T = 20, 3, 4, 10
    model = _build(cfg, sd, "EETLlamaForCausalLM", "convert_llama_weights", B, 4, T)
    lm = OracleLM(sd, cfg, max_len=T, batch=B)
    gen = torch.Generator().manual_seed(18)
    ids = torch.randint(0, cfg.vocab_size, (B, S + NEW), generator=gen)
    assert _logits_close(model(ids[:, :S].cuda(), first_pass=True).logits, lm(ids[:, :S], True))
    from eet_b200 import EET
    for t in range(S, S + 2):
        with EET.deferred_epilogue():   # what decode_step does: epilogues finished by the next op
            hidden = model.model(input_ids=ids[:, t:t + 1].cuda(), first_pass=False)
        logits = model.lm_head(hidden)
        assert _logits_close(logits, lm(ids[:, t:t + 1], False)), f"decode step {t}"
    eager = model.generate(ids[:, :S].cuda(), NEW).cpu()
    model.use_cuda_graph = True
    graphed = model.generate(ids[:, :S].cuda(), NEW).cpu()
    assert torch.equal(eager, graphed)
    from eet_b200 import _lib
    assert _lib.device_status() == 0


def test_int8_lm_head_logits_and_greedy_choice():
    """lm_head_int8=True (an option beyond the reference): the head is quantized like the other projections; its
    logits against the oracle with the same quantized head, and the fused greedy kernel against argmax of them."""
    from eet_b200 import modeling
    cfg = tiny_config(vocab=320)
    sd = random_hf_state_dict(cfg, seed=11)
    B, S, T = 2, 6, 16
    eet_dict = modeling.convert_llama_weights({k: v.clone() for k, v in sd.items()}, torch.int8)
    model = modeling.EETLlamaForCausalLM.from_eet(eet_dict, cfg, B, 8, T, torch.int8, lm_head_int8=True)
    assert model.lm_head.int8 and model.lm_head.w.dtype == torch.int8
    lm = OracleLM(sd, cfg, max_len=T, batch=B, lm_head_int8=True)
    gen = torch.Generator().manual_seed(12)
    ids = torch.randint(0, cfg.vocab_size, (B, S + 3), generator=gen)
    assert _logits_close(model(ids[:, :S].cuda(), first_pass=True).logits, lm(ids[:, :S], True))
    for t in range(S, S + 3):
        logits = model.decode_logits(ids[:, t:t + 1].cuda())
        assert _logits_close(logits, lm(ids[:, t:t + 1], False))
    # greedy: the fused kernel works on the fp32 sums and must agree with argmax over the fp16 logits
    hidden = torch.randn(B, cfg.hidden_size, generator=gen).half().cuda()
    want = model.lm_head(hidden).float().argmax(-1).view(B, 1)
    assert torch.equal(model.lm_head.greedy(hidden), want)
    eager = model.generate(ids[:, :S].cuda(), 5).cpu()
    model.use_cuda_graph = True
    assert torch.equal(model.generate(ids[:, :S].cuda(), 5).cpu(), eager)


@pytest.mark.parametrize("M,n", [(1, 64), (5, 320), (8, 32000), (64, 4096)])
def test_lm_head_argmax_kernel(M, n):
    from eet_b200._lib import check, lib
    gen = torch.Generator().manual_seed(M + n)
    sums = (torch.randn(M, n, generator=gen) * 500).cuda()
    scale = (torch.rand(n, generator=gen) * 1e-3 + 1e-4).half().cuda()
    logits_ref = (sums * scale.float()[None]).half()
    # plant exact ties at the maximum: the smallest index must win
    top = logits_ref.float().amax(1)
    for r in range(M):
        j = int(torch.randint(0, n, (1,), generator=gen))
        sums[r, j] = float(top[r]) / float(scale[j].float()) if float(scale[j]) > 0 else sums[r, j]
    logits_ref = (sums * scale.float()[None]).half()
    out = torch.full((M,), -1, dtype=torch.int64, device="cuda")
    logits = torch.empty(M, n, dtype=torch.float16, device="cuda")
    check(lib.eet_lm_head_argmax(sums.data_ptr(), scale.data_ptr(), M, n, 7 * 64, None, 1, 0, None, out.data_ptr(),
                                 logits.data_ptr(), torch.cuda.current_stream().cuda_stream))
    torch.cuda.synchronize()
    assert torch.equal(logits, logits_ref)
    assert torch.equal(out.cpu(), logits_ref.float().argmax(1).cpu() + 7 * 64)
    assert float(sums.abs().max()) == 0
