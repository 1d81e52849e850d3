"""Host-side logic that needs no GPU: descriptor validation, quantizer input checks, weight-dictionary
conversion rules, tensor-parallel shard plans."""
import pytest
import torch

from eet_b200 import EET, tp
from eet_b200.modeling import convert_name, gen_alibi_mask


def test_metadesc_validation():
    d = EET.MetaDesc(dtype=torch.float16, batch_size=2, head_num=2, hidden_units=256, layer_num=1, max_seq_len=8,
                     max_full_seq_len=16, activation_fn="silu", d_ff=512, cuda_device="cuda:0", layernorm_eps=1e-6,
                     is_int8=True)
    assert d.max_full_seq_len == 16 and d.is_int8
    with pytest.raises(RuntimeError):
        EET.MetaDesc(torch.float16, 0, 2, 256, 1, 8)
    with pytest.raises(RuntimeError):
        EET.MetaDesc(torch.float16, 1, 2, 256, 1, 8, cuda_device="cpu")
    with pytest.raises(RuntimeError):
        EET.MetaDesc(torch.float16, 1, 2, 256, 1, 8, requires_grad=True)


def test_quant_weights_rejects_what_the_reference_rejects():
    with pytest.raises(RuntimeError, match="contiguous"):
        EET.quant_weights(torch.zeros(64, 128).t(), torch.int8)
    with pytest.raises(RuntimeError, match="empty"):
        EET.quant_weights(torch.zeros(0, 64), torch.int8)
    with pytest.raises(RuntimeError, match="dim"):
        EET.quant_weights(torch.zeros(64), torch.int8)
    with pytest.raises(RuntimeError, match="FP16 or FP32"):
        EET.quant_weights(torch.zeros(64, 64, dtype=torch.float64), torch.int8)
    with pytest.raises(RuntimeError, match="int8"):
        EET.quant_weights(torch.zeros(64, 64), torch.float16)


def test_convert_name_rules():
    assert convert_name("layers.0.mlp.down_proj.weight") == "layer.0.ffn.output.weight"
    assert convert_name("layers.7.self_attn.qkv_proj.weight") == "layer.7.self_attn.qkv_proj.weight"
    with pytest.raises(KeyError):
        convert_name("layers.0.x", "gpt2")


def test_shard_plan():
    plan = tp.shard_plan(32, 11008, 2)
    assert plan == [((0, 16), (0, 5504)), ((16, 32), (5504, 11008))]
    # 86 strips of 128 over 8 ranks: uneven, contiguous, complete
    plan8 = tp.shard_plan(32, 11008, 8)
    widths = [hi - lo for _, (lo, hi) in plan8]
    assert sum(widths) == 11008 and set(widths) == {10 * 128, 11 * 128}
    assert all(plan8[i][1][1] == plan8[i + 1][1][0] for i in range(7))
    with pytest.raises(ValueError):
        tp.shard_plan(32, 11008, 3)     # heads do not divide
    with pytest.raises(ValueError):
        tp.ff_range(128, 0, 4)          # fewer tiles than ranks


def test_alibi_mask_shape():
    m = gen_alibi_mask(8, 5)
    assert m.shape == (8, 5, 5) and torch.isinf(m[0, 0, 1]) and m[0, 4, 0] == 0


def test_every_name_the_reference_models_import_exists():
    """The import lines of python/eet/transformers/modeling_llama.py:35-42, modeling_baichuan.py:34-42 and
    encoder_decoder.py:22 must keep working against this module."""
    import sys
    import eet_b200
    eet_b200.install_as_EET()
    try:
        from EET import MetaDesc, Embedding, GatedFeedForwardNetworkInt8, GatedFeedForwardNetwork  # noqa: F401
        from EET import LlamaMmha, BaichuanMmha, LayerNorm, preprocess_weights, quant_weights      # noqa: F401
    finally:
        sys.modules.pop("EET", None)


def test_convert_weights_data_types():
    from eet_b200 import modeling
    with pytest.raises(RuntimeError):
        modeling.convert_llama_weights({}, torch.float32)
    w = {"model.layers.0.mlp.down_proj.weight": torch.randn(8, 16).half(),
         "model.layers.0.self_attn.q_proj.weight": torch.randn(8, 8).half(),
         "model.layers.0.self_attn.k_proj.weight": torch.randn(8, 8).half(),
         "model.layers.0.self_attn.v_proj.weight": torch.randn(8, 8).half()}
    d = modeling.convert_llama_weights(w, torch.float16)
    # [K = in, N = out] like the reference's fp branch (modeling_llama.py:773-782); no scales
    assert d["layer.0.ffn.output.weight"].shape == (16, 8) and d["layer.0.ffn.output.weight"].dtype == torch.float16
    assert d["layer.0.self_attn.qkv_proj.weight"].shape == (8, 24)
    assert not any(k.endswith(".scale") for k in d)


def test_fp16_weight_shards_are_plain_slices():
    """Tensor-parallel shards of the fp16 twin's weights: columns [lo, hi) of each of the Q | K | V blocks
    (column-parallel) and rows [lo, hi) (row-parallel); no scales."""
    import types
    from eet_b200 import modeling
    fake_tp = types.SimpleNamespace(size=2, rank=1)
    w = torch.arange(4 * 12, dtype=torch.float16).view(4, 12)          # K = 4, N = 3 blocks of 4
    cols, s = modeling._shard_cols(w, modeling._EMPTY, fake_tp, 2, 4, 3)
    assert s.numel() == 0 and cols.shape == (4, 6)
    assert torch.equal(cols, torch.cat([w[:, 2:4], w[:, 6:8], w[:, 10:12]], 1))
    rows, s = modeling._shard_rows(w, modeling._EMPTY, fake_tp, 1, 3)
    assert torch.equal(rows, w[1:3]) and rows.is_contiguous()
    same, _ = modeling._shard_cols(w, modeling._EMPTY, None, 0, 4, 3)
    assert same is w


def test_graph_mode_decode_step_refuses_to_run_past_the_cache():
    """With use_cuda_graph the step advances on the device, out of sight of the eager path's check
    ("Exceed the maximum step length", LlamaMmha::forward_inc): decode_step must raise on the host before
    anything is launched - here there is no GPU at all, so a launch would fail differently."""
    import types
    from eet_b200 import modeling
    lm = modeling.EETLlamaForCausalLM.__new__(modeling.EETLlamaForCausalLM)
    attn = types.SimpleNamespace(step_=16)
    lm.model = types.SimpleNamespace(desc=types.SimpleNamespace(device=torch.device("cpu"), tp=None),
                                     reorder_state=torch.empty(0).long(), layers=[types.SimpleNamespace(attention=attn)],
                                     max_full_seq_len=16, past_kv_length=16)
    lm.use_cuda_graph, lm._graph = True, None
    with pytest.raises(RuntimeError, match="Exceed the maximum step length"):
        lm.decode_step(torch.zeros(2, 1, dtype=torch.long))
    assert attn.step_ == 16


def test_device_status_codes_are_named():
    assert set(EET._STATUS_TEXT) == {1, 2, 3, 4, 5}


def test_vocab_range_covers_the_vocabulary_in_whole_tiles():
    for vocab, size in ((32000, 8), (32000, 4), (64000, 8), (1024, 8), (320, 2)):
        ranges = [tp.vocab_range(vocab, r, size) for r in range(size)]
        assert ranges[0][0] == 0 and ranges[-1][1] == vocab
        assert all(ranges[i][1] == ranges[i + 1][0] for i in range(size - 1))
        assert all(lo % 64 == 0 and hi % 64 == 0 and hi > lo for lo, hi in ranges)
    widths = {hi - lo for lo, hi in (tp.vocab_range(32000, r, 8) for r in range(8))}
    assert widths == {31 * 128, 32 * 128}        # 250 strips of 128 over 8 ranks: uneven
    with pytest.raises(ValueError):
        tp.vocab_range(32001, 0, 2)
    with pytest.raises(ValueError):
        tp.vocab_range(128, 0, 4)
