"""Host-side model wrappers for int8 weight-only LLaMA and Baichuan, mirroring the reference's
python/eet/transformers/modeling_llama.py and modeling_baichuan.py for ``data_type=torch.int8``: the same
converted-weight dictionary schema, the same class names, constructor arguments and call signatures,
built on the ops of eet_b200.EET.

Beyond the reference: `tp=` shards the model Megatron-style over a tensor-parallel group
(eet_b200.tp), and the decode step can be replayed as a CUDA graph (`use_cuda_graph=True`), which removes
the host launch cost of the ~300 kernels of one step.
"""
import re

import torch
import torch.nn as nn

from . import EET
from . import tp as tp_mod
from .EET import GatedFeedForwardNetworkInt8 as eet_gated_ffn
from .EET import GatedFeedForwardNetwork as eet_gated_ffn_fp16
from .EET import LayerNorm as eet_layernorm
from .EET import LlamaMmha as eet_masked_attention
from .EET import BaichuanMmha as eet_baichuan_13b_attention
from .EET import MetaDesc as meta_desc
from .EET import quant_weights as quant_and_preprocess_weights
from ._lib import check, lib

__all__ = ["convert_name", "convert_llama_weights", "convert_baichuan_weights", "EETLlamaModel",
           "EETLlamaForCausalLM", "EETBaichuanModel", "EETBaichuanForCausalLM", "CausalLMOutput", "gen_alibi_mask"]

_EMPTY = torch.empty(0)

# transformers_llama_mapping / transformers_baichuan_mapping (python/eet/utils/mapping.py:256-296)
_RENAMES = (
    (r"^layers\.", "layer."),
    (r"\.self_attn\.W_pack\.", ".self_attn.qkv_proj."),
    (r"\.self_attn\.o_proj\.", ".self_attn.out_proj."),
    (r"\.input_layernorm\.", ".self_attn.layernorm."),
    (r"\.mlp\.gate_proj\.", ".ffn.intermediate_0."),
    (r"\.mlp\.up_proj\.", ".ffn.intermediate_1."),
    (r"\.mlp\.down_proj\.", ".ffn.output."),
    (r"\.post_attention_layernorm\.", ".ffn.layernorm."),
)


def convert_name(org_key, model_name="llama"):
    """HF parameter name -> EET name (python/eet/utils/mapping.py:298-324 with the llama / baichuan
    tables): layers.N.self_attn.o_proj.weight -> layer.N.self_attn.out_proj.weight, and so on."""
    if model_name not in ("llama", "baichuan"):
        raise KeyError(model_name)
    key = org_key
    for pat, rep in _RENAMES:
        key = re.sub(pat, rep, key)
    return key


def _check_data_type(data_type):
    if data_type not in (torch.int8, torch.float16):
        raise RuntimeError("this library serves data_type=torch.int8 (W8A16) and torch.float16 only")


def _convert(model_dict, data_type, model_attr, fuse_qkv):
    model_dict = dict(model_dict)
    if fuse_qkv:
        # q, k, v -> one [3h, h] matrix in Q, K, V block order (modeling_llama.py:745-753)
        qkv = {}
        for k in [k for k in model_dict if any(p in k for p in ("q_proj", "k_proj", "v_proj"))]:
            v = model_dict.pop(k)
            kk = k[k.find("layers."):]
            qkv.setdefault(kk.split(".")[1], {})[kk.split(".")[3]] = v
        for layer_id, parts in qkv.items():
            model_dict[f"layers.{layer_id}.self_attn.qkv_proj.weight"] = torch.cat(
                [parts["q_proj"], parts["k_proj"], parts["v_proj"]], dim=0)
    out = {}
    for k, v in model_dict.items():
        if k.startswith(model_attr + "."):
            k = k[len(model_attr) + 1:]
        if "layers." in k:
            k = convert_name(k[k.find("layers."):])
            if ".weight" in k and v.dim() == 2:
                w = v.transpose(0, 1).contiguous()  # [K, N], K = in-features (modeling_llama.py:764-768)
                if data_type == torch.int8:
                    packed, scale = quant_and_preprocess_weights(w.half() if w.dtype == torch.bfloat16 else w,
                                                                 torch.int8, False)
                    out[k] = packed
                    out[k.replace(".weight", ".scale")] = scale
                    continue
                v = w
        out[k] = v if data_type == torch.int8 else v.to(data_type)
    return out


def convert_llama_weights(model_dict, data_type=torch.int8, model_attr="model"):
    """HF LLaMA state dict -> EET dictionary (modeling_llama.py:739-784).  With data_type=torch.int8 every
    2-D layer weight becomes `<name>.weight` (packed int8 [K, N]) + `<name>.scale` ([N]); with
    torch.float16 it is the transposed fp16 matrix [K, N]."""
    _check_data_type(data_type)
    return _convert(model_dict, data_type, model_attr, fuse_qkv=True)


def convert_baichuan_weights(model_dict, data_type=torch.int8, model_attr="model"):
    """HF Baichuan state dict (fused W_pack) -> EET dictionary (modeling_baichuan.py:572-603)."""
    _check_data_type(data_type)
    return _convert(model_dict, data_type, model_attr, fuse_qkv=False)


def gen_alibi_mask(n_head, max_pos):
    """_gen_alibi_mask (modeling_baichuan.py:70-80): [H, L, L] fp32, slope_h * j on and below the diagonal,
    -inf above."""
    slopes = torch.tensor(EET.alibi_slopes(n_head), dtype=torch.float32)
    alibi = slopes[:, None, None] * torch.arange(max_pos)[None, None, :]
    upper = torch.triu(torch.full((max_pos, max_pos), float("-inf")), 1)
    return upper[None] + alibi


class CausalLMOutput:
    """The fields of transformers' CausalLMOutputWithPast that the reference fills (modeling_llama.py:485-491)."""

    def __init__(self, logits, hidden_states, loss=None):
        self.loss, self.logits, self.hidden_states = loss, logits, hidden_states
        self.past_key_values = None
        self.attentions = None


# ---------------------------------------------------------------------------------------------------
def _shard_cols(packed, scale, tp, lo, hi, blocks=1):
    """Column-parallel shard of a packed [K, N] weight: N is seen as `blocks` equal blocks (3 for the fused
    Q|K|V matrix) and the rank keeps columns [lo, hi) of every block.  Per-channel scales shard with the
    columns, so quantizing before sharding gives the single-GPU values."""
    if tp is None or tp.size == 1:
        return packed, scale
    K, N = packed.shape
    if packed.dtype != torch.int8:   # fp16 twin: plain [K, N] matrix, no scale
        return packed.view(K, blocks, N // blocks)[:, :, lo:hi].reshape(K, -1).contiguous(), scale
    q = EET.unpack_weights(packed).view(K, blocks, N // blocks)
    s = scale.view(blocks, N // blocks)
    return EET.preprocess_weights(q[:, :, lo:hi].reshape(K, -1).contiguous()), s[:, lo:hi].reshape(-1).contiguous()


def _shard_rows(packed, scale, tp, lo, hi):
    """Row-parallel shard: the full matrix was quantized first (so the scales equal the single-GPU ones
    and are replicated); the rank keeps rows [lo, hi) of K."""
    if tp is None or tp.size == 1:
        return packed, scale
    if packed.dtype != torch.int8:
        return packed[lo:hi].contiguous(), scale
    q = EET.unpack_weights(packed)
    return EET.preprocess_weights(q[lo:hi].contiguous()), scale


class _DecoderLayer:
    """EETLlamaDecoderLayer / EETBaichuanDecoderLayer (modeling_llama.py:150-199): attention op + FFN op
    and the tensors they point at."""

    NAMES = ("ln1", "ln2", "qkv_w", "qkv_s", "out_w", "out_s", "w0", "s0", "w1", "s1", "w2", "s2")

    @staticmethod
    def _tensors(config, model_dict, layer_id):
        """This rank's tensors of one layer, in NAMES order, from an EET dictionary."""
        dev = config.device
        tp = config.tp
        p = f"layer.{layer_id}."

        def cuda(name):
            return model_dict[p + name].to(dev)

        def scale(name):
            # the fp16 twin has no scales: the reference passes torch.empty(0) (modeling_llama.py:63-64)
            return cuda(name).half() if config.is_int8 else _EMPTY

        a_lo, a_hi = config.shard_attn   # inner-dim columns of this rank inside each of Q, K, V
        f_lo, f_hi = config.shard_ffn    # d_ff channels of this rank
        qkv_w, qkv_s = _shard_cols(cuda("self_attn.qkv_proj.weight"), scale("self_attn.qkv_proj.scale"), tp, a_lo, a_hi, 3)
        out_w, out_s = _shard_rows(cuda("self_attn.out_proj.weight"), scale("self_attn.out_proj.scale"), tp, a_lo, a_hi)
        w0, s0 = _shard_cols(cuda("ffn.intermediate_0.weight"), scale("ffn.intermediate_0.scale"), tp, f_lo, f_hi)
        w1, s1 = _shard_cols(cuda("ffn.intermediate_1.weight"), scale("ffn.intermediate_1.scale"), tp, f_lo, f_hi)
        w2, s2 = _shard_rows(cuda("ffn.output.weight"), scale("ffn.output.scale"), tp, f_lo, f_hi)
        return (cuda("self_attn.layernorm.weight").half(), cuda("ffn.layernorm.weight").half(), qkv_w, qkv_s, out_w,
                out_s, w0, s0, w1, s1, w2, s2)

    def __init__(self, config, model_dict, layer_id, attention_cls):
        for name, t in zip(self.NAMES, self._tensors(config, model_dict, layer_id)):
            setattr(self, name, t)
        self.config = config
        self.attention = attention_cls(config, self.qkv_w, self.qkv_s, _EMPTY, _EMPTY, _EMPTY, self.out_w, self.out_s,
                                       _EMPTY, self.ln1, _EMPTY)
        if config.is_int8:
            self.feedforward = eet_gated_ffn(config, self.w0, self.s0, _EMPTY, self.w1, self.s1, _EMPTY, self.w2,
                                             self.s2, _EMPTY, self.ln2, _EMPTY, "decoder_out_cache")
        else:
            self.feedforward = eet_gated_ffn_fp16(config, self.w0, _EMPTY, self.w1, _EMPTY, self.w2, _EMPTY, self.ln2,
                                                  _EMPTY, "decoder_out_cache")

    def update(self, model_dict, layer_id):
        """New weights into the tensors the ops (and any captured CUDA graph) already point at: the in-place
        `.copy_()` of EETLlamaSelfMaskedAttention.update / EETGatedFeedForward.update
        (modeling_llama.py:80-93,133-149)."""
        for name, t in zip(self.NAMES, self._tensors(self.config, model_dict, layer_id)):
            getattr(self, name).copy_(t)

    def __call__(self, hidden_states, first_pass=True, pre_padding_len=_EMPTY, reorder_state=_EMPTY,
                 relative_attention_bias=_EMPTY):
        x = self.attention.forward(hidden_states, pre_padding_len, reorder_state, True, True, first_pass,
                                   relative_attention_bias)
        return self.feedforward.forward(x, True, True)


class _ModelBase:
    """EETLlamaModel / EETBaichuanModel (modeling_llama.py:248-437, modeling_baichuan.py:249-330):
    embedding (torch, fp16) -> decoder layers -> final RMSNorm."""

    ATTENTION = eet_masked_attention
    ALIBI = False

    def __init__(self, config, layers, layer_norm, embedding, desc, max_batch, max_prompt_len, max_full_seq_len):
        self.config, self.layers, self.layer_norm, self.embedding, self.desc = config, layers, layer_norm, embedding, desc
        self.max_batch, self.max_prompt_len, self.max_full_seq_len = max_batch, max_prompt_len, max_full_seq_len
        self.pre_padding_len = torch.empty(0).long()
        self.reorder_state = torch.empty(0).long()
        self.past_kv_length = 0
        self.future_mask = None

    @classmethod
    def from_eet(cls, model_dict, cfg, max_batch, max_prompt_seq_len, max_full_seq_len, data_type=torch.int8,
                 device_id=0, tp=None):
        """Same arguments as the reference (modeling_llama.py:330-377) plus `tp`.  data_type torch.int8
        builds the W8A16 ops, torch.float16 the fp16 twins (:336-337)."""
        _check_data_type(data_type)
        torch.set_grad_enabled(False)
        size = 1 if tp is None else tp.size
        rank = 0 if tp is None else tp.rank
        device = f"cuda:{device_id}"
        heads, d_ff = cfg.num_attention_heads, cfg.intermediate_size
        head_dim = cfg.hidden_size // heads
        h_lo, h_hi = tp_mod.head_range(heads, rank, size)
        f_lo, f_hi = tp_mod.ff_range(d_ff, rank, size)
        desc = meta_desc(dtype=torch.float16, batch_size=max_batch, head_num=h_hi - h_lo, hidden_units=cfg.hidden_size,
                         layer_num=cfg.num_hidden_layers, max_seq_len=max_prompt_seq_len,
                         max_full_seq_len=max_full_seq_len, activation_fn=cfg.hidden_act,
                         d_kv=head_dim, d_ff=f_hi - f_lo, cuda_device=device,
                         layernorm_eps=cfg.rms_norm_eps, is_int8=(data_type == torch.int8), tp=tp)
        desc.shard_attn = (h_lo * head_dim, h_hi * head_dim)
        desc.shard_ffn = (f_lo, f_hi)
        embedding = nn.Embedding(cfg.vocab_size, cfg.hidden_size, getattr(cfg, "pad_token_id", None))
        embedding.load_state_dict({"weight": model_dict["embed_tokens.weight"]})
        embedding = embedding.half().to(device)
        attention_cls = cls._attention_class(cfg)
        layers = [_DecoderLayer(desc, model_dict, i, attention_cls) for i in range(cfg.num_hidden_layers)]
        if attention_cls is eet_baichuan_13b_attention:
            slopes = torch.tensor(EET.alibi_slopes(heads), dtype=torch.float32)
            for layer in layers:
                layer.attention.set_alibi_slopes(slopes[h_lo:h_hi])
        layer_norm = eet_layernorm(desc, model_dict["norm.weight"].half().to(device), _EMPTY)
        return cls(cfg, layers, layer_norm, embedding, desc, max_batch, max_prompt_seq_len, max_full_seq_len)

    @classmethod
    def _attention_class(cls, cfg):
        return eet_masked_attention

    def update(self, model_dict):
        """Reloads every weight from an EET dictionary of the same architecture, in place
        (EETLlamaModel.update, modeling_llama.py:299-327)."""
        self.embedding.weight.copy_(model_dict["embed_tokens.weight"].to(self.embedding.weight))
        for i, layer in enumerate(self.layers):
            layer.update(model_dict, i)
        self.layer_norm.gamma.copy_(model_dict["norm.weight"].to(self.layer_norm.gamma))

    def _bias(self, first_pass, seq_len, like):
        return _EMPTY

    def _embed(self, input_ids):
        """Token embeddings [B, S, hidden] into a pooled buffer (the reference calls torch.nn.Embedding,
        modeling_llama.py:281-283; this is the same lookup as one small kernel of this library, which also
        takes part in the programmatic launch chain of a decode step)."""
        B, S = input_ids.shape
        h = self.config.hidden_size
        cap = self.max_batch * self.max_prompt_len
        buf = EET._pool.get("embed_out", cap * h, torch.float16, self.desc.device)[: B * S * h].view(B * S, h)
        return EET.gather_rows(self.embedding.weight, input_ids, out=buf).view(B, S, h)

    def __call__(self, input_ids, first_pass=True, position_ids=None, token_type_ids=None, attention_mask=None,
                 reorder_state=None, context_lengths=None):
        shape = input_ids.size()
        assert shape[0] <= self.max_batch, f"[EET][ERROR] batch size must less than max_batch {self.max_batch}"
        assert shape[1] <= self.max_prompt_len, f"[EET][ERROR] input_ids length must less than max_prompt_len {self.max_prompt_len}"
        if first_pass:
            self.past_kv_length = 0
        if attention_mask is None:
            pre_padding_len = self.pre_padding_len
        else:
            pre_padding_len = torch.sum(1 - attention_mask, 1, True).to(self.desc.device).long()
        if reorder_state is not None:
            self.reorder_state = reorder_state.long()
        x = self._embed(input_ids)
        self.past_kv_length += shape[1]
        bias = self._bias(first_pass, self.past_kv_length, x)
        for layer in self.layers:
            x = layer(x, first_pass=first_pass, pre_padding_len=pre_padding_len, reorder_state=self.reorder_state,
                      relative_attention_bias=bias)
        return self.layer_norm.layer_norm(x)


class EETLlamaModel(_ModelBase):
    pass


class EETBaichuanModel(_ModelBase):
    """Baichuan: 32 layers = the 7B model with rotary embedding (LlamaMmha), anything else = the 13B model
    with ALiBi (BaichuanMmha) - the reference's own switch (modeling_baichuan.py:235,261,308)."""

    @classmethod
    def _attention_class(cls, cfg):
        return eet_masked_attention if cfg.num_hidden_layers == 32 else eet_baichuan_13b_attention

    def _bias(self, first_pass, seq_len, like):
        if self.config.num_hidden_layers == 32:
            return _EMPTY
        heads = self.config.num_attention_heads
        if self.future_mask is None or seq_len > self.future_mask.shape[-1]:
            n = max(seq_len, self.max_full_seq_len)
            self.future_mask = gen_alibi_mask(heads, n).to(like)   # modeling_baichuan.py:270-282
        size = 1 if self.desc.tp is None else self.desc.tp.size
        rank = 0 if self.desc.tp is None else self.desc.tp.rank
        h_lo, h_hi = tp_mod.head_range(heads, rank, size)
        mask = self.future_mask[h_lo:h_hi, :seq_len, :seq_len]
        if not first_pass:
            mask = mask[:, -1:, :]
        return mask.contiguous()


class _LmHead:
    """The lm_head of a causal LM.  By default the reference's: an fp16 torch.nn.Linear, replicated on every rank
    (modeling_llama.py:370-372, called at :471).  With int8=True (not in the reference) the weight is quantized
    like every other projection and runs through this library's W8A16 GEMM, and under tensor parallelism each rank
    keeps only its vocabulary columns (whole 128- or 64-column blocks, tp.vocab_range): a decode step then reads 1/size of
    half the bytes, and the greedy token is chosen from the GEMM's fp32 sums by one kernel that also settles the
    choice between the ranks (eet_lm_head_argmax)."""

    def __init__(self, weight_vh, device, int8, tp, max_rows):
        self.vocab, self.hidden = weight_vh.shape
        self.device, self.int8, self.max_rows = torch.device(device), bool(int8), int(max_rows)
        self.tp = tp if (tp is not None and tp.size > 1 and int8) else None
        self.lo, self.hi = 0, self.vocab
        if not self.int8:
            self.linear = nn.Linear(self.hidden, self.vocab, bias=False)
            self.linear.load_state_dict({"weight": weight_vh})
            self.linear = self.linear.half().to(self.device)
            return
        if self.tp is not None:
            self.lo, self.hi = tp_mod.vocab_range(self.vocab, self.tp.rank, self.tp.size)
        self.w, self.s = self._quantize(weight_vh)

    def _quantize(self, weight_vh):
        w = weight_vh.to(self.device).half().t().contiguous()       # [K = hidden, N = vocab]
        packed, scale = quant_and_preprocess_weights(w, torch.int8, False)
        return _shard_cols(packed, scale.half(), self.tp, self.lo, self.hi)

    @property
    def weight(self):
        return self.linear.weight if not self.int8 else self.w

    def load(self, weight_vh):
        """New weights into the tensors a captured graph already points at."""
        if not self.int8:
            self.linear.weight.copy_(weight_vh.to(self.linear.weight))
            return
        w, s = self._quantize(weight_vh)
        self.w.copy_(w)
        self.s.copy_(s)

    def __call__(self, hidden):
        """Logits [..., vocab] (fp16) for hidden [..., hidden]; a sharded head gathers the ranks' columns."""
        if not self.int8:
            return self.linear(hidden)
        x2d = hidden.reshape(-1, self.hidden)
        local = EET.gemm_w8a16(x2d.contiguous(), self.w, self.s)
        if self.tp is not None:
            import torch.distributed as dist
            ranges = [tp_mod.vocab_range(self.vocab, r, self.tp.size) for r in range(self.tp.size)]
            width = max(hi - lo for lo, hi in ranges)
            padded = torch.zeros((local.shape[0], width), dtype=local.dtype, device=local.device)
            padded[:, : local.shape[1]] = local
            parts = [torch.empty_like(padded) for _ in ranges]
            dist.all_gather(parts, padded, group=self.tp.group)
            local = torch.cat([p[:, : hi - lo] for p, (lo, hi) in zip(parts, ranges)], 1)
        return local.view(*hidden.shape[:-1], self.vocab)

    def greedy(self, hidden2d):
        """Next token ids [B, 1] (int64) for hidden2d [B, hidden]: argmax of the fp16 logits, the smallest index on
        ties, identical on every rank."""
        B = hidden2d.shape[0]
        hidden2d = hidden2d.contiguous()
        world = 1 if self.tp is None else self.tp.size
        if not self.int8 or B > self.max_rows or (world > 1 and B > tp_mod.PeerBuffers.ROWS):
            return EET.argmax_rows(self(hidden2d)).view(-1, 1)
        n = self.hi - self.lo
        sums = EET._pool.zeros("lm_head_sums", self.max_rows * n, torch.float32, self.device)[: B * n].view(B, n)
        out = EET._pool.get("lm_head_ids", self.max_rows, torch.int64, self.device)[:B]
        EET.gemm_w8a16_accum(hidden2d, self.w, sums)
        inbox = epochs = None
        rank = 0
        if world > 1:
            pb = self.tp.peer_buffers(self.hidden, self.device)
            inbox, epochs, rank = pb.argmax_ptrs, pb.argmax_epochs.data_ptr(), self.tp.rank
        check(lib.eet_lm_head_argmax(sums.data_ptr(), self.s.data_ptr(), B, n, self.lo, inbox, world, rank, epochs,
                                     out.data_ptr(), None, torch.cuda.current_stream().cuda_stream))
        return out.view(B, 1)


class _CausalLMBase:
    """EETLlamaForCausalLM / EETBaichuanForCausalLM (modeling_llama.py:441-579): model + lm_head (fp16 through
    torch as in the reference, or int8 and vocabulary-sharded, see _LmHead), called as
    model(input_ids, first_pass=..., attention_mask=...) -> .logits."""

    MODEL = EETLlamaModel

    def __init__(self, config, model, lm_head=None):
        self.config, self.model, self.lm_head = config, model, lm_head
        self.main_input_name = "input_ids"
        self.use_cuda_graph = False
        self._graph = None

    @classmethod
    def from_eet(cls, model_dict, config, max_batch, max_prompt_seq_len, max_full_seq_len, data_type=torch.int8,
                 device_id=0, tp=None, lm_head_int8=False):
        """The reference's arguments (modeling_llama.py:525-546) plus `tp` and `lm_head_int8` (quantize the lm_head
        as well and shard its vocabulary over the tensor-parallel group; the reference keeps it in fp16)."""
        torch.set_grad_enabled(False)
        body = {k: v for k, v in model_dict.items() if "lm_head" not in k}
        model = cls.MODEL.from_eet(body, config, max_batch, max_prompt_seq_len, max_full_seq_len, data_type,
                                   device_id=device_id, tp=tp)
        lm_head = _LmHead(model_dict["lm_head.weight"], f"cuda:{device_id}", lm_head_int8, tp, max_batch)
        return cls(config, model, lm_head)

    @classmethod
    def from_torch(cls, torch_model, max_batch, max_prompt_seq_len, max_full_seq_len, data_type=torch.int8,
                   device_id=0, tp=None, lm_head_int8=False):
        """Converts a HF causal LM held in memory (the directory branch of from_pretrained,
        modeling_llama.py:559-561, without the disk read)."""
        sd = {k: v.half() if v.is_floating_point() else v for k, v in torch_model.state_dict().items()}
        conv = convert_baichuan_weights if any("W_pack" in k for k in sd) else convert_llama_weights
        return cls.from_eet(conv(sd, data_type), torch_model.config, max_batch, max_prompt_seq_len, max_full_seq_len,
                            data_type, device_id=device_id, tp=tp, lm_head_int8=lm_head_int8)

    def update(self, torch_model):
        """Takes new weights from a HF model of the same architecture (re-quantizing them when the model is
        int8) without reallocating anything: EETLlamaForCausalLM.update (modeling_llama.py:518-522)."""
        data_type = torch.int8 if self.model.desc.is_int8 else torch.float16
        sd = {k: v.half() if v.is_floating_point() else v for k, v in torch_model.state_dict().items()}
        conv = convert_baichuan_weights if any("W_pack" in k for k in sd) else convert_llama_weights
        model_dict = conv(sd, data_type)
        self.lm_head.load(model_dict["lm_head.weight"])
        self.model.update({k: v for k, v in model_dict.items() if "lm_head" not in k})

    def __call__(self, input_ids, first_pass=True, position_ids=None, attention_mask=None, reorder_state=None,
                 labels=None, **kwargs):
        hidden = self.model(input_ids=input_ids, first_pass=first_pass, position_ids=position_ids,
                            attention_mask=attention_mask, reorder_state=reorder_state)
        logits = self.lm_head(hidden)
        loss = None
        if labels is not None:
            shift_logits = logits[..., :-1, :].contiguous().view(-1, self.config.vocab_size)
            loss = nn.functional.cross_entropy(shift_logits.float(), labels[..., 1:].contiguous().view(-1))
        return CausalLMOutput(logits, hidden, loss)

    def prepare_inputs_for_generation(self, input_ids, first_pass=True, attention_mask=None, **kwargs):
        """modeling_llama.py:493-516: after the first pass only the newest token is fed."""
        if not first_pass:
            input_ids = input_ids[:, -1:]
        return {"input_ids": input_ids, "attention_mask": attention_mask}

    # -- greedy generation ------------------------------------------------------------------------------
    def _decode_eager(self, ids, pad):
        # the whole chain of ops below belongs to this library, so every projection's epilogue may run
        # inside the kernel that consumes it
        with EET.deferred_epilogue():
            hidden = self.model(input_ids=ids, first_pass=False)
        return self.lm_head.greedy(hidden[:, -1, :])

    def decode_logits(self, ids):
        """Logits [B, 1, vocab] of one decode step for ids [B, 1], computed by the same chain of kernels that
        decode_step() and generate() run (deferred epilogues, fused tensor-parallel exchange), eagerly."""
        with EET.deferred_epilogue():
            hidden = self.model(input_ids=ids, first_pass=False)
        return self.lm_head(hidden)

    def _capture(self, B):
        """Captures one decode step (embedding -> layers -> norm -> lm_head -> argmax) as a CUDA graph.  The
        attention ops read their step from device memory inside the graph; one extra launch at the head of
        the graph advances all of them."""
        m = self.model
        attn = [layer.attention for layer in m.layers]
        arena, first = attn[0]._arena, attn[0]._slot
        assert [a._slot for a in attn] == list(range(first, first + len(attn))), "step slots must be contiguous"
        for a in attn:
            a.sync_device_step()
            a.use_device_step = True
        g = {"ids": torch.zeros((B, 1), dtype=torch.long, device=m.desc.device), "B": B}
        saved = (m.past_kv_length, [a.step_ for a in attn])
        torch.cuda.synchronize()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            check(lib.eet_advance_steps(arena.data_ptr() + 4 * first, len(attn), 1,
                                        torch.cuda.current_stream().cuda_stream))
            g["next"] = self._decode_eager(g["ids"], None)
        # capturing ran the host-side bookkeeping once without executing anything: undo it
        m.past_kv_length = saved[0]
        for a, s in zip(attn, saved[1]):
            a.step_ = s
        g["graph"] = graph
        self._graph = g

    def decode_step(self, ids):
        """One greedy decode step for ids [B, 1] (int64, on the device or in host memory): returns the next ids
        [B, 1] on the device.  With use_cuda_graph the step is captured on its second use and replayed
        afterwards."""
        m = self.model
        dev = m.desc.device
        if not self.use_cuda_graph or m.reorder_state.numel() != 0:
            return self._decode_eager(ids.to(dev, non_blocking=True), None)
        B = ids.shape[0]
        # the captured graph advances the step on the device, where no host check sees it: refuse here, before
        # anything is launched, exactly where the eager path raises (LlamaMmha::forward_inc asserts the same)
        if any(layer.attention.step_ + 1 > m.max_full_seq_len for layer in m.layers):
            raise RuntimeError("Exceed the maximum step length")
        if self._graph is None or self._graph["B"] != B:
            if not getattr(self, "_warmed", False):
                self._warmed = True
                return self._decode_eager(ids.to(dev, non_blocking=True), None)   # first step eagerly: sizes every pooled buffer
            self._capture(B)
        # ids may live in (pinned) host memory: they are copied straight into the graph's input tensor
        g = self._graph
        g["ids"].copy_(ids, non_blocking=True)
        g["graph"].replay()
        m.past_kv_length += 1
        for layer in m.layers:
            layer.attention.step_ += 1
        return g["next"]

    def end_graph(self):
        """Leaves graph mode (e.g. before a new prompt): the ops go back to host-side step counters."""
        for layer in self.model.layers:
            layer.attention.use_device_step = False
        self._graph = None
        self._warmed = False

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens, attention_mask=None):
        """Greedy search in the shape of GenerationMixin_EET.greedy_search
        (python/eet/pipelines/generation.py:1080-1243): one first_pass=True call over the prompt, then one
        token per call; no EOS stop.  Returns [B, prompt + max_new_tokens] ids."""
        self.end_graph()
        if attention_mask is not None and self.use_cuda_graph:
            self.model.pre_padding_len = torch.sum(1 - attention_mask, 1, True).to(self.model.desc.device).long()
        # only the last position's logits are needed to choose the first new token: the lm_head runs on that
        # row alone (the reference computes and discards the logits of every prompt position, modeling_llama.py:471)
        hidden = self.model(input_ids=input_ids, first_pass=True, attention_mask=attention_mask)
        nxt = self.lm_head.greedy(hidden[:, -1, :].contiguous()).clone()
        toks = [input_ids, nxt]
        for _ in range(max_new_tokens - 1):
            if attention_mask is not None and not self.use_cuda_graph:
                hidden = self.model(input_ids=nxt, first_pass=False, attention_mask=attention_mask)
                nxt = self.lm_head.greedy(hidden[:, -1, :]).clone()
            else:
                nxt = self.decode_step(nxt).clone()
            toks.append(nxt)
        if attention_mask is not None:
            self.model.pre_padding_len = torch.empty(0).long()
        out = torch.cat(toks, dim=1)
        EET.check_device_status(self.model.desc.tp)   # a kernel that gave up on a wait must not go unnoticed
        return out

    @torch.no_grad()
    def beam_search(self, input_ids, num_beams, max_new_tokens):
        """Fixed-length beam search in the shape of GenerationMixin_EET.beam_search
        (python/eet/pipelines/generation.py:1399-1600): the prompt is repeated num_beams times (the model must
        have been built with max_batch >= B * num_beams), candidates are ranked by the sum of token
        log-probabilities, and before every step the ops reorder their KV caches with `reorder_state`
        (:1564-1580; LlamaMmha::forward_inc, csrc/op/llama_mmha.cpp:250-252).  No EOS stop and no length
        penalty.  Returns (best sequences [B, prompt + max_new_tokens], their scores [B])."""
        self.end_graph()
        B, S = input_ids.shape
        nb = num_beams
        dev = input_ids.device
        ids = input_ids.repeat_interleave(nb, 0)
        scores = torch.zeros(B, nb, device=dev)
        scores[:, 1:] = -1e9          # the beams start identical: only the first may spawn candidates
        logits = self(ids, first_pass=True).logits[:, -1]
        offs = (torch.arange(B, device=dev) * nb).view(B, 1)
        try:
            for t in range(max_new_tokens):
                logp = torch.log_softmax(logits.float(), -1)
                V = logp.shape[-1]
                cand = (scores.view(B, nb, 1) + logp.view(B, nb, V)).view(B, nb * V)
                scores, idx = cand.topk(nb, -1)
                beam, tok = idx // V, idx % V
                reorder = (beam + offs).view(-1)
                ids = torch.cat([ids[reorder], tok.view(-1, 1)], 1)
                if t + 1 < max_new_tokens:
                    logits = self(ids[:, -1:].contiguous(), first_pass=False, reorder_state=reorder).logits[:, -1]
        finally:
            self.model.reorder_state = torch.empty(0).long()
        EET.check_device_status(self.model.desc.tp)
        best = scores.argmax(-1)
        rows = torch.arange(B, device=dev)
        return ids.view(B, nb, -1)[rows, best], scores[rows, best]


class EETLlamaForCausalLM(_CausalLMBase):
    MODEL = EETLlamaModel


class EETBaichuanForCausalLM(_CausalLMBase):
    MODEL = EETBaichuanModel
