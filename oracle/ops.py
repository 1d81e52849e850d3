"""TEST INFRASTRUCTURE - not part of the product.

torch-on-CPU restatement of the reference's W8A16 GEMM, the decode / prefill attention around it and
the glue kernels between them, written from the reference's CUDA sources (which cannot run on sm_90+
and have no CPU path).  Only ``tests/``, the smoke check and the CPU-baseline legs of ``bench.py`` may
import this module.

PARITY UNPINNED for everything in this file: the reference ships no test, golden vector or CPU
implementation for these functions, and its GPU kernels refuse to run on the build hardware, so these
restatements are anchored on the cited source lines only.  (The quantizer/packer in ``w8.py`` is pinned.)

All functions take and return CPU tensors; "fp16" below means the value is rounded through
torch.float16 at the point where the reference holds it in a ``half``.
"""
import math

import torch

F16 = torch.float16
F32 = torch.float32


def _h(x):
    """Round through fp16 and come back to fp32 (a value the reference keeps in a `half`)."""
    return x.to(F16).to(F32)


# ------------------------------------------------------------------------------------------ GEMM
def dequant(q: torch.Tensor, scale: torch.Tensor, exact: bool = True) -> torch.Tensor:
    """q int8 [K,N], scale fp16 [N] -> fp32 [K,N].  exact=True mirrors the reference, which multiplies
    fp16(q) by the fp16 scale in fp16 (cutlass_extensions/.../warp/mma_tensorop_dequantizer.h:259-274)
    so every weight is rounded to fp16 before the MMA; exact=False is the plain fp32 product."""
    w = q.to(F32) * scale.to(F32)[None, :]
    return _h(w) if exact else w


def gemm_w8a16(x: torch.Tensor, q: torch.Tensor, scale: torch.Tensor, exact: bool = True) -> torch.Tensor:
    """C[M,N] fp16 = A[M,K] fp16 x dequant(B) with fp32 accumulation and one fp16 rounding at the end
    (fpA_intB_gemm/fpA_intB_gemm_template.h:48-177, default_fpA_intB_traits.h:110,
    epilogue_helpers.h:73-80).  No bias, no activation: every hot-path call passes nullptr
    (csrc/op/llama_mmha.cpp:319-331)."""
    return (x.to(F32) @ dequant(q, scale, exact)).to(F16)


def gemm_fp16(x: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    """The fp16 twin of the projection: x [M,K] fp16 times w [K,N] fp16 (cublasGemmEx in
    csrc/op/llama_mmha.cpp:288-310 with the compute type of csrc/op/meta_desc.hpp:47).  Restated with fp32
    accumulation and one fp16 rounding; the reference accumulates in fp16, whose extra error the tests'
    tolerance covers."""
    return _h(x.float() @ w.float())


def linear(x, w, scale, exact=True):
    """Dispatch used by DecoderOracle: scale None means fp16 weights [K,N]."""
    return gemm_fp16(x, w) if scale is None else gemm_w8a16(x, w, scale, exact)


def gemm_w8a16_fp32(x, q, scale):
    """The tolerance reference: fp32 dequantize-then-matmul computed in float64, returned as float64."""
    return x.double() @ (q.double() * scale.double()[None, :])


# ------------------------------------------------------------------------------------------ glue
def rmsnorm(x: torch.Tensor, gamma: torch.Tensor, eps: float) -> torch.Tensor:
    """T5norm1_kernel_opt<half> (csrc/core/layer_norm.cu:490-531): fp32 sum of squares over the row,
    rsqrtf(mean + eps), x * inv * gamma in fp32, one rounding to fp16."""
    xf = x.to(F32)
    inv = torch.rsqrt((xf * xf).sum(-1, keepdim=True) / x.shape[-1] + eps)
    return (xf * inv * gamma.to(F32)).to(F16)


def rope_coef(dim: int, t, base: float = 10000.0):
    """rotary_embedding_coefficient (csrc/core/common.cuh:176-180): for pair index i in [0, dim/2):
    angle = t / base^(2i/dim) in fp32; returns (cos, sin) fp32 [..., dim/2]."""
    i = torch.arange(dim // 2, dtype=F32)
    denom = torch.pow(torch.tensor(base, dtype=F32), (2 * i) / float(dim))
    ang = torch.as_tensor(t, dtype=F32)[..., None] / denom
    return torch.cos(ang), torch.sin(ang)


def rope_neox(v: torch.Tensor, t) -> torch.Tensor:
    """apply_rotary_embedding (csrc/core/common.cuh:213-226) as used by fused_QKV_neox_rotary_transpose
    (csrc/core/self_add_bias.cu:369-403): pairs (i, i + D/2), fp32 math, each output rounded to fp16.
    v: [..., D] fp16; t broadcastable to v.shape[:-1] (the position of every row)."""
    D = v.shape[-1]
    c, s = rope_coef(D, t)
    a, b = v[..., : D // 2].to(F32), v[..., D // 2:].to(F32)
    return torch.cat([(a * c - b * s).to(F16), (b * c + a * s).to(F16)], -1)


def gated_silu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """gated_silu<half> (csrc/core/activation_kernel.cu:106-124): exp(-gate) in fp32 rounded to fp16,
    then up * gate / (1 + e) evaluated left to right in fp16 arithmetic."""
    e = torch.exp(-gate.to(F32)).to(F16)
    prod = _h(up.to(F32) * gate.to(F32))          # in2 * in1 (half2 multiply)
    den = _h(1.0 + e.to(F32))                     # half_one2 + e
    return (prod / den).to(F16)


def add_residual(out: torch.Tensor, inp: torch.Tensor) -> torch.Tensor:
    """add_input<half> (csrc/core/add_bias.cu:22-28): out + in in fp16."""
    return (out.to(F32) + inp.to(F32)).to(F16)


# ------------------------------------------------------------------------------------------ attention
def decode_attention(q, k_new, v_new, k_cache, v_cache, step, pad_len=None, alibi=None):
    """masked_attention_kernel_opt (csrc/core/attention_dispatch.cu:140-324) and, with `alibi`,
    t5_masked_attention_kernel (:1155-1336).

    q, k_new, v_new: [B, H, D] fp16 (already rotated for LLaMA).  k_cache, v_cache: [B, H, T, D] fp16 -
    the history of each (batch, head); which physical layout holds it is private to an implementation.
    The new K,V are written at index step-1 (:224-229, :288-294) before use.  pad_len: [B] int or None;
    positions t < pad_len get logit -1e20 -> -inf in fp16 (:219-220).  alibi: [H, step] fp16 added to the
    fp16 logit in fp16 arithmetic (:1249).  Returns ctx [B, H, D] fp16.

    Numerics kept: fp32 dot of fp16 values times fp16(1/sqrt(D)), logit rounded to fp16 (:238), fp32
    softmax with max subtraction, denominator + 1e-6 (:255-271), fp32 P.V (:278-297).  Not kept: the
    bounce of per-warp partial sums through fp16 shared memory (:298-313), which depends on the
    launch shape."""
    B, H, D = q.shape
    k_cache[:, :, step - 1] = k_new
    v_cache[:, :, step - 1] = v_new
    scalar = torch.tensor(math.sqrt(1.0 / D), dtype=F32).to(F16).to(F32)
    kf = k_cache[:, :, :step].to(F32)
    logits = torch.einsum("bhd,bhtd->bht", q.to(F32), kf) * scalar
    logits = _h(logits)
    if alibi is not None:
        logits = _h(logits + alibi.to(F32)[None, :, :step])
    if pad_len is not None:
        t = torch.arange(step)[None, None, :]
        logits = torch.where(t < pad_len.view(B, 1, 1), torch.tensor(float("-inf")), logits)
    m = torch.maximum(logits.max(-1, keepdim=True).values, torch.tensor(-1e20))
    p = torch.exp(logits - m)
    p = p * (1.0 / (p.sum(-1, keepdim=True) + 1e-6))
    ctx = torch.einsum("bht,bhtd->bhd", p, v_cache[:, :, :step].to(F32))
    return ctx.to(F16)


def prefill_attention(q, k, v, pad_len=None, alibi=None):
    """Prefill self-attention of LlamaMmha::forward_full (csrc/op/llama_mmha.cpp:354-426): scores =
    fp16(1/sqrt(D)) * Q.K^T held in fp16 (:354-373), softmax_kernel_gpt2 (csrc/core/gpt2_self_softmax.cu
    :8-57: causal, columns left of pad_len masked, rows above pad_len zeroed, denominator + 1e-6,
    probabilities stored in fp16), then P.V (:397-416) to fp16.  With `alibi` ([H, S, S] fp16):
    masked_softmax_kernel (:161-240) = softmax(scores + alibi) over j <= i, no padding handling.

    q, k, v: [B, H, S, D] fp16 -> ctx [B, H, S, D] fp16.  The reference's cuBLAS calls accumulate in
    fp16 (csrc/op/meta_desc.hpp:45-48); this restatement accumulates in fp32 and rounds where the
    reference stores fp16, so it is the tighter of the two."""
    B, H, S, D = q.shape
    scalar = torch.tensor(math.sqrt(1.0 / D), dtype=F32).to(F16).to(F32)
    sc = _h(torch.einsum("bhid,bhjd->bhij", q.to(F32), k.to(F32)) * scalar)
    i = torch.arange(S)[:, None]
    j = torch.arange(S)[None, :]
    causal = (j <= i)[None, None]
    neg = torch.tensor(-1e20)
    if alibi is not None:
        sc = sc + alibi.to(F32)[None]
        sc = torch.where(causal, sc, neg)
        row_ok = torch.ones(B, 1, S, 1, dtype=torch.bool)
    else:
        if pad_len is None:
            pad_len = torch.zeros(B, dtype=torch.long)
        pl = pad_len.view(B, 1, 1, 1)
        sc = torch.where(j[None, None] < pl, sc + neg, sc)
        sc = torch.where(causal, sc, neg)
        row_ok = (i[None, None] >= pl)
    m = sc.max(-1, keepdim=True).values
    p = torch.where(causal, torch.exp(sc - m), torch.tensor(0.0))
    p = p / (p.sum(-1, keepdim=True) + 1e-6)
    p = torch.where(row_ok, p, torch.tensor(0.0))
    p = _h(p)
    return torch.einsum("bhij,bhjd->bhid", p, v.to(F32)).to(F16)


# ------------------------------------------------------------------------------------------ ALiBi
def alibi_slopes(n_head: int):
    """_get_interleave (python/eet/transformers/modeling_baichuan.py:51-64)."""
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]
    if math.log2(n_head).is_integer():
        return pow2(n_head)
    c = 2 ** math.floor(math.log2(n_head))
    return pow2(c) + alibi_slopes(2 * c)[0::2][: n_head - c]


def alibi_mask(n_head: int, max_pos: int) -> torch.Tensor:
    """_gen_alibi_mask (modeling_baichuan.py:70-80): [H, L, L] fp32.  Its `position_point - diag` step
    turns the positions -(L-1)..0 into 0..L-1, so the bias is slope_h * j on and below the diagonal and
    -inf above it, the same for every row."""
    slopes = torch.tensor(alibi_slopes(n_head), dtype=F32)
    alibi = slopes[:, None, None] * torch.arange(max_pos)[None, None, :]
    upper = torch.triu(torch.full((max_pos, max_pos), float("-inf")), 1)
    return upper[None] + alibi


# ------------------------------------------------------------------------------------------ blocks
class LayerWeights:
    """One decoder layer in un-packed form: row-major int8 [K,N] + fp16 scale [N] per projection (or fp16
    [K,N] with scale None for the fp16 twin ops), RMSNorm gammas in fp16.  qkv is the fused [h, 3*inner] matrix in Q-block, K-block, V-block column order
    (python/eet/transformers/modeling_llama.py:745-753)."""

    def __init__(self, qkv, qkv_s, out, out_s, gate, gate_s, up, up_s, down, down_s, ln1, ln2):
        self.qkv, self.qkv_s, self.out, self.out_s = qkv, qkv_s, out, out_s
        self.gate, self.gate_s, self.up, self.up_s, self.down, self.down_s = gate, gate_s, up, up_s, down, down_s
        self.ln1, self.ln2 = ln1, ln2


class DecoderOracle:
    """LlamaMmha / BaichuanMmha + GatedFeedForwardNetworkInt8 for a stack of layers
    (csrc/op/llama_mmha.cpp:114-266, csrc/op/baichuan_mmha.cpp:80-216, csrc/op/gated_ffn_int8.cpp:98-132;
    layer loop python/eet/transformers/modeling_llama.py:161-297).  rope=True is LLaMA / Baichuan-7B,
    rope=False with ALiBi is Baichuan-13B."""

    def __init__(self, layers, n_head, head_dim, eps, max_len, batch, rope=True, exact=True):
        self.layers, self.H, self.D, self.eps, self.rope, self.exact = layers, n_head, head_dim, eps, rope, exact
        self.kc = [torch.zeros(batch, n_head, max_len, head_dim, dtype=F16) for _ in layers]
        self.vc = [torch.zeros(batch, n_head, max_len, head_dim, dtype=F16) for _ in layers]
        self.step = 0
        self.alibi = None if rope else alibi_mask(n_head, max_len).to(F16)
        self.max_len = max_len

    def _attn_block(self, li, x, first_pass, pad_len):
        L = self.layers[li]
        B, S, h = x.shape
        H, D = self.H, self.D
        xn = rmsnorm(x, L.ln1, self.eps)
        qkv = linear(xn.reshape(B * S, h), L.qkv, L.qkv_s, self.exact).view(B, S, 3, H, D)
        q, k, v = (qkv[:, :, i].transpose(1, 2).contiguous() for i in range(3))  # [B,H,S,D]
        if first_pass:
            if self.rope:
                t = torch.arange(S).view(1, 1, S)       # position = index in the prompt, padding ignored
                q, k = rope_neox(q, t), rope_neox(k, t)
            self.kc[li][:B, :, :S] = k
            self.vc[li][:B, :, :S] = v
            # the model hands the [:S, :S] corner of the mask to the op (modeling_baichuan.py:284-287,312-315)
            al = None if self.rope else self.alibi[:, :S, :S]
            ctx = prefill_attention(q, k, v, pad_len, al)
        else:
            step = self.step
            if self.rope:
                q, k = rope_neox(q, step - 1), rope_neox(k, step - 1)
            al = None if self.rope else self.alibi[:, step - 1, :step]
            ctx = decode_attention(q[:, :, 0], k[:, :, 0], v[:, :, 0], self.kc[li][:B], self.vc[li][:B], step,
                                   pad_len, al).unsqueeze(2)
        ctx = ctx.transpose(1, 2).reshape(B * S, H * D)
        o = linear(ctx, L.out, L.out_s, self.exact).view(B, S, h)
        return add_residual(o, x)   # the residual is always added (llama_mmha.cpp:461-463)

    def _ffn_block(self, li, x):
        L = self.layers[li]
        B, S, h = x.shape
        xn = rmsnorm(x, L.ln2, self.eps).reshape(B * S, h)
        g = linear(xn, L.gate, L.gate_s, self.exact)
        u = linear(xn, L.up, L.up_s, self.exact)
        a = gated_silu(g, u)
        o = linear(a, L.down, L.down_s, self.exact).view(B, S, h)
        return add_residual(o, x)

    def reorder(self, index):
        """Beam search: cache row b takes the history of row index[b] before the step
        (reorderKV_kernel, csrc/core/transpose.cu:136-162; called first in llama_mmha.cpp:250-252)."""
        n = len(index)
        for li in range(len(self.layers)):
            self.kc[li][:n] = self.kc[li][index].clone()
            self.vc[li][:n] = self.vc[li][index].clone()

    def forward(self, x, first_pass, pad_len=None):
        """x: [B, S, h] fp16.  first_pass resets the step counter to S (llama_mmha.cpp:121,195); every
        later call advances it by one (:210)."""
        if first_pass:
            self.step = x.shape[1]
        else:
            self.step += 1
        for li in range(len(self.layers)):
            x = self._attn_block(li, x, first_pass, pad_len)
            x = self._ffn_block(li, x)
        return x
