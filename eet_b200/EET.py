"""Drop-in for the int8 weight-only part of the reference's pybind11 module ``EET``
(csrc/py11/eet2py.cpp:17-156): the same class and function names, argument order and meaning, backed
by the sm_100a kernels of libeet_b200.so through ctypes.

    import eet_b200.EET as EET            # or eet_b200.install_as_EET(); then `from EET import ...`
    from eet_b200.EET import MetaDesc, LlamaMmha, BaichuanMmha, GatedFeedForwardNetworkInt8, LayerNorm
    from eet_b200.EET import quant_weights, preprocess_weights

Covered: MetaDesc, LlamaMmha, BaichuanMmha, GatedFeedForwardNetworkInt8, LayerNorm (RMSNorm form),
quant_weights, preprocess_weights - everything python/eet/transformers/modeling_llama.py and
modeling_baichuan.py import for ``data_type=torch.int8``.  The fp16/fp32 ops of the reference module
(GatedFeedForwardNetwork, Embedding, the BERT/GPT-2/T5 ops) are not part of this path.

Additions that the reference does not have, all optional: `tp` (a tensor-parallel handle, see
eet_b200.tp) on MetaDesc, and device-resident step counters so that a decode step can be replayed as a
CUDA graph (eet_b200.modeling).
"""
import math

import torch

from . import _lib
from ._lib import EETError, check, lib

__all__ = ["MetaDesc", "LlamaMmha", "BaichuanMmha", "GatedFeedForwardNetworkInt8", "LayerNorm", "quant_weights",
           "preprocess_weights", "unpack_weights", "repack_reference_weights", "gemm_w8a16", "gemm_w8a16_accum",
           "deferred_epilogue", "check_device_status", "EETError"]


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t):
    """Device address of a tensor, or None (NULL) for an empty one - the reference turns
    torch.empty(0) arguments into nullptr the same way (csrc/op/llama_mmha.cpp:27-36,46)."""
    if t is None or t.numel() == 0:
        return None
    return t.data_ptr()


# ---------------------------------------------------------------------------------------------------
# buffer pool (the reference's MManager, csrc/op/mmanager.hpp:118-224): named scratch buffers shared by
# all ops of a device; a request larger than the cached buffer replaces it.
# ---------------------------------------------------------------------------------------------------
class _Pool:
    def __init__(self):
        self.buffers = {}
        self.gemm_ws = {}
        self.step_arena = {}

    def get(self, name, numel, dtype, device):
        key = (name, str(device), dtype)
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.empty(max(int(numel), 1), dtype=dtype, device=device)
            self.buffers[key] = buf
        return buf

    def zeros(self, name, numel, dtype, device):
        """Like get(), but zero-filled when (re)allocated: the fp32 sum buffers of the decode GEMMs, which
        every reader leaves zero again."""
        key = ("z:" + name, str(device), dtype)
        buf = self.buffers.get(key)
        if buf is None or buf.numel() < numel:
            buf = torch.zeros(max(int(numel), 1), dtype=dtype, device=device)
            self.buffers[key] = buf
        return buf

    def gemm_workspace(self, nbytes, device):
        """Zero-initialised split-K scratch; the GEMM leaves it zero after every call."""
        key = str(device)
        buf = self.gemm_ws.get(key)
        if buf is None or buf.numel() < nbytes:
            buf = torch.zeros(int(nbytes), dtype=torch.uint8, device=device)
            self.gemm_ws[key] = buf
        return buf

    def new_step_slot(self, device):
        """One int32 of a per-device arena; the arena is contiguous so that one launch advances all slots."""
        key = str(device)
        arena = self.step_arena.get(key)
        if arena is None:
            arena = {"tensor": torch.zeros(4096, dtype=torch.int32, device=device), "used": 0}
            self.step_arena[key] = arena
        if arena["used"] >= arena["tensor"].numel():
            raise EETError("step arena exhausted: more than 4096 attention ops on one device")
        idx = arena["used"]
        arena["used"] += 1
        return arena["tensor"], idx

    def clear(self):
        self.buffers.clear()
        self.gemm_ws.clear()

    def rezero(self):
        """Puts every buffer that the kernels expect to find zero (the fp32 sum buffers, the split-K scratch) back
        to zero: what a kernel that gave up on a wait left in them is undefined."""
        for key, buf in self.buffers.items():
            if key[0].startswith("z:"):
                buf.zero_()
        for buf in self.gemm_ws.values():
            buf.zero_()


_pool = _Pool()


def clear_buffers():
    """Drops the pooled scratch buffers (MManager::clear, csrc/op/mmanager.hpp:211-214)."""
    _pool.clear()


_STATUS_TEXT = {
    1: "decode GEMM: a shared-memory pipeline wait ran out",
    2: "tensor-core GEMM: a pipeline or tensor-memory wait ran out",
    3: "decode attention: a pipeline wait ran out",
    4: "tensor-parallel exchange: a peer's partial sums never arrived",
    5: "decode attention: the step ran past the end of the KV cache",
}


def check_device_status(tp=None):
    """Reads the device-side status word (synchronises the device).  If a kernel gave up since the last check,
    the pooled fp32 scratch is put back to zero - every later GEMM would otherwise add onto what the failed
    kernel left there - the deferred-output table is dropped, and EETError is raised, as the reference raises
    from check_cuda_error at its next synchronisation point (csrc/op/common.hpp:55-64).  With tensor
    parallelism pass the handle: this rank's peer buffers are cleared as well; the other ranks must do the
    same (TensorParallel.reset_peer_buffers is collective) before the group decodes again."""
    status = _lib.device_status()
    if status == 0:
        return
    _pending.clear()
    _pool.rezero()
    if tp is not None and getattr(tp, "_peer", None) is not None:
        tp._peer.clear_local()
    raise EETError(f"device status {status}: {_STATUS_TEXT.get(status, 'unknown code')}; scratch buffers were re-zeroed")


# ---------------------------------------------------------------------------------------------------
# quantizer / packer entry points
# ---------------------------------------------------------------------------------------------------
def _check_quant_input(weight, quant_type):
    # the checks of symmetric_quantize_last_axis_of_tensor (fpA_intB_gemm_wrapper.cu:31-44)
    if not weight.is_contiguous():
        raise RuntimeError("weight must be contiguous")
    if weight.numel() == 0:
        raise RuntimeError("weight should not be empty tensor")
    if weight.dim() not in (2, 3):
        raise RuntimeError("Invalid dim. The dim of weight should be 2 or 3")
    if weight.dtype not in (torch.float16, torch.float32):
        raise RuntimeError("Invalid datatype. Weight must be FP16 or FP32")
    if quant_type != torch.int8:
        raise RuntimeError("Must be int8 quantization (the int4 path of the reference is not part of this library)")


def quant_weights(origin_weight, quant_type=torch.int8, return_unprocessed_quantized_tensor=False, variant=0,
                  device=None):
    """EET.quant_weights (csrc/py11/eet2py.cpp:152-155 -> symmetric_quantize_last_axis_of_tensor,
    3rdparty/cutlass_kernels/fpA_intB_gemm_wrapper.cu:27-105).

    origin_weight: contiguous fp16/fp32 [K, N] (or [E, K, N]), on the CPU as the reference requires; a
    CUDA tensor is accepted too.  Returns [packed int8 [K,N], scales [N]] or, with
    return_unprocessed_quantized_tensor, [row-major int8, packed, scales]; results live where the input
    lives.  `packed` holds the W8T64 bytes this library's GEMM consumes (opaque, like the reference's).
    The int8 values and scales are bit-identical to the reference's.  variant=1 selects amax/127 with
    clip [-127,127] instead of the reference's amax/128, [-128,127]."""
    _check_quant_input(origin_weight, quant_type)
    src_device = origin_weight.device
    dev = torch.device(device) if device is not None else (
        src_device if src_device.type == "cuda" else torch.device("cuda", torch.cuda.current_device()))
    w = origin_weight.to(dev)
    three_d = w.dim() == 3
    w3 = w if three_d else w.unsqueeze(0)
    E, K, N = w3.shape
    if K % 64 or N % 64:
        raise RuntimeError(f"quant_weights: K={K} and N={N} must be multiples of 64")
    q = torch.empty((E, K, N), dtype=torch.int8, device=dev) if return_unprocessed_quantized_tensor else None
    packed = torch.empty((E, K, N), dtype=torch.int8, device=dev)
    scales = torch.empty((E, N), dtype=w.dtype, device=dev)
    ws_bytes = lib.eet_quantize_w8_workspace_bytes(K, N)
    ws = torch.empty(ws_bytes, dtype=torch.uint8, device=dev)
    with torch.cuda.device(dev):
        for e in range(E):
            check(lib.eet_quantize_w8(w3[e].data_ptr(), int(w.dtype == torch.float32), K, N,
                                      q[e].data_ptr() if q is not None else None, packed[e].data_ptr(),
                                      scales[e].data_ptr(), variant, ws.data_ptr(), ws_bytes, _stream()))
    outs = ([q] if q is not None else []) + [packed, scales]
    outs = [o if three_d else o[0] for o in outs]
    if src_device.type != "cuda":
        outs = [o.cpu() for o in outs]
    return outs


def preprocess_weights(origin_weight, is_int4=False):
    """EET.preprocess_weights (csrc/py11/eet2py.cpp:148-150 -> preprocess_weights_cuda,
    fpA_intB_gemm_wrapper.cu:107-126): row-major int8 [K, N] -> packed bytes of the same shape."""
    if is_int4:
        raise RuntimeError("int4 packing is not part of this library")
    if origin_weight.dtype != torch.int8 or origin_weight.dim() != 2:
        raise RuntimeError("preprocess_weights expects a 2-D int8 tensor")
    src_device = origin_weight.device
    w = origin_weight.contiguous()
    w = w if w.is_cuda else w.cuda()
    K, N = w.shape
    out = torch.empty_like(w)
    with torch.cuda.device(w.device):
        check(lib.eet_pack_w8(w.data_ptr(), K, N, out.data_ptr(), _stream()))
    return out if src_device.type == "cuda" else out.cpu()


def unpack_weights(packed):
    """Inverse of preprocess_weights: W8T64 bytes [K, N] -> row-major int8 [K, N]."""
    src_device = packed.device
    p = packed.contiguous()
    p = p if p.is_cuda else p.cuda()
    K, N = p.shape
    out = torch.empty_like(p)
    with torch.cuda.device(p.device):
        check(lib.eet_unpack_w8(p.data_ptr(), K, N, out.data_ptr(), _stream()))
    return out if src_device.type == "cuda" else out.cpu()


def repack_reference_weights(ref_packed):
    """Bytes packed by the reference for sm75-89 (what an `eet_*_int8.pt` file produced by the reference
    holds) -> W8T64 bytes."""
    src_device = ref_packed.device
    p = ref_packed.contiguous()
    p = p if p.is_cuda else p.cuda()
    K, N = p.shape
    out = torch.empty_like(p)
    with torch.cuda.device(p.device):
        check(lib.eet_repack_ref_w8(p.data_ptr(), K, N, out.data_ptr(), _stream()))
    return out if src_device.type == "cuda" else out.cpu()


# ---------------------------------------------------------------------------------------------------
# GEMM helper shared by the ops
# ---------------------------------------------------------------------------------------------------
def gemm_w8a16(x, packed_w, scale, out=None, residual=None, gate=None):
    """out[M, N] = x[M, K] @ dequant(packed_w) (+ residual), or gated_silu(gate, x @ dequant(packed_w)) with `gate`
    (the gate projection of a gated FFN; may be `out` itself).  x fp16 CUDA contiguous; packed_w int8 [K, N]
    W8T64 bytes; scale fp16 [N].  The functional form of fastertransformer::gemm_fp16_int_bias_act as the
    ops call it (csrc/op/llama_mmha.cpp:319-331)."""
    K, N = packed_w.shape
    M = x.numel() // K
    if out is None:
        out = torch.empty((M, N), dtype=torch.float16, device=x.device)
    if gate is not None and residual is not None:
        raise RuntimeError("gemm_w8a16: residual and gate exclude each other")
    second, epilogue = (gate, 2) if gate is not None else (residual, 1 if residual is not None else 0)
    ws_bytes = lib.eet_gemm_w8a16_workspace_bytes(M, N, K)
    ws = _pool.gemm_workspace(ws_bytes, x.device)
    check(lib.eet_gemm_w8a16(x.data_ptr(), packed_w.data_ptr(), scale.data_ptr(), out.data_ptr(), M, N, K,
                             _ptr(second), epilogue, ws.data_ptr(), ws.numel(), _stream()))
    return out


def _linear(x, w, scale, out, residual=None):
    """One projection of an op: W8A16 when w is int8 (packed), else the fp16 twin - w fp16 [K, N] row-major
    through cuBLAS, as the reference's is_int8 == false branches do (cublasGemmEx in
    csrc/op/llama_mmha.cpp:288-310, csrc/op/gated_ffn.cpp), then the residual with this library's kernel."""
    if w.dtype == torch.int8:
        return gemm_w8a16(x, w, scale, out=out, residual=residual)
    torch.matmul(x, w, out=out)
    if residual is not None:
        check(lib.eet_add_residual(out.data_ptr(), residual.data_ptr(), out.numel(), _stream()))
    return out


def gemm_w8a16_accum(x, packed_w, sums, packed_w2=None, sums2=None):
    """sums[M, N] += x[M, K] @ q (unscaled int8 values); optionally the same for a second weight in the same
    launch.  The decode-regime half of gemm_w8a16: whoever reads `sums` applies scale / residual."""
    K, N = packed_w.shape
    M = x.numel() // K
    check(lib.eet_gemm_w8a16_accum(x.data_ptr(), packed_w.data_ptr(), sums.data_ptr(), M, N, K,
                                   None if packed_w2 is None else packed_w2.data_ptr(),
                                   None if sums2 is None else sums2.data_ptr(), _stream()))


def argmax_rows(logits2d):
    """Greedy token choice: [rows] int64 index of the largest value of each row of a CUDA fp16 matrix (the
    smallest index on ties, like torch.argmax); rows may be strided."""
    rows, n = logits2d.shape
    if logits2d.dtype != torch.float16 or not logits2d.is_cuda or logits2d.stride(1) != 1:
        raise RuntimeError("argmax_rows: a CUDA fp16 matrix with contiguous rows is required")
    out = torch.empty(rows, dtype=torch.int64, device=logits2d.device)
    check(lib.eet_argmax_rows(logits2d.data_ptr(), out.data_ptr(), rows, n, logits2d.stride(0) if rows > 1 else n,
                              _stream()))
    return out


def gather_rows(table, ids, out=None):
    """Token-embedding lookup: out[..., :] = table[ids[...]] for a CUDA fp16 table [V, n] and int64 ids."""
    V, n = table.shape
    if table.dtype != torch.float16 or not table.is_cuda or not table.is_contiguous():
        raise RuntimeError("gather_rows: a contiguous CUDA fp16 table is required")
    flat = ids.reshape(-1).to(device=table.device, dtype=torch.int64).contiguous()
    if out is None:
        out = torch.empty((flat.numel(), n), dtype=torch.float16, device=table.device)
    check(lib.eet_gather_rows(table.data_ptr(), flat.data_ptr(), out.data_ptr(), flat.numel(), n, V, _stream()))
    return out.view(*ids.shape, n)


# ---------------------------------------------------------------------------------------------------
# deferred epilogues (decode fast path)
# ---------------------------------------------------------------------------------------------------
class _Pending:
    """An op output whose fp16 values do not exist yet: fp32 GEMM sums + scale + residual.  The next op of
    this module that receives the tensor finishes it inside its own first kernel.  With tensor parallelism
    `peer` = (PeerBuffers, which buffer): the sums are this rank's partial sums and the finishing kernel
    also adds the other ranks' over NVLink."""
    __slots__ = ("sums", "scale", "residual", "out", "peer")

    def __init__(self, sums, scale, residual, out, peer=None):
        self.sums, self.scale, self.residual, self.out, self.peer = sums, scale, residual, out, peer


_pending = {}
_defer = [False]
_DECODE_MAX_M = 64       # below the tensor-core GEMM's first M
_DECODE_MAX_M_TP = 64    # rows of the tensor-parallel peer buffers (tp.PeerBuffers.ROWS)


def _defer_ok(M, desc):
    """Whether an op called with M rows may leave its last projection unfinished for the next op."""
    if not (_defer[0] and desc.is_int8):
        return False
    tp = desc.tp
    return M <= (_DECODE_MAX_M_TP if tp is not None and tp.size > 1 else _DECODE_MAX_M)


class deferred_epilogue:
    """Context manager for a chain of decode-step ops of this module (M <= 64): inside
    it an attention / FFN op returns its output tensor *before* the last GEMM's epilogue has run, and the next
    op (attention, FFN or LayerNorm of this module) completes it in its RMSNorm kernel.  Outputs still
    unfinished when the context ends are completed then, so callers outside never see stale memory."""

    def __enter__(self):
        self.prev = _defer[0]
        _defer[0] = True
        return self

    def __exit__(self, *exc):
        _defer[0] = self.prev
        if not _defer[0]:
            flush_pending()
        return False


def flush_pending():
    for p in list(_pending.values()):
        M, N = p.sums.shape
        if p.peer is not None:
            p.peer[0].tp.all_reduce(p.sums)   # not consumed by an op of this module: plain NCCL path
        check(lib.eet_gemm_w8a16_finalize(p.sums.data_ptr(), p.scale.data_ptr(), _ptr(p.residual), p.out.data_ptr(),
                                          M, N, _stream()))
    _pending.clear()


def _norm_head(x2d, gamma, eps, xn):
    """RMSNorm at the head of a block; completes x first when it is a deferred output of the previous block."""
    M, n = x2d.shape
    p = _pending.pop(x2d.data_ptr(), None)
    if p is not None and p.peer is not None:
        pb, which = p.peer
        check(lib.eet_rmsnorm_finalize_tp(p.sums.data_ptr(), pb.inbox_ptrs, pb.tp.size, pb.tp.rank, which,
                                          pb.epochs.data_ptr(), p.scale.data_ptr(), p.residual.data_ptr(),
                                          x2d.data_ptr(), gamma.data_ptr(), xn.data_ptr(), M, n, eps, _stream()))
    elif p is not None:
        check(lib.eet_rmsnorm_finalize(p.sums.data_ptr(), p.scale.data_ptr(), p.residual.data_ptr(), x2d.data_ptr(),
                                       gamma.data_ptr(), xn.data_ptr(), M, n, eps, _stream()))
    else:
        check(lib.eet_rmsnorm(x2d.data_ptr(), gamma.data_ptr(), xn.data_ptr(), M, n, eps, _stream()))
    return xn


# ---------------------------------------------------------------------------------------------------
# MetaDesc
# ---------------------------------------------------------------------------------------------------
class MetaDesc:
    """Shape / dtype descriptor handed to every op (csrc/op/meta_desc.hpp:9-101, binding
    csrc/py11/eet2py.cpp:26-42).  max_seq_len is the prompt cap (sizes scratch), max_full_seq_len the
    KV-cache length.  dtype must be torch.float16; is_int8 selects packed int8 weights (the accelerated
    path) or plain fp16 weights (the twin ops, GEMMs through cuBLAS like the reference).

    `tp` (not in the reference) is an optional eet_b200.tp.TensorParallel handle: the ops then treat their
    weights as this rank's shard (head_num / d_ff already divided by the caller) and all-reduce the output
    of the row-parallel projections before the residual is added."""

    def __init__(self, dtype, batch_size, head_num, hidden_units, layer_num, max_seq_len, max_full_seq_len=1,
                 activation_fn="gelu", d_kv=0, d_ff=0, cuda_device="cuda:0", requires_grad=False, layernorm_eps=1e-6,
                 is_int8=False, tp=None):
        if not (batch_size > 0 and head_num > 0 and layer_num > 0 and max_seq_len > 0 and max_full_seq_len > 0):
            raise RuntimeError("MetaDesc: batch_size, head_num, layer_num, max_seq_len, max_full_seq_len must be > 0")
        if requires_grad:
            raise RuntimeError("EET now only support inference")
        self.dtype = dtype
        self.batch_size = int(batch_size)
        self.head_num = int(head_num)
        self.hidden_units = int(hidden_units)
        self.layer_num = int(layer_num)
        self.max_seq_len = int(max_seq_len)
        self.max_full_seq_len = int(max_full_seq_len)
        self.activation_fn = activation_fn
        self.d_kv = int(d_kv)
        self.d_ff = int(d_ff)
        self.device = torch.device(cuda_device)
        if self.device.type != "cuda":
            raise RuntimeError("EET now only support CUDA")
        self.layernorm_eps = float(layernorm_eps)
        self.is_int8 = bool(is_int8)
        self.tp = tp

    def _require_half(self, who, int8=None):
        if self.dtype != torch.float16:
            raise RuntimeError(f"{who}: this library serves dtype=torch.float16 only")
        if int8 is not None and self.is_int8 != int8:
            raise RuntimeError(f"{who}: MetaDesc.is_int8 must be {int8} for this op")

    @property
    def weight_dtype(self):
        return torch.int8 if self.is_int8 else torch.float16


def _rmsnorm(x2d, gamma, eps, out):
    M, n = x2d.shape
    check(lib.eet_rmsnorm(x2d.data_ptr(), gamma.data_ptr(), out.data_ptr(), M, n, eps, _stream()))
    return out


# ---------------------------------------------------------------------------------------------------
# attention ops
# ---------------------------------------------------------------------------------------------------
class _MmhaBase:
    """State and flow shared by LlamaMmha and BaichuanMmha: RMSNorm -> W8A16 QKV GEMM -> (rotary) ->
    attention over the per-layer KV cache -> W8A16 output GEMM + residual
    (csrc/op/llama_mmha.cpp:114-266, csrc/op/baichuan_mmha.cpp:80-216)."""

    ROPE = True

    def __init__(self, desc, QKV_weights, QKV_scale, Q_bias, K_bias, V_bias, Output_weights, Output_scale,
                 Output_bias, layernorm_weights, layernorm_bias):
        desc._require_half(type(self).__name__)
        for name, b in (("Q_bias", Q_bias), ("K_bias", K_bias), ("V_bias", V_bias), ("Output_bias", Output_bias),
                        ("layernorm_bias", layernorm_bias)):
            if b is not None and b.numel() != 0:
                # the half-precision rotary kernel of the reference refuses biases as well
                # (csrc/core/self_add_bias.cu:479-481); LLaMA/Baichuan have none
                raise RuntimeError(f"{type(self).__name__}: {name} must be empty (RMSNorm, bias-free projections)")
        self.desc = desc
        # the op keeps the tensors alive itself; the reference keeps raw pointers and relies on Python
        self.qkv_w, self.qkv_s = QKV_weights, QKV_scale
        self.out_w, self.out_s = Output_weights, Output_scale
        self.ln_w = layernorm_weights
        if desc.d_kv == 0:
            self.size_per_head = desc.hidden_units // desc.head_num
            self.inner_dim = desc.hidden_units
        else:
            self.size_per_head = desc.d_kv
            self.inner_dim = desc.d_kv * desc.head_num
        if self.size_per_head != 128:
            raise RuntimeError("attention: only head size 128 is supported")
        for t, shape, what in ((self.qkv_w, (desc.hidden_units, 3 * self.inner_dim), "QKV_weights"),
                               (self.out_w, (self.inner_dim, desc.hidden_units), "Output_weights")):
            if tuple(t.shape) != shape or t.dtype != desc.weight_dtype or not t.is_cuda or not t.is_contiguous():
                raise RuntimeError(f"{what} must be a contiguous CUDA {desc.weight_dtype} tensor of shape {shape}, "
                                   f"got {tuple(t.shape)} {t.dtype}")
        dev = desc.device
        H, D, T = desc.head_num, self.size_per_head, desc.max_full_seq_len
        # per-layer caches, [batch][head][time][dim] so that one (batch, head) history is contiguous
        self.k_cache = torch.zeros((desc.batch_size, H, T, D), dtype=torch.float16, device=dev)
        self.v_cache = torch.zeros_like(self.k_cache)
        self.step_ = 1
        self._arena, self._slot = _pool.new_step_slot(dev)
        self.use_device_step = False
        self.rope_base = 10000.0
        self._slopes = None

    # -- helpers ------------------------------------------------------------------------------------
    def _project(self, ctx2d, inp, B, S):
        """Output projection + residual (LlamaMmha::project, llama_mmha.cpp:428-469: the residual is added
        whatever add_residual says)."""
        d = self.desc
        out = _pool.get("self_mask_attn_cache", d.batch_size * d.max_seq_len * d.hidden_units, torch.float16, d.device)
        out = out[: B * S * d.hidden_units].view(B * S, d.hidden_units)
        inp2d = inp.reshape(B * S, d.hidden_units)
        if _defer_ok(B * S, d):
            peer = None
            if d.tp is not None and d.tp.size > 1:
                # row-parallel: the ranks' fp32 partial sums are added before scale, residual and rounding -
                # by the next block's first kernel, straight from the peers' memory
                pb = d.tp.peer_buffers(d.hidden_units, d.device)
                sums, peer = pb.buffer(0, B * S), (pb, 0)
            else:
                sums = _pool.zeros("out_sums", d.batch_size * d.hidden_units, torch.float32, d.device)
                sums = sums[: B * S * d.hidden_units].view(B * S, d.hidden_units)
            gemm_w8a16_accum(ctx2d, self.out_w, sums)
            _pending[out.data_ptr()] = _Pending(sums, self.out_s, inp2d, out, peer)
        elif d.tp is None or d.tp.size == 1:
            _linear(ctx2d, self.out_w, self.out_s, out, residual=inp2d)
        else:
            _linear(ctx2d, self.out_w, self.out_s, out)
            d.tp.all_reduce(out)
            check(lib.eet_add_residual(out.data_ptr(), inp2d.data_ptr(), out.numel(), _stream()))
        return out.view(B, S, d.hidden_units)

    def _check_input(self, inp):
        d = self.desc
        if inp.dtype != torch.float16 or not inp.is_cuda or inp.dim() != 3 or inp.shape[2] != d.hidden_units:
            raise RuntimeError("input must be a CUDA fp16 tensor [batch, seq, hidden]")
        if not inp.is_contiguous():
            raise RuntimeError("input must be contiguous")
        if inp.shape[0] > d.batch_size:
            raise RuntimeError("cur_batch_size_ must be less than or equal to max_batch_size_")

    def forward(self, input, pre_padding_len, reorder_state, pre_layernorm, add_residual, first_pass,
                relative_attention_bias=None):
        """Same signature as the reference (csrc/py11/eet2py.cpp:73-86).  pre_layernorm / add_residual are
        accepted and ignored exactly as the reference ignores them: the norm always comes first and the
        residual is always added."""
        self._check_input(input)
        with torch.cuda.device(self.desc.device):
            if first_pass:
                return self._forward_full(input, pre_padding_len, relative_attention_bias)
            return self._forward_inc(input, pre_padding_len, reorder_state, relative_attention_bias)

    __call__ = forward

    def _forward_full(self, inp, pre_padding_len, bias):
        d = self.desc
        B, S, h = inp.shape
        if S > d.max_seq_len or S > d.max_full_seq_len:
            raise RuntimeError("cur_seq_len must be less than or equal to max_seq_len / max_full_seq_len")
        H, D = d.head_num, self.size_per_head
        M = B * S
        cap = d.batch_size * d.max_seq_len
        xn = _pool.get("layernorm", cap * h, torch.float16, d.device)[: M * h].view(M, h)
        _norm_head(inp.view(M, h), self.ln_w, d.layernorm_eps, xn)
        qkv = _pool.get("qkv_full", cap * 3 * self.inner_dim, torch.float16, d.device)[: M * 3 * self.inner_dim]
        qkv = qkv.view(M, 3 * self.inner_dim)
        _linear(xn, self.qkv_w, self.qkv_s, qkv)
        q = _pool.get("q_buf", cap * self.inner_dim, torch.float16, d.device)[: M * self.inner_dim]
        check(lib.eet_qkv_split_store(qkv.data_ptr(), q.data_ptr(), self.k_cache.data_ptr(), self.v_cache.data_ptr(),
                                      B, S, H, D, d.max_full_seq_len, int(self.ROPE), self.rope_base, _stream()))
        ctx = _pool.get("dst", cap * self.inner_dim, torch.float16, d.device)[: M * self.inner_dim]
        alibi = None
        if not self.ROPE:
            if bias is None or bias.numel() == 0:
                raise RuntimeError("BaichuanMmha: relative_attention_bias [H, S, S] is required")
            if tuple(bias.shape) != (H, S, S) or bias.dtype != torch.float16 or not bias.is_contiguous():
                raise RuntimeError(f"relative_attention_bias must be contiguous fp16 [{H}, {S}, {S}]")
            alibi = bias
        check(lib.eet_prefill_mha(q.data_ptr(), self.k_cache.data_ptr(), self.v_cache.data_ptr(), ctx.data_ptr(),
                                  B, S, H, D, d.max_full_seq_len, _ptr(pre_padding_len), _ptr(alibi), S, _stream()))
        out = self._project(ctx.view(M, self.inner_dim), inp, B, S)
        self.step_ = S
        return out

    def _forward_inc(self, inp, pre_padding_len, reorder_state, bias):
        d = self.desc
        B, S, h = inp.shape
        if S != 1:
            raise RuntimeError("incremental decoding takes one token per sequence")
        self.step_ += 1
        if self.step_ > d.max_full_seq_len:
            raise RuntimeError("Exceed the maximum step length")
        H, D = d.head_num, self.size_per_head
        xn = _pool.get("layernorm_inc", d.batch_size * h, torch.float16, d.device)[: B * h].view(B, h)
        _norm_head(inp.view(B, h), self.ln_w, d.layernorm_eps, xn)
        qkv, qkv_sums = None, None
        if _defer_ok(B, d):
            # the attention kernel finishes the projection itself: fp16(sums * scale)
            qkv_sums = _pool.zeros("qkv_sums", d.batch_size * 3 * self.inner_dim, torch.float32, d.device)
            qkv_sums = qkv_sums[: B * 3 * self.inner_dim].view(B, 3 * self.inner_dim)
            gemm_w8a16_accum(xn, self.qkv_w, qkv_sums)
        else:
            qkv = _pool.get("qkv_inc", d.batch_size * 3 * self.inner_dim, torch.float16, d.device)
            qkv = qkv[: B * 3 * self.inner_dim].view(B, 3 * self.inner_dim)
            _linear(xn, self.qkv_w, self.qkv_s, qkv)
        if reorder_state is not None and reorder_state.numel() != 0:
            self._reorder(reorder_state, B)
        ctx = _pool.get("context_buf", d.batch_size * self.inner_dim, torch.float16, d.device)[: B * self.inner_dim]
        alibi, alibi_stride, slopes = None, 0, None
        if not self.ROPE:
            if self.use_device_step:
                slopes = self._alibi_slopes()
            else:
                if bias is None or bias.numel() == 0:
                    raise RuntimeError("BaichuanMmha: relative_attention_bias [H, 1, step] is required")
                if bias.shape[0] != H or bias.shape[-1] < self.step_ or not bias.is_contiguous():
                    raise RuntimeError(f"relative_attention_bias must be contiguous fp16 [{H}, 1, >={self.step_}]")
                alibi, alibi_stride = bias, bias.shape[-1]
        step_dev = None
        if self.use_device_step:
            step_dev = self._arena.data_ptr() + 4 * self._slot
        check(lib.eet_decode_mha(_ptr(qkv), _ptr(qkv_sums), _ptr(self.qkv_s), self.k_cache.data_ptr(),
                                 self.v_cache.data_ptr(), ctx.data_ptr(),
                                 B, H, D, d.max_full_seq_len, self.step_, step_dev, _ptr(pre_padding_len),
                                 _ptr(alibi), alibi_stride, _ptr(slopes), int(self.ROPE), self.rope_base, 0,
                                 _stream()))
        return self._project(ctx.view(B, self.inner_dim), inp, B, 1)

    def _reorder(self, reorder_state, B):
        """Beam search: reorder the cache rows first, as LlamaMmha::forward_inc does
        (llama_mmha.cpp:250-252); step_ already counts the token being added, whose slot is still empty."""
        d = self.desc
        H, D = d.head_num, self.size_per_head
        hist = self.step_ - 1
        nbytes = lib.eet_reorder_kv_workspace_bytes(B, H, D, hist)
        ws = _pool.get("reorder_ws", nbytes // 2, torch.float16, d.device)
        idx = reorder_state.to(device=d.device, dtype=torch.int64).contiguous()
        check(lib.eet_reorder_kv(self.k_cache.data_ptr(), self.v_cache.data_ptr(), idx.data_ptr(), B, H, D,
                                 d.max_full_seq_len, hist, ws.data_ptr(), nbytes, _stream()))

    def _alibi_slopes(self):
        return self._slopes

    # -- device-resident step (used by the CUDA-graph decode path) -------------------------------------
    def sync_device_step(self):
        """Copies the host step counter into this op's device slot."""
        self._arena[self._slot] = self.step_


class LlamaMmha(_MmhaBase):
    """EET.LlamaMmha (csrc/py11/eet2py.cpp:73-86, csrc/op/llama_mmha.{hpp,cpp}): LLaMA / Baichuan-7B
    attention block with NeoX rotary embedding."""
    ROPE = True


class BaichuanMmha(_MmhaBase):
    """EET.BaichuanMmha (csrc/py11/eet2py.cpp:58-71, csrc/op/baichuan_mmha.{hpp,cpp}): Baichuan-13B
    attention block, no rotary embedding, ALiBi bias passed as relative_attention_bias."""
    ROPE = False

    def set_alibi_slopes(self, slopes):
        """fp32 [head_num] slopes of this op's heads; lets the decode kernel form the bias row
        fp16(slope * t) itself, which is what the mask the reference's Python builds contains
        (python/eet/transformers/modeling_baichuan.py:70-80)."""
        self._slopes = slopes.to(device=self.desc.device, dtype=torch.float32).contiguous()


# ---------------------------------------------------------------------------------------------------
# feed-forward op
# ---------------------------------------------------------------------------------------------------
class GatedFeedForwardNetworkInt8:
    """EET.GatedFeedForwardNetworkInt8 (csrc/py11/eet2py.cpp:126-134, csrc/op/gated_ffn_int8.{hpp,cpp}):
    RMSNorm -> act(x.W0) * (x.W1) -> .W_out (+ residual)."""

    INT8 = True

    def __init__(self, desc, Intermediate_0_weights, Intermediate_0_scale, Intermediate_0_bias,
                 Intermediate_1_weights, Intermediate_1_scale, Intermediate_1_bias, Output_weights, Output_scale,
                 Output_bias, layernorm_weights, layernorm_bias, ffn_cache_name="out_cache"):
        desc._require_half(type(self).__name__, int8=self.INT8)
        if desc.activation_fn != "silu":
            # the reference prints "unsupported activation" for unknown names and supports gelu/relu gates
            # too (gated_ffn_int8.cpp:40-61); the LLaMA/Baichuan path uses silu only
            raise RuntimeError(f"GatedFeedForwardNetworkInt8: activation '{desc.activation_fn}' is not supported (silu only)")
        for name, b in (("Intermediate_0_bias", Intermediate_0_bias), ("Intermediate_1_bias", Intermediate_1_bias),
                        ("Output_bias", Output_bias), ("layernorm_bias", layernorm_bias)):
            if b is not None and b.numel() != 0:
                raise RuntimeError(f"GatedFeedForwardNetworkInt8: {name} must be empty")
        self.desc = desc
        self.d_ff = desc.d_ff if desc.d_ff != 0 else desc.hidden_units * 4
        self.w0, self.s0 = Intermediate_0_weights, Intermediate_0_scale
        self.w1, self.s1 = Intermediate_1_weights, Intermediate_1_scale
        self.w_out, self.s_out = Output_weights, Output_scale
        self.ln_w = layernorm_weights
        self.cache_name = ffn_cache_name
        h = desc.hidden_units
        for t, shape, what in ((self.w0, (h, self.d_ff), "Intermediate_0_weights"),
                               (self.w1, (h, self.d_ff), "Intermediate_1_weights"),
                               (self.w_out, (self.d_ff, h), "Output_weights")):
            if tuple(t.shape) != shape or t.dtype != desc.weight_dtype or not t.is_cuda or not t.is_contiguous():
                raise RuntimeError(f"{what} must be a contiguous CUDA {desc.weight_dtype} tensor of shape {shape}, "
                                   f"got {tuple(t.shape)} {t.dtype}")

    def forward(self, input, pre_layernorm=True, add_residual=True):
        d = self.desc
        if input.dtype != torch.float16 or not input.is_cuda or not input.is_contiguous():
            raise RuntimeError("input must be a contiguous CUDA fp16 tensor [batch, seq, hidden]")
        if not pre_layernorm:
            raise RuntimeError("GatedFeedForwardNetworkInt8: the post-layernorm form is not part of the int8 LLaMA path")
        B, S, h = input.shape
        M = B * S
        cap = d.batch_size * d.max_seq_len
        with torch.cuda.device(d.device):
            xn = _pool.get("layernorm_tensor", cap * h, torch.float16, d.device)[: M * h].view(M, h)
            _norm_head(input.view(M, h), self.ln_w, d.layernorm_eps, xn)
            act = _pool.get("ffn_inner_act", cap * self.d_ff, torch.float16, d.device)[: M * self.d_ff].view(M, self.d_ff)
            out = _pool.get(self.cache_name, cap * h, torch.float16, d.device)[: M * h].view(M, h)
            inp2d = input.view(M, h)
            deferred = _defer_ok(M, d)
            if deferred:
                # gate and up in one launch, their epilogues inside the SwiGLU kernel
                gs = _pool.zeros("gate_sums", d.batch_size * self.d_ff, torch.float32, d.device)[: M * self.d_ff].view(M, self.d_ff)
                us = _pool.zeros("up_sums", d.batch_size * self.d_ff, torch.float32, d.device)[: M * self.d_ff].view(M, self.d_ff)
                gemm_w8a16_accum(xn, self.w0, gs, self.w1, us)
                check(lib.eet_swiglu_finalize(gs.data_ptr(), self.s0.data_ptr(), us.data_ptr(), self.s1.data_ptr(),
                                              act.data_ptr(), M, self.d_ff, _stream()))
            else:
                _linear(xn, self.w0, self.s0, act)
                if self.w1.dtype == torch.int8:
                    # the gated activation runs in the up projection's epilogue, on the gate values already in `act`
                    gemm_w8a16(xn, self.w1, self.s1, out=act, gate=act)
                else:
                    lin = _pool.get("ffn_inner_linear", cap * self.d_ff, torch.float16, d.device)[: M * self.d_ff].view(M, self.d_ff)
                    _linear(xn, self.w1, self.s1, lin)
                    check(lib.eet_swiglu(act.data_ptr(), lin.data_ptr(), M, self.d_ff, _stream()))
            if deferred and add_residual:
                peer = None
                if d.tp is not None and d.tp.size > 1:
                    pb = d.tp.peer_buffers(h, d.device)   # row-parallel partial sums, see LlamaMmha._project
                    sums, peer = pb.buffer(1, M), (pb, 1)
                else:
                    sums = _pool.zeros("down_sums", d.batch_size * h, torch.float32, d.device)[: M * h].view(M, h)
                gemm_w8a16_accum(act, self.w_out, sums)
                _pending[out.data_ptr()] = _Pending(sums, self.s_out, inp2d, out, peer)
            elif d.tp is None or d.tp.size == 1:
                _linear(act, self.w_out, self.s_out, out, residual=inp2d if add_residual else None)
            else:
                _linear(act, self.w_out, self.s_out, out)
                d.tp.all_reduce(out)
                if add_residual:
                    check(lib.eet_add_residual(out.data_ptr(), inp2d.data_ptr(), out.numel(), _stream()))
        return out.view(B, S, h)

    __call__ = forward


class GatedFeedForwardNetwork(GatedFeedForwardNetworkInt8):
    """EET.GatedFeedForwardNetwork (csrc/py11/eet2py.cpp:117-124, csrc/op/gated_ffn.{hpp,cpp}): the fp16 twin
    the reference builds when data_type is torch.float16 (modeling_llama.py:118-123).  Same flow with fp16
    weights [in, out] and no scales."""

    INT8 = False

    def __init__(self, desc, Intermediate_0_weights, Intermediate_0_bias, Intermediate_1_weights, Intermediate_1_bias,
                 Output_weights, Output_bias, layernorm_weights, layernorm_bias, ffn_cache_name="out_cache"):
        super().__init__(desc, Intermediate_0_weights, None, Intermediate_0_bias, Intermediate_1_weights, None,
                         Intermediate_1_bias, Output_weights, None, Output_bias, layernorm_weights, layernorm_bias,
                         ffn_cache_name)


# ---------------------------------------------------------------------------------------------------
# Embedding op
# ---------------------------------------------------------------------------------------------------
class Embedding:
    """EET.Embedding (csrc/py11/eet2py.cpp:136-141, csrc/op/embedding.{hpp,cpp}).  The reference's LLaMA and
    Baichuan models import this name but look tokens up with torch.nn.Embedding
    (modeling_llama.py:36,281-283); it is provided so that `from EET import Embedding` keeps working and
    is plain tensor indexing: word + token-type + position rows (embedding.cpp:105-137), optional
    LayerNorm with bias (the BERT/GPT form; :83-94)."""

    def __init__(self, desc, embedding_weights, position_weights, token_type_weights, layernorm_weights, layernorm_bias,
                 emb_cache_name="emb_cache"):
        self.desc = desc
        self.word, self.pos, self.tok = embedding_weights, position_weights, token_type_weights
        self.ln_w, self.ln_b = layernorm_weights, layernorm_bias
        self.cache_name = emb_cache_name

    def forward_transformers(self, input_ids, position_ids, token_type_ids, if_layernorm):
        d = self.desc
        B, S = input_ids.shape
        if B > d.batch_size or S > d.max_seq_len:
            raise RuntimeError("Embedding: input exceeds batch_size / max_seq_len of the MetaDesc")
        out = _pool.get(self.cache_name, d.batch_size * d.max_seq_len * d.hidden_units, d.dtype, d.device)
        out = out[: B * S * d.hidden_units].view(B, S, d.hidden_units)
        torch.index_select(self.word, 0, input_ids.reshape(-1), out=out.view(B * S, -1))
        if token_type_ids is not None and token_type_ids.numel() != 0:
            out += self.tok[token_type_ids].expand(B, S, -1)
        if position_ids is not None and position_ids.numel() != 0:
            out += self.pos[position_ids].expand(B, S, -1)
        if if_layernorm:
            out.copy_(torch.nn.functional.layer_norm(out.float(), (d.hidden_units,), self.ln_w.float(),
                                                     None if self.ln_b is None or self.ln_b.numel() == 0
                                                     else self.ln_b.float(), d.layernorm_eps))
        return out

    def forward_fairseq(self, *args, **kwargs):
        raise RuntimeError("Embedding.forward_fairseq: the fairseq sinusoidal form is not part of the LLaMA/Baichuan path")


# ---------------------------------------------------------------------------------------------------
# LayerNorm op
# ---------------------------------------------------------------------------------------------------
class LayerNorm:
    """EET.LayerNorm (csrc/py11/eet2py.cpp:143-145, csrc/op/layer_norm.cpp:8-33).  With an empty beta it is
    RMSNorm, the only form on the LLaMA/Baichuan path; the op owns its output tensor
    [batch, max_seq_len, hidden]."""

    def __init__(self, desc, gamma, beta):
        if desc.dtype != torch.float16:
            raise RuntimeError("LayerNorm: fp16 only")
        if beta is not None and beta.numel() != 0:
            raise RuntimeError("LayerNorm: only the RMSNorm form (empty beta) is part of this library")
        self.desc = desc
        self.gamma = gamma
        self.output = torch.zeros((desc.batch_size, desc.max_seq_len, desc.hidden_units), dtype=torch.float16,
                                  device=desc.device)

    def layer_norm(self, input_tensor):
        B, S, h = input_tensor.shape
        out = self.output.view(-1)[: B * S * h].view(B * S, h)
        with torch.cuda.device(self.desc.device):
            _norm_head(input_tensor.reshape(B * S, h), self.gamma, self.desc.layernorm_eps, out)
        return out.view(B, S, h)


def alibi_slopes(n_head):
    """Slopes of _get_interleave (python/eet/transformers/modeling_baichuan.py:51-64)."""
    def pow2(n):
        start = 2 ** (-(2 ** -(math.log2(n) - 3)))
        return [start * start ** i for i in range(n)]
    if math.log2(n_head).is_integer():
        return pow2(n_head)
    c = 2 ** math.floor(math.log2(n_head))
    return pow2(c) + alibi_slopes(2 * c)[0::2][: n_head - c]
