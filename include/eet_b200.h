/*
 * eet_b200 - C ABI of the B200 (sm_100a) int8 weight-only inference path.
 *
 * Every entry point takes plain pointers and sizes; device pointers are raw CUDA device addresses owned
 * by the caller, `stream` is a cudaStream_t passed as void*.  Every function enqueues its work on
 * `stream` and returns immediately: 0 on success, non-zero on failure, in which case eet_last_error()
 * returns a message.  The library allocates no device memory; kernels that need scratch take it from
 * the caller, sized by the matching *_workspace_bytes() function.
 *
 * Each declaration names the interface of the reference project (NetEase-FuXi/EET, paths inside that
 * project) that it stands in for.
 */
#ifndef EET_B200_H
#define EET_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ABI version of this header (4); bumped when a signature changes. */
int eet_abi_version(void);

/* Message of the last failure on the calling thread ("" if none). */
const char* eet_last_error(void);

/* Reads (and clears) the device-side status word of the current device; 0 = no kernel gave up since the last
 * call.  Every wait inside the kernels is bounded: a kernel that gives up records a code and returns normally.
 *   1  decode GEMM: a shared-memory pipeline wait ran out
 *   2  tensor-core GEMM: a pipeline or tensor-memory wait ran out
 *   3  decode attention: a pipeline wait ran out
 *   4  tensor-parallel exchange: a peer's partial sums never arrived
 *   5  decode attention: the device-resident step was outside [1, T_max]; nothing was appended to the cache
 * After a non-zero status the fp32 scratch buffers of the failed call hold undefined values: zero them (and, for
 * the tensor-parallel exchange, the inboxes and epoch counters of every rank) before the next call.
 * Synchronises the device.  The reference reports asynchronous failures the same way, at its next
 * check_cuda_error (csrc/op/common.hpp:55-64). */
int eet_device_status(int* status_out);

/* Number of polls after which a wait on another GPU (the tensor-parallel inbox) gives up
 * on the current device; the default, 1 << 22, is a second or more.  Takes effect for kernels launched after the
 * call; synchronises the device.  No counterpart in the reference (it has no such waits). */
int eet_set_wait_limit(unsigned int polls);

/* ------------------------------------------------------------------------------------------------
 * Quantizer and packer
 * ---------------------------------------------------------------------------------------------- */

/* Scratch needed by eet_quantize_w8: N floats. */
size_t eet_quantize_w8_workspace_bytes(int K, int N);

/*
 * Symmetric per-output-channel int8 quantization of a row-major weight W[K][N] (K = reduction dim),
 * bit-exact with the reference.
 * Replaces: fastertransformer::symmetric_quantize<half,half> / <float,float>
 *           (3rdparty/cutlass_kernels/cutlass_preprocessors.cc:581-678) as reached through
 *           symmetric_quantize_last_axis_of_tensor (3rdparty/cutlass_kernels/fpA_intB_gemm_wrapper.cu:27-105,
 *           Python name EET.quant_weights, csrc/py11/eet2py.cpp:152-155).
 *   w            device, fp16 (w_is_fp32 = 0) or fp32 (1), K % 64 == 0, N % 64 == 0
 *   q_rowmajor   device int8 [K][N], the "unprocessed" tensor; may be NULL
 *   packed       device, K*N bytes in the W8T64 layout consumed by eet_gemm_w8a16
 *   scales       device [N], fp16 when w is fp16, fp32 when w is fp32
 *   variant      0 = reference (amax/128, clip [-128,127]); 1 = amax/127, clip [-127,127]
 *   ws           device scratch of eet_quantize_w8_workspace_bytes(K, N) bytes
 */
int eet_quantize_w8(const void* w, int w_is_fp32, int K, int N, int8_t* q_rowmajor, void* packed, void* scales,
                    int variant, void* ws, size_t ws_bytes, void* stream);

/*
 * Row-major int8 [K][N] -> W8T64 bytes.
 * Replaces: fastertransformer::preprocess_weights (cutlass_preprocessors.cc:536-544; Python name
 *           EET.preprocess_weights, csrc/py11/eet2py.cpp:148-150, wrapper fpA_intB_gemm_wrapper.cu:107-126).
 */
int eet_pack_w8(const int8_t* q_rowmajor, int K, int N, void* packed, void* stream);

/* W8T64 bytes -> row-major int8 [K][N] (no counterpart in the reference; used to re-shard packed
 * weights for tensor parallelism and in tests). */
int eet_unpack_w8(const void* packed, int K, int N, int8_t* q_rowmajor, void* stream);

/* Bytes packed by the reference for sm75-89 (preprocess_weights_for_mixed_gemm,
 * cutlass_preprocessors.cc:497-534) -> W8T64, so checkpoints converted by the reference load unchanged. */
int eet_repack_ref_w8(const void* ref_packed, int K, int N, void* packed, void* stream);

/* ------------------------------------------------------------------------------------------------
 * W8A16 GEMM
 * ---------------------------------------------------------------------------------------------- */

/* Scratch needed by eet_gemm_w8a16 for a problem of this size: M * N fp32 sums up to M = 512 (the stream-K
 * kernels add partial sums there), 128 rows above that (only used when the shape has no large-tile kernel).
 * The scratch must be zero before its first use (e.g. cudaMemset once after allocation); every call leaves
 * it zero again.  Calls that share one scratch buffer must not overlap on the GPU. */
size_t eet_gemm_w8a16_workspace_bytes(int M, int N, int K);

/*
 * C[M][N] (fp16) = A[M][K] (fp16, row-major) x dequant(B), B = W8T64 bytes of a [K][N] int8 matrix,
 * scale fp16 [N].
 * Replaces: fastertransformer::gemm_fp16_int_bias_act<uint8_t>
 *           (3rdparty/cutlass_kernels/fpA_intB_gemm.cu:36-62 -> CutlassFpAIntBGemmRunner::gemm,
 *           fpA_intB_gemm/fpA_intB_gemm_template.h:545-558) as called from
 *           csrc/op/llama_mmha.cpp:313-337,428-447 and csrc/op/gated_ffn_int8.cpp:253-326.
 *   epilogue  0: C = A.B;  1: C = fp16(A.B) + residual in fp16, the add_input kernel that follows the
 *             projection GEMMs in the reference (csrc/core/add_bias.cu:22-28) fused in;  2: C =
 *             gated_silu(residual, fp16(A.B)), i.e. this GEMM is the up projection of a gated FFN and `residual`
 *             holds the gate projection: the reference's gated_act kernel (csrc/core/activation_kernel.cu:106-124,
 *             called from csrc/op/gated_ffn_int8.cpp:290-301) fused in, with its mix of fp32 and fp16 arithmetic.
 *   residual  device fp16 [M][N] for epilogues 1 and 2, else NULL (may alias C)
 * M may be any value >= 0; K and N must be multiples of 64; pointers 16-byte aligned.
 * Kernels: M <= 16 TMA-staged skinny kernel; 16 < M <= 512 (N % 128 == 0) stream-K tcgen05 kernel; above
 * that - and from M = 65 on for shapes (N % 256 == 0) whose 256 x 256 tiles, whole or with their k-blocks split
 * over clusters of 2-4 CTAs, can occupy most of the GPU - tcgen05 kernels with 256 x 256 or 128 x 256 output
 * tiles that need no scratch; shapes none of them takes fall back to the skinny kernel in groups of 128 rows.
 */
int eet_gemm_w8a16(const void* A, const void* packedB, const void* scale, void* C, int M, int N, int K,
                   const void* residual, int epilogue, void* ws, size_t ws_bytes, void* stream);

/*
 * The two halves of eet_gemm_w8a16 for M <= 512 (the decode regime and small prefills), exposed so that the
 * second half can be fused into the kernel that consumes the product.
 *
 * eet_gemm_w8a16_accum ADDS sum_k A[m][k] * q[k][n] (q = the int8 weight values, unscaled) into the fp32
 * buffer sums[M][N]; with packedB2 / sums2 a second weight of the same shape (the FFN "up" projection next
 * to "gate", csrc/op/gated_ffn_int8.cpp:253-301) is walked by the same launch.  Buffers must be zero on
 * entry unless accumulation onto earlier sums is wanted.
 *
 * eet_gemm_w8a16_finalize turns sums into C = fp16(sums * scale) (+ residual, fp16 add) - the epilogue of
 * the reference GEMM (cutlass_extensions epilogue_helpers.h:73-80) and its add_input kernel
 * (csrc/core/add_bias.cu:22-28) - and puts sums back to zero.  eet_rmsnorm_finalize, eet_swiglu_finalize
 * and eet_decode_mha (qkv_sums) do the same inside the next kernel of a decode step.
 */
int eet_gemm_w8a16_accum(const void* A, const void* packedB, float* sums, int M, int N, int K, const void* packedB2,
                         float* sums2, void* stream);
int eet_gemm_w8a16_finalize(float* sums, const void* scale, const void* residual, void* C, int M, int N, void* stream);

/*
 * eet_gemm_w8a16 for M <= 16 without a caller-provided scratch buffer.  It has no counterpart in the
 * reference.  It exists for hosts that may not allocate device memory - a server that gave all of HBM to
 * one arena at start-up, a plugin inside somebody else's process, a decode loop that cannot take the
 * device-wide stall of cudaMalloc - and therefore cannot hand eet_gemm_w8a16 its zeroed fp32 scratch.
 * The scratch is a fixed 2 MiB array inside the library's device image (held by every GPU that loads the
 * library, until the process ends): M * N may not exceed 16 * 32768, M may not exceed 16; larger problems
 * are refused with an error.  The call allocates
 * nothing.  Its first use on a device looks up the array's device address, so make that first call outside
 * any stream capture.  All calls on a device share the array: it is cleared at the start of each call, and
 * two calls that overlap on the GPU (different streams) race.
 */
int eet_gemm_w8a16_noalloc(const void* A, const void* packedB, const void* scale, void* C, int M, int N, int K,
                           const void* residual, int epilogue, void* stream);

/* ------------------------------------------------------------------------------------------------
 * Kernels between the GEMMs
 * ---------------------------------------------------------------------------------------------- */

/* y = x * rsqrt(mean(x^2) + eps) * gamma over rows of length n.
 * Replaces: RMSnorm<half> (csrc/core/layer_norm.cu:580-625 -> T5norm1_kernel_opt :490-531). */
int eet_rmsnorm(const void* x, const void* gamma, void* y, int M, int n, float eps, void* stream);

/*
 * Decode-step head of an attention or FFN block: with sums != NULL, first h = fp16(sums * scale) + residual
 * (finishing the projection GEMM that feeds the block, see eet_gemm_w8a16_finalize) is written to h_out and
 * sums is zeroed; with sums == NULL, h = residual.  Then xn_out = RMSNorm(h) * gamma.
 * Replaces: add_input<half> (csrc/core/add_bias.cu:22-28) + RMSnorm<half> (csrc/core/layer_norm.cu:580-625).
 */
int eet_rmsnorm_finalize(float* sums, const void* scale, const void* residual, void* h_out, const void* gamma,
                         void* xn_out, int M, int n, float eps, void* stream);

/*
 * Tensor-parallel form of eet_rmsnorm_finalize (decode, M <= 64): the all-reduce of a row-parallel projection
 * fused into the kernel that consumes it.  local_sums: this rank's partial sums [M][n] fp32 (zeroed by the call).
 * peer_inbox[r] (host array of `world` device pointers, r = rank): every rank's inbox, 2 * 8 * 64 * (n / 8) * 3
 * packets of 16 bytes {value, value, value, int32 epoch} (zero at start), in memory all ranks can reach (CUDA IPC /
 * peer access); an aligned 16-byte store is assumed to arrive there as one piece.  which: 0 or 1, the inbox of this
 * exchange - consecutive exchanges must alternate.  epochs: 128 int32 of this rank, zero at start.  Each row's CTAs
 * push the partial row into every peer's inbox, then poll their own
 * inbox - a bounded wait, status 4 in eet_device_status if a peer never arrives - and adds the partial rows in
 * fp32 in rank order; then scale, residual, RMSNorm as eet_rmsnorm_finalize.  The reference is single-GPU: no
 * counterpart.
 */
int eet_rmsnorm_finalize_tp(float* local_sums, void* const* peer_inbox, int world, int rank, int which, int* epochs,
                            const void* scale, const void* residual, void* h_out, const void* gamma, void* xn_out, int M,
                            int n, float eps, void* stream);

/* act_out = up * silu(gate) where gate = fp16(gate_sums * gate_scale), up = fp16(up_sums * up_scale) are the
 * unfinished products of eet_gemm_w8a16_accum; both sum buffers are zeroed.
 * Replaces: the epilogues of the gate / up GEMMs + gated_silu<half> (csrc/core/activation_kernel.cu:106-124). */
int eet_swiglu_finalize(float* gate_sums, const void* gate_scale, float* up_sums, const void* up_scale, void* act_out,
                        int M, int n, void* stream);

/* gate <- up * silu(gate), in place.  Replaces: gated_act_kernel<half> with act_type silu
 * (csrc/core/activation_kernel.cu:275-338 -> gated_silu :106-124). */
int eet_swiglu(void* gate_inout, const void* up, int M, int n, void* stream);

/* out += in (fp16), `count` elements.  Replaces: add_bias_input_kernel<half> with a null bias
 * (csrc/core/add_bias.cu:51-73 -> add_input :22-28). */
int eet_add_residual(void* out, const void* in, size_t count, void* stream);

/*
 * Prefill: fused projection output qkv[B][S][3][H][D] -> q_out[B][H][S][D], and K, V written into the
 * caches [B_max][H][T_max][D] at positions 0..S-1; rope != 0 applies the NeoX rotary embedding
 * (base rope_base) to q and k at position s.
 * Replaces: fused_QKV_bias_rotary_kernel<half> (csrc/core/self_add_bias.cu:442-487 -> :369-403) or, with
 *           rope = 0, fused_add_QKV_bias_kernel without bias, followed by copyKV_transpose_kernel
 *           (csrc/core/transpose.cu:116-124).
 */
int eet_qkv_split_store(const void* qkv, void* q_out, void* kcache, void* vcache, int B, int S, int H, int D,
                        int T_max, int rope, float rope_base, void* stream);

/*
 * Prefill causal self-attention over the freshly stored cache: ctx[B][S][H*D].
 * pad_len: device int64 [B] left-padding lengths or NULL; alibi: device fp16 [H][S][S] bias
 * (alibi_stride = S) or NULL.
 * Replaces: q_k_mul + qk_softmax + attn_v_mul + transpose of LlamaMmha::forward_full /
 *           BaichuanMmha::forward_full (csrc/op/llama_mmha.cpp:354-426, csrc/op/baichuan_mmha.cpp:117-150;
 *           softmax kernels csrc/core/gpt2_self_softmax.cu:8-57,161-240).
 */
int eet_prefill_mha(const void* q, const void* kcache, const void* vcache, void* ctx, int B, int S, int H, int D,
                    int T_max, const int64_t* pad_len, const void* alibi, int alibi_stride, void* stream);

/*
 * One decode step of masked multi-head attention for every (batch, head): rotates the new q,k
 * (rope != 0), appends k,v to the caches at position step-1 and attends over positions
 * [pad_len[b], step).  qkv[B][3][H][D] is the fused projection of the new token; ctx[B][H*D].
 *   qkv_sums    alternative to qkv (pass qkv = NULL): the fp32 sums [B][3*H*D] left by
 *               eet_gemm_w8a16_accum, finished here as fp16(sums * qkv_scale) and zeroed
 *   step        history length including the new token, used when step_dev is NULL
 *   step_dev    optional device int32 holding the same number (lets a captured CUDA graph be replayed
 *               while the step advances on the device, see eet_advance_steps)
 *   alibi       device fp16 [H][alibi_stride] bias for the newest row (what the reference's Python
 *               passes as alibi_mask[:, -1:, :]) or NULL;  alibi_slopes: device fp32 [H] or NULL, the
 *               closed form of the same row: bias[h][t] = fp16(slope[h] * t)
 *   splits      CTAs cooperating on one (batch, head): 0 = choose, else 1, 2, 4 or 8
 * Replaces: masked_attention_dispatch<half> (csrc/core/attention_dispatch.cu:888-928 -> :140-324),
 *           fused_masked_attention_dispatch<half> (:1338-1426 -> :1155-1336) and the decode call of
 *           fused_QKV_bias_rotary_kernel (csrc/op/llama_mmha.cpp:241).
 */
int eet_decode_mha(const void* qkv, float* qkv_sums, const void* qkv_scale, void* kcache, void* vcache, void* ctx,
                   int B, int H, int D, int T_max, int step, const int* step_dev, const int64_t* pad_len,
                   const void* alibi, int alibi_stride, const float* alibi_slopes, int rope, float rope_base, int splits,
                   void* stream);

/* Scratch needed by eet_reorder_kv: 2 * B * H * step * D halves. */
size_t eet_reorder_kv_workspace_bytes(int B, int H, int D, int step);

/* Beam search: cache[b] <- cache[index[b]] for positions [0, step).  index: device int64 [B].
 * Replaces: reorderKV_kernel<half> (csrc/core/transpose.cu:136-162). */
int eet_reorder_kv(void* kcache, void* vcache, const int64_t* index, int B, int H, int D, int T_max, int step,
                   void* ws, size_t ws_bytes, void* stream);

/* steps[i] += delta for i < count (device int32).  The reference keeps its step counter on the host
 * (LlamaMmha::step_, csrc/op/llama_mmha.cpp:121,195,210); this is its device-resident twin. */
int eet_advance_steps(int* steps, int count, int delta, void* stream);

/* out[r] (int64) = index of the largest of the n fp16 values of row r (rows row_stride elements apart), the
 * smallest index on ties: the greedy token choice.  The reference leaves it to torch.argmax
 * (python/eet/pipelines/generation.py:1185-1190). */
int eet_argmax_rows(const void* logits, int64_t* out, int rows, int n, size_t row_stride, void* stream);

/*
 * Greedy token choice straight from the fp32 sums of an int8 lm_head projection (eet_gemm_w8a16_accum), for a
 * vocabulary that may be sharded over tensor-parallel ranks: logit = fp16(sums * scale), out_ids[r] = global index
 * of the largest logit of row r (the smallest index on ties); sums is zeroed.  This rank holds the vocabulary
 * columns [col_offset, col_offset + n_local).  With world > 1 each row's {logit, index, epoch} is pushed into every
 * peer's inbox as one 16-byte packet and the best of all ranks is taken, the same on every rank: peer_inbox[r] is
 * rank r's inbox of 2 * 8 * 64 packets of 16 bytes (zero at start, reachable by every rank), epochs 64 int32 of
 * this rank (zero at start), M <= 64; the wait for the peers is bounded (status 4).  With world == 1 peer_inbox and
 * epochs may be NULL and M is not limited.  logits_out, if not NULL, receives the fp16 logits [M][n_local].
 * Replaces: the fp16 lm_head + torch.argmax of the reference's generation loop
 *           (python/eet/transformers/modeling_llama.py:471, python/eet/pipelines/generation.py:1185-1190); the
 *           int8 weights and the sharding have no counterpart there.
 */
int eet_lm_head_argmax(float* sums, const void* scale, int M, int n_local, int64_t col_offset, void* const* peer_inbox,
                       int world, int rank, int* epochs, int64_t* out_ids, void* logits_out, void* stream);

/* out[r][0..n) = table[ids[r]][0..n), fp16, n a multiple of 8, ids device int64 (an id outside
 * [0, rows_in_table) reads row 0): the token-embedding lookup, torch.nn.Embedding in the reference
 * (python/eet/transformers/modeling_llama.py:281-283). */
int eet_gather_rows(const void* table, const int64_t* ids, void* out, int rows, int n, int64_t rows_in_table, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* EET_B200_H */
