// Internal launcher declarations shared between the kernel files and the C ABI (api.cu).  Every
// launcher enqueues on the given stream, allocates nothing, and returns 0 or a non-zero status after
// recording a message with set_error().
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stddef.h>
#include <stdint.h>

namespace eet {

// quantize.cu
int launch_quantize_w8(const void* w, bool fp32, int K, int N, int8_t* q_rowmajor, void* packed, void* scales,
                       int variant, float* amax_ws, cudaStream_t stream);
int launch_pack_w8(const int8_t* q, int K, int N, void* packed, cudaStream_t stream);
int launch_unpack_w8(const void* packed, int K, int N, int8_t* q, cudaStream_t stream);
int launch_repack_ref_w8(const void* ref_packed, int K, int N, void* packed, cudaStream_t stream);

// gemm_skinny.cu
struct GemmArgs {
    const __half* A;    // [M][K] fp16 activations
    const uint8_t* B;   // W8T64 [N/64][K/64][64][64]
    const uint8_t* B2;  // optional second weight of the same shape (FFN up projection) or null
    float* ws;          // [M][N] fp32: sum over k of A[m][k] * q[k][n] is ADDED here
    float* ws2;         // the same for B2
    int M, N, K;
};
size_t skinny_sum_bytes(int M, int N);
int launch_gemm_skinny(const GemmArgs& a, cudaStream_t stream);

// gemm_tc.cu (tcgen05 / TMEM)
bool gemm_tc_supported(int M, int N, int K);
int tc2_split(int M, int N, int K);  // 0: the 256 x 256 kernel does not take this shape; else its split-K cluster size
int launch_gemm_tc(const __half* A, const uint8_t* B, const __half* scale, __half* C, const __half* residual, int gate,
                   int M, int N, int K, cudaStream_t stream);

// gemm_mid.cu (stream-K tcgen05, fp32 sums like the skinny kernel)
constexpr int kMidMaxM = 512;
bool gemm_mid_supported(int M, int N, int K);
int launch_gemm_mid(const GemmArgs& a, cudaStream_t stream);

// noalloc.cu
int gemm_w8a16_noalloc(const __half* A, const uint8_t* B, const __half* scale, __half* C, int M, int N, int K,
                       const __half* residual, cudaStream_t stream);

// glue.cu
int launch_rmsnorm(const __half* x, const __half* gamma, __half* y, int M, int n, float eps, cudaStream_t stream);
int launch_finalize(float* sums, const __half* scale, const __half* residual, __half* C, int M, int N,
                    cudaStream_t stream, int gate = 0);   // gate: C = gated_silu(residual, fp16(sums * scale))
int launch_rmsnorm_finalize(float* sums, const __half* scale, const __half* residual, __half* h_out,
                            const __half* gamma, __half* xn_out, int M, int n, float eps, cudaStream_t stream);
int launch_rmsnorm_finalize_tp(float* local_sums, void* const* peer_inbox, int world, int rank, int which, int* epochs,
                               const __half* scale, const __half* residual, __half* h_out, const __half* gamma,
                               __half* xn_out, int M, int n, float eps, cudaStream_t stream);
int launch_swiglu_finalize(float* gate_sums, const __half* gate_scale, float* up_sums, const __half* up_scale,
                           __half* act_out, int M, int n, cudaStream_t stream);
int launch_swiglu(__half* gate_inout, const __half* up, int M, int n, cudaStream_t stream);
int launch_add_residual(__half* out, const __half* in, size_t count, cudaStream_t stream);
int launch_qkv_split_store(const __half* qkv, __half* q_out, __half* kcache, __half* vcache, int B, int S, int H,
                           int D, int T_max, int rope, float rope_base, cudaStream_t stream);
int launch_reorder_kv(__half* kcache, __half* vcache, const int64_t* index, int B, int H, int D, int T_max, int step,
                      __half* ws, cudaStream_t stream);
int launch_advance_steps(int* steps, int count, int delta, cudaStream_t stream);
int launch_argmax_rows(const __half* logits, int64_t* out, int rows, int n, size_t row_stride, cudaStream_t stream);
int launch_lm_head_argmax(float* sums, const __half* scale, int M, int n, long long col_offset, void* const* peer_inbox,
                          int world, int rank, int* epochs, int64_t* out, __half* logits_out, cudaStream_t stream);
int launch_gather_rows(const __half* table, const int64_t* ids, __half* out, int rows, int n, int64_t rows_in_table,
                       cudaStream_t stream);

// attention.cu
struct DecodeAttnArgs {
    const __half* qkv;        // [B][3][H][D] fused projection output of the new token, or null with:
    float* qkv_sums;          // [B][3*H*D] fp32 sums of the projection GEMM, finalized (and zeroed) here
    const __half* qkv_scale;  // [3*H*D] per-channel scales of that projection
    __half* kcache;           // [B_max][H][T_max][D]
    __half* vcache;
    __half* ctx;              // [B][H*D]
    int B, H, D, T_max;
    int step;                 // history length including the new token (used when step_dev is null)
    const int* step_dev;      // optional device-resident step
    const int64_t* pad_len;   // [B] or null
    const __half* alibi;      // [H][alibi_stride] bias row for the newest position, or null
    int alibi_stride;
    const float* alibi_slopes;  // [H] or null: bias = fp16(slope * t), the closed form of the same row
    int rope;                 // 1: rotate q,k (NeoX pairing) at position step-1
    float rope_base;
    int splits;               // CTAs per (batch, head): 1, 2, 4 or 8; 0 = choose
};
int launch_decode_mha(const DecodeAttnArgs& a, cudaStream_t stream);
int launch_prefill_mha(const __half* q, const __half* kcache, const __half* vcache, __half* ctx, int B, int S, int H,
                       int D, int T_max, const int64_t* pad_len, const __half* alibi, int alibi_stride,
                       cudaStream_t stream);


// attention_tc.cu (tcgen05 prefill attention for long prompts)
bool prefill_mha_tc_supported(int S, int D);
int launch_prefill_mha_tc(const __half* q, const __half* kcache, const __half* vcache, __half* ctx, int B, int S, int H,
                          int T_max, const int64_t* pad_len, const __half* alibi, int alibi_stride, cudaStream_t stream);

}  // namespace eet
