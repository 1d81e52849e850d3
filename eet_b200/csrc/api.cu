// The C ABI of the library (declared in include/eet_b200.h): argument validation, then a launcher from
// one of the kernel files.  The library is one translation unit - the kernel files are included below -
// so that the device-side status word and the inline helpers are shared without relocatable device code.
#include "../../include/eet_b200.h"

#include <cstring>
#include <string>

#include "common.cuh"
#include "kernels.h"

namespace eet {

static thread_local std::string t_last_error;

void set_error(const char* fmt, ...)
{
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    t_last_error = buf;
}

int sm_count()
{
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    dev &= 63;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

static inline bool aligned16(const void* p)
{
    return (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

}  // namespace eet

#include "attention.cu"
#include "gemm_skinny.cu"
#include "gemm_tc.cu"
#include "gemm_mid.cu"
#include "attention_tc.cu"
#include "glue.cu"
#include "noalloc.cu"
#include "quantize.cu"

using namespace eet;

extern "C" {

int eet_abi_version(void)
{
    return 4;
}

const char* eet_last_error(void)
{
    return t_last_error.c_str();
}

int eet_device_status(int* status_out)
{
    EET_CHECK(status_out != nullptr, "eet_device_status: status_out is NULL");
    int v = 0;
    EET_CUDA(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        EET_CUDA(cudaMemcpyToSymbol(g_device_status, &zero, sizeof(int)));
    }
    *status_out = v;
    return 0;
}

int eet_set_wait_limit(unsigned int polls)
{
    EET_CHECK(polls >= 1, "eet_set_wait_limit: the limit must be at least 1");
    EET_CUDA(cudaMemcpyToSymbol(g_wait_limit, &polls, sizeof(polls)));
    return 0;
}

size_t eet_quantize_w8_workspace_bytes(int K, int N)
{
    (void)K;
    return N > 0 ? sizeof(float) * (size_t)N : 0;
}

static int check_kn(const char* who, int K, int N)
{
    EET_CHECK(K > 0 && N > 0, "%s: weight must not be empty (K=%d, N=%d)", who, K, N);
    EET_CHECK(K % 64 == 0 && N % 64 == 0, "%s: K=%d and N=%d must be multiples of 64", who, K, N);
    return 0;
}

int eet_quantize_w8(const void* w, int w_is_fp32, int K, int N, int8_t* q_rowmajor, void* packed, void* scales,
                    int variant, void* ws, size_t ws_bytes, void* stream)
{
    if (check_kn("eet_quantize_w8", K, N)) return 1;
    EET_CHECK(w && packed && scales, "eet_quantize_w8: weight, packed and scales must not be NULL");
    EET_CHECK(variant == 0 || variant == 1, "eet_quantize_w8: unknown variant %d", variant);
    EET_CHECK(ws && ws_bytes >= eet_quantize_w8_workspace_bytes(K, N), "eet_quantize_w8: workspace too small");
    EET_CHECK(aligned16(w) && aligned16(packed) && (q_rowmajor == nullptr || aligned16(q_rowmajor)),
              "eet_quantize_w8: pointers must be 16-byte aligned");
    return launch_quantize_w8(w, w_is_fp32 != 0, K, N, q_rowmajor, packed, scales, variant, (float*)ws,
                              (cudaStream_t)stream);
}

int eet_pack_w8(const int8_t* q_rowmajor, int K, int N, void* packed, void* stream)
{
    if (check_kn("eet_pack_w8", K, N)) return 1;
    EET_CHECK(q_rowmajor && packed && aligned16(q_rowmajor) && aligned16(packed),
              "eet_pack_w8: pointers must be non-NULL and 16-byte aligned");
    return launch_pack_w8(q_rowmajor, K, N, packed, (cudaStream_t)stream);
}

int eet_unpack_w8(const void* packed, int K, int N, int8_t* q_rowmajor, void* stream)
{
    if (check_kn("eet_unpack_w8", K, N)) return 1;
    EET_CHECK(q_rowmajor && packed && aligned16(q_rowmajor) && aligned16(packed),
              "eet_unpack_w8: pointers must be non-NULL and 16-byte aligned");
    return launch_unpack_w8(packed, K, N, q_rowmajor, (cudaStream_t)stream);
}

int eet_repack_ref_w8(const void* ref_packed, int K, int N, void* packed, void* stream)
{
    if (check_kn("eet_repack_ref_w8", K, N)) return 1;
    EET_CHECK(ref_packed && packed && ref_packed != packed, "eet_repack_ref_w8: needs two distinct buffers");
    return launch_repack_ref_w8(ref_packed, K, N, packed, (cudaStream_t)stream);
}

static const int kSkinnyGroupRows = 128;  // rows finished per accumulate + finalize pair when M is large

// Largest M that eet_gemm_w8a16 gives to the stream-K kernel; above it the large-tile kernels take over.
static int mid_use_max_m()
{
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("EET_MID_MAX_M");
        v = e ? atoi(e) : 512;
        if (v > kMidMaxM) v = kMidMaxM;
    }
    return v;
}

size_t eet_gemm_w8a16_workspace_bytes(int M, int N, int K)
{
    (void)K;
    if (N <= 0 || M <= 0) return 0;
    return skinny_sum_bytes(M <= kMidMaxM ? M : kSkinnyGroupRows, N);
}

// sums += A x q(B) for any M: the decode kernel up to 16 rows, the stream-K tensor-core kernel above
static int launch_gemm_accum(const GemmArgs& a, cudaStream_t stream)
{
    if (gemm_mid_supported(a.M, a.N, a.K)) return launch_gemm_mid(a, stream);
    return launch_gemm_skinny(a, stream);
}

static int check_gemm(const char* who, const void* A, const void* B, int M, int N, int K)
{
    if (check_kn(who, K, N)) return 1;
    EET_CHECK(M >= 0, "%s: M=%d is negative", who, M);
    EET_CHECK(M == 0 || (A && B), "%s: A and B must not be NULL", who);
    EET_CHECK(aligned16(A) && aligned16(B), "%s: pointers must be 16-byte aligned", who);
    return 0;
}

int eet_gemm_w8a16_accum(const void* A, const void* packedB, float* sums, int M, int N, int K, const void* packedB2,
                         float* sums2, void* stream)
{
    if (check_gemm("eet_gemm_w8a16_accum", A, packedB, M, N, K)) return 1;
    if (M == 0) return 0;
    EET_CHECK(sums != nullptr && aligned16(sums), "eet_gemm_w8a16_accum: sums must be a 16-byte aligned buffer");
    EET_CHECK((packedB2 == nullptr) == (sums2 == nullptr), "eet_gemm_w8a16_accum: B2 and sums2 go together");
    EET_CHECK(aligned16(packedB2) && aligned16(sums2), "eet_gemm_w8a16_accum: pointers must be 16-byte aligned");
    GemmArgs a = {};
    a.A = (const __half*)A;
    a.B = (const uint8_t*)packedB;
    a.B2 = (const uint8_t*)packedB2;
    a.ws = sums;
    a.ws2 = sums2;
    a.M = M;
    a.N = N;
    a.K = K;
    return launch_gemm_accum(a, (cudaStream_t)stream);
}

int eet_gemm_w8a16_finalize(float* sums, const void* scale, const void* residual, void* C, int M, int N, void* stream)
{
    EET_CHECK(M >= 0 && N > 0 && N % 8 == 0, "eet_gemm_w8a16_finalize: bad shape M=%d N=%d", M, N);
    if (M == 0) return 0;
    EET_CHECK(sums && scale && C, "eet_gemm_w8a16_finalize: sums, scale and C must not be NULL");
    EET_CHECK(aligned16(sums) && aligned16(scale) && aligned16(C) && aligned16(residual),
              "eet_gemm_w8a16_finalize: pointers must be 16-byte aligned");
    return launch_finalize(sums, (const __half*)scale, (const __half*)residual, (__half*)C, M, N, (cudaStream_t)stream);
}

int eet_gemm_w8a16(const void* A, const void* packedB, const void* scale, void* C, int M, int N, int K,
                   const void* residual, int epilogue, void* ws, size_t ws_bytes, void* stream)
{
    if (check_gemm("eet_gemm_w8a16", A, packedB, M, N, K)) return 1;
    if (M == 0) return 0;
    EET_CHECK(scale && C && aligned16(C) && aligned16(scale), "eet_gemm_w8a16: scale and C must be 16-byte aligned buffers");
    EET_CHECK(epilogue >= 0 && epilogue <= 2, "eet_gemm_w8a16: unknown epilogue %d", epilogue);
    EET_CHECK(epilogue == 0 || (residual != nullptr && aligned16(residual)),
              "eet_gemm_w8a16: epilogues 1 and 2 need a 16-byte aligned second operand");
    const __half* res = epilogue != 0 ? (const __half*)residual : nullptr;
    const int gate = epilogue == 2 ? 1 : 0;
    // Above 64 tokens a shape that the 256 x 256 kernel can spread over the machine (plain tiles or split-K
    // clusters) goes there: one launch, epilogue fused, no fp32 scratch.
    const bool tiles_first = M > 64 && gemm_tc_supported(M, N, K) && tc2_split(M, N, K) > 0;
    if (!tiles_first && M <= mid_use_max_m() && gemm_mid_supported(M, N, K)) {
        // stream-K tensor-core kernel into the fp32 scratch, then one epilogue pass over all rows
        EET_CHECK(ws && aligned16(ws) && ws_bytes >= skinny_sum_bytes(M, N),
                  "eet_gemm_w8a16: workspace of %zu bytes is smaller than the %zu needed", ws_bytes, skinny_sum_bytes(M, N));
        GemmArgs a = {};
        a.A = (const __half*)A;
        a.B = (const uint8_t*)packedB;
        a.ws = (float*)ws;
        a.M = M;
        a.N = N;
        a.K = K;
        if (int rc = launch_gemm_mid(a, (cudaStream_t)stream)) return rc;
        return launch_finalize((float*)ws, (const __half*)scale, res, (__half*)C, M, N, (cudaStream_t)stream, gate);
    }
    if (gemm_tc_supported(M, N, K)) {
        // prefill regime: tcgen05 tensor-core kernel, epilogue fused, no scratch
        return launch_gemm_tc((const __half*)A, (const uint8_t*)packedB, (const __half*)scale, (__half*)C, res, gate, M, N,
                              K, (cudaStream_t)stream);
    }
    EET_CHECK(ws && aligned16(ws) && ws_bytes >= eet_gemm_w8a16_workspace_bytes(M, N, K),
              "eet_gemm_w8a16: workspace of %zu bytes is smaller than the %zu needed", ws_bytes,
              eet_gemm_w8a16_workspace_bytes(M, N, K));
    for (int r0 = 0; r0 < M; r0 += kSkinnyGroupRows) {
        const int rows = (M - r0 < kSkinnyGroupRows) ? (M - r0) : kSkinnyGroupRows;
        GemmArgs a = {};
        a.A = (const __half*)A + (size_t)r0 * K;
        a.B = (const uint8_t*)packedB;
        a.ws = (float*)ws;
        a.M = rows;
        a.N = N;
        a.K = K;
        if (int rc = launch_gemm_skinny(a, (cudaStream_t)stream)) return rc;
        if (int rc = launch_finalize((float*)ws, (const __half*)scale, res ? res + (size_t)r0 * N : nullptr,
                                     (__half*)C + (size_t)r0 * N, rows, N, (cudaStream_t)stream, gate))
            return rc;
    }
    return 0;
}

int eet_gemm_w8a16_noalloc(const void* A, const void* packedB, const void* scale, void* C, int M, int N, int K,
                           const void* residual, int epilogue, void* stream)
{
    if (check_gemm("eet_gemm_w8a16_noalloc", A, packedB, M, N, K)) return 1;
    if (M == 0) return 0;
    EET_CHECK(scale && C && aligned16(C) && aligned16(scale) && aligned16(residual),
              "eet_gemm_w8a16_noalloc: scale, C and residual must be 16-byte aligned buffers");
    EET_CHECK(epilogue == 0 || epilogue == 1, "eet_gemm_w8a16_noalloc: unknown epilogue %d", epilogue);
    EET_CHECK(epilogue != 1 || residual != nullptr, "eet_gemm_w8a16_noalloc: epilogue 1 needs a residual");
    return gemm_w8a16_noalloc((const __half*)A, (const uint8_t*)packedB, (const __half*)scale, (__half*)C, M, N, K,
                              epilogue == 1 ? (const __half*)residual : nullptr, (cudaStream_t)stream);
}

int eet_rmsnorm(const void* x, const void* gamma, void* y, int M, int n, float eps, void* stream)
{
    EET_CHECK(M >= 0 && x && gamma && y, "eet_rmsnorm: bad arguments");
    EET_CHECK(aligned16(x) && aligned16(gamma) && aligned16(y), "eet_rmsnorm: pointers must be 16-byte aligned");
    return launch_rmsnorm((const __half*)x, (const __half*)gamma, (__half*)y, M, n, eps, (cudaStream_t)stream);
}

int eet_rmsnorm_finalize(float* sums, const void* scale, const void* residual, void* h_out, const void* gamma,
                         void* xn_out, int M, int n, float eps, void* stream)
{
    EET_CHECK(M >= 0 && residual && gamma && xn_out, "eet_rmsnorm_finalize: bad arguments");
    EET_CHECK(sums == nullptr || (scale != nullptr && h_out != nullptr),
              "eet_rmsnorm_finalize: sums need their scale and an output for the finished rows");
    EET_CHECK(aligned16(sums) && aligned16(scale) && aligned16(residual) && aligned16(h_out) && aligned16(gamma) &&
                  aligned16(xn_out),
              "eet_rmsnorm_finalize: pointers must be 16-byte aligned");
    return launch_rmsnorm_finalize(sums, (const __half*)scale, (const __half*)residual, (__half*)h_out,
                                   (const __half*)gamma, (__half*)xn_out, M, n, eps, (cudaStream_t)stream);
}

int eet_rmsnorm_finalize_tp(float* local_sums, void* const* peer_inbox, int world, int rank, int which, int* epochs,
                            const void* scale, const void* residual, void* h_out, const void* gamma, void* xn_out, int M,
                            int n, float eps, void* stream)
{
    EET_CHECK(local_sums && peer_inbox && epochs && scale && residual && h_out && gamma && xn_out,
              "eet_rmsnorm_finalize_tp: NULL argument");
    EET_CHECK(aligned16(local_sums) && aligned16(scale) && aligned16(residual) && aligned16(h_out) && aligned16(gamma) &&
                  aligned16(xn_out),
              "eet_rmsnorm_finalize_tp: pointers must be 16-byte aligned");
    return launch_rmsnorm_finalize_tp(local_sums, peer_inbox, world, rank, which, epochs, (const __half*)scale,
                                      (const __half*)residual, (__half*)h_out, (const __half*)gamma, (__half*)xn_out, M,
                                      n, eps, (cudaStream_t)stream);
}

int eet_swiglu_finalize(float* gate_sums, const void* gate_scale, float* up_sums, const void* up_scale, void* act_out,
                        int M, int n, void* stream)
{
    EET_CHECK(M >= 0 && gate_sums && gate_scale && up_sums && up_scale && act_out, "eet_swiglu_finalize: bad arguments");
    EET_CHECK(aligned16(gate_sums) && aligned16(gate_scale) && aligned16(up_sums) && aligned16(up_scale) &&
                  aligned16(act_out),
              "eet_swiglu_finalize: pointers must be 16-byte aligned");
    return launch_swiglu_finalize(gate_sums, (const __half*)gate_scale, up_sums, (const __half*)up_scale,
                                  (__half*)act_out, M, n, (cudaStream_t)stream);
}

int eet_swiglu(void* gate_inout, const void* up, int M, int n, void* stream)
{
    EET_CHECK(M >= 0 && gate_inout && up && aligned16(gate_inout) && aligned16(up), "eet_swiglu: bad arguments");
    return launch_swiglu((__half*)gate_inout, (const __half*)up, M, n, (cudaStream_t)stream);
}

int eet_add_residual(void* out, const void* in, size_t count, void* stream)
{
    EET_CHECK(out && in && aligned16(out) && aligned16(in), "eet_add_residual: bad arguments");
    return launch_add_residual((__half*)out, (const __half*)in, count, (cudaStream_t)stream);
}

int eet_qkv_split_store(const void* qkv, void* q_out, void* kcache, void* vcache, int B, int S, int H, int D,
                        int T_max, int rope, float rope_base, void* stream)
{
    EET_CHECK(qkv && q_out && kcache && vcache && B >= 0 && S >= 0 && H > 0, "eet_qkv_split_store: bad arguments");
    return launch_qkv_split_store((const __half*)qkv, (__half*)q_out, (__half*)kcache, (__half*)vcache, B, S, H, D,
                                  T_max, rope, rope_base, (cudaStream_t)stream);
}

int eet_prefill_mha(const void* q, const void* kcache, const void* vcache, void* ctx, int B, int S, int H, int D,
                    int T_max, const int64_t* pad_len, const void* alibi, int alibi_stride, void* stream)
{
    EET_CHECK(q && kcache && vcache && ctx && B >= 0 && S >= 0 && H > 0, "eet_prefill_mha: bad arguments");
    EET_CHECK(aligned16(q) && aligned16(kcache) && aligned16(vcache) && aligned16(ctx),
              "eet_prefill_mha: pointers must be 16-byte aligned");
    // long prompts: tcgen05 kernel (128 x 128 tiles); short ones: the mma.sync kernel with 64 x 64 tiles
    static const bool no_tc = getenv("EET_NO_PREFILL_TC") != nullptr;
    if (!no_tc && prefill_mha_tc_supported(S, D) && B > 0) {
        EET_CHECK(S <= T_max, "prefill attention: prompt length %d exceeds the cache length %d", S, T_max);
        return launch_prefill_mha_tc((const __half*)q, (const __half*)kcache, (const __half*)vcache, (__half*)ctx, B, S, H,
                                     T_max, pad_len, (const __half*)alibi, alibi_stride, (cudaStream_t)stream);
    }
    return launch_prefill_mha((const __half*)q, (const __half*)kcache, (const __half*)vcache, (__half*)ctx, B, S, H, D,
                              T_max, pad_len, (const __half*)alibi, alibi_stride, (cudaStream_t)stream);
}

int eet_decode_mha(const void* qkv, float* qkv_sums, const void* qkv_scale, void* kcache, void* vcache, void* ctx,
                   int B, int H, int D, int T_max, int step, const int* step_dev, const int64_t* pad_len,
                   const void* alibi, int alibi_stride, const float* alibi_slopes, int rope, float rope_base, int splits,
                   void* stream)
{
    EET_CHECK(kcache && vcache && ctx && B >= 0 && H > 0, "eet_decode_mha: bad arguments");
    EET_CHECK((qkv != nullptr) != (qkv_sums != nullptr), "eet_decode_mha: pass either qkv or qkv_sums");
    EET_CHECK(qkv_sums == nullptr || qkv_scale != nullptr, "eet_decode_mha: qkv_sums need qkv_scale");
    EET_CHECK(aligned16(qkv) && aligned16(qkv_sums) && aligned16(kcache) && aligned16(vcache) && aligned16(ctx),
              "eet_decode_mha: pointers must be 16-byte aligned");
    DecodeAttnArgs a = {};
    a.qkv = (const __half*)qkv;
    a.qkv_sums = qkv_sums;
    a.qkv_scale = (const __half*)qkv_scale;
    a.kcache = (__half*)kcache;
    a.vcache = (__half*)vcache;
    a.ctx = (__half*)ctx;
    a.B = B;
    a.H = H;
    a.D = D;
    a.T_max = T_max;
    a.step = step;
    a.step_dev = step_dev;
    a.pad_len = pad_len;
    a.alibi = (const __half*)alibi;
    a.alibi_stride = alibi_stride;
    a.alibi_slopes = alibi_slopes;
    a.rope = rope;
    a.rope_base = rope_base;
    a.splits = splits;
    return launch_decode_mha(a, (cudaStream_t)stream);
}

size_t eet_reorder_kv_workspace_bytes(int B, int H, int D, int step)
{
    return (size_t)2 * B * H * step * D * sizeof(__half);
}

int eet_reorder_kv(void* kcache, void* vcache, const int64_t* index, int B, int H, int D, int T_max, int step,
                   void* ws, size_t ws_bytes, void* stream)
{
    EET_CHECK(kcache && vcache && index && ws, "eet_reorder_kv: bad arguments");
    EET_CHECK(step >= 0 && step <= T_max, "eet_reorder_kv: step %d outside the cache length %d", step, T_max);
    EET_CHECK(ws_bytes >= eet_reorder_kv_workspace_bytes(B, H, D, step), "eet_reorder_kv: workspace too small");
    if (B == 0 || step == 0) return 0;
    return launch_reorder_kv((__half*)kcache, (__half*)vcache, index, B, H, D, T_max, step, (__half*)ws,
                             (cudaStream_t)stream);
}

int eet_advance_steps(int* steps, int count, int delta, void* stream)
{
    EET_CHECK(steps != nullptr || count == 0, "eet_advance_steps: steps is NULL");
    return launch_advance_steps(steps, count, delta, (cudaStream_t)stream);
}

int eet_argmax_rows(const void* logits, int64_t* out, int rows, int n, size_t row_stride, void* stream)
{
    EET_CHECK(rows >= 0 && n > 0 && (rows == 0 || (logits && out)), "eet_argmax_rows: bad arguments");
    return launch_argmax_rows((const __half*)logits, out, rows, n, row_stride, (cudaStream_t)stream);
}

int eet_lm_head_argmax(float* sums, const void* scale, int M, int n_local, int64_t col_offset, void* const* peer_inbox,
                       int world, int rank, int* epochs, int64_t* out_ids, void* logits_out, void* stream)
{
    EET_CHECK(M >= 0 && (M == 0 || (sums && scale && out_ids)), "eet_lm_head_argmax: NULL argument");
    EET_CHECK(aligned16(sums) && aligned16(scale) && aligned16(logits_out), "eet_lm_head_argmax: pointers must be 16-byte aligned");
    return launch_lm_head_argmax(sums, (const __half*)scale, M, n_local, (long long)col_offset, peer_inbox, world, rank, epochs,
                                 out_ids, (__half*)logits_out, (cudaStream_t)stream);
}

int eet_gather_rows(const void* table, const int64_t* ids, void* out, int rows, int n, int64_t rows_in_table, void* stream)
{
    EET_CHECK(rows >= 0 && n > 0 && rows_in_table > 0 && (rows == 0 || (table && ids && out)), "eet_gather_rows: bad arguments");
    EET_CHECK(aligned16(table) && aligned16(out), "eet_gather_rows: pointers must be 16-byte aligned");
    return launch_gather_rows((const __half*)table, ids, (__half*)out, rows, n, rows_in_table, (cudaStream_t)stream);
}

}  // extern "C"
