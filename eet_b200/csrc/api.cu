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
#include "glue.cu"
#include "quantize.cu"

using namespace eet;

extern "C" {

int eet_abi_version(void)
{
    return 1;
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

size_t eet_gemm_w8a16_workspace_bytes(int M, int N, int K)
{
    (void)K;
    if (N <= 0) return 0;
    return skinny_workspace_bytes(M, N, 0);
}

int eet_gemm_w8a16(const void* A, const void* packedB, const void* scale, void* C, int M, int N, int K,
                   const void* residual, int epilogue, void* ws, size_t ws_bytes, void* stream)
{
    if (check_kn("eet_gemm_w8a16", K, N)) return 1;
    EET_CHECK(M >= 0, "eet_gemm_w8a16: M=%d is negative", M);
    if (M == 0) return 0;
    EET_CHECK(A && packedB && scale && C, "eet_gemm_w8a16: A, B, scale and C must not be NULL");
    EET_CHECK(aligned16(A) && aligned16(packedB) && aligned16(C), "eet_gemm_w8a16: pointers must be 16-byte aligned");
    EET_CHECK(epilogue == 0 || epilogue == 1, "eet_gemm_w8a16: unknown epilogue %d", epilogue);
    EET_CHECK(epilogue != 1 || residual != nullptr, "eet_gemm_w8a16: epilogue 1 needs a residual");
    EET_CHECK(ws && ws_bytes >= eet_gemm_w8a16_workspace_bytes(M, N, K),
              "eet_gemm_w8a16: workspace of %zu bytes is smaller than the %zu needed", ws_bytes,
              eet_gemm_w8a16_workspace_bytes(M, N, K));
    GemmArgs a = {};
    a.A = (const __half*)A;
    a.B = (const uint8_t*)packedB;
    a.scale = (const __half*)scale;
    a.C = (__half*)C;
    a.residual = (const __half*)residual;
    a.M = M;
    a.N = N;
    a.K = K;
    a.epilogue = epilogue;
    a.ws = (float*)ws;
    a.ws_bytes = ws_bytes;
    return launch_gemm_skinny(a, (cudaStream_t)stream);
}

int eet_rmsnorm(const void* x, const void* gamma, void* y, int M, int n, float eps, void* stream)
{
    EET_CHECK(M >= 0 && x && gamma && y, "eet_rmsnorm: bad arguments");
    EET_CHECK(aligned16(x) && aligned16(gamma) && aligned16(y), "eet_rmsnorm: pointers must be 16-byte aligned");
    return launch_rmsnorm((const __half*)x, (const __half*)gamma, (__half*)y, M, n, eps, (cudaStream_t)stream);
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
    return launch_prefill_mha((const __half*)q, (const __half*)kcache, (const __half*)vcache, (__half*)ctx, B, S, H, D,
                              T_max, pad_len, (const __half*)alibi, alibi_stride, (cudaStream_t)stream);
}

int eet_decode_mha(const void* qkv, void* kcache, void* vcache, void* ctx, int B, int H, int D, int T_max, int step,
                   const int* step_dev, const int64_t* pad_len, const void* alibi, int alibi_stride,
                   const float* alibi_slopes, int rope, float rope_base, int splits, void* stream)
{
    EET_CHECK(qkv && kcache && vcache && ctx && B >= 0 && H > 0, "eet_decode_mha: bad arguments");
    EET_CHECK(aligned16(qkv) && aligned16(kcache) && aligned16(vcache) && aligned16(ctx),
              "eet_decode_mha: pointers must be 16-byte aligned");
    DecodeAttnArgs a = {};
    a.qkv = (const __half*)qkv;
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

}  // extern "C"
