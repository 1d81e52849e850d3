// Shared device/host helpers for the sm_100a kernels of this library: error plumbing for the C ABI,
// mbarrier / bulk-copy (TMA engine) wrappers with bounded waits, and the int8 -> fp16 register
// conversion used by both GEMM kernels.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

namespace eet {

// ------------------------------------------------------------------------------------------ host errors
// Every extern "C" entry point returns 0 on success; on failure it returns non-zero and leaves a message
// that eet_last_error() hands out (thread-local, overwritten by the next failure on the same thread).
void set_error(const char* fmt, ...);

#define EET_CHECK(cond, ...)                                                                                 \
    do {                                                                                                     \
        if (!(cond)) {                                                                                       \
            ::eet::set_error(__VA_ARGS__);                                                                   \
            return 1;                                                                                        \
        }                                                                                                    \
    } while (0)

#define EET_CUDA(call)                                                                                       \
    do {                                                                                                     \
        cudaError_t err__ = (call);                                                                          \
        if (err__ != cudaSuccess) {                                                                          \
            ::eet::set_error("%s failed: %s (%s:%d)", #call, cudaGetErrorString(err__), __FILE__, __LINE__); \
            return 2;                                                                                        \
        }                                                                                                    \
    } while (0)

#define EET_LAUNCH_CHECK() EET_CUDA(cudaGetLastError())

// Device-side status word.  A kernel that had to give up stores a non-zero code here and returns normally (uniform
// control flow, tensor memory freed, nothing left in flight); the host reads and clears it with eet_device_status().
//   1  decode GEMM (gemm_skinny): a shared-memory pipeline wait ran out
//   2  tensor-core GEMMs (gemm_mid, gemm_tc): a pipeline or tensor-memory wait ran out
//   3  decode attention: a pipeline wait ran out
//   4  tensor-parallel exchange: a peer's partial sums never arrived in this rank's inbox
//   5  decode attention: the device-resident step was outside [1, cache length]; nothing was appended
// After a non-zero status the contents of every fp32 scratch buffer the failed kernel used are undefined.
// (The library is built as one translation unit, so these definitions are seen exactly once.)
#ifdef __CUDACC__
__device__ int g_device_status = 0;
// Polls allowed in the waits on other GPUs (tensor-parallel inbox) before they give up;
// eet_set_wait_limit() changes it.  The mbarrier waits inside one CTA use the compile-time kSpinLimit below.
__device__ unsigned int g_wait_limit = 1u << 22;
#endif

int sm_count();  // multiprocessors of the current device (cached per device)

// ------------------------------------------------------------------------------------------ device helpers
#ifdef __CUDACC__

constexpr int kTile = 64;              // W8T64 tile edge (channels and reduction indices)
constexpr int kTileBytes = kTile * kTile;

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}

__device__ __forceinline__ void mbar_fence_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t* bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint64_t* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

// Waits for the phase with the given parity to complete, but never forever: after kSpinLimit failed
// polls it gives up and returns false.  Each failed try_wait already blocks for a hardware-defined
// interval, so the limit amounts to a second or more of wall time.
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kSpinLimit; ++i) {
        if (mbar_try_wait(bar, parity)) {
            return true;
        }
    }
    return false;
}

// 1-D bulk copy global -> shared through the TMA engine; completion is signalled on `bar` as
// transaction bytes.  Both addresses must be 16-byte aligned and `bytes` a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(smem_dst)),
                 "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}

// Same with an L2 evict-first hint for data that is streamed once (the weights).
__device__ __forceinline__ void bulk_g2s_stream(void* smem_dst, const void* gmem_src, uint32_t bytes, uint64_t* bar)
{
    uint64_t policy;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(policy));
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(
            smem_u32(smem_dst)),
        "l"(gmem_src), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

// gate <- up * gate / (1 + exp(-gate)) with the reference's mix of precisions: exp in fp32 rounded to
// fp16, the multiply, add and divide in fp16 (gated_silu<half>, csrc/core/activation_kernel.cu:106-124).
__device__ __forceinline__ __half2 gated_silu2(__half2 g, __half2 u)
{
    const float2 gf = __half22float2(g);
    const __half2 e = __floats2half2_rn(expf(-gf.x), expf(-gf.y));
    const __half2 one = __floats2half2_rn(1.f, 1.f);
    return __h2div(__hmul2(u, g), __hadd2(one, e));
}

// Four biased bytes (value + 128 each) -> four fp16 values, as two half2 registers {b0,b1} and {b2,b3}.
// Placing a byte under the exponent pattern 0x64 yields the fp16 number 1024 + byte; subtracting 1152
// gives byte - 128 exactly.
__device__ __forceinline__ void cvt_u8x4_to_f16x4(uint32_t w, uint32_t& lo, uint32_t& hi)
{
    const uint32_t magic = 0x64646464u;
    const uint32_t bias = 0x64806480u;  // {1152, 1152} in fp16
    uint32_t a, b;
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(w), "r"(magic));
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(w), "r"(magic));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(lo) : "r"(a), "r"(bias));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(hi) : "r"(b), "r"(bias));
}

__device__ __forceinline__ void mma_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1)
{
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Programmatic dependent launch (PDL).  A kernel launched with launch_pdl() may begin while the kernel
// before it in the stream is still running; pdl_wait() blocks until that kernel has completed and its
// writes are visible, so everything that reads or writes data of the dependency chain comes after it.
// pdl_launch_dependents() tells the scheduler that the next kernel may be started.  Both are no-ops for
// a kernel launched without the attribute.
__device__ __forceinline__ void pdl_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

__device__ __forceinline__ void pdl_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

__device__ __forceinline__ float warp_sum(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v += __shfl_xor_sync(0xffffffffu, v, o);
    }
    return v;
}

__device__ __forceinline__ float warp_max(float v)
{
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    }
    return v;
}

// Launches `kernel` with the programmatic-stream-serialization attribute (see pdl_wait above).
template<typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              Args... args)
{
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#endif  // __CUDACC__

}  // namespace eet
