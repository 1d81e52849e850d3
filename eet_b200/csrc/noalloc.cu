// eet_gemm_w8a16_noalloc: the decode-regime W8A16 GEMM for callers that cannot provide scratch memory.
//
// Some hosts of this library must not allocate device memory at all: an inference server that hands its
// whole HBM budget to one arena at start-up and forbids any later cudaMalloc, a plugin loaded into a
// process whose allocator is owned by somebody else, or a latency-critical decode loop that cannot afford
// the device-wide synchronisation a cudaMalloc / cudaFree implies.  eet_gemm_w8a16 asks such callers for a
// zeroed fp32 scratch buffer; this variant brings its own, a fixed array that lives in the library's
// device image (every GPU that loads the library holds it until the process exits).
#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

// fp32 sums of at most 16 tokens x 32768 output channels: 2 MiB
constexpr size_t kNoAllocMaxSums = (size_t)16 * 32768;
static __device__ __align__(256) float g_noalloc_sums[kNoAllocMaxSums];

// In host code the array's name stands for a host-side shadow, not for device memory: handing it to a
// kernel would fault (or silently touch the wrong memory where the GPU can reach host memory).  The device
// address is looked up once per device, with that device current.
int noalloc_scratch(float** out)
{
    static float* cached[64] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    EET_CHECK(dev >= 0 && dev < 64, "eet_gemm_w8a16_noalloc: device index %d out of range", dev);
    if (cached[dev] == nullptr) {
        void* p = nullptr;
        EET_CUDA(cudaGetSymbolAddress(&p, g_noalloc_sums));
        cached[dev] = static_cast<float*>(p);
    }
    *out = cached[dev];
    return 0;
}

}  // namespace

int gemm_w8a16_noalloc(const __half* A, const uint8_t* B, const __half* scale, __half* C, int M, int N, int K,
                       const __half* residual, cudaStream_t stream)
{
    EET_CHECK(M <= 16, "eet_gemm_w8a16_noalloc: M=%d exceeds 16 (use eet_gemm_w8a16 with a caller-provided scratch)", M);
    EET_CHECK((size_t)M * (size_t)N <= kNoAllocMaxSums,
              "eet_gemm_w8a16_noalloc: M*N = %zu exceeds the built-in scratch of %zu sums", (size_t)M * (size_t)N,
              kNoAllocMaxSums);
    float* sums = nullptr;
    if (int rc = noalloc_scratch(&sums)) return rc;
    // the array keeps whatever the previous call (or an aborted one) left: start from zero
    EET_CUDA(cudaMemsetAsync(sums, 0, (size_t)M * N * sizeof(float), stream));
    GemmArgs a = {};
    a.A = A;
    a.B = B;
    a.ws = sums;
    a.M = M;
    a.N = N;
    a.K = K;
    if (int rc = launch_gemm_skinny(a, stream)) return rc;
    return launch_finalize(sums, scale, residual, C, M, N, stream);
}

}  // namespace eet
