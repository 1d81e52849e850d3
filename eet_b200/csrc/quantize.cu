// Symmetric per-output-channel int8 quantizer and the W8T64 weight packer.
//
// Replaces, for the int8 path, the reference's host-side symmetric_quantize
// (3rdparty/cutlass_kernels/cutlass_preprocessors.cc:581-678) and preprocess_weights_for_mixed_gemm
// (:497-534).  The arithmetic is kept operation for operation so that the int8 values and the scales
// are bit-identical: per-column max of |w| ignoring NaN, scale = amax * (1/128) in fp32, quotient by
// the un-rounded fp32 scale with IEEE division, C round() (half away from zero), clamp with the
// operand order of std::min / std::max (NaN -> 127).
//
// Layout produced ("W8T64"): tiles of 64 output channels x 64 reduction indices, ordered
// [N/64][K/64]; byte (n % 64) * 64 + (k % 64) inside a tile; each byte is q + 128.  One tile is a
// contiguous 4 KiB block, so a GEMM CTA streams its share of the weights as one linear byte range.
#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

template<typename T>
struct Vec8;
template<>
struct Vec8<__half> {
    uint4 raw;
    __device__ __forceinline__ void load(const __half* p) { raw = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ float get(int i) const
    {
        const __half* h = reinterpret_cast<const __half*>(&raw);
        return __half2float(h[i]);
    }
};
template<>
struct Vec8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p)
    {
        a = *reinterpret_cast<const float4*>(p);
        b = *reinterpret_cast<const float4*>(p + 4);
    }
    __device__ __forceinline__ float get(int i) const
    {
        const float* f = reinterpret_cast<const float*>(&a);
        return i < 4 ? f[i] : reinterpret_cast<const float*>(&b)[i - 4];
    }
};

// Per-column max |w| over a slab of 64 rows x 256 columns, merged into amax[N] with an integer atomic
// max (valid because the values are non-negative floats).  NaN never becomes the maximum:
// fmaxf returns its non-NaN operand, as std::max(acc, x) does when x is NaN.
template<typename T>
__global__ void __launch_bounds__(256) colmax_kernel(const T* __restrict__ w, int K, int N, float* __restrict__ amax)
{
    __shared__ float red[8][256];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int n0 = blockIdx.x * 256 + tx * 8;
    const int k0 = blockIdx.y * 64;
    float m[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) m[i] = 0.f;
    if (n0 < N) {
#pragma unroll 4
        for (int r = ty; r < 64; r += 8) {
            Vec8<T> v;
            v.load(w + (size_t)(k0 + r) * N + n0);
#pragma unroll
            for (int i = 0; i < 8; ++i) m[i] = fmaxf(m[i], fabsf(v.get(i)));
        }
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) red[ty][tx * 8 + i] = m[i];
    __syncthreads();
    const int c = threadIdx.x;
    float v = red[0][c];
#pragma unroll
    for (int r = 1; r < 8; ++r) v = fmaxf(v, red[r][c]);
    const int n = blockIdx.x * 256 + c;
    if (n < N) {
        atomicMax(reinterpret_cast<int*>(amax) + n, __float_as_int(v));
    }
}

__device__ __forceinline__ float col_scale(float amax, int variant)
{
    return variant ? __fdiv_rn(amax, 127.f) : amax * (1.f / 128.f);
}

__device__ __forceinline__ int quantize_one(float w, float s, float lo)
{
    float r = roundf(__fdiv_rn(w, s));
    float c = (r < 127.f) ? r : 127.f;  // std::min(127.f, r)
    c = (lo < c) ? c : lo;              // std::max(lo, c)
    return (int)c;
}

// One 64(k) x 64(n) tile per block: quantize, optionally emit the row-major int8 matrix, and write the
// tile's 4 KiB of the W8T64 layout with fully coalesced 16-byte stores after a transpose in shared
// memory.  Blocks with blockIdx.y == 0 also write the scales.
template<typename T>
__global__ void __launch_bounds__(256)
quant_pack_kernel(const T* __restrict__ w, int K, int N, const float* __restrict__ amax, int variant,
                  int8_t* __restrict__ q_rowmajor, uint8_t* __restrict__ packed, void* __restrict__ scales)
{
    __shared__ __align__(16) uint8_t tile[64][64 + 16];
    const int nt = blockIdx.x, kt = blockIdx.y;
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;  // 8 column groups x 32 rows
    const int n0 = nt * 64 + tx * 8;
    const float lo = variant ? -127.f : -128.f;
    float s[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) s[i] = col_scale(amax[n0 + i], variant);
    if (kt == 0 && ty == 0) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            if (sizeof(T) == 4) {
                reinterpret_cast<float*>(scales)[n0 + i] = s[i];
            }
            else {
                reinterpret_cast<__half*>(scales)[n0 + i] = __float2half_rn(s[i]);
            }
        }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int kl = ty + half * 32;
        const size_t k = (size_t)kt * 64 + kl;
        Vec8<T> v;
        v.load(w + k * N + n0);
        uint32_t lo4 = 0, hi4 = 0;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int q = quantize_one(v.get(i), s[i], lo);
            tile[tx * 8 + i][kl] = (uint8_t)(q + 128);
            const uint32_t byte = (uint32_t)(q & 0xff);
            if (i < 4) {
                lo4 |= byte << (8 * i);
            }
            else {
                hi4 |= byte << (8 * (i - 4));
            }
        }
        if (q_rowmajor != nullptr) {
            *reinterpret_cast<uint2*>(q_rowmajor + k * N + n0) = make_uint2(lo4, hi4);
        }
    }
    __syncthreads();
    const int row = threadIdx.x >> 2, seg = threadIdx.x & 3;
    const uint4 out = *reinterpret_cast<const uint4*>(&tile[row][seg * 16]);
    uint8_t* dst = packed + ((size_t)nt * (K / 64) + kt) * kTileBytes;
    *reinterpret_cast<uint4*>(dst + threadIdx.x * 16) = out;
}

// Row-major int8 [K][N] -> W8T64 (the role of the reference's preprocess_weights, :536-544).
__global__ void __launch_bounds__(256)
pack_kernel(const int8_t* __restrict__ q, int K, int N, uint8_t* __restrict__ packed)
{
    __shared__ __align__(16) uint8_t tile[64][64 + 16];
    const int nt = blockIdx.x, kt = blockIdx.y;
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int kl = ty + half * 32;
        const uint2 v = *reinterpret_cast<const uint2*>(q + ((size_t)kt * 64 + kl) * N + nt * 64 + tx * 8);
        const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) tile[tx * 8 + i][kl] = (uint8_t)(b[i] ^ 0x80u);  // two's complement + 128
    }
    __syncthreads();
    const int row = threadIdx.x >> 2, seg = threadIdx.x & 3;
    uint8_t* dst = packed + ((size_t)nt * (K / 64) + kt) * kTileBytes;
    *reinterpret_cast<uint4*>(dst + threadIdx.x * 16) = *reinterpret_cast<const uint4*>(&tile[row][seg * 16]);
}

// W8T64 -> row-major int8 [K][N].
__global__ void __launch_bounds__(256)
unpack_kernel(const uint8_t* __restrict__ packed, int K, int N, int8_t* __restrict__ q)
{
    __shared__ __align__(16) uint8_t tile[64][64 + 16];
    const int nt = blockIdx.x, kt = blockIdx.y;
    const int row = threadIdx.x >> 2, seg = threadIdx.x & 3;
    const uint8_t* src = packed + ((size_t)nt * (K / 64) + kt) * kTileBytes;
    *reinterpret_cast<uint4*>(&tile[row][seg * 16]) = *reinterpret_cast<const uint4*>(src + threadIdx.x * 16);
    __syncthreads();
    const int tx = threadIdx.x & 7, ty = threadIdx.x >> 3;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int kl = ty + half * 32;
        uint2 v;
        uint8_t* b = reinterpret_cast<uint8_t*>(&v);
#pragma unroll
        for (int i = 0; i < 8; ++i) b[i] = (uint8_t)(tile[tx * 8 + i][kl] ^ 0x80u);
        *reinterpret_cast<uint2*>(q + ((size_t)kt * 64 + kl) * N + nt * 64 + tx * 8) = v;
    }
}

// Bytes packed by the reference for sm75-89 (cutlass_preprocessors.cc:497-534) -> W8T64.  The reference
// layout, in closed form: rows permuted in groups of 16 by {0,1,8,9,2,3,10,11,4,5,12,13,6,7,14,15},
// transposed, column pairs interleaved per 64-row tile (byte position
// (n/2)*2K + 128*(k/64) + 64*(n%2) + k%64), +128, bytes 1 and 2 of each 32-bit word swapped.
__global__ void __launch_bounds__(256)
repack_ref_kernel(const uint8_t* __restrict__ ref, int K, int N, uint8_t* __restrict__ packed)
{
    const int nt = blockIdx.x, kt = blockIdx.y;
    uint8_t* dst = packed + ((size_t)nt * (K / 64) + kt) * kTileBytes;
    for (int e = threadIdx.x; e < kTileBytes; e += 256) {
        const int n = nt * 64 + (e >> 6);
        const int k = kt * 64 + (e & 63);  // logical reduction index wanted at this byte
        // the reference stored logical row `k` at permuted row p where perm(p % 16) == k % 16
        const int t = k & 15;
        // inverse of perm(t) = 8*((t%4)/2) + t%2 + 2*(t/4)
        const int p16 = ((t & 7) >> 1) * 4 + ((t >> 3) << 1) + (t & 1);
        const int p = (k & ~15) + p16;
        size_t pos = (size_t)(n >> 1) * (2 * (size_t)K) + 128 * (p >> 6) + 64 * (n & 1) + (p & 63);
        const int in_word = (int)(pos & 3);
        pos = (pos & ~(size_t)3) | (in_word == 1 ? 2 : (in_word == 2 ? 1 : in_word));
        dst[e] = ref[pos];
    }
}

}  // namespace

int launch_quantize_w8(const void* w, bool fp32, int K, int N, int8_t* q_rowmajor, void* packed, void* scales,
                       int variant, float* amax_ws, cudaStream_t stream)
{
    EET_CUDA(cudaMemsetAsync(amax_ws, 0, sizeof(float) * N, stream));
    dim3 g1((N + 255) / 256, K / 64), g2(N / 64, K / 64);
    if (fp32) {
        colmax_kernel<float><<<g1, 256, 0, stream>>>((const float*)w, K, N, amax_ws);
        quant_pack_kernel<float><<<g2, 256, 0, stream>>>((const float*)w, K, N, amax_ws, variant, q_rowmajor,
                                                         (uint8_t*)packed, scales);
    }
    else {
        colmax_kernel<__half><<<g1, 256, 0, stream>>>((const __half*)w, K, N, amax_ws);
        quant_pack_kernel<__half><<<g2, 256, 0, stream>>>((const __half*)w, K, N, amax_ws, variant, q_rowmajor,
                                                          (uint8_t*)packed, scales);
    }
    EET_LAUNCH_CHECK();
    return 0;
}

int launch_pack_w8(const int8_t* q, int K, int N, void* packed, cudaStream_t stream)
{
    pack_kernel<<<dim3(N / 64, K / 64), 256, 0, stream>>>(q, K, N, (uint8_t*)packed);
    EET_LAUNCH_CHECK();
    return 0;
}

int launch_unpack_w8(const void* packed, int K, int N, int8_t* q, cudaStream_t stream)
{
    unpack_kernel<<<dim3(N / 64, K / 64), 256, 0, stream>>>((const uint8_t*)packed, K, N, q);
    EET_LAUNCH_CHECK();
    return 0;
}

int launch_repack_ref_w8(const void* ref_packed, int K, int N, void* packed, cudaStream_t stream)
{
    repack_ref_kernel<<<dim3(N / 64, K / 64), 256, 0, stream>>>((const uint8_t*)ref_packed, K, N, (uint8_t*)packed);
    EET_LAUNCH_CHECK();
    return 0;
}

}  // namespace eet
