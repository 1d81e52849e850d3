// The small kernels between the GEMMs of one decoder layer: RMSNorm, gated SiLU, residual add, the
// prefill-side QKV split + rotary embedding + KV-cache store, KV-cache reordering for beam search and
// the device-resident step counters used when a decode step is replayed as a CUDA graph.
//
// Each mirrors the arithmetic of a reference kernel (cited per function) and is sized for HBM:
// 16-byte accesses, one pass over the data where the reference makes two.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

// y = x * rsqrt(mean(x^2) + eps) * gamma, fp32 math, one fp16 rounding.
// Reference: T5norm1_kernel_opt<half> (csrc/core/layer_norm.cu:490-531).  One CTA per row; the row is
// kept in registers between the two phases (n <= 8 * 2 * blockDim).
__global__ void __launch_bounds__(1024)
rmsnorm_kernel(const __half* __restrict__ x, const __half* __restrict__ gamma, __half* __restrict__ y, int n, float eps)
{
    __shared__ float red[32];
    __shared__ float s_inv;
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    const int nv = n >> 3;
    const uint4* xr = reinterpret_cast<const uint4*>(x + (size_t)row * n);
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    uint4* yr = reinterpret_cast<uint4*>(y + (size_t)row * n);
    uint4 v[2];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            v[j] = xr[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        if (threadIdx.x == 0) s_inv = rsqrtf(t / n + eps);
    }
    __syncthreads();
    const float inv = s_inv;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const uint4 g = g4[i];
            const __half2* h = reinterpret_cast<const __half2*>(&v[j]);
            const __half2* gh = reinterpret_cast<const __half2*>(&g);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(h[e]);
                const float2 gg = __half22float2(gh[e]);
                oh[e] = __float22half2_rn(make_float2(f.x * inv * gg.x, f.y * inv * gg.y));
            }
            yr[i] = o;
        }
    }
}

// ---- consumers of the skinny GEMM's fp32 sums -------------------------------------------------------
// The decode-regime GEMM leaves sum_k x[m][k] * q[k][n] in an fp32 buffer; what the reference's GEMM
// epilogue does next (multiply by the per-channel scale, round once to fp16: epilogue_helpers.h:73-80) and
// what its add_input kernel does after that (fp16 add of the residual, csrc/core/add_bias.cu:22-28) happen
// in the kernel that reads the sums.  Every reader restores the buffer to zero for the next GEMM.

__device__ __forceinline__ void load_sums8(float* p, float (&v)[8])
{
    const float4 a = __ldcg(reinterpret_cast<const float4*>(p));
    const float4 b = __ldcg(reinterpret_cast<const float4*>(p) + 1);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
    v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
    __stcg(reinterpret_cast<float4*>(p), z);
    __stcg(reinterpret_cast<float4*>(p) + 1, z);
}

// 8 outputs: fp16(sum * scale) (+ residual in fp16)
__device__ __forceinline__ uint4 finalize8(const float (&v)[8], const uint4& scale, const uint4* residual, bool gate = false)
{
    const __half2* sh = reinterpret_cast<const __half2*>(&scale);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 sc = __half22float2(sh[e]);
        oh[e] = __floats2half2_rn(v[2 * e] * sc.x, v[2 * e + 1] * sc.y);
    }
    if (residual != nullptr) {
        const __half2* rh = reinterpret_cast<const __half2*>(residual);
        if (gate) {
#pragma unroll
            for (int e = 0; e < 4; ++e) oh[e] = gated_silu2(rh[e], oh[e]);
        }
        else {
#pragma unroll
            for (int e = 0; e < 4; ++e) oh[e] = __hadd2(oh[e], rh[e]);
        }
    }
    return o;
}

// C = fp16(sums * scale) (+ residual, or gated_silu(residual, .) with gate set); sums <- 0.
__global__ void __launch_bounds__(256)
finalize_kernel(float* __restrict__ sums, const __half* __restrict__ scale, const __half* __restrict__ residual,
                __half* __restrict__ C, int N, size_t nvec, int gate)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    const int col = (int)((i * 8) % (size_t)N);
    float v[8];
    load_sums8(sums + i * 8, v);
    const uint4 sc = *reinterpret_cast<const uint4*>(scale + col);
    uint4 r;
    if (residual != nullptr) r = reinterpret_cast<const uint4*>(residual)[i];
    reinterpret_cast<uint4*>(C)[i] = finalize8(v, sc, residual ? &r : nullptr, gate != 0);
}

// Row kernel at the head of an attention or FFN block during decode.  With sums != null it first finishes
// the projection GEMM that produced this block's input: h = fp16(sums * scale) + residual, written to
// h_out as the new residual stream; with sums == null the input is `residual` itself.  Then
// xn = h * rsqrt(mean(h^2) + eps) * gamma as in rmsnorm_kernel above.
__global__ void __launch_bounds__(1024)
rmsnorm_finalize_kernel(float* __restrict__ sums, const __half* __restrict__ scale, const __half* __restrict__ residual,
                        __half* __restrict__ h_out, const __half* __restrict__ gamma, __half* __restrict__ xn_out, int n,
                        float eps)
{
    __shared__ float red[32];
    pdl_launch_dependents();
    const int row = blockIdx.x;
    const int nv = n >> 3;
    // the per-channel scales and the norm weights are constants: fetched while the preceding GEMM still runs,
    // so that neither of the two phases below waits for them
    uint4 scv[2], gv[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        scv[j] = make_uint4(0u, 0u, 0u, 0u);
        gv[j] = scv[j];
        if (i < nv) {
            gv[j] = reinterpret_cast<const uint4*>(gamma)[i];
            if (sums != nullptr) scv[j] = reinterpret_cast<const uint4*>(scale)[i];
        }
    }
    pdl_wait();
    const uint4* rr = reinterpret_cast<const uint4*>(residual + (size_t)row * n);
    uint4 h[2];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            h[j] = rr[i];
            if (sums != nullptr) {
                float v[8];
                load_sums8(sums + (size_t)row * n + (size_t)i * 8, v);
                h[j] = finalize8(v, scv[j], &h[j]);
                reinterpret_cast<uint4*>(h_out + (size_t)row * n)[i] = h[j];
            }
            const __half2* hh = reinterpret_cast<const __half2*>(&h[j]);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(hh[e]);
                ss += f.x * f.x + f.y * f.y;
            }
        }
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    // every warp adds the (at most 32) per-warp sums itself, in the same order: one barrier instead of two
    float tot = (threadIdx.x & 31) < (blockDim.x >> 5) ? red[threadIdx.x & 31] : 0.f;
    tot = warp_sum(tot);
    const float inv = rsqrtf(tot / n + eps);
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = threadIdx.x + j * blockDim.x;
        if (i < nv) {
            const __half2* hh = reinterpret_cast<const __half2*>(&h[j]);
            const __half2* gh = reinterpret_cast<const __half2*>(&gv[j]);
            uint4 o;
            __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(hh[e]);
                const float2 gg = __half22float2(gh[e]);
                oh[e] = __float22half2_rn(make_float2(f.x * inv * gg.x, f.y * inv * gg.y));
            }
            reinterpret_cast<uint4*>(xn_out + (size_t)row * n)[i] = o;
        }
    }
}

// Tensor-parallel form of rmsnorm_finalize_kernel: the all-reduce of a row-parallel projection fused into
// the kernel that consumes it, with the latency of ONE NVLink hop.  Every rank's GEMM has left its partial
// sums in local memory.  A row's CTAs push them into an inbox in every peer's memory (peer stores over
// NVLink) as 16-byte packets {v0, v1, v2, epoch}: the receiver needs no separate flag and no fence - it polls
// its own (local) inbox until the packets carry the epoch of this exchange, the scheme of NCCL's low-latency
// protocols.  ASSUMPTION: an aligned 16-byte vector store arrives in the peer's memory as one piece, i.e. a
// 16-byte load never sees the new epoch word beside old value words (NVLink delivers such a store as one
// packet; NCCL's 128-byte protocol rests on the same property).  The partial rows are added in fp32 in rank
// order, so every rank forms bit-identical sums; then scale, residual and RMSNorm as on one GPU.  Two
// inboxes alternate (attention output projection / FFN down projection): a peer can overwrite an inbox only
// after the exchange in between, which needs this rank's push, which follows this rank's reads.
struct TpPeers {
    uint4* inbox[8];   // every rank's inbox [2][8 source ranks][64 rows][n/8][3] packets (index = rank)
    int world, rank, which;
};

constexpr int kTpRows = 64;       // rows an inbox holds: decode batches up to 64
constexpr int kTpPackets = 3;     // 16-byte packets per 8 values: {v0,v1,v2,e} {v3,v4,v5,e} {v6,v7,-,e}

__device__ __forceinline__ uint4 ld_volatile_u4(const void* p)
{
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// One row is split over the CTAs of a thread-block cluster (up to 8): the peer stores of a row leave from
// up to 8 SMs instead of one (what one SM can push over NVLink per microsecond bounded the exchange at 4 and 8
// ranks), and the row's sum of squares meets through distributed shared memory.  One 8-float vector per thread.
// kMaxThreads = 256 (every hidden size up to 16384 with a cluster of 8) leaves the registers for polling all peers
// at once; 1024 is the fallback for rows that a smaller cluster has to cover.
template<int kMaxThreads>
__global__ void __launch_bounds__(kMaxThreads)
rmsnorm_finalize_tp_kernel(TpPeers peers, float* __restrict__ local_sums, int* __restrict__ epochs,
                           const __half* __restrict__ scale, const __half* __restrict__ residual,
                           __half* __restrict__ h_out, const __half* __restrict__ gamma, __half* __restrict__ xn_out,
                           int n, float eps)
{
    namespace cgx = cooperative_groups;
    cgx::cluster_group cluster = cgx::this_cluster();
    __shared__ float red[32];
    __shared__ float s_parts[8]; // every CTA's share of the row's sum of squares, written by the owners
    __shared__ int s_epoch;
    pdl_launch_dependents();
    const int slices = (int)cluster.num_blocks();
    const int slice = (int)cluster.block_rank();
    const int row = blockIdx.x / slices;
    // constants first, while the preceding GEMM still runs
    const uint4 sc = reinterpret_cast<const uint4*>(scale)[slice * blockDim.x + threadIdx.x];
    const uint4 g = reinterpret_cast<const uint4*>(gamma)[slice * blockDim.x + threadIdx.x];
    pdl_wait();   // this rank's GEMM (and everything before it) is complete
    const uint32_t spin_limit = g_wait_limit;
    // every CTA of the row derives the epoch from the counter; the row's first CTA advances it afterwards
    if (threadIdx.x == 0) s_epoch = epochs[peers.which * kTpRows + row] + 1;
    __syncthreads();
    const uint32_t epoch = (uint32_t)s_epoch;
    const int i = slice * blockDim.x + threadIdx.x;   // this thread's vector of 8 columns
    const size_t row_packets = (size_t)(n >> 3) * kTpPackets;
    // packet index of this thread's first packet inside the inbox of source rank `src`
    auto slot = [&](int src) -> size_t {
        return ((size_t)(peers.which * 8 + src) * kTpRows + row) * row_packets + (size_t)i * kTpPackets;
    };

    // ---- push this rank's partial row to every peer, keep a copy, zero the local sums for the next GEMM ----
    float mine[8];
    {
        float4* lp = reinterpret_cast<float4*>(local_sums + (size_t)row * n + (size_t)i * 8);
        const float4 a = lp[0], b = lp[1];
        mine[0] = a.x; mine[1] = a.y; mine[2] = a.z; mine[3] = a.w;
        mine[4] = b.x; mine[5] = b.y; mine[6] = b.z; mine[7] = b.w;
        const float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
        lp[0] = z;
        lp[1] = z;
#pragma unroll
        for (int p = 0; p < 8; ++p) {
            if (p < peers.world && p != peers.rank) {
                uint4* dst = peers.inbox[p] + slot(peers.rank);
                dst[0] = make_uint4(__float_as_uint(mine[0]), __float_as_uint(mine[1]), __float_as_uint(mine[2]), epoch);
                dst[1] = make_uint4(__float_as_uint(mine[3]), __float_as_uint(mine[4]), __float_as_uint(mine[5]), epoch);
                dst[2] = make_uint4(__float_as_uint(mine[6]), __float_as_uint(mine[7]), 0u, epoch);
            }
        }
    }

    // ---- collect: poll the local inbox until every peer's packets carry this epoch, add in rank order ----
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = 0.f;
    if (kMaxThreads <= 256) {
        // All pending peers are polled in the same round trip: a poll is a load from this GPU's memory, and with one
        // peer after the other every rank that had already arrived still cost its own round trip (measured at 4
        // ranks: the decode step 1.4 % shorter this way).
        uint4 c[8][kTpPackets];
        uint32_t pending = 0;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < peers.world && r != peers.rank) pending |= 1u << r;
        }
        uint32_t spins = 0;
        while (pending != 0) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (pending & (1u << r)) {
                    const uint4* src = peers.inbox[peers.rank] + slot(r);
#pragma unroll
                    for (int e = 0; e < kTpPackets; ++e) c[r][e] = ld_volatile_u4(src + e);
                }
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (pending & (1u << r)) {
                    bool ok = true;
#pragma unroll
                    for (int e = 0; e < kTpPackets; ++e) ok = ok && c[r][e].w == epoch;
                    if (ok) pending &= ~(1u << r);
                }
            }
            if (pending != 0 && ++spins > spin_limit) {
                g_device_status = 4;   // a peer never arrived: give up, the host reads the status word
                break;
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= peers.world) continue;
            if (r == peers.rank) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += mine[e];
                continue;
            }
            v[0] += __uint_as_float(c[r][0].x); v[1] += __uint_as_float(c[r][0].y); v[2] += __uint_as_float(c[r][0].z);
            v[3] += __uint_as_float(c[r][1].x); v[4] += __uint_as_float(c[r][1].y); v[5] += __uint_as_float(c[r][1].z);
            v[6] += __uint_as_float(c[r][2].x); v[7] += __uint_as_float(c[r][2].y);
        }
    }
    else {
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= peers.world) continue;
            if (r == peers.rank) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] += mine[e];
                continue;
            }
            const uint4* src = peers.inbox[peers.rank] + slot(r);
            uint4 c[kTpPackets];
            uint32_t spins = 0;
            while (true) {
#pragma unroll
                for (int e = 0; e < kTpPackets; ++e) c[e] = ld_volatile_u4(src + e);
                bool ok = true;
#pragma unroll
                for (int e = 0; e < kTpPackets; ++e) ok = ok && c[e].w == epoch;
                if (ok) break;
                if (++spins > spin_limit) {
                    g_device_status = 4;   // a peer never arrived: give up, the host reads the status word
                    break;
                }
            }
            v[0] += __uint_as_float(c[0].x); v[1] += __uint_as_float(c[0].y); v[2] += __uint_as_float(c[0].z);
            v[3] += __uint_as_float(c[1].x); v[4] += __uint_as_float(c[1].y); v[5] += __uint_as_float(c[1].z);
            v[6] += __uint_as_float(c[2].x); v[7] += __uint_as_float(c[2].y);
        }
    }
    uint4 h = reinterpret_cast<const uint4*>(residual + (size_t)row * n)[i];
    h = finalize8(v, sc, &h);
    reinterpret_cast<uint4*>(h_out + (size_t)row * n)[i] = h;
    float ss = 0.f;
    const __half2* hh = reinterpret_cast<const __half2*>(&h);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(hh[e]);
        ss += f.x * f.x + f.y * f.y;
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x < 32) {
        float t = (threadIdx.x < (blockDim.x >> 5)) ? red[threadIdx.x] : 0.f;
        t = warp_sum(t);
        // this CTA's share goes into EVERY CTA's shared memory (lane c writes to CTA c): after the cluster
        // barrier each CTA adds the shares from its own memory and nobody touches a peer's any more
        if ((int)threadIdx.x < slices) *cluster.map_shared_rank(&s_parts[slice], threadIdx.x) = t;
    }
    cluster.sync();   // every share is written (and every CTA has read the old epoch counter)
    float total = 0.f;
    for (int c = 0; c < slices; ++c) total += s_parts[c];   // same order in every CTA
    if (slice == 0 && threadIdx.x == 0) epochs[peers.which * kTpRows + row] = (int)epoch;
    const float inv = rsqrtf(total / n + eps);
    {
        const __half2* gh = reinterpret_cast<const __half2*>(&g);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(hh[e]);
            const float2 gg = __half22float2(gh[e]);
            oh[e] = __float22half2_rn(make_float2(f.x * inv * gg.x, f.y * inv * gg.y));
        }
        reinterpret_cast<uint4*>(xn_out + (size_t)row * n)[i] = o;
    }
}

// (gated_silu2, the reference's gated SiLU on half2, lives in common.cuh: the GEMM epilogues use it too)

__global__ void __launch_bounds__(256)
swiglu_kernel(__half* __restrict__ gate, const __half* __restrict__ up, size_t nvec)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    uint4 g = reinterpret_cast<uint4*>(gate)[i];
    const uint4 u = reinterpret_cast<const uint4*>(up)[i];
    __half2* gh = reinterpret_cast<__half2*>(&g);
    const __half2* uh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
    for (int e = 0; e < 4; ++e) gh[e] = gated_silu2(gh[e], uh[e]);
    reinterpret_cast<uint4*>(gate)[i] = g;
}

// act = gated_silu(fp16(gate_sums * gate_scale), fp16(up_sums * up_scale)); both sum buffers <- 0.
__global__ void __launch_bounds__(256)
swiglu_finalize_kernel(float* __restrict__ gate_sums, const __half* __restrict__ gate_scale, float* __restrict__ up_sums,
                       const __half* __restrict__ up_scale, __half* __restrict__ act, int n, size_t nvec)
{
    pdl_launch_dependents();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const bool live = i < nvec;
    const int col = live ? (int)((i * 8) % (size_t)n) : 0;
    // constants first, while the preceding GEMM still runs
    const uint4 gsc = *reinterpret_cast<const uint4*>(gate_scale + col);
    const uint4 usc = *reinterpret_cast<const uint4*>(up_scale + col);
    pdl_wait();
    if (!live) return;
    float gv[8], uv[8];
    load_sums8(gate_sums + i * 8, gv);
    load_sums8(up_sums + i * 8, uv);
    const uint4 g = finalize8(gv, gsc, nullptr);
    const uint4 u = finalize8(uv, usc, nullptr);
    const __half2* gh = reinterpret_cast<const __half2*>(&g);
    const __half2* uh = reinterpret_cast<const __half2*>(&u);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = gated_silu2(gh[e], uh[e]);
    reinterpret_cast<uint4*>(act)[i] = o;
}

// out += in in fp16 (add_input<half>, csrc/core/add_bias.cu:22-28).
__global__ void __launch_bounds__(256)
add_residual_kernel(__half* __restrict__ out, const __half* __restrict__ in, size_t nvec)
{
    pdl_launch_dependents();
    pdl_wait();
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nvec) return;
    uint4 o = reinterpret_cast<uint4*>(out)[i];
    const uint4 a = reinterpret_cast<const uint4*>(in)[i];
    __half2* oh = reinterpret_cast<__half2*>(&o);
    const __half2* ah = reinterpret_cast<const __half2*>(&a);
#pragma unroll
    for (int e = 0; e < 4; ++e) oh[e] = __hadd2(oh[e], ah[e]);
    reinterpret_cast<uint4*>(out)[i] = o;
}

// Prefill: fused projection output [B][S][3][H][D] -> Q [B][H][S][D] and K,V straight into the caches
// [B_max][H][T_max][D] at positions 0..S-1; with rope != 0 Q and K get the NeoX rotary embedding at
// position s (the index inside the prompt; left padding is not subtracted, as in the reference).
// Reference: fused_QKV_neox_rotary_transpose (csrc/core/self_add_bias.cu:369-403) with the math of
// apply_rotary_embedding (csrc/core/common.cuh:176-226) followed by copyKV_transpose
// (csrc/core/transpose.cu:40-54); without rope, fused_QKV_transpose + copyKV_transpose as
// BaichuanMmha::forward_full does (csrc/op/baichuan_mmha.cpp:112-137).
__global__ void qkv_split_store_kernel(const __half* __restrict__ qkv, __half* __restrict__ q_out,
                                       __half* __restrict__ kcache, __half* __restrict__ vcache, int S, int H, int D,
                                       int T_max, int rope, float rope_base)
{
    // a thread owns 8 consecutive dims of the first half of a head and their partners in the second half
    // (the NeoX pairing is (i, i + D/2)): 16-byte loads and stores; blockDim / (D/16) heads per CTA
    const int half_d = D >> 1;
    const int tph = half_d >> 3;                       // threads per head
    const int s = blockIdx.x, b = blockIdx.z;
    const int h = blockIdx.y * (blockDim.x / tph) + threadIdx.x / tph;
    if (h >= H) return;
    const int i0 = (threadIdx.x % tph) * 8;
    const size_t inner = (size_t)H * D;
    const __half* src = qkv + ((size_t)b * S + s) * 3 * inner + (size_t)h * D;
    uint4 q1 = *reinterpret_cast<const uint4*>(src + i0), q2 = *reinterpret_cast<const uint4*>(src + i0 + half_d);
    uint4 k1 = *reinterpret_cast<const uint4*>(src + inner + i0);
    uint4 k2 = *reinterpret_cast<const uint4*>(src + inner + i0 + half_d);
    const uint4 v1 = *reinterpret_cast<const uint4*>(src + 2 * inner + i0);
    const uint4 v2 = *reinterpret_cast<const uint4*>(src + 2 * inner + i0 + half_d);
    if (rope) {
        __half* q1h = reinterpret_cast<__half*>(&q1);
        __half* q2h = reinterpret_cast<__half*>(&q2);
        __half* k1h = reinterpret_cast<__half*>(&k1);
        __half* k2h = reinterpret_cast<__half*>(&k2);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float ang = (float)s / powf(rope_base, (float)(2 * (i0 + e)) / (float)D);
            const float c = cosf(ang), sn = sinf(ang);
            const float a1 = __half2float(q1h[e]), a2 = __half2float(q2h[e]);
            const float b1 = __half2float(k1h[e]), b2 = __half2float(k2h[e]);
            q1h[e] = __float2half(a1 * c - a2 * sn);
            q2h[e] = __float2half(a2 * c + a1 * sn);
            k1h[e] = __float2half(b1 * c - b2 * sn);
            k2h[e] = __float2half(b2 * c + b1 * sn);
        }
    }
    __half* qd = q_out + (((size_t)b * H + h) * S + s) * D;
    *reinterpret_cast<uint4*>(qd + i0) = q1;
    *reinterpret_cast<uint4*>(qd + i0 + half_d) = q2;
    const size_t c_off = (((size_t)b * H + h) * T_max + s) * D;
    *reinterpret_cast<uint4*>(kcache + c_off + i0) = k1;
    *reinterpret_cast<uint4*>(kcache + c_off + i0 + half_d) = k2;
    *reinterpret_cast<uint4*>(vcache + c_off + i0) = v1;
    *reinterpret_cast<uint4*>(vcache + c_off + i0 + half_d) = v2;
}

// Beam-search cache reordering: cache[b] <- cache[index[b]] for the first `step` positions
// (reorderKV, csrc/core/transpose.cu:136-162).  The reference gathers in place and notes that the
// read/write order is not guaranteed; here the rows are gathered into scratch first and copied back by
// a second launch, so the result is well defined.
__global__ void __launch_bounds__(256)
gather_kv_kernel(const __half* __restrict__ kcache, const __half* __restrict__ vcache, const int64_t* __restrict__ index,
                 int H, int T_max, int step, int rowvec, uint4* __restrict__ ws, size_t per_cache_vec)
{
    // grid: (ceil(step*rowvec/256), H, B)
    const int b = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= step * rowvec) return;
    const int src_b = (int)index[b];
    const size_t src = (((size_t)src_b * H + h) * T_max) * rowvec + e;
    const size_t dst = (((size_t)b * H + h) * step) * rowvec + e;
    ws[dst] = reinterpret_cast<const uint4*>(kcache)[src];
    ws[per_cache_vec + dst] = reinterpret_cast<const uint4*>(vcache)[src];
}

__global__ void __launch_bounds__(256)
scatter_kv_kernel(__half* __restrict__ kcache, __half* __restrict__ vcache, int H, int T_max, int step, int rowvec,
                  const uint4* __restrict__ ws, size_t per_cache_vec)
{
    const int b = blockIdx.z, h = blockIdx.y;
    const int e = blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= step * rowvec) return;
    const size_t dst = (((size_t)b * H + h) * T_max) * rowvec + e;
    const size_t src = (((size_t)b * H + h) * step) * rowvec + e;
    reinterpret_cast<uint4*>(kcache)[dst] = ws[src];
    reinterpret_cast<uint4*>(vcache)[dst] = ws[per_cache_vec + src];
}

// Greedy token choice: index of the largest of n fp16 logits per row, the smallest index on ties (what
// torch.argmax returns for the reference's generation loop, python/eet/pipelines/generation.py:1185-1190).
// One CTA per row; NaN compares false and is never chosen unless the whole row is NaN (index 0).
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const __half* __restrict__ logits, int64_t* __restrict__ out, int n, size_t row_stride, int vec_ok)
{
    __shared__ float s_val[8];
    __shared__ int s_idx[8];
    pdl_launch_dependents();
    pdl_wait();
    const __half* row = logits + (size_t)blockIdx.x * row_stride;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    const int nv = vec_ok ? (n >> 3) : 0;   // 16-byte loads only when every row is 16-byte aligned
    for (int i = threadIdx.x; i < nv; i += blockDim.x) {
        const uint4 v = reinterpret_cast<const uint4*>(row)[i];
        const __half* hv = reinterpret_cast<const __half*>(&v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float f = __half2float(hv[e]);
            if (f > best) {   // strictly greater: the first (smallest) index of a maximum stays
                best = f;
                best_i = i * 8 + e;
            }
        }
    }
    for (int i = nv * 8 + threadIdx.x; i < n; i += blockDim.x) {   // tail, or everything for unaligned rows
        const float f = __half2float(row[i]);
        if (f > best) {
            best = f;
            best_i = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) {
            best = ov;
            best_i = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        s_val[threadIdx.x >> 5] = best;
        s_idx[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
            if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
                best = s_val[w];
                best_i = s_idx[w];
            }
        }
        out[blockIdx.x] = (best_i == 0x7fffffff) ? 0 : best_i;
    }
}

// Greedy token choice straight from the lm_head GEMM's fp32 sums, optionally over a vocabulary that is sharded
// across tensor-parallel ranks.  One CTA per row: logit = fp16(sum * scale) - the value the reference's fp16
// lm_head (torch.nn.Linear, python/eet/transformers/modeling_llama.py:471) would have stored - then the index
// of the largest logit, the smallest index on ties (torch.argmax, python/eet/pipelines/generation.py:1185-1190);
// the sums go back to zero.  With world > 1 every rank holds the columns [col_offset, col_offset + n) of the
// vocabulary: the row's {logit bits, global index, epoch} goes into every peer's inbox as one 16-byte packet
// (peer stores over NVLink, same delivery assumption as the partial-sum exchange above), this rank polls its
// own inbox (bounded, status 4) and takes the best of all ranks - every rank the same token.  Two inbox
// halves alternate with the epoch's parity: a peer's next packet for the same half needs this rank's packet
// of the step in between, which is sent after this rank has read.
struct ArgmaxPeers {
    uint4* inbox[8];   // every rank's inbox [2][8 source ranks][64 rows] packets (index = rank)
    int world, rank;
};

__global__ void __launch_bounds__(256)
lm_head_argmax_kernel(ArgmaxPeers peers, float* __restrict__ sums, const __half* __restrict__ scale, int n, long long col_offset,
                      int* __restrict__ epochs, int64_t* __restrict__ out, __half* __restrict__ logits_out)
{
    __shared__ float s_val[8];
    __shared__ int s_idx[8];
    pdl_launch_dependents();
    pdl_wait();
    const int row = blockIdx.x;
    float* srow = sums + (size_t)row * n;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = threadIdx.x; i < (n >> 3); i += blockDim.x) {
        float v[8];
        load_sums8(srow + (size_t)i * 8, v);
        const uint4 sc = __ldg(reinterpret_cast<const uint4*>(scale) + i);
        const uint4 lg = finalize8(v, sc, nullptr);
        if (logits_out != nullptr) reinterpret_cast<uint4*>(logits_out + (size_t)row * n)[i] = lg;
        const __half* hv = reinterpret_cast<const __half*>(&lg);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float f = __half2float(hv[e]);
            if (f > best) {   // strictly greater: the first (smallest) index of a maximum stays
                best = f;
                best_i = i * 8 + e;
            }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
        if (ov > best || (ov == best && oi < best_i)) {
            best = ov;
            best_i = oi;
        }
    }
    if ((threadIdx.x & 31) == 0) {
        s_val[threadIdx.x >> 5] = best;
        s_idx[threadIdx.x >> 5] = best_i;
    }
    __syncthreads();
    if (threadIdx.x != 0) return;
    for (int w = 1; w < (int)(blockDim.x >> 5); ++w) {
        if (s_val[w] > best || (s_val[w] == best && s_idx[w] < best_i)) {
            best = s_val[w];
            best_i = s_idx[w];
        }
    }
    // a row of NaNs chooses nothing: local index 0, value -inf (it loses against any real logit of a peer)
    long long best_g = col_offset + (best_i == 0x7fffffff ? 0 : best_i);
    if (peers.world > 1) {
        const uint32_t epoch = (uint32_t)epochs[row] + 1u;
        const size_t half = (size_t)(epoch & 1u) * 8 * kTpRows;
        const uint4 mine = make_uint4(__float_as_uint(best), (uint32_t)best_g, epoch, 0u);
        for (int p = 0; p < peers.world; ++p) {
            if (p != peers.rank) peers.inbox[p][half + (size_t)peers.rank * kTpRows + row] = mine;
        }
        const uint32_t spin_limit = g_wait_limit;
        // all pending peers are polled in the same round trip (each poll is a load from this GPU's memory)
        uint4 c[8];
        uint32_t pending = 0;
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r < peers.world && r != peers.rank) pending |= 1u << r;
        }
        uint32_t spins = 0;
        while (pending != 0) {
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if (pending & (1u << r)) c[r] = ld_volatile_u4(peers.inbox[peers.rank] + half + (size_t)r * kTpRows + row);
            }
#pragma unroll
            for (int r = 0; r < 8; ++r) {
                if ((pending & (1u << r)) && c[r].z == epoch) pending &= ~(1u << r);
            }
            if (pending != 0 && ++spins > spin_limit) {
                g_device_status = 4;
                break;
            }
        }
#pragma unroll
        for (int r = 0; r < 8; ++r) {
            if (r >= peers.world || r == peers.rank || (pending & (1u << r))) continue;
            const float ov = __uint_as_float(c[r].x);
            const long long og = (long long)c[r].y;
            if (ov > best || (ov == best && og < best_g)) {
                best = ov;
                best_g = og;
            }
        }
        epochs[row] = (int)epoch;
    }
    out[row] = best_g;
}

// out[r] = table[ids[r]] for rows of n fp16 values (n a multiple of 8): the token-embedding lookup that the
// reference leaves to torch.nn.Embedding (python/eet/transformers/modeling_llama.py:281-283).
__global__ void __launch_bounds__(256)
gather_rows_kernel(const __half* __restrict__ table, const int64_t* __restrict__ ids, __half* __restrict__ out, int n,
                   int64_t rows_in_table)
{
    pdl_launch_dependents();
    pdl_wait();
    int64_t id = ids[blockIdx.x];
    if (id < 0 || id >= rows_in_table) id = 0;   // never read outside the table
    const uint4* src = reinterpret_cast<const uint4*>(table + (size_t)id * n);
    uint4* dst = reinterpret_cast<uint4*>(out + (size_t)blockIdx.x * n);
    for (int i = threadIdx.x; i < (n >> 3); i += blockDim.x) dst[i] = src[i];
}

__global__ void advance_steps_kernel(int* steps, int count, int delta)
{
    pdl_launch_dependents();
    pdl_wait();
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < count) steps[i] += delta;
}

}  // namespace

int launch_rmsnorm(const __half* x, const __half* gamma, __half* y, int M, int n, float eps, cudaStream_t stream)
{
    EET_CHECK(n % 8 == 0 && n > 0 && n <= 16384, "rmsnorm: hidden size %d must be a multiple of 8 and <= 16384", n);
    if (M == 0) return 0;
    const int nv = n / 8;
    int threads = ((nv + 1) / 2 + 31) / 32 * 32;
    if (threads < 32) threads = 32;
    if (threads > 1024) threads = 1024;
    EET_CUDA(launch_pdl(rmsnorm_kernel, dim3(M), dim3(threads), 0, stream, x, gamma, y, n, eps));
    return 0;
}

int launch_finalize(float* sums, const __half* scale, const __half* residual, __half* C, int M, int N,
                    cudaStream_t stream, int gate)
{
    EET_CHECK(N % 8 == 0, "finalize: N must be a multiple of 8");
    const size_t nvec = (size_t)M * N / 8;
    if (nvec == 0) return 0;
    EET_CUDA(launch_pdl(finalize_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, sums, scale,
                        residual, C, N, nvec, gate));
    return 0;
}

int launch_rmsnorm_finalize(float* sums, const __half* scale, const __half* residual, __half* h_out,
                            const __half* gamma, __half* xn_out, int M, int n, float eps, cudaStream_t stream)
{
    EET_CHECK(n % 8 == 0 && n > 0 && n <= 16384, "rmsnorm: hidden size %d must be a multiple of 8 and <= 16384", n);
    if (M == 0) return 0;
    const int nv = n / 8;
    int threads = ((nv + 1) / 2 + 31) / 32 * 32;
    if (threads < 32) threads = 32;
    if (threads > 1024) threads = 1024;
    EET_CUDA(launch_pdl(rmsnorm_finalize_kernel, dim3(M), dim3(threads), 0, stream, sums, scale, residual, h_out, gamma,
                        xn_out, n, eps));
    return 0;
}

int launch_rmsnorm_finalize_tp(float* local_sums, void* const* peer_inbox, int world, int rank, int which, int* epochs,
                               const __half* scale, const __half* residual, __half* h_out, const __half* gamma,
                               __half* xn_out, int M, int n, float eps, cudaStream_t stream)
{
    EET_CHECK(n % 8 == 0 && n > 0 && n <= 16384, "rmsnorm: hidden size %d must be a multiple of 8 and <= 16384", n);
    EET_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world, "tensor-parallel rmsnorm: bad world %d / rank %d",
              world, rank);
    EET_CHECK(which == 0 || which == 1, "tensor-parallel rmsnorm: inbox index %d must be 0 or 1", which);
    EET_CHECK(M <= kTpRows, "tensor-parallel rmsnorm: at most 64 rows (decode regime), got %d", M);
    if (M == 0) return 0;
    TpPeers peers = {};
    for (int r = 0; r < world; ++r) {
        EET_CHECK(peer_inbox[r] != nullptr, "tensor-parallel rmsnorm: NULL peer pointer");
        EET_CHECK((reinterpret_cast<uintptr_t>(peer_inbox[r]) & 15u) == 0, "tensor-parallel rmsnorm: inboxes must be 16-byte aligned");
        peers.inbox[r] = reinterpret_cast<uint4*>(peer_inbox[r]);
    }
    peers.world = world;
    peers.rank = rank;
    peers.which = which;
    // the row is split over the largest cluster (8, 4, 2 or 1 CTAs) that leaves every CTA whole warps
    const int nv = n / 8;
    int slices = 8;
    while (slices > 1 && (nv % (slices * 32) != 0 || nv / slices > 1024)) slices >>= 1;
    // whole warps only: the block reductions shuffle with the full mask
    EET_CHECK(nv % slices == 0 && (nv / slices) % 32 == 0 && nv / slices <= 1024,
              "tensor-parallel rmsnorm: hidden size %d is not supported (a multiple of 256 up to 65536 is required)", n);
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)(M * slices));
    cfg.blockDim = dim3((unsigned)(nv / slices));
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)slices;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    if (nv / slices <= 256) {
        EET_CUDA(cudaLaunchKernelEx(&cfg, rmsnorm_finalize_tp_kernel<256>, peers, local_sums, epochs, scale, residual, h_out,
                                    gamma, xn_out, n, eps));
    }
    else {
        EET_CUDA(cudaLaunchKernelEx(&cfg, rmsnorm_finalize_tp_kernel<1024>, peers, local_sums, epochs, scale, residual, h_out,
                                    gamma, xn_out, n, eps));
    }
    return 0;
}

int launch_swiglu_finalize(float* gate_sums, const __half* gate_scale, float* up_sums, const __half* up_scale,
                           __half* act_out, int M, int n, cudaStream_t stream)
{
    EET_CHECK(n % 8 == 0, "swiglu: inner size %d must be a multiple of 8", n);
    const size_t nvec = (size_t)M * n / 8;
    if (nvec == 0) return 0;
    EET_CUDA(launch_pdl(swiglu_finalize_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, gate_sums,
                        gate_scale, up_sums, up_scale, act_out, n, nvec));
    return 0;
}

int launch_swiglu(__half* gate_inout, const __half* up, int M, int n, cudaStream_t stream)
{
    EET_CHECK(n % 8 == 0, "swiglu: inner size %d must be a multiple of 8", n);
    const size_t nvec = (size_t)M * n / 8;
    if (nvec == 0) return 0;
    EET_CUDA(launch_pdl(swiglu_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, gate_inout, up, nvec));
    return 0;
}

int launch_add_residual(__half* out, const __half* in, size_t count, cudaStream_t stream)
{
    EET_CHECK(count % 8 == 0, "add_residual: element count must be a multiple of 8");
    const size_t nvec = count / 8;
    if (nvec == 0) return 0;
    EET_CUDA(launch_pdl(add_residual_kernel, dim3((unsigned)((nvec + 255) / 256)), dim3(256), 0, stream, out, in, nvec));
    return 0;
}

int launch_qkv_split_store(const __half* qkv, __half* q_out, __half* kcache, __half* vcache, int B, int S, int H,
                           int D, int T_max, int rope, float rope_base, cudaStream_t stream)
{
    EET_CHECK(D % 16 == 0 && D <= 2048, "qkv_split_store: head size %d unsupported (multiples of 16 up to 2048)", D);
    EET_CHECK(S <= T_max, "qkv_split_store: prompt length %d exceeds the cache length %d", S, T_max);
    EET_CHECK(B <= 65535, "qkv_split_store: batch too large for the grid");
    if (B == 0 || S == 0) return 0;
    const int tph = D / 16;                         // threads per head
    int heads_per_cta = 256 / tph;
    if (heads_per_cta < 1) heads_per_cta = 1;
    if (heads_per_cta > H) heads_per_cta = H;
    const int threads = heads_per_cta * tph;
    qkv_split_store_kernel<<<dim3(S, (H + heads_per_cta - 1) / heads_per_cta, B), threads, 0, stream>>>(
        qkv, q_out, kcache, vcache, S, H, D, T_max, rope, rope_base);
    EET_LAUNCH_CHECK();
    return 0;
}

int launch_reorder_kv(__half* kcache, __half* vcache, const int64_t* index, int B, int H, int D, int T_max, int step,
                      __half* ws, cudaStream_t stream)
{
    EET_CHECK(D % 8 == 0, "reorder_kv: head size must be a multiple of 8");
    const int rowvec = D / 8;
    const size_t per_cache_vec = (size_t)B * H * step * rowvec;
    dim3 grid((step * rowvec + 255) / 256, H, B);
    gather_kv_kernel<<<grid, 256, 0, stream>>>(kcache, vcache, index, H, T_max, step, rowvec, (uint4*)ws,
                                               per_cache_vec);
    scatter_kv_kernel<<<grid, 256, 0, stream>>>(kcache, vcache, H, T_max, step, rowvec, (const uint4*)ws,
                                                per_cache_vec);
    EET_LAUNCH_CHECK();
    return 0;
}

int launch_argmax_rows(const __half* logits, int64_t* out, int rows, int n, size_t row_stride, cudaStream_t stream)
{
    if (rows == 0) return 0;
    const int vec_ok = (reinterpret_cast<uintptr_t>(logits) % 16 == 0 && row_stride % 8 == 0) ? 1 : 0;
    EET_CUDA(launch_pdl(argmax_rows_kernel, dim3(rows), dim3(256), 0, stream, logits, out, n, row_stride, vec_ok));
    return 0;
}

int launch_lm_head_argmax(float* sums, const __half* scale, int M, int n, long long col_offset, void* const* peer_inbox,
                          int world, int rank, int* epochs, int64_t* out, __half* logits_out, cudaStream_t stream)
{
    EET_CHECK(n > 0 && n % 8 == 0, "lm_head argmax: the local vocabulary size %d must be a multiple of 8", n);
    EET_CHECK(world >= 1 && world <= 8 && rank >= 0 && rank < world, "lm_head argmax: bad world %d / rank %d", world, rank);
    EET_CHECK(col_offset >= 0 && col_offset + n <= 0x7fffffffLL, "lm_head argmax: vocabulary range out of bounds");
    ArgmaxPeers peers = {};
    peers.world = world;
    peers.rank = rank;
    if (world > 1) {
        EET_CHECK(M <= kTpRows, "lm_head argmax: at most 64 rows with a sharded vocabulary, got %d", M);
        EET_CHECK(peer_inbox != nullptr && epochs != nullptr, "lm_head argmax: a sharded vocabulary needs inboxes and epochs");
        for (int r = 0; r < world; ++r) {
            EET_CHECK(peer_inbox[r] != nullptr && (reinterpret_cast<uintptr_t>(peer_inbox[r]) & 15u) == 0,
                      "lm_head argmax: inboxes must be non-NULL and 16-byte aligned");
            peers.inbox[r] = reinterpret_cast<uint4*>(peer_inbox[r]);
        }
    }
    if (M == 0) return 0;
    EET_CUDA(launch_pdl(lm_head_argmax_kernel, dim3(M), dim3(256), 0, stream, peers, sums, scale, n, col_offset, epochs,
                        out, logits_out));
    return 0;
}

int launch_gather_rows(const __half* table, const int64_t* ids, __half* out, int rows, int n, int64_t rows_in_table,
                       cudaStream_t stream)
{
    EET_CHECK(n % 8 == 0, "gather_rows: row length %d must be a multiple of 8", n);
    if (rows == 0) return 0;
    EET_CUDA(launch_pdl(gather_rows_kernel, dim3(rows), dim3(256), 0, stream, table, ids, out, n, rows_in_table));
    return 0;
}

int launch_advance_steps(int* steps, int count, int delta, cudaStream_t stream)
{
    if (count <= 0) return 0;
    EET_CUDA(launch_pdl(advance_steps_kernel, dim3((count + 127) / 128), dim3(128), 0, stream, steps, count, delta));
    return 0;
}

}  // namespace eet
