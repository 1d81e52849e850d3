// Decode-step masked multi-head attention over the KV cache, and the prefill self-attention that
// fills it.
//
// Decode replaces masked_attention_kernel_opt (csrc/core/attention_dispatch.cu:140-324, LLaMA /
// Baichuan-7B) and t5_masked_attention_kernel (:1155-1336, Baichuan-13B with ALiBi), plus the decode
// branch of fused_QKV_neox_rotary_transpose (csrc/core/self_add_bias.cu:369-403) that precedes them:
// the rotary embedding of the new q,k and the cache append happen inside this kernel.
//
// B200 design: the cache is [B][H][T][D], so one (batch, head) history is a contiguous stream.  A
// thread-block cluster of 1-8 CTAs shares one (batch, head): every CTA walks its slice of the history
// once, a half-warp per time step with 16-byte loads of K and V, keeping a running (max, sum,
// accumulator) per half-warp; the partial results meet in shared memory, then across the cluster
// through distributed shared memory, so no global scratch and no second launch are needed, and the
// history length is not capped by shared memory (the reference stores all logits there: < 4096).
//
// Numerics kept from the reference: logits are rounded to fp16 before the softmax (:238), the ALiBi
// bias is added in fp16 (:1249), padded positions are excluded (:219-220), the softmax denominator
// gets + 1e-6 (:264), P.V accumulates in fp32.
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"

namespace cg = cooperative_groups;

namespace eet {

namespace {

constexpr int kAttnConsumerWarps = 4;
constexpr int kAttnConsumerThreads = kAttnConsumerWarps * 32;
constexpr int kAttnThreads = kAttnConsumerThreads + 32;  // + one producer warp
constexpr int kHalfWarps = kAttnConsumerThreads / 16;
#ifndef EET_ATTN_TILE
#define EET_ATTN_TILE 32
#define EET_ATTN_STAGES 2
#define EET_ATTN_CTAS 5
#endif
constexpr int kAttnTile = EET_ATTN_TILE;                     // time steps per shared-memory stage
constexpr int kAttnStages = EET_ATTN_STAGES;
constexpr int kAttnCtasPerSm = EET_ATTN_CTAS;
constexpr int kAttnRowBytes = 256;                        // D = 128 halves
constexpr int kAttnStageBytes = 2 * kAttnTile * kAttnRowBytes;  // K tile + V tile

struct OnlineState {
    float m;       // running max
    float l;       // running sum of exp(s - m)
    float acc[8];  // this lane's 8 of the D accumulators
};

// Sum over the 16 lanes of one half-warp.  The two half-warps of a warp work on different time steps
// and may diverge, so the shuffle names only the caller's own half.
__device__ __forceinline__ float half_warp_sum(float v)
{
    const uint32_t mask = 0xffffu << (threadIdx.x & 16);
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) v += __shfl_xor_sync(mask, v, o);
    return v;
}

__device__ __forceinline__ float dot8(const uint4& k, const float (&q)[8])
{
    const __half2* h = reinterpret_cast<const __half2*>(&k);
    float s = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        s += f.x * q[2 * e] + f.y * q[2 * e + 1];
    }
    return s;
}

__device__ __forceinline__ void online_update(OnlineState& st, float s, const uint4& v)
{
    // s may be -inf (never NaN); st.m starts at -1e20 so the differences below stay finite or -inf
    const float m_new = fmaxf(st.m, s);
    const float corr = __expf(st.m - m_new);
    const float p = __expf(s - m_new);
    st.l = st.l * corr + p;
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float2 f = __half22float2(h[e]);
        st.acc[2 * e] = st.acc[2 * e] * corr + p * f.x;
        st.acc[2 * e + 1] = st.acc[2 * e + 1] * corr + p * f.y;
    }
    st.m = m_new;
}

struct AttnSmem {
    uint64_t full[kAttnStages];
    uint64_t empty[kAttnStages];
    __half q[128], k[128], v[128];
    float m[kHalfWarps], l[kHalfWarps];
    float acc[kHalfWarps][128];
    // the merged partial (max, sum, accumulator) of every CTA of the cluster, written into cluster rank 0's
    // copy of this structure through distributed shared memory
    float c_acc[8][128];
    float c_ml[8][2];
    volatile int abort;
};

// D is fixed at 128 (16 lanes x 8 halves); the dispatch rejects other head sizes.
//
// Data path: the history slice of a CTA is contiguous in the [B][H][T][D] caches, so a producer warp
// streams it with 1-D bulk copies (TMA engine) of 32 time steps of K and of V per stage into a two-stage
// ring; five CTAs per SM keep ~160 KiB in flight.  Register-level loads of the same bytes stall on the
// number of outstanding L1 misses long before HBM is busy.  Four consumer warps take a half-warp per time
// step from shared memory.
__global__ void __launch_bounds__(kAttnThreads, kAttnCtasPerSm)
decode_mha_kernel(DecodeAttnArgs a)
{
    constexpr int D = 128;
    extern __shared__ __align__(128) uint8_t attn_dyn[];
    __shared__ __align__(16) AttnSmem sm;
    cg::cluster_group cluster = cg::this_cluster();
    const int splits = (int)cluster.num_blocks();
    const int split = (int)cluster.block_rank();
    const int bh = blockIdx.y;
    const int b = bh / a.H, h = bh % a.H;
    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int hw = tid >> 4;  // half-warp index inside the CTA (consumers: 0..7)
    const int hl = tid & 15;  // lane inside the half-warp: owns dims 8*hl .. 8*hl+7

    if (tid == 0) {
        for (int s = 0; s < kAttnStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kAttnConsumerWarps);
        }
        sm.abort = 0;
        mbar_fence_init();
    }

    pdl_launch_dependents();
    __syncthreads();  // barriers initialised (before the wait below, so that nothing stands between it and the
                      // producer's first request)
    // everything this kernel reads that an earlier kernel of the same step produced (the projection of the
    // new token, the device-resident step) comes after this wait
    pdl_wait();
    int step = a.step_dev ? *a.step_dev : a.step;
    // A device-resident step is not seen by the host-side range check.  Outside [1, T_max] the append would land in
    // another head's cache (or past the allocation) and the tile sizes below would go negative: record status 5,
    // touch no cache row and request no tile; every CTA still walks the same path to the cluster barrier and the
    // context of this (batch, head) comes out as zeros.
    const bool step_ok = (step >= 1 && step <= a.T_max);
    if (!step_ok) {
        if (tid == 0) g_device_status = 5;
        step = 1;
    }
    const size_t inner = (size_t)a.H * D;

    // ---- slice of the history owned by this CTA: equal numbers of time steps (not of tiles: with 580 steps
    // and two CTAs that is 290 + 290, ten tiles each, instead of 320 + 260) ----
    const int chunk = (step + splits - 1) / splits;
    const int t_begin = split * chunk;
    const int t_end = min(step, t_begin + chunk);
    int pad = 0;
    if (a.pad_len != nullptr) pad = (int)a.pad_len[b];
    const int t_first = max(t_begin, pad / kAttnTile * kAttnTile);  // whole tiles left of the padding are skipped
    const int n_tiles = (step_ok && t_end > t_first) ? (t_end - t_first + kAttnTile - 1) / kAttnTile : 0;
    const size_t cache_row0 = ((size_t)b * a.H + h) * a.T_max;

    if (warp == kAttnConsumerWarps) {
        // ------------------------------------------------------------------ producer warp (one lane)
        if ((tid & 31) == 0) {
            for (int j = 0; j < n_tiles; ++j) {
                const int s = j % kAttnStages;
                if (j >= kAttnStages && !sm.abort) {
                    if (!mbar_wait_bounded(&sm.empty[s], ((j / kAttnStages) - 1) & 1)) {
                        sm.abort = 1;
                        g_device_status = 3;
                    }
                }
                const int t = t_first + j * kAttnTile;
                // rows up to the cache end may be copied: rows at or beyond `step` are never used
                const int rows = min(kAttnTile, a.T_max - t);
                if (rows <= 0) break;   // cannot happen for a step inside the cache; never hand the copy engine a negative size
                uint8_t* dst = attn_dyn + (size_t)s * kAttnStageBytes;
                mbar_arrive_expect_tx(&sm.full[s], (uint32_t)(2 * rows * kAttnRowBytes));
                bulk_g2s(dst, a.kcache + (cache_row0 + t) * D, (uint32_t)(rows * kAttnRowBytes), &sm.full[s]);
                bulk_g2s(dst + kAttnTile * kAttnRowBytes, a.vcache + (cache_row0 + t) * D,
                         (uint32_t)(rows * kAttnRowBytes), &sm.full[s]);
            }
        }
    }
    else {
        // ---- new token: rotate q,k at position step-1, round to fp16 as the reference's buffers do ----
        // The projection arrives either as fp16 [B][3][H][D] or as the fp32 sums of the skinny GEMM, which
        // are finished here: fp16(sum * scale), the value the reference's GEMM epilogue would have stored.
        auto proj = [&](int which, int i) -> __half {
            const size_t col = (size_t)which * inner + (size_t)h * D + i;
            if (a.qkv_sums != nullptr) {
                return __float2half(__ldcg(a.qkv_sums + (size_t)b * 3 * inner + col) * __half2float(a.qkv_scale[col]));
            }
            return a.qkv[(size_t)b * 3 * inner + col];
        };
        if (tid < D / 2) {
            const int i = tid;
            const __half hq1 = proj(0, i), hq2 = proj(0, i + D / 2), hk1 = proj(1, i), hk2 = proj(1, i + D / 2);
            if (a.rope) {
                const float q1 = __half2float(hq1), q2 = __half2float(hq2);
                const float k1 = __half2float(hk1), k2 = __half2float(hk2);
                const float ang = (float)(step - 1) / powf(a.rope_base, (float)(2 * i) / (float)D);
                const float c = cosf(ang), sn = sinf(ang);
                sm.q[i] = __float2half(q1 * c - q2 * sn);
                sm.q[i + D / 2] = __float2half(q2 * c + q1 * sn);
                sm.k[i] = __float2half(k1 * c - k2 * sn);
                sm.k[i + D / 2] = __float2half(k2 * c + k1 * sn);
            }
            else {
                sm.q[i] = hq1;
                sm.q[i + D / 2] = hq2;
                sm.k[i] = hk1;
                sm.k[i + D / 2] = hk2;
            }
        }
        else {
            const int i = tid - D / 2;
            sm.v[i] = proj(2, i);
            sm.v[i + D / 2] = proj(2, i + D / 2);
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kAttnConsumerThreads) : "memory");

        // cache append: done by the CTA whose slice holds the newest position
        if (step_ok && step - 1 >= t_begin && step - 1 < t_end && tid < 32) {
            uint4* kd = reinterpret_cast<uint4*>(a.kcache + (cache_row0 + step - 1) * D);
            uint4* vd = reinterpret_cast<uint4*>(a.vcache + (cache_row0 + step - 1) * D);
            if (tid < 16) {
                kd[tid] = reinterpret_cast<const uint4*>(sm.k)[tid];
            }
            else {
                vd[tid - 16] = reinterpret_cast<const uint4*>(sm.v)[tid - 16];
            }
        }

        float q[8];
        {
            const uint4 qv = reinterpret_cast<const uint4*>(sm.q)[hl];
            const __half2* qh = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f = __half22float2(qh[e]);
                q[2 * e] = f.x;
                q[2 * e + 1] = f.y;
            }
        }
        // the reference multiplies by the fp16-rounded 1/sqrt(D) (csrc/op/llama_mmha.cpp:80-84)
        const float scalar = __half2float(__float2half(sqrtf(1.0f / D)));
        const float slope = a.alibi_slopes ? a.alibi_slopes[h] : 0.f;

        OnlineState st;
        st.m = -1e20f;
        st.l = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) st.acc[e] = 0.f;

        constexpr int U = kAttnTile / kHalfWarps;  // time steps per half-warp and tile
        for (int j = 0; j < n_tiles; ++j) {
            const int s = j % kAttnStages;
            if (!sm.abort) {
                if (!mbar_wait_bounded(&sm.full[s], (j / kAttnStages) & 1)) {
                    sm.abort = 1;
                    g_device_status = 3;
                }
            }
            const uint4* kt = reinterpret_cast<const uint4*>(attn_dyn + (size_t)s * kAttnStageBytes);
            const uint4* vt = kt + kAttnTile * (kAttnRowBytes / 16);
            const int t0 = t_first + j * kAttnTile;
            uint4 kv[U], vv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int r = hw + u * kHalfWarps;
                const int t = t0 + r;
                if (t == step - 1) {  // the newest row is not in the cache copy: take it from the projection
                    kv[u] = reinterpret_cast<const uint4*>(sm.k)[hl];
                    vv[u] = reinterpret_cast<const uint4*>(sm.v)[hl];
                }
                else {
                    kv[u] = kt[r * (kAttnRowBytes / 16) + hl];
                    vv[u] = vt[r * (kAttnRowBytes / 16) + hl];
                }
            }
            // the tile's bytes are in registers: hand the stage back to the producer
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&sm.empty[s]);
            // the U time steps of this half-warp are folded into the running softmax together: independent
            // dot products and shuffle chains, one rescale of the accumulators per tile
            float sc[U];
#pragma unroll
            for (int u = 0; u < U; ++u) sc[u] = dot8(kv[u], q);
            const uint32_t hmask = 0xffffu << (tid & 16);
#pragma unroll
            for (int o = 8; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < U; ++u) sc[u] += __shfl_xor_sync(hmask, sc[u], o);
            }
            float m_new = st.m;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int t = t0 + hw + u * kHalfWarps;
                __half sh = __float2half(sc[u] * scalar);
                if (a.alibi != nullptr) {
                    sh = __hadd(sh, a.alibi[(size_t)h * a.alibi_stride + min(t, step - 1)]);
                }
                else if (a.alibi_slopes != nullptr) {
                    sh = __hadd(sh, __float2half_rn(slope * (float)t));
                }
                // positions outside [pad, t_end) get -inf, i.e. probability 0 (m_new stays >= -1e20)
                const bool valid = (t < t_end && t >= pad);
                sc[u] = valid ? __half2float(sh) : -INFINITY;
                if (!valid) vv[u] = make_uint4(0, 0, 0, 0);  // rows past the history may hold anything, even NaN
                m_new = fmaxf(m_new, sc[u]);
            }
            const float corr = __expf(st.m - m_new);
            float p[U];
            float psum = 0.f;
#pragma unroll
            for (int u = 0; u < U; ++u) {
                p[u] = __expf(sc[u] - m_new);
                psum += p[u];
            }
            st.l = st.l * corr + psum;
            st.m = m_new;
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                float a0 = st.acc[2 * e] * corr, a1 = st.acc[2 * e + 1] * corr;
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    const float2 f = __half22float2(reinterpret_cast<const __half2*>(&vv[u])[e]);
                    a0 += p[u] * f.x;
                    a1 += p[u] * f.y;
                }
                st.acc[2 * e] = a0;
                st.acc[2 * e + 1] = a1;
            }
        }

        // ---- merge the half-warps of this CTA ----
        if (hl == 0) {
            sm.m[hw] = st.m;
            sm.l[hw] = st.l;
        }
#pragma unroll
        for (int e = 0; e < 8; ++e) sm.acc[hw][hl * 8 + e] = st.acc[e];
        asm volatile("bar.sync 1, %0;" ::"n"(kAttnConsumerThreads) : "memory");
        if (tid < D) {
            float m = -1e20f;
#pragma unroll
            for (int w = 0; w < kHalfWarps; ++w) m = fmaxf(m, sm.m[w]);
            float l = 0.f, acc = 0.f;
#pragma unroll
            for (int w = 0; w < kHalfWarps; ++w) {
                const float c = __expf(sm.m[w] - m);
                l += sm.l[w] * c;
                acc += sm.acc[w][tid] * c;
            }
            // push the partial into rank 0's shared memory: after the cluster barrier rank 0 merges from its
            // own memory, and the other CTAs may leave at once
            float* dst_acc = cluster.map_shared_rank(&sm.c_acc[0][0], 0);
            dst_acc[split * 128 + tid] = acc;
            if (tid == 0) {
                float* dst_ml = cluster.map_shared_rank(&sm.c_ml[0][0], 0);
                dst_ml[split * 2 + 0] = m;
                dst_ml[split * 2 + 1] = l;
            }
        }
    }

    // ---- merge the CTAs of the cluster; rank 0 writes the context ----
    cluster.sync();
    if (split != 0) return;
    if (a.qkv_sums != nullptr) {
        // every CTA of the cluster has read the projection sums of this (batch, head): put them back to zero
        for (int e = tid; e < 3 * D; e += kAttnThreads) {
            __stcg(a.qkv_sums + (size_t)b * 3 * inner + (size_t)(e / D) * inner + (size_t)h * D + (e % D), 0.f);
        }
    }
    if (tid < D) {
        float m = -1e20f;
        for (int r = 0; r < splits; ++r) m = fmaxf(m, sm.c_ml[r][0]);
        float l = 0.f, acc = 0.f;
        for (int r = 0; r < splits; ++r) {
            const float c = __expf(sm.c_ml[r][0] - m);
            l += sm.c_ml[r][1] * c;
            acc += sm.c_acc[r][tid] * c;
        }
        a.ctx[(size_t)b * inner + (size_t)h * D + tid] = __float2half(acc * __fdividef(1.0f, l + 1e-6f));
    }
}

// Prefill self-attention, causal with optional left padding (LLaMA) or ALiBi bias (Baichuan-13B).
// Reference: q_k_mul + qk_softmax + attn_v_mul + transpose of LlamaMmha::forward_full
// (csrc/op/llama_mmha.cpp:354-426; softmax_kernel_gpt2 csrc/core/gpt2_self_softmax.cu:8-57; ALiBi
// variant masked_softmax_kernel :161-240).  The reference materialises [B,H,S,S] scores in fp16 and runs
// two cuBLAS batched GEMMs around a row-serial softmax; this kernel is blockwise (no S x S buffer):
// a CTA takes 64 consecutive queries of one (batch, head), four warps of 16 query rows each; K and V of 64
// keys at a time are staged in shared memory (cp.async, 16-byte chunks XOR-swizzled so ldmatrix is
// conflict-free, double buffered); Q.K^T and P.V run on the tensor cores (mma.sync m16n8k16, fp16 in, fp32
// accumulate) with the online softmax between them in registers.  Key blocks above the diagonal are
// never visited.
// Numerics kept: scores are scaled by the fp16-rounded 1/sqrt(D) and rounded to fp16 where the reference
// stores them in fp16, the ALiBi bias is added in fp32 after that rounding, probabilities enter P.V as
// fp16 (the reference's score buffer is fp16 too), denominator + 1e-6, rows above the left padding are
// zero.
constexpr int kPfQ = 64;         // queries per CTA
constexpr int kPfK = 64;         // keys per shared-memory block
constexpr int kPfThreads = 128;
constexpr int kPfTileBytes = 64 * 256;   // 64 rows of 128 halves

__device__ __forceinline__ uint32_t pf_swz(int row, int chunk)
{
    return (uint32_t)(row * 256 + ((chunk ^ (row & 7)) << 4));
}

__device__ __forceinline__ void cp_async16(uint32_t smem_addr, const void* gptr, bool valid)
{
    const int bytes = valid ? 16 : 0;   // src-size 0 zero-fills the destination
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_addr), "l"(gptr), "r"(bytes) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ void ldsm_x4_trans(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3)
{
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}

__device__ __forceinline__ uint32_t pack_half2(float a, float b)
{
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t*>(&h);
}

__global__ void __launch_bounds__(kPfThreads)
prefill_mha_kernel(const __half* __restrict__ q, const __half* __restrict__ kcache, const __half* __restrict__ vcache,
                   __half* __restrict__ ctx, int S, int H, int T_max, const int64_t* __restrict__ pad_len,
                   const __half* __restrict__ alibi, int alibi_stride)
{
    constexpr int D = 128;
    extern __shared__ __align__(128) uint8_t pf_smem[];   // Q tile | K[2] | V[2]
    const uint32_t sQ = smem_u32(pf_smem);
    const uint32_t sK = sQ + kPfTileBytes;
    const uint32_t sV = sK + 2 * kPfTileBytes;
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int qb = blockIdx.x;
    const int i0 = qb * kPfQ;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const int pad = (pad_len != nullptr && alibi == nullptr) ? (int)pad_len[b] : 0;
    const size_t cache_row0 = ((size_t)b * H + h) * T_max;
    const __half* qbase = q + (((size_t)b * H + h) * S) * D;
    const __half* kbase = kcache + cache_row0 * D;
    const __half* vbase = vcache + cache_row0 * D;

    auto load_tile = [&](uint32_t sdst, const __half* gsrc, int row0, int row_limit) {
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int e = tid + it * kPfThreads;   // 1024 chunks of 16 bytes
            const int r = e >> 4, c = e & 15;
            const bool ok = (row0 + r) < row_limit;
            cp_async16(sdst + pf_swz(r, c), gsrc + (size_t)(ok ? row0 + r : 0) * D + c * 8, ok);
        }
    };

    const int kb_first = pad / kPfK;                       // key blocks left of the padding are skipped
    const int kb_last = min(qb, (S - 1) / kPfK);           // causal: nothing above the diagonal block
    load_tile(sQ, qbase, i0, S);
    load_tile(sK, kbase, kb_first * kPfK, S);
    load_tile(sV, vbase, kb_first * kPfK, S);
    asm volatile("cp.async.commit_group;" ::: "memory");

    float o[16][4];
#pragma unroll
    for (int n = 0; n < 16; ++n)
#pragma unroll
        for (int c = 0; c < 4; ++c) o[n][c] = 0.f;
    float m_run[2] = {-1e20f, -1e20f}, l_run[2] = {0.f, 0.f};
    const float scalar = __half2float(__float2half(sqrtf(1.0f / D)));
    const int row_a = i0 + warp * 16 + g, row_b = row_a + 8;   // this lane's two query rows

    uint32_t qf[8][4];
    bool q_loaded = false;

    for (int kb = kb_first; kb <= kb_last; ++kb) {
        const int buf = (kb - kb_first) & 1;
        if (kb < kb_last) {   // prefetch the next key block into the other buffer
            load_tile(sK + (buf ^ 1) * kPfTileBytes, kbase, (kb + 1) * kPfK, S);
            load_tile(sV + (buf ^ 1) * kPfTileBytes, vbase, (kb + 1) * kPfK, S);
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        }
        else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        if (!q_loaded) {
            // A fragments of this warp's 16 query rows for the 8 k-steps of D = 128
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
                ldsm_x4(sQ + pf_swz(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)), qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3]);
            }
            q_loaded = true;
        }
        const uint32_t kt = sK + buf * kPfTileBytes, vt = sV + buf * kPfTileBytes;

        // ---- S = Q K^T for 64 keys: 8 n-tiles of 8 keys ----
        float sc[8][4];
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int c = 0; c < 4; ++c) sc[n][c] = 0.f;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
#pragma unroll
            for (int np = 0; np < 4; ++np) {   // two n-tiles (16 keys) per ldmatrix.x4
                uint32_t b0, b1, b2, b3;
                const int krow = np * 16 + (lane & 7) + ((lane >> 4) << 3);
                const int chunk = kk * 2 + ((lane >> 3) & 1);
                ldsm_x4(kt + pf_swz(krow, chunk), b0, b1, b2, b3);
                mma_m16n8k16(sc[2 * np], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b0, b1);
                mma_m16n8k16(sc[2 * np + 1], qf[kk][0], qf[kk][1], qf[kk][2], qf[kk][3], b2, b3);
            }
        }

        // ---- scale, fp16 rounding, bias, masks; online softmax ----
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int n = 0; n < 8; ++n) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int i = (c < 2) ? row_a : row_b;
                const int j = kb * kPfK + n * 8 + 2 * t + (c & 1);
                float v = __half2float(__float2half(sc[n][c] * scalar));
                if (alibi != nullptr && i < S && j <= i) {
                    v += __half2float(alibi[((size_t)h * alibi_stride + i) * alibi_stride + j]);
                }
                v = (j <= i && j >= pad && j < S) ? v : -INFINITY;
                sc[n][c] = v;
                mx[c >> 1] = fmaxf(mx[c >> 1], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int r = 0; r < 2; ++r) {
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
            mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
            const float m_new = fmaxf(m_run[r], mx[r]);
            corr[r] = __expf(m_run[r] - m_new);
            m_run[r] = m_new;
            l_run[r] *= corr[r];
        }
        uint32_t pfrag[4][4];   // P as A fragments: 4 k-steps of 16 keys
#pragma unroll
        for (int n = 0; n < 8; ++n) {
            const float p0 = __expf(sc[n][0] - m_run[0]), p1 = __expf(sc[n][1] - m_run[0]);
            const float p2 = __expf(sc[n][2] - m_run[1]), p3 = __expf(sc[n][3] - m_run[1]);
            l_run[0] += p0 + p1;
            l_run[1] += p2 + p3;
            pfrag[n >> 1][(n & 1) * 2] = pack_half2(p0, p1);
            pfrag[n >> 1][(n & 1) * 2 + 1] = pack_half2(p2, p3);
        }
#pragma unroll
        for (int n = 0; n < 16; ++n) {
            o[n][0] *= corr[0];
            o[n][1] *= corr[0];
            o[n][2] *= corr[1];
            o[n][3] *= corr[1];
        }

        // ---- O += P V: k-steps of 16 keys, 16 n-tiles of 8 head dims ----
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {
#pragma unroll
            for (int dp = 0; dp < 8; ++dp) {   // two d-tiles (16 dims) per ldmatrix.x4.trans
                uint32_t b0, b1, b2, b3;
                const int vrow = kk * 16 + (lane & 7) + (((lane >> 3) & 1) << 3);
                const int chunk = dp * 2 + (lane >> 4);
                ldsm_x4_trans(vt + pf_swz(vrow, chunk), b0, b1, b2, b3);
                mma_m16n8k16(o[2 * dp], pfrag[kk][0], pfrag[kk][1], pfrag[kk][2], pfrag[kk][3], b0, b1);
                mma_m16n8k16(o[2 * dp + 1], pfrag[kk][0], pfrag[kk][1], pfrag[kk][2], pfrag[kk][3], b2, b3);
            }
        }
        __syncthreads();   // all warps are done with this buffer before the next prefetch overwrites it
    }

    asm volatile("cp.async.wait_group 0;" ::: "memory");   // nothing in flight at exit when no key block was visited

    // ---- normalise and store: context layout [B][S][H*D] (the transpose of llama_mmha.cpp:418-426) ----
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
        l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
    }
#pragma unroll
    for (int r = 0; r < 2; ++r) {
        const int i = r ? row_b : row_a;
        if (i < S) {
            // rows above the left padding are zeroed by the reference (gpt2_self_softmax.cu:24-30)
            const float inv = (i < pad) ? 0.f : 1.0f / (l_run[r] + 1e-6f);
            __half* dst = ctx + (((size_t)b * S + i) * H + h) * D;
#pragma unroll
            for (int n = 0; n < 16; ++n) {
                *reinterpret_cast<uint32_t*>(dst + n * 8 + 2 * t) = pack_half2(o[n][2 * r] * inv, o[n][2 * r + 1] * inv);
            }
        }
    }
}

}  // namespace

int launch_decode_mha(const DecodeAttnArgs& a, cudaStream_t stream)
{
    EET_CHECK(a.D == 128, "decode attention: head size %d is not supported (128 only)", a.D);
    EET_CHECK(a.step_dev != nullptr || (a.step >= 1 && a.step <= a.T_max),
              "decode attention: step %d outside the cache length %d", a.step, a.T_max);
    if (a.B == 0) return 0;
    int splits = a.splits;
    if (splits == 0) {
        // as many CTAs as fit on the machine at once (5 per SM); at least 64 time steps per CTA
        const int len = a.step_dev ? a.T_max : a.step;
        const int room = kAttnCtasPerSm * sm_count() / (a.B * a.H);
        splits = 1;
        while (splits < 8 && splits * 2 <= room && len / (splits * 2) >= 64) splits *= 2;
        // more (batch, head) pairs than CTA slots: the launch runs in waves, and for long histories halves
        // balance the last wave better (measured at 1024 pairs: +13 % at 1060 steps, -10 % at 320)
        if (room == 0 && len >= 768) splits = 2;
    }
    EET_CHECK(splits == 1 || splits == 2 || splits == 4 || splits == 8, "decode attention: splits must be 1,2,4,8");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, a.B * a.H, 1);
    cfg.blockDim = dim3(kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = kAttnStages * kAttnStageBytes;
    if (kAttnStages * kAttnStageBytes > 48 * 1024) {
        static bool attr_set[64] = {};
        int dev = 0;
        EET_CUDA(cudaGetDevice(&dev));
        dev &= 63;
        if (!attr_set[dev]) {
            EET_CUDA(cudaFuncSetAttribute(decode_mha_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          kAttnStages * kAttnStageBytes));
            attr_set[dev] = true;
        }
    }
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = splits;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 2;
    EET_CUDA(cudaLaunchKernelEx(&cfg, decode_mha_kernel, a));
    return 0;
}

int launch_prefill_mha(const __half* q, const __half* kcache, const __half* vcache, __half* ctx, int B, int S, int H,
                       int D, int T_max, const int64_t* pad_len, const __half* alibi, int alibi_stride,
                       cudaStream_t stream)
{
    EET_CHECK(D == 128, "prefill attention: head size %d is not supported (128 only)", D);
    EET_CHECK(S <= T_max, "prefill attention: prompt length %d exceeds the cache length %d", S, T_max);
    if (B == 0 || S == 0) return 0;
    static bool attr_set[64] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    dev &= 63;
    const int smem = 5 * kPfTileBytes;
    if (!attr_set[dev]) {
        EET_CUDA(cudaFuncSetAttribute(prefill_mha_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
        attr_set[dev] = true;
    }
    dim3 grid((S + kPfQ - 1) / kPfQ, B * H);
    prefill_mha_kernel<<<grid, kPfThreads, smem, stream>>>(q, kcache, vcache, ctx, S, H, T_max, pad_len, alibi,
                                                          alibi_stride);
    EET_LAUNCH_CHECK();
    return 0;
}

}  // namespace eet
