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
constexpr int kAttnTile = 32;                             // time steps per shared-memory stage
constexpr int kAttnStages = 2;
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
    float c_acc[128];  // this CTA's merged partial, read by cluster rank 0 through distributed shared memory
    float c_ml[2];
    volatile int abort;
};

// D is fixed at 128 (16 lanes x 8 halves); the dispatch rejects other head sizes.
//
// Data path: the history slice of a CTA is contiguous in the [B][H][T][D] caches, so a producer warp
// streams it with 1-D bulk copies (TMA engine) of 32 time steps of K and of V per stage into a two-stage
// ring; five CTAs per SM keep ~160 KiB in flight.  Register-level loads of the same bytes stall on the
// number of outstanding L1 misses long before HBM is busy.  Four consumer warps take a half-warp per time
// step from shared memory.
__global__ void __launch_bounds__(kAttnThreads, 5)
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

    // everything this kernel reads that an earlier kernel of the same step produced (the projection of the
    // new token, the device-resident step) comes after this wait
    pdl_launch_dependents();
    pdl_wait();
    const int step = a.step_dev ? *a.step_dev : a.step;
    const size_t inner = (size_t)a.H * D;

    // ---- slice of the history owned by this CTA ----
    const int chunk = (((step + splits - 1) / splits) + kAttnTile - 1) / kAttnTile * kAttnTile;
    const int t_begin = split * chunk;
    const int t_end = min(step, t_begin + chunk);
    int pad = 0;
    if (a.pad_len != nullptr) pad = (int)a.pad_len[b];
    const int t_first = max(t_begin, pad / kAttnTile * kAttnTile);  // whole tiles left of the padding are skipped
    const int n_tiles = (t_end > t_first) ? (t_end - t_first + kAttnTile - 1) / kAttnTile : 0;
    const size_t cache_row0 = ((size_t)b * a.H + h) * a.T_max;
    __syncthreads();  // barriers initialised

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
        if (step - 1 >= t_begin && step - 1 < t_end && tid < 32) {
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
            sm.c_acc[tid] = acc;
            if (tid == 0) {
                sm.c_ml[0] = m;
                sm.c_ml[1] = l;
            }
        }
    }

    // ---- merge the CTAs of the cluster; rank 0 writes the context ----
    cluster.sync();
    if (split == 0 && a.qkv_sums != nullptr) {
        // every CTA of the cluster has read the projection sums of this (batch, head): put them back to zero
        for (int e = tid; e < 3 * D; e += kAttnThreads) {
            __stcg(a.qkv_sums + (size_t)b * 3 * inner + (size_t)(e / D) * inner + (size_t)h * D + (e % D), 0.f);
        }
    }
    if (split == 0 && tid < D) {
        float m = -1e20f;
        for (int r = 0; r < splits; ++r) {
            const float* rml = cluster.map_shared_rank(sm.c_ml, r);
            m = fmaxf(m, rml[0]);
        }
        float l = 0.f, acc = 0.f;
        for (int r = 0; r < splits; ++r) {
            const float* rml = cluster.map_shared_rank(sm.c_ml, r);
            const float* racc = cluster.map_shared_rank(sm.c_acc, r);
            const float c = __expf(rml[0] - m);
            l += rml[1] * c;
            acc += racc[tid] * c;
        }
        a.ctx[(size_t)b * inner + (size_t)h * D + tid] = __float2half(acc * __fdividef(1.0f, l + 1e-6f));
    }
    cluster.sync();  // keep every CTA's shared memory alive until rank 0 has read it
}

// Prefill self-attention, causal with optional left padding (LLaMA) or ALiBi bias (Baichuan-13B).
// Reference: q_k_mul + qk_softmax + attn_v_mul + transpose of LlamaMmha::forward_full
// (csrc/op/llama_mmha.cpp:354-426; softmax_kernel_gpt2 csrc/core/gpt2_self_softmax.cu:8-57; ALiBi
// variant masked_softmax_kernel :161-240).  The reference materialises [B,H,S,S] scores; this kernel is
// blockwise: a CTA takes 16 consecutive queries of one (batch, head), stages 32 keys/values at a time in
// shared memory and each warp runs the same online softmax as the decode kernel for its query.
// Scores are rounded to fp16 where the reference stores them in fp16; probabilities are kept in fp32.
constexpr int kPfQueries = 16;
constexpr int kPfKeys = 32;

__global__ void __launch_bounds__(kPfQueries * 32)
prefill_mha_kernel(const __half* __restrict__ q, const __half* __restrict__ kcache, const __half* __restrict__ vcache,
                   __half* __restrict__ ctx, int S, int H, int T_max, const int64_t* __restrict__ pad_len,
                   const __half* __restrict__ alibi, int alibi_stride)
{
    constexpr int D = 128;
    __shared__ __align__(16) uint4 s_k[kPfKeys][D / 8];
    __shared__ __align__(16) uint4 s_v[kPfKeys][D / 8];
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int i0 = blockIdx.x * kPfQueries;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane >> 4, hl = lane & 15;  // two half-warps per query: even / odd keys
    const int i = i0 + warp;                    // this warp's query row
    const int pad = pad_len ? (int)pad_len[b] : 0;
    const size_t cache_row0 = ((size_t)b * H + h) * T_max;
    const uint4* kc = reinterpret_cast<const uint4*>(kcache + cache_row0 * D);
    const uint4* vc = reinterpret_cast<const uint4*>(vcache + cache_row0 * D);

    float qf[8];
    if (i < S) {
        const uint4 qv = reinterpret_cast<const uint4*>(q + (((size_t)b * H + h) * S + i) * D)[hl];
        const __half2* qh = reinterpret_cast<const __half2*>(&qv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float2 f = __half22float2(qh[e]);
            qf[2 * e] = f.x;
            qf[2 * e + 1] = f.y;
        }
    }
    const float scalar = __half2float(__float2half(sqrtf(1.0f / D)));
    OnlineState st;
    st.m = -1e20f;
    st.l = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) st.acc[e] = 0.f;

    const int j_hi = min(S, i0 + kPfQueries);  // keys needed by the last query of the tile
    const int j_lo = (alibi ? 0 : pad) / kPfKeys * kPfKeys;
    for (int j0 = j_lo; j0 < j_hi; j0 += kPfKeys) {
        __syncthreads();
        for (int e = threadIdx.x; e < kPfKeys * (D / 8); e += blockDim.x) {
            const int r = e / (D / 8), c = e % (D / 8);
            if (j0 + r < S) {
                s_k[r][c] = __ldg(kc + (size_t)(j0 + r) * (D / 8) + c);
                s_v[r][c] = __ldg(vc + (size_t)(j0 + r) * (D / 8) + c);
            }
        }
        __syncthreads();
        if (i < S) {
#pragma unroll 4
            for (int r = sub; r < kPfKeys; r += 2) {
                const int j = j0 + r;
                if (j <= i && (alibi != nullptr || j >= pad)) {
                    float s = half_warp_sum(dot8(s_k[r][hl], qf)) * scalar;
                    s = __half2float(__float2half(s));
                    if (alibi != nullptr) {
                        s += __half2float(alibi[((size_t)h * alibi_stride + i) * alibi_stride + j]);
                    }
                    online_update(st, s, s_v[r][hl]);
                }
            }
        }
    }
    if (i >= S) return;
    // merge the two half-warps of the query
    const float m_o = __shfl_xor_sync(0xffffffffu, st.m, 16);
    const float l_o = __shfl_xor_sync(0xffffffffu, st.l, 16);
    const float m = fmaxf(st.m, m_o);
    const float c_self = __expf(st.m - m), c_oth = __expf(m_o - m);
    const float l = st.l * c_self + l_o * c_oth;
    float out[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
        const float o = __shfl_xor_sync(0xffffffffu, st.acc[e], 16);
        out[e] = st.acc[e] * c_self + o * c_oth;
    }
    if (sub == 0) {
        // rows above the left padding are zeroed by the reference (gpt2_self_softmax.cu:24-30)
        const bool zero_row = (alibi == nullptr) && (i < pad);
        const float inv = zero_row ? 0.f : 1.0f / (l + 1e-6f);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int e = 0; e < 4; ++e) oh[e] = __floats2half2_rn(out[2 * e] * inv, out[2 * e + 1] * inv);
        // context layout [B][S][H*D], ready for the output projection (transpose, llama_mmha.cpp:418-426)
        reinterpret_cast<uint4*>(ctx + (((size_t)b * S + i) * H + h) * D)[hl] = o;
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
        const int room = 5 * sm_count() / (a.B * a.H);
        splits = 1;
        while (splits < 8 && splits * 2 <= room && len / (splits * 2) >= 64) splits *= 2;
    }
    EET_CHECK(splits == 1 || splits == 2 || splits == 4 || splits == 8, "decode attention: splits must be 1,2,4,8");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(splits, a.B * a.H, 1);
    cfg.blockDim = dim3(kAttnThreads, 1, 1);
    cfg.dynamicSmemBytes = kAttnStages * kAttnStageBytes;
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
    dim3 grid((S + kPfQueries - 1) / kPfQueries, B * H);
    prefill_mha_kernel<<<grid, kPfQueries * 32, 0, stream>>>(q, kcache, vcache, ctx, S, H, T_max, pad_len, alibi,
                                                            alibi_stride);
    EET_LAUNCH_CHECK();
    return 0;
}

}  // namespace eet
