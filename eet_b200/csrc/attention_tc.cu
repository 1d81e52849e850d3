// Prefill self-attention on the 5th-generation tensor cores (tcgen05 / TMEM), causal with optional left padding
// (LLaMA) or ALiBi bias (Baichuan-13B).
//
// Reference: q_k_mul + qk_softmax + attn_v_mul + transpose of LlamaMmha::forward_full
// (csrc/op/llama_mmha.cpp:354-426; softmax_kernel_gpt2 csrc/core/gpt2_self_softmax.cu:8-57; ALiBi variant
// masked_softmax_kernel :161-240): two cuBLAS batched GEMMs around a row-serial softmax over a materialised
// [B,H,S,S] fp16 score buffer.  Here one CTA owns 128 consecutive queries of one (batch, head) and walks the keys
// in blocks of 64, never past the diagonal and never left of the padding; nothing of size S x S exists.
//
// B200 design (two CTAs per SM, 256 tensor-memory columns and 97 KiB of shared memory each: what one CTA cannot
// overlap by itself the other fills):
//   warp 0 (one lane)  TMA producer: the Q tile once, then K and V tiles of 64 keys into two-stage rings (a K
//                      stage is free again when its Q.K^T has completed, a V stage when its P.V has); 3-D tensor
//                      maps with the 128-byte swizzle, rows past the prompt read as zeros.  It sets the barriers
//                      up itself and requests Q and the first two blocks before the block-wide barrier and the
//                      tensor-memory allocation.
//   warp 1 (one lane)  MMA issuer: S = Q.K^T (M128 x N64 x K16, eight per block, both operands K-major from
//                      shared memory) into one of two score buffers in tensor memory - the scores of block j+1
//                      are computed while the softmax of block j runs; O += P.V (four per block) with P read FROM
//                      TENSOR MEMORY as the A operand and V straight from its [key][dim] tile as an MN-major B
//                      operand - V is never transposed and P never touches shared memory.
//   warps 2-5          softmax, one thread per query row (= TMEM lane): tcgen05.ld of the row's 64 scores,
//                      scale / fp16 rounding / bias / masks, running max and sum, probabilities back INTO THE
//                      SCORE COLUMNS as fp16 pairs (tcgen05.st: a row only ever touches its own lane, and the
//                      tensor core overwrites a score buffer only after the P.V that read it, in issue order);
//                      the O accumulator is rescaled only when some row of the warp saw a new maximum.  At the
//                      end they read O, normalise and store the context.
// Every wait is bounded (device status 2) and the CTA frees its tensor memory on every path.
//
// Numerics kept from the reference and from the mma.sync kernel this one replaces for long prompts: scores scaled
// by the fp16-rounded 1/sqrt(D) and rounded to fp16 where the reference stores them in fp16, the ALiBi bias added
// in fp32 after that rounding, probabilities enter P.V as fp16, denominator + 1e-6, rows above the left padding
// are zero.
#include <cuda.h>

#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

constexpr int kPtQ = 128;                      // queries per CTA
constexpr int kPtK = 64;                       // keys per block
constexpr int kPtThreads = 192;
constexpr int kPtQHalf = 128 * 128;            // bytes of the [128 queries][64 halves] swizzled half of the Q tile
constexpr int kPtQTile = 2 * kPtQHalf;         // dims 0-63, then dims 64-127
constexpr int kPtKvHalf = kPtK * 128;          // the same for a [64 keys][64 halves] half of a K or V tile
constexpr int kPtKvTile = 2 * kPtKvHalf;
constexpr int kPtStages = 2;
constexpr uint32_t kPtTmemCols = 256;
constexpr uint32_t kPtColS = 0;                // two score buffers of 64 fp32 columns; a block's probabilities
                                               // (32 columns: 64 fp16 as pairs) go over the first half of its scores
constexpr uint32_t kPtColO = 128;              // the context accumulator, 128 fp32 columns
constexpr int kPtSmem = kPtQTile + 2 * kPtStages * kPtKvTile + 1024;

struct PtSmem {
    uint64_t q_full;
    uint64_t k_full[kPtStages], k_empty[kPtStages];   // K tile landed / its Q.K^T has completed
    uint64_t v_full[kPtStages], v_empty[kPtStages];   // V tile landed / its P.V has completed
    uint64_t s_full[2];         // Q.K^T of a block has completed
    uint64_t p_ready[2];        // probabilities written, O rescaled (four softmax warps): P.V may be issued
    uint64_t pv_done[2];        // a block's P.V has completed (blocks alternate between the two: a softmax warp can
                                // be a whole block ahead of the slowest one, and one barrier's parity could then
                                // no longer tell "the previous P.V" from "the one before it")
    uint32_t tmem_base;
    volatile int abort;
};

__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ float ex2_approx(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// x rounded to the 11 significant bits of an fp16 value, in fp32 arithmetic (Veltkamp's splitting: three FP32
// operations instead of a conversion to half and back - the conversion unit is the one that also evaluates the
// exponentials, and it is what bounds the softmax).  Equal to fp16(x) for |x| inside fp16's normal range except
// on exact ties, where it may pick the other neighbour; scores outside that range (|x| < 6e-5) keep more bits
// than fp16 would, which no softmax can see.
__device__ __forceinline__ float round_to_half_precision(float x)
{
    // (intrinsics: the compiler must not contract these into fused multiply-adds, which would skip a rounding)
    const float big = __fmul_rn(x, 8193.0f);   // 2^13 + 1
    return __fsub_rn(big, __fsub_rn(big, x));
}

// B operand held [k][n] with n contiguous (MN-major), 128-byte swizzle: 64 n-values per 128-byte row, 8 k-rows per
// 1024-byte group (stride byte offset), the next 64 n-values `lbo_bytes` further (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_mn_sw128(uint32_t smem_addr, uint32_t lbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)(lbo_bytes >> 4) << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

__global__ void __launch_bounds__(kPtThreads, 2)
prefill_mha_tc_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                      const __grid_constant__ CUtensorMap map_v, __half* __restrict__ ctx, int S, int H,
                      const int64_t* __restrict__ pad_len, const __half* __restrict__ alibi, int alibi_stride)
{
    constexpr int D = 128;
    extern __shared__ __align__(1024) uint8_t pt_dyn[];
    __shared__ PtSmem sm;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(pt_dyn) + 1023) & ~(uintptr_t)1023);
    uint8_t* q_tile = base;
    uint8_t* k_ring = q_tile + kPtQTile;
    uint8_t* v_ring = k_ring + kPtStages * kPtKvTile;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int bh = blockIdx.y;
    const int b = bh / H, h = bh % H;
    const int qb = (int)gridDim.x - 1 - (int)blockIdx.x;   // the long tiles (late queries) are scheduled first
    const int i0 = qb * kPtQ;
    const int pad = (pad_len != nullptr && alibi == nullptr) ? (int)pad_len[b] : 0;
    const int kb_first = pad / kPtK;                                        // key blocks left of the padding are skipped
    const int kb_last = min((i0 + kPtQ - 1) / kPtK, (S - 1) / kPtK);        // causal: nothing above the diagonal
    const int n_blocks = kb_last - kb_first + 1;                            // <= 0: the whole tile lies inside the padding

    auto load_kv = [&](uint8_t* tile, const CUtensorMap* map, int key0, uint64_t* bar) {
        mbar_arrive_expect_tx(bar, (uint32_t)kPtKvTile);
        tma_load_3d(tile, map, 0, key0, bh, bar);
        tma_load_3d(tile + kPtKvHalf, map, 64, key0, bh, bar);
    };
    if (threadIdx.x == 0) {
        mbar_init(&sm.q_full, 1);
        for (int st = 0; st < kPtStages; ++st) {
            mbar_init(&sm.k_full[st], 1);
            mbar_init(&sm.k_empty[st], 1);
            mbar_init(&sm.v_full[st], 1);
            mbar_init(&sm.v_empty[st], 1);
        }
        for (int st = 0; st < 2; ++st) {
            mbar_init(&sm.s_full[st], 1);
            mbar_init(&sm.p_ready[st], 4);
        }
        mbar_init(&sm.pv_done[0], 1);
        mbar_init(&sm.pv_done[1], 1);
        sm.abort = 0;
        mbar_fence_init();
        // nobody else touches the barriers before the block-wide barrier below: the first loads go out now
        if (n_blocks > 0) {
            mbar_arrive_expect_tx(&sm.q_full, (uint32_t)kPtQTile);
            tma_load_3d(q_tile, &map_q, 0, i0, bh, &sm.q_full);
            tma_load_3d(q_tile + kPtQHalf, &map_q, 64, i0, bh, &sm.q_full);
            for (int jl = 0; jl < kPtStages && jl < n_blocks; ++jl) {
                load_kv(k_ring + jl * kPtKvTile, &map_k, (kb_first + jl) * kPtK, &sm.k_full[jl]);
                load_kv(v_ring + jl * kPtKvTile, &map_v, (kb_first + jl) * kPtK, &sm.v_full[jl]);
            }
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kPtTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            for (int jl = kPtStages; jl < n_blocks; ++jl) {
                const int st = jl % kPtStages;
                const uint32_t ph = (uint32_t)((jl / kPtStages - 1) & 1);
                const int key0 = (kb_first + jl) * kPtK;
                if (!tc_wait(&sm.k_empty[st], ph, &sm.abort)) break;
                load_kv(k_ring + st * kPtKvTile, &map_k, key0, &sm.k_full[st]);
                if (!tc_wait(&sm.v_empty[st], ph, &sm.abort)) break;
                load_kv(v_ring + st * kPtKvTile, &map_v, key0, &sm.v_full[st]);
            }
        }
    }
    else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0 && n_blocks > 0) {
            constexpr uint32_t idesc_qk = umma_idesc_f16(128, kPtK);                  // both operands K-major
            constexpr uint32_t idesc_pv = umma_idesc_f16(128, D) | (1u << 16);        // B operand MN-major
            const uint64_t q_desc = umma_desc_sw128(smem_u32(q_tile));
            const uint64_t k_desc0 = umma_desc_sw128(smem_u32(k_ring));
            const uint64_t v_desc0 = umma_desc_mn_sw128(smem_u32(v_ring), (uint32_t)kPtKvHalf);
            // Q.K^T of block jl into score buffer jl & 1.  That buffer last held the probabilities of block jl - 2,
            // whose P.V was issued before this: the tensor core executes in issue order.
            auto issue_qk = [&](int jl) -> bool {
                const int st = jl % kPtStages;
                if (!tc_wait(&sm.k_full[st], (uint32_t)((jl / kPtStages) & 1), &sm.abort)) return false;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t kd = k_desc0 + (uint64_t)(st * (kPtKvTile >> 4));
#pragma unroll
                for (int kk = 0; kk < 8; ++kk) {
                    // 16 head dims per MMA: 32 bytes along the swizzled row; dims 64-127 sit in the second half tile
                    const uint64_t qoff = (uint64_t)((kk >> 2) * (kPtQHalf >> 4) + (kk & 3) * 2);
                    const uint64_t koff = (uint64_t)((kk >> 2) * (kPtKvHalf >> 4) + (kk & 3) * 2);
                    umma_f16(tmem + kPtColS + (uint32_t)((jl & 1) * kPtK), q_desc + qoff, kd + koff, idesc_qk, kk != 0);
                }
                umma_commit(&sm.s_full[jl & 1]);
                umma_commit(&sm.k_empty[st]);
                return true;
            };
            bool ok = tc_wait(&sm.q_full, 0, &sm.abort) && issue_qk(0);
            for (int jl = 0; jl < n_blocks && ok; ++jl) {
                if (jl + 1 < n_blocks) ok = issue_qk(jl + 1);   // runs while the softmax of block jl does
                if (!ok) break;
                const int st = jl % kPtStages;
                if (!tc_wait(&sm.p_ready[jl & 1], (uint32_t)((jl >> 1) & 1), &sm.abort) ||
                    !tc_wait(&sm.v_full[st], (uint32_t)((jl / kPtStages) & 1), &sm.abort)) {
                    break;
                }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t vd = v_desc0 + (uint64_t)(st * (kPtKvTile >> 4));
#pragma unroll
                for (int kk = 0; kk < kPtK / 16; ++kk) {
                    // 16 keys per MMA: 8 columns of P, two 8-row groups (2048 bytes) of the V tile
                    umma_f16_ts(tmem + kPtColO, tmem + kPtColS + (uint32_t)((jl & 1) * kPtK + kk * 8),
                                vd + (uint64_t)(kk * (2048 >> 4)), idesc_pv, jl != 0 || kk != 0);
                }
                umma_commit(&sm.pv_done[jl & 1]);
                umma_commit(&sm.v_empty[st]);
            }
        }
    }
    else {
        // ------------------------------------------------------------------ softmax warps, then the epilogue
        const int lane_base = (warp & 3) * 32;               // the TMEM lanes this warp may access
        const int r = lane_base + lane;                      // query row inside the tile
        const int i = i0 + r;
        const uint32_t t_lane = (uint32_t)lane_base << 16;
        const float scalar = __half2float(__float2half(sqrtf(1.0f / D)));
        float m_run = -1e20f, l_run = 0.f;
        bool ok = n_blocks > 0;
        for (int jl = 0; jl < n_blocks && ok; ++jl) {
            const int key0 = (kb_first + jl) * kPtK;
            const uint32_t t_s = tmem + t_lane + kPtColS + (uint32_t)((jl & 1) * kPtK);   // this block's score buffer
            int got = 1;
            if (lane == 0) got = tc_wait(&sm.s_full[jl & 1], (uint32_t)((jl >> 1) & 1), &sm.abort) ? 1 : 0;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) {
                ok = false;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float sc[kPtK];
#pragma unroll
            for (int c0 = 0; c0 < kPtK; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(t_s + (uint32_t)c0, v);
#pragma unroll
                for (int c = 0; c < 32; ++c) sc[c0 + c] = __uint_as_float(v[c]);
            }

            float mx = -INFINITY;
            const __half* arow = (alibi != nullptr && i < S) ? alibi + ((size_t)h * alibi_stride + i) * alibi_stride : nullptr;
            // a block left of the diagonal, right of the padding and inside the prompt needs no per-element mask
            const bool whole = (key0 + kPtK - 1 <= i) && (key0 >= pad) && (key0 + kPtK <= S) && (arow == nullptr);
            if (whole) {
#pragma unroll
                for (int c = 0; c < kPtK; ++c) {
                    sc[c] = round_to_half_precision(sc[c] * scalar);
                    mx = fmaxf(mx, sc[c]);
                }
            }
            else {
#pragma unroll
                for (int c = 0; c < kPtK; ++c) {
                    const int j = key0 + c;
                    float v = round_to_half_precision(sc[c] * scalar);
                    if (arow != nullptr && j <= i) v += __half2float(arow[j]);
                    v = (j <= i && j >= pad && j < S) ? v : -INFINITY;
                    sc[c] = v;
                    mx = fmaxf(mx, v);
                }
            }
            constexpr float kLog2e = 1.4426950408889634f;
            const float m_new = fmaxf(m_run, mx);
            const float corr = ex2_approx((m_run - m_new) * kLog2e);
            m_run = m_new;
            const float m_l2 = -m_new * kLog2e;
            float psum = 0.f;
            uint32_t pk[kPtK / 2];
#pragma unroll
            for (int c = 0; c < kPtK; c += 2) {
                // exp(s - m) as one FMA and one ex2 (-inf stays -inf and gives 0)
                const float p0 = ex2_approx(fmaf(sc[c], kLog2e, m_l2)), p1 = ex2_approx(fmaf(sc[c + 1], kLog2e, m_l2));
                psum += p0 + p1;
                const __half2 hp = __floats2half2_rn(p0, p1);
                pk[c >> 1] = *reinterpret_cast<const uint32_t*>(&hp);
            }
            l_run = l_run * corr + psum;
            // probabilities as the A operand of P.V: lane = query, 16-bit pairs along the columns, written over the
            // first half of this row's scores (which are in registers by now)
            {
                uint32_t v[32];
#pragma unroll
                for (int c0 = 0; c0 < kPtK / 2; c0 += 32) {
#pragma unroll
                    for (int c = 0; c < 32; ++c) v[c] = pk[c0 + c];
                    tmem_st32(t_s + (uint32_t)c0, v);
                }
            }
            // O accumulates under the old maximum: rescale it if any row of this warp moved, after the previous
            // block's P.V has completed
            if (jl > 0) {
                const unsigned moved = __ballot_sync(0xffffffffu, corr != 1.0f);
                if (moved != 0u) {
                    int done = 1;
                    if (lane == 0) done = tc_wait(&sm.pv_done[(jl - 1) & 1], (uint32_t)(((jl - 1) >> 1) & 1), &sm.abort) ? 1 : 0;
                    done = __shfl_sync(0xffffffffu, done, 0);
                    if (!done) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll 1
                    for (int c0 = 0; c0 < D; c0 += 32) {
                        uint32_t v[32];
                        tmem_ld32(tmem + t_lane + kPtColO + (uint32_t)c0, v);
#pragma unroll
                        for (int c = 0; c < 32; ++c) v[c] = __float_as_uint(__uint_as_float(v[c]) * corr);
                        tmem_st32(tmem + t_lane + kPtColO + (uint32_t)c0, v);
                    }
                }
            }
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.p_ready[jl & 1]);
        }

        // ---- normalise and store: context layout [B][S][H*D] (the transpose of llama_mmha.cpp:418-426) ----
        if (n_blocks > 0 && ok) {
            int done = 1;
            if (lane == 0) {
                done = tc_wait(&sm.pv_done[(n_blocks - 1) & 1], (uint32_t)(((n_blocks - 1) >> 1) & 1), &sm.abort) ? 1 : 0;
            }
            done = __shfl_sync(0xffffffffu, done, 0);
            ok = done != 0;
        }
        if (i < S) {
            __half* dst = ctx + (((size_t)b * S + i) * H + h) * D;
            if (n_blocks <= 0 || !ok) {
                // the whole tile lies inside the left padding (or a wait ran out): rows of zeros
                const uint4 z = make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
                for (int c = 0; c < D / 8; ++c) reinterpret_cast<uint4*>(dst)[c] = z;
            }
        }
        if (n_blocks > 0 && ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // rows above the left padding are zeroed by the reference (gpt2_self_softmax.cu:24-30)
            const float inv = (i < pad) ? 0.f : 1.0f / (l_run + 1e-6f);
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + t_lane + kPtColO + (uint32_t)c0, v);   // (warp-collective: rows past the prompt take part)
                if (i < S) {
                    __half* dst = ctx + (((size_t)b * S + i) * H + h) * D + c0;
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint4 o;
                        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            oh[e] = __floats2half2_rn(__uint_as_float(v[c + 2 * e]) * inv, __uint_as_float(v[c + 2 * e + 1]) * inv);
                        }
                        *reinterpret_cast<uint4*>(dst + c) = o;
                    }
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kPtTmemCols) : "memory");
    }
}

// [rows_per_bh rows of 128 halves] x n_bh, of which the first `rows` of every (batch, head) are valid: reads past
// them return zeros, so a key block that reaches beyond the prompt never feeds stale cache rows (possibly NaN)
// into P.V.
int encode_rows_map(CUtensorMap* map, const __half* basep, int rows, size_t rows_per_bh, int n_bh, int box_rows)
{
    EncodeTiledFn encode = encode_tiled_fn();
    EET_CHECK(encode != nullptr, "prefill attention: cuTensorMapEncodeTiled is not available from the driver");
    const cuuint64_t dims[3] = {128, (cuuint64_t)rows, (cuuint64_t)n_bh};
    const cuuint64_t strides[2] = {256, (cuuint64_t)rows_per_bh * 256};
    const cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult rc = encode(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<__half*>(basep), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    EET_CHECK(rc == CUDA_SUCCESS, "prefill attention: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    return 0;
}

}  // namespace

// Prompts of at least this many tokens go to the tensor-core kernel (its tiles are 128 queries x 64 keys).
constexpr int kPrefillTcMinS = 96;

bool prefill_mha_tc_supported(int S, int D)
{
    return D == 128 && S >= kPrefillTcMinS;
}

int launch_prefill_mha_tc(const __half* q, const __half* kcache, const __half* vcache, __half* ctx, int B, int S, int H,
                          int T_max, const int64_t* pad_len, const __half* alibi, int alibi_stride, cudaStream_t stream)
{
    EET_CHECK((long long)B * H <= 65535, "prefill attention: batch x heads = %lld exceeds the grid limit", (long long)B * H);
    CUtensorMap map_q, map_k, map_v;
    if (int rc = encode_rows_map(&map_q, q, S, (size_t)S, B * H, kPtQ)) return rc;
    if (int rc = encode_rows_map(&map_k, kcache, S, (size_t)T_max, B * H, kPtK)) return rc;
    if (int rc = encode_rows_map(&map_v, vcache, S, (size_t)T_max, B * H, kPtK)) return rc;
    static bool attr_set[64] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    dev &= 63;
    if (!attr_set[dev]) {
        EET_CUDA(cudaFuncSetAttribute(prefill_mha_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPtSmem));
        attr_set[dev] = true;
    }
    dim3 grid((S + kPtQ - 1) / kPtQ, B * H);
    prefill_mha_tc_kernel<<<grid, kPtThreads, kPtSmem, stream>>>(map_q, map_k, map_v, ctx, S, H, pad_len, alibi, alibi_stride);
    EET_LAUNCH_CHECK();
    return 0;
}

}  // namespace eet
