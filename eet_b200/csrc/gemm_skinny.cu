// W8A16 skinny GEMM for the decode regime (M <= 16 per pass): C[M,N] = A[M,K] (fp16) x dequant(B),
// B in the W8T64 layout, fp16 per-channel scale applied once per output.
//
// Replaces the reference's fpA_intB GEMM (3rdparty/cutlass_kernels/fpA_intB_gemm/fpA_intB_gemm_template.h
// :48-177, kernel cutlass_extensions/.../gemm/kernel/fpA_intB_gemm.h:60-486) for small M, where that
// kernel pads M to a 32-row tile and launches only N/128 CTAs with no split-K (cutlass_heuristic.cc
// :80-84), far too few bytes in flight for HBM.
//
// B200 design.  The job is HBM-bound: N*K weight bytes are read once.
//  * Stream-K partition: the W8T64 tiles are numbered [N/64][K/64] in memory order; the grid is two
//    persistent CTAs per SM and CTA c owns an equal, contiguous run of tiles, i.e. one linear byte range
//    of the weight array, whatever N and K are.
//  * A producer warp feeds a ring of shared-memory stages with 1-D bulk copies (TMA engine,
//    cp.async.bulk + mbarrier complete_tx, L2 evict-first hint): 32 KiB of weights (eight tiles) per stage,
//    two stages per CTA, two CTAs per SM (measured best among 16-40 KiB stages x 2-5 stages and 2-3 CTAs
//    per SM).  The matching slice of the activations (a few KiB, L2 resident) is staged beside it by the
//    consumer warps with plain 16-byte loads, one stage ahead.
//  * Eight consumer warps share a stage by channel group and tile half: 16-byte shared loads deliver
//    exactly the A fragments of mma.m16n8k16 (16 channels x 64 reduction indices per pair of loads),
//    bytes become fp16 in registers (prmt + sub.f16x2) and feed the tensor cores with up to 8 tokens as
//    the B operand; the reduction index is permuted identically on both operands, so no shuffles or
//    transposes are needed, and a warp's accumulators stay in registers for a whole tile row.
//  * The kernel's result is the fp32 sum over k of x[m][k] * q[k][n], ADDED into a caller-provided fp32
//    buffer with red.global.add at the end of each CTA's share of a tile row (one to three CTAs
//    contribute to a row).  Scale, residual and the fp16 rounding are left to whoever reads the sums -
//    the generic finalize kernel below, or the next kernel of a decode step (RMSNorm, attention, SwiGLU),
//    which also puts the buffer back to zero.  Nothing in this kernel waits on another CTA.
//  * Programmatic dependent launch: the kernel may start while its predecessor in the stream is still
//    draining.  Weights do not depend on earlier kernels, so the producer streams them at once; only the
//    consumers wait (griddepcontrol.wait) before they touch activations, scratch or the output.  Back to
//    back GEMMs of a decode step therefore keep HBM busy across kernel boundaries.
//
//  * Two weight matrices with the same K and N (the gate and up projections of the FFN) can be walked by
//    one launch: the tile list is the concatenation of both and each has its own sum buffer.
//
// Numerics: products of fp16 activations with exact integer weights, fp32 accumulation; the finalize step
// multiplies once by the fp16 scale and rounds once to fp16 (the reference rounds every q*scale to fp16
// first and rounds the fp32 accumulator once: mma_tensorop_dequantizer.h:259-274,
// epilogue_helpers.h:73-80).
#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kSkinnyThreads = kConsumerThreads + 32;
constexpr int kStageTiles = 8;  // W8T64 tiles per stage: four for each half of the consumer warps
constexpr int kStageWBytes = kStageTiles * kTileBytes;
constexpr int kXRowBytes = kStageTiles * 128 + 16;  // one token's slice of a stage, padded: conflict-free loads
constexpr int kMaxStages = 2;
constexpr int kSkinnyCtasPerSm = 2;

__host__ __device__ constexpr int stage_bytes(int nb)
{
    return kStageWBytes + 8 * nb * kXRowBytes;
}
__host__ __device__ constexpr int stage_count(int nb)
{
    (void)nb;
    return 2;  // 2 x 40.1 KiB (8 tokens) or 2 x 48.3 KiB (16 tokens): two CTAs fit in one SM's shared memory
}

struct SkinnySmem {
    uint64_t full[kMaxStages];
    uint64_t empty[kMaxStages];
    float fold[4][2][32][4];  // fragments of warps 4-7 on their way to warps 0-3 at the end of a tile row
    volatile int abort;
};

__device__ __forceinline__ void consumer_bar()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// NB = token groups of 8 handled per pass (1: M <= 8, 2: M <= 16).
// The launch bound asks for three CTAs per SM although the grid is two per SM: that caps the kernel at 72
// registers (it would take 86), and a 72-register CTA of this kernel - started early by programmatic
// dependent launch - fits beside the CTAs of the attention kernel that runs before the output projection
// and fills its ring while they finish.  Measured on the decode step: +1.6 % (56 registers: -0.7 %).
template<int NB>
__global__ void __launch_bounds__(kSkinnyThreads, kSkinnyCtasPerSm + 1)
gemm_skinny_kernel(GemmArgs a)
{
    extern __shared__ __align__(128) uint8_t dyn_smem[];
    __shared__ SkinnySmem sm;

    // let the next kernel in the stream start its own weight streaming as soon as SM resources allow
    pdl_launch_dependents();

    const int KT = a.K / kTile, NT = a.N / kTile;
    const long long G1 = (long long)NT * KT;               // tiles of one matrix
    const long long G = a.B2 ? 2 * G1 : G1;
    const int g0 = (int)(G * blockIdx.x / gridDim.x);
    const int g1 = (int)(G * (blockIdx.x + 1) / gridDim.x);
    const int m0 = blockIdx.y * 16;
    const int rows = min(8 * NB, a.M - m0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    constexpr int kStages = stage_count(NB);
    constexpr int kStageBytes = stage_bytes(NB);

    // The producer lane sets the barriers up itself and requests the first stages BEFORE the block-wide
    // barrier: nobody else touches the ring until then, and on a 5-10 us kernel the few hundred nanoseconds
    // that the other warps need to arrive are worth having the first 64 KiB in flight.
    // Weights are constant inputs: no need to wait for the preceding kernel either.
    const bool is_producer = (warp == kConsumerWarps) && (lane == 0);
    int p_it = 0, p_g = g0;
    auto issue_stage = [&]() {
        const int nt = p_g / KT, kb = p_g - nt * KT;
        const int nb_tiles = min(min(kStageTiles, KT - kb), g1 - p_g);
        const int s = p_it % kStages;
        mbar_arrive_expect_tx(&sm.full[s], (uint32_t)(nb_tiles * kTileBytes));
        const uint8_t* src = (p_g < G1) ? a.B + (size_t)p_g * kTileBytes : a.B2 + (size_t)(p_g - G1) * kTileBytes;
        bulk_g2s_stream(dyn_smem + (size_t)s * kStageBytes, src, (uint32_t)(nb_tiles * kTileBytes), &sm.full[s]);
        p_g += nb_tiles;
        ++p_it;
    };
    if (is_producer) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kConsumerWarps);
        }
        sm.abort = 0;
        mbar_fence_init();
        while (p_it < kStages && p_g < g1) issue_stage();
    }
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer warp (one lane)
        if (lane == 0) {
            while (p_g < g1) {
                const int s = p_it % kStages;
                if (!sm.abort) {
                    if (!mbar_wait_bounded(&sm.empty[s], ((p_it / kStages) - 1) & 1)) {
                        sm.abort = 1;
                        g_device_status = 1;
                    }
                }
                issue_stage();
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    // mma.m16n8k16 with the WEIGHTS as the 16-row A operand (16 channels x 16 reduction indices) and the
    // activations as the 8-column B operand (8 tokens): a batch of up to 8 tokens costs one MMA per 256
    // weights.  The legacy mma.sync path of this GPU is slow enough (about 32 cycles per instruction and
    // SM sub-partition) that the instruction count decides whether the kernel stays HBM-bound.
    //
    // Warp w owns channel group cg = w % 4 (channels 16cg .. 16cg+15 of the tile row) and half kh = w / 4
    // of the tiles of each stage, so its accumulators never leave registers until the tile row ends; then
    // the two halves meet through 4 KiB of shared memory and warps 0-3 run the epilogue from registers.
    const int gq = lane >> 2, tq = lane & 3;  // mma fragment coordinates
    const int cg = warp & 3, kh = warp >> 2;
    float acc[NB][4];
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[nb][c] = 0.f;

    // activations, scratch and output belong to the dependency chain: wait for the preceding kernel
    pdl_wait();

    // The four warps of a half stage the activations of their four tiles themselves: 16-byte global loads
    // (L2 hits) one stage ahead into registers, then into the stage's padded slab.
    constexpr int kHalfTiles = kStageTiles / 2;
    constexpr int kXChunks = 8 * NB * kHalfTiles * 8;          // 16-byte chunks per half and stage
    constexpr int kXPerThread = (kXChunks + 127) / 128;
    const int hl = threadIdx.x & 127;
    uint4 xr[kXPerThread];
    auto fetch_x = [&](int kb_stage, int nb_tiles_stage) {
#pragma unroll
        for (int u = 0; u < kXPerThread; ++u) {
            const int c = hl + u * 128;
            const int row = c / (kHalfTiles * 8), col = c % (kHalfTiles * 8);
            const int tile = kh * kHalfTiles + (col >> 3);
            xr[u] = make_uint4(0, 0, 0, 0);
            if (c < kXChunks && row < rows && tile < nb_tiles_stage) {
                xr[u] = __ldg(reinterpret_cast<const uint4*>(a.A + (size_t)(m0 + row) * a.K +
                                                             (size_t)(kb_stage + kh * kHalfTiles) * kTile) + col);
            }
        }
    };

    // schedule walk shared with the producer: stage `it` holds tiles [g, g + nb_tiles) of one tile row
    int it = 0;
    if (g0 < g1) {
        const int nt = g0 / KT, kb = g0 - nt * KT;
        fetch_x(kb, min(min(kStageTiles, KT - kb), g1 - g0));
    }
    for (int g = g0; g < g1; ++it) {
        const int nt = g / KT, kb = g - nt * KT;
        const int nb_tiles = min(min(kStageTiles, KT - kb), g1 - g);
        const int s = it % kStages;
        {
            uint8_t* xdst = dyn_smem + (size_t)s * kStageBytes + kStageWBytes + kh * kHalfTiles * 128;
#pragma unroll
            for (int u = 0; u < kXPerThread; ++u) {
                const int c = hl + u * 128;
                if (c < kXChunks) {
                    const int row = c / (kHalfTiles * 8), col = c % (kHalfTiles * 8);
                    *reinterpret_cast<uint4*>(xdst + row * kXRowBytes + col * 16) = xr[u];
                }
            }
            // next stage's activations: in flight while this stage is computed
            const int gn = g + nb_tiles;
            if (gn < g1) {
                const int ntn = gn / KT, kbn = gn - ntn * KT;
                fetch_x(kbn, min(min(kStageTiles, KT - kbn), g1 - gn));
            }
            // slab complete for the four warps of this half (a warp can be at most one stage ahead of the
            // others, and the ring has at least two stages, so the slab being refilled is no longer read)
            if (kh == 0) {
                asm volatile("bar.sync 2, 128;" ::: "memory");
            }
            else {
                asm volatile("bar.sync 3, 128;" ::: "memory");
            }
        }
        if (!sm.abort) {
            if (!mbar_wait_bounded(&sm.full[s], (it / kStages) & 1)) {
                sm.abort = 1;
                g_device_status = 1;
            }
        }
        // channels 16cg + gq and 16cg + gq + 8, reduction indices 16*tq .. 16*tq + 15 of each tile
        const uint8_t* stage = dyn_smem + (size_t)s * kStageBytes;
        const uint8_t* ws = stage + cg * 1024 + lane * 16;
        const uint8_t* xs = stage + kStageWBytes + tq * 32;
#pragma unroll
        for (int t = 0; t < kStageTiles / 2; ++t) {
            const int tile = kh * (kStageTiles / 2) + t;
            if (tile < nb_tiles) {
                // activations (B operand): token gq (+8 per group), the same 16 reduction indices
                uint32_t xw[NB][8];
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    // (rows beyond the batch were stored as zeros)
                    const uint8_t* xp = xs + (gq + 8 * nb) * kXRowBytes + tile * 128;
                    const uint4 x0 = *reinterpret_cast<const uint4*>(xp);
                    const uint4 x1 = *reinterpret_cast<const uint4*>(xp + 16);
                    xw[nb][0] = x0.x; xw[nb][1] = x0.y; xw[nb][2] = x0.z; xw[nb][3] = x0.w;
                    xw[nb][4] = x1.x; xw[nb][5] = x1.y; xw[nb][6] = x1.z; xw[nb][7] = x1.w;
                }
                const uint4 wa = *reinterpret_cast<const uint4*>(ws + tile * kTileBytes);
                const uint4 wb = *reinterpret_cast<const uint4*>(ws + tile * kTileBytes + 512);
                const uint32_t wa4[4] = {wa.x, wa.y, wa.z, wa.w};
                const uint32_t wb4[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t a0, a1, a2, a3;
                    cvt_u8x4_to_f16x4(wa4[i], a0, a2);
                    cvt_u8x4_to_f16x4(wb4[i], a1, a3);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        mma_m16n8k16(acc[nb], a0, a1, a2, a3, xw[nb][2 * i], xw[nb][2 * i + 1]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[s]);
        g += nb_tiles;

        const bool row_end = (kb + nb_tiles == KT);
        if (row_end || g == g1) {
            // ---- end of this CTA's share of the tile row: fold the two k-halves, then the epilogue ----
            if (kh == 1) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    *reinterpret_cast<float4*>(&sm.fold[cg][nb][lane][0]) =
                        make_float4(acc[nb][0], acc[nb][1], acc[nb][2], acc[nb][3]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[nb][c] = 0.f;
                }
            }
            consumer_bar();
            if (kh == 0) {
                // fragment element c of group nb: token 8nb + 2tq + (c & 1), channel n0 + 8 * (c >> 1)
                float* sums = (nt < NT) ? a.ws : a.ws2;
                const int n0 = (nt < NT ? nt : nt - NT) * kTile + cg * 16 + gq;
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const float4 o = *reinterpret_cast<const float4*>(&sm.fold[cg][nb][lane][0]);
                    const float v[4] = {acc[nb][0] + o.x, acc[nb][1] + o.y, acc[nb][2] + o.z, acc[nb][3] + o.w};
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int m = 8 * nb + 2 * tq + (c & 1);
                        if (m < rows) atomicAdd(sums + (size_t)(m0 + m) * a.N + n0 + 8 * (c >> 1), v[c]);
                        acc[nb][c] = 0.f;
                    }
                }
            }
            consumer_bar();   // the fold buffer may be rewritten by the next tile row
        }
    }
}

}  // namespace

size_t skinny_sum_bytes(int M, int N)
{
    return (size_t)(M > 0 ? M : 0) * (size_t)N * sizeof(float);
}

// Adds A[M,K] x q(B) (and, with B2, A x q(B2)) into the fp32 buffers sums (sums2), rows [0, M).
int launch_gemm_skinny(const GemmArgs& a, cudaStream_t stream)
{
    if (a.M == 0) return 0;
    static bool attr_set[64][2] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    dev &= 63;
    const long long G = (long long)(a.N / kTile) * (a.K / kTile) * (a.B2 ? 2 : 1);
    int grid_x = kSkinnyCtasPerSm * sm_count();
    if (grid_x > G) grid_x = (int)G;
    const int total_chunks = (a.M + 15) / 16;
    for (int c0 = 0; c0 < total_chunks; c0 += 8) {
        const int chunks = (total_chunks - c0 < 8) ? (total_chunks - c0) : 8;
        GemmArgs b = a;
        b.A = a.A + (size_t)c0 * 16 * a.K;
        b.ws = a.ws + (size_t)c0 * 16 * a.N;
        if (a.ws2) b.ws2 = a.ws2 + (size_t)c0 * 16 * a.N;
        b.M = a.M - c0 * 16;
        if (b.M > chunks * 16) b.M = chunks * 16;
        const bool one_group = (b.M <= 8);
        auto kern = one_group ? gemm_skinny_kernel<1> : gemm_skinny_kernel<2>;
        const int nbg = one_group ? 1 : 2;
        const size_t smem = (size_t)stage_count(nbg) * stage_bytes(nbg);
        if (!attr_set[dev][one_group ? 0 : 1]) {
            EET_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set[dev][one_group ? 0 : 1] = true;
        }
        EET_CUDA(launch_pdl(kern, dim3(grid_x, chunks), dim3(kSkinnyThreads), smem, stream, b));
    }
    return 0;
}

}  // namespace eet
