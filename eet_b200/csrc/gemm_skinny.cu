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
//  * A producer warp feeds a ring of three 32 KiB shared-memory stages with 1-D bulk copies (TMA engine,
//    cp.async.bulk + mbarrier complete_tx, L2 evict-first).  Two CTAs per SM keep six stages in flight.
//  * Eight consumer warps each take one 64x64 tile of a stage: 16-byte shared loads deliver exactly the
//    A fragments of mma.m16n8k16 (16 channels x 64 reduction indices per pair of loads), bytes become
//    fp16 in registers (prmt + sub.f16x2) and feed the tensor cores with up to 8 tokens as the B operand,
//    which comes straight from global memory (L1/L2 resident, prefetched one tile ahead); the reduction
//    index is permuted identically on both operands, so no shuffles or transposes are needed.
//  * When a CTA's run ends inside a tile row, partial sums go to an fp32 scratch with red.global.add and
//    a per-tile-row arrival counter; the CTA that completes the count applies the scale (and residual),
//    writes fp16, and restores the scratch to zero.  Tile rows covered by one CTA skip the scratch.
//  * Programmatic dependent launch: the kernel may start while its predecessor in the stream is still
//    draining.  Weights do not depend on earlier kernels, so the producer streams them at once; only the
//    consumers wait (griddepcontrol.wait) before they touch activations, scratch or the output.  Back to
//    back GEMMs of a decode step therefore keep HBM busy across kernel boundaries.
//
// Numerics: products of fp16 activations with exact integer weights, fp32 accumulation, one multiply by
// the fp16 scale, one rounding to fp16 (the reference rounds every q*scale to fp16 first and rounds the
// fp32 accumulator once: mma_tensorop_dequantizer.h:259-274, epilogue_helpers.h:73-80).
#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

constexpr int kConsumerWarps = 8;
constexpr int kConsumerThreads = kConsumerWarps * 32;
constexpr int kSkinnyThreads = kConsumerThreads + 32;
constexpr int kStageTiles = 8;  // W8T64 tiles per stage
constexpr int kStageBytes = kStageTiles * kTileBytes;
constexpr int kStages = 3;
constexpr int kTilePitch = 72;  // padded row of the shared accumulation tile
constexpr int kSkinnyCtasPerSm = 2;

struct SkinnySmem {
    uint64_t full[kStages];
    uint64_t empty[kStages];
    float tile[16][kTilePitch];  // cross-warp accumulation of one tile row's [tokens][64 channels]
    int flag;
    volatile int abort;
};

__device__ __forceinline__ void consumer_bar()
{
    asm volatile("bar.sync 1, %0;" ::"n"(kConsumerThreads) : "memory");
}

// Activation fragment of one 64-wide reduction tile for this lane: token `row`, 16 consecutive reduction
// indices starting at 16 * tq (two 16-byte loads; L1/L2 hits after the first touch).
__device__ __forceinline__ void load_x(uint32_t (&xw)[8], const __half* A, int K, int row, int rows, int m0, int kb,
                                       int tq)
{
    uint4 x0 = make_uint4(0, 0, 0, 0), x1 = x0;
    if (row < rows) {
        const uint4* p = reinterpret_cast<const uint4*>(A + (size_t)(m0 + row) * K + (size_t)kb * kTile + tq * 16);
        x0 = __ldg(p);
        x1 = __ldg(p + 1);
    }
    xw[0] = x0.x; xw[1] = x0.y; xw[2] = x0.z; xw[3] = x0.w;
    xw[4] = x1.x; xw[5] = x1.y; xw[6] = x1.z; xw[7] = x1.w;
}

// NB = token groups of 8 handled per pass (1: M <= 8, 2: M <= 16).
template<int NB>
__global__ void __launch_bounds__(kSkinnyThreads, kSkinnyCtasPerSm)
gemm_skinny_kernel(GemmArgs a)
{
    extern __shared__ __align__(128) uint8_t dyn_smem[];
    __shared__ SkinnySmem sm;

    // let the next kernel in the stream start its own weight streaming as soon as SM resources allow
    pdl_launch_dependents();

    const int KT = a.K / kTile, NT = a.N / kTile;
    const long long G = (long long)NT * KT;
    const int g0 = (int)(G * blockIdx.x / gridDim.x);
    const int g1 = (int)(G * (blockIdx.x + 1) / gridDim.x);
    const int m0 = blockIdx.y * 16;
    const int rows = min(8 * NB, a.M - m0);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.empty[s], kConsumerWarps);
        }
        sm.abort = 0;
        mbar_fence_init();
    }
    for (int e = threadIdx.x; e < 16 * kTilePitch; e += blockDim.x) (&sm.tile[0][0])[e] = 0.f;
    __syncthreads();

    if (warp == kConsumerWarps) {
        // ------------------------------------------------------------------ producer warp (one lane)
        // Weights are constant inputs: no need to wait for the preceding kernel.
        if (lane == 0) {
            int it = 0;
            for (int g = g0; g < g1; ++it) {
                const int nt = g / KT, kb = g - nt * KT;
                const int nb_tiles = min(min(kStageTiles, KT - kb), g1 - g);
                const int s = it % kStages;
                if (it >= kStages && !sm.abort) {
                    if (!mbar_wait_bounded(&sm.empty[s], ((it / kStages) - 1) & 1)) {
                        sm.abort = 1;
                        g_device_status = 1;
                    }
                }
                mbar_arrive_expect_tx(&sm.full[s], (uint32_t)(nb_tiles * kTileBytes));
                bulk_g2s_stream(dyn_smem + (size_t)s * kStageBytes, a.B + (size_t)g * kTileBytes,
                                (uint32_t)(nb_tiles * kTileBytes), &sm.full[s]);
                g += nb_tiles;
            }
        }
        return;
    }

    // ---------------------------------------------------------------------- consumer warps
    // mma.m16n8k16 with the WEIGHTS as the 16-row A operand (16 channels x 16 reduction indices) and the
    // activations as the 8-column B operand (8 tokens): a batch of up to 8 tokens costs one MMA per 256
    // weights.  The legacy mma.sync path of this GPU is slow enough (about 32 cycles per instruction and
    // SM sub-partition) that the instruction count decides whether the kernel stays HBM-bound.
    const int gq = lane >> 2, tq = lane & 3;  // mma fragment coordinates
    float acc[4][NB][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[j][nb][c] = 0.f;

    // activations, scratch and output belong to the dependency chain: wait for the preceding kernel
    pdl_wait();

    // schedule walk shared with the producer: stage `it` holds tiles [g, g + nb_tiles) of one tile row
    int it = 0;
    int tile_first_kb = -1;  // first k-tile of the current tile row handled by this CTA
    uint32_t xw[NB][8], xn[NB][8];
    {
        // prefetch the activations of this warp's tile in the first stage
        const int nt = g0 / KT, kb = g0 - nt * KT;
        const int nb_tiles = (g0 < g1) ? min(min(kStageTiles, KT - kb), g1 - g0) : 0;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            load_x(xn[nb], a.A, a.K, (warp < nb_tiles) ? gq + 8 * nb : rows, rows, m0, kb + warp, tq);
        }
    }
    for (int g = g0; g < g1; ++it) {
        const int nt = g / KT, kb = g - nt * KT;
        const int nb_tiles = min(min(kStageTiles, KT - kb), g1 - g);
        const int s = it % kStages;
        if (tile_first_kb < 0) tile_first_kb = kb;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb)
#pragma unroll
            for (int w = 0; w < 8; ++w) xw[nb][w] = xn[nb][w];
        {
            // prefetch the next stage's activations before blocking on this stage's weights
            const int gn = g + nb_tiles;
            const int ntn = gn / KT, kbn = gn - ntn * KT;
            const int nbn = (gn < g1) ? min(min(kStageTiles, KT - kbn), g1 - gn) : 0;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                load_x(xn[nb], a.A, a.K, (warp < nbn) ? gq + 8 * nb : rows, rows, m0, kbn + warp, tq);
            }
        }
        if (!sm.abort) {
            if (!mbar_wait_bounded(&sm.full[s], (it / kStages) & 1)) {
                sm.abort = 1;
                g_device_status = 1;
            }
        }
        if (warp < nb_tiles) {
            const uint8_t* ws = dyn_smem + (size_t)s * kStageBytes + warp * kTileBytes + lane * 16;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                // channels 16j + gq and 16j + gq + 8, reduction indices 16*tq .. 16*tq + 15 of this tile
                const uint4 wa = *reinterpret_cast<const uint4*>(ws + j * 1024);
                const uint4 wb = *reinterpret_cast<const uint4*>(ws + j * 1024 + 512);
                const uint32_t wa4[4] = {wa.x, wa.y, wa.z, wa.w};
                const uint32_t wb4[4] = {wb.x, wb.y, wb.z, wb.w};
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    uint32_t a0, a1, a2, a3;
                    cvt_u8x4_to_f16x4(wa4[i], a0, a2);
                    cvt_u8x4_to_f16x4(wb4[i], a1, a3);
#pragma unroll
                    for (int nb = 0; nb < NB; ++nb) {
                        mma_m16n8k16(acc[j][nb], a0, a1, a2, a3, xw[nb][2 * i], xw[nb][2 * i + 1]);
                    }
                }
            }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&sm.empty[s]);
        g += nb_tiles;

        const bool row_end = (kb + nb_tiles == KT);
        if (row_end || g == g1) {
            // ---- flush the tile row: reduce the 8 warps' fragments through shared memory ----
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
                for (int nb = 0; nb < NB; ++nb) {
                    const int m = nb * 8 + tq * 2, n = j * 16 + gq;
                    atomicAdd(&sm.tile[m][n], acc[j][nb][0]);
                    atomicAdd(&sm.tile[m + 1][n], acc[j][nb][1]);
                    atomicAdd(&sm.tile[m][n + 8], acc[j][nb][2]);
                    atomicAdd(&sm.tile[m + 1][n + 8], acc[j][nb][3]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) acc[j][nb][c] = 0.f;
                }
            }
            consumer_bar();
            const bool whole_row = (tile_first_kb == 0) && row_end;
            const int n_base = nt * kTile;
            float* ws_tile = a.ws + (size_t)m0 * a.N + n_base;
            int* counter = reinterpret_cast<int*>(a.ws + (size_t)gridDim.y * 16 * a.N) + blockIdx.y * NT + nt;
            bool finalize = whole_row;
            if (!whole_row) {
                for (int e = threadIdx.x; e < rows * 64; e += kConsumerThreads) {
                    const int m = e >> 6, n = e & 63;
                    atomicAdd(ws_tile + (size_t)m * a.N + n, sm.tile[m][n]);
                }
                __threadfence();
                consumer_bar();
                if (threadIdx.x == 0) {
                    const int contributed = kb + nb_tiles - tile_first_kb;
                    const int old = atomicAdd(counter, contributed);
                    sm.flag = (old + contributed == KT);
                }
                consumer_bar();
                finalize = sm.flag != 0;
                if (finalize) __threadfence();
            }
            if (finalize) {
                for (int e = threadIdx.x; e < rows * 64; e += kConsumerThreads) {
                    const int m = e >> 6, n = e & 63;
                    float v;
                    if (whole_row) {
                        v = sm.tile[m][n];
                    }
                    else {
                        v = __ldcg(ws_tile + (size_t)m * a.N + n);
                        __stcg(ws_tile + (size_t)m * a.N + n, 0.f);
                    }
                    const size_t o = (size_t)(m0 + m) * a.N + n_base + n;
                    __half r = __float2half(v * __half2float(a.scale[n_base + n]));
                    if (a.epilogue == 1) r = __hadd(r, a.residual[o]);
                    a.C[o] = r;
                }
                if (!whole_row && threadIdx.x == 0) *counter = 0;
            }
            // each thread clears exactly the elements it read above (same e -> (m, n) mapping), so no
            // barrier is needed between the reads and the clearing
            for (int e = threadIdx.x; e < 16 * 64; e += kConsumerThreads) sm.tile[e >> 6][e & 63] = 0.f;
            consumer_bar();
            tile_first_kb = -1;
        }
    }
}

}  // namespace

size_t skinny_workspace_bytes(int M, int N, int dual)
{
    (void)dual;
    const size_t chunks = (size_t)((M + 15) / 16 > 0 ? (M + 15) / 16 : 1);
    const size_t chunks_per_launch = chunks < 8 ? chunks : 8;
    return chunks_per_launch * 16 * (size_t)N * sizeof(float) + chunks_per_launch * (size_t)(N / kTile) * sizeof(int);
}

int launch_gemm_skinny(const GemmArgs& a, cudaStream_t stream)
{
    EET_CHECK(a.epilogue == 0 || a.epilogue == 1, "skinny GEMM: epilogue %d is not supported", a.epilogue);
    if (a.M == 0) return 0;
    static bool attr_set[64][2] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    dev &= 63;
    const long long G = (long long)(a.N / kTile) * (a.K / kTile);
    int grid_x = kSkinnyCtasPerSm * sm_count();
    if (grid_x > G) grid_x = (int)G;
    const int total_chunks = (a.M + 15) / 16;
    const size_t smem = (size_t)kStages * kStageBytes;
    for (int c0 = 0; c0 < total_chunks; c0 += 8) {
        const int chunks = (total_chunks - c0 < 8) ? (total_chunks - c0) : 8;
        GemmArgs b = a;
        b.A = a.A + (size_t)c0 * 16 * a.K;
        b.C = a.C + (size_t)c0 * 16 * a.N;
        if (a.residual) b.residual = a.residual + (size_t)c0 * 16 * a.N;
        b.M = a.M - c0 * 16;
        if (b.M > chunks * 16) b.M = chunks * 16;
        const bool one_group = (b.M <= 8);
        auto kern = one_group ? gemm_skinny_kernel<1> : gemm_skinny_kernel<2>;
        if (!attr_set[dev][one_group ? 0 : 1]) {
            EET_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set[dev][one_group ? 0 : 1] = true;
        }
        EET_CUDA(launch_pdl(kern, dim3(grid_x, chunks), dim3(kSkinnyThreads), smem, stream, b));
    }
    return 0;
}

}  // namespace eet
