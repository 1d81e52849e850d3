// W8A16 tensor-core GEMM for the prefill regime (M > 512; smaller M go to the stream-K kernel):
// C[M,N] = A[M,K] (fp16) x dequant(B), B in the W8T64 layout, per-channel fp16 scale (and optional fp16 residual) in the epilogue.
//
// Replaces the reference's fpA_intB GEMM (kernel cutlass_extensions/.../gemm/kernel/fpA_intB_gemm.h:60-486,
// mainloop .../threadblock/dq_mma_multistage.h:490-583: mma.sync m16n8k16 with int8 -> fp16 conversion in
// registers after ldmatrix), which has no path for sm_90 or later.
//
// B200 design (tcgen05 / TMEM, one CTA per 128-channel x BN-token output tile):
//  * "swap AB": the weights are the 128-row M operand of tcgen05.mma, the tokens the N operand (BN up to
//    256), so any batch of tokens fills the tensor core and the per-channel scale is per TMEM lane.
//  * warp 0 (one lane) is the TMA producer: per 64-wide k-block it requests the two 4 KiB W8T64 tiles of
//    the 128 channels with 1-D bulk copies and the BN x 64 activation tile with one 2-D tensor-map copy
//    that lands in the 128-byte-swizzled K-major layout the MMA reads.
//  * warps 2-5 turn each int8 weight tile into fp16 (prmt + sub.f16x2, exact) and write it into shared
//    memory in the same swizzled K-major layout - the int8 bytes never go through the tensor core as int8
//    and the weights are never materialised as fp16 in global memory.
//  * warp 1 (one lane) issues four tcgen05.mma (M128 x BN x K16, fp16 in, fp32 accumulate in TMEM) per
//    k-block and commits them to the stage's "empty" mbarrier, which releases the stage to the producer.
//  * after the last k-block warps 2-5 read the accumulator with tcgen05.ld (lane = channel), multiply by
//    the channel's scale, round once to fp16, and pass 128 x 32 blocks through shared memory so that the
//    stores (and the residual loads) are 16-byte accesses of whole 256-byte row segments.
//  Three-stage ring of {8 KiB int8 weights, 16 KiB fp16 weights, BN x 128 B activations}.
//  Every wait is bounded; a wait that runs out sets the device status word, and the CTA still frees its
//  tensor memory before it returns.
//
// Numerics: exact integer weights as fp16, fp32 accumulation, one multiply by the fp16 scale, one rounding
// to fp16 - the same as the skinny kernel's finalize step.
#include <cuda.h>
#include <cooperative_groups.h>

#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

constexpr int kTcThreads = 192;     // warp 0 producer, warp 1 MMA issuer + TMEM owner, warps 2-5 transform/epilogue
constexpr int kTcStages = 3;
constexpr int kTcW8Bytes = 2 * kTileBytes;          // 128 channels x 64 k, int8
constexpr int kTcWhBytes = 128 * 128;               // 128 channels x 64 k, fp16, 128 B per row
constexpr uint32_t kTcSpin = 1u << 24;

__host__ __device__ constexpr int tc_stage_bytes(int bn)
{
    return kTcW8Bytes + kTcWhBytes + bn * 128;
}

struct TcSmem {
    uint64_t full[kTcStages];    // TMA bytes of a stage have landed (int8 weights + activations)
    uint64_t ready[kTcStages];   // fp16 weights of a stage are written (4 transform warps)
    uint64_t empty[kTcStages];   // the MMAs that read a stage have completed (tcgen05.commit)
    uint64_t accum;              // all MMAs of the tile have completed
    uint32_t tmem_base;
    volatile int abort;
};

// Bounded wait of the warp-specialised kernels.  The roles that issue work are SINGLE threads whose loop
// is a chain of dependent instructions (a few cycles each at best): the common case - the phase has
// already completed - must cost one try_wait and nothing else.
__device__ __noinline__ bool tc_wait_slow(uint64_t* bar, uint32_t parity, volatile int* abort)
{
    for (uint32_t i = 0; i < kTcSpin; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort) return false;
    }
    *abort = 1;
    g_device_status = 2;
    return false;
}

__device__ __forceinline__ bool tc_wait(uint64_t* bar, uint32_t parity, volatile int* abort)
{
    if (mbar_try_wait(bar, parity)) return true;
    return tc_wait_slow(bar, parity, abort);
}

// shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 128 bytes, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t umma_desc_sw128(uint32_t smem_addr)
{
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);        // start address, 16-byte units
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused with swizzle)
    d |= (uint64_t)(1024 >> 4) << 32;                   // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                             // descriptor version of this architecture
    d |= (uint64_t)2 << 61;                             // SWIZZLE_128B
    return d;
}

// instruction descriptor for kind::f16: fp16 A and B, fp32 accumulate, both operands K-major
__host__ __device__ constexpr uint32_t umma_idesc_f16(int m, int n)
{
    return (1u << 4) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(m >> 4) << 24);
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}

__device__ __forceinline__ void umma_commit(uint64_t* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, int x, int y, uint64_t* bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(
            smem_u32(smem_dst)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
        : "memory");
}

__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
          "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
          "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Epilogue of one block of 128 channels x 32 tokens.  After tcgen05.ld every epilogue thread holds the 32
// token sums of ONE channel, while the output is channel-contiguous; the block therefore goes through a
// [32 tokens][128 channels] fp16 staging tile in shared memory (the operand rings are idle by then) and
// leaves as 16-byte stores of whole 256-byte row segments, with the residual fetched the same way and all
// four residual loads of a thread in flight before the first add.  Two staging tiles alternate so one named
// barrier per block is enough.  Called by all 128 epilogue threads.
constexpr int kEpiStageHalves = 32 * 128;

template<int kBarId = 1>
__device__ __forceinline__ void epilogue_block(const uint32_t (&v)[32], float sc, __half* stage, int channel, int tw,
                                               __half* C, const __half* residual, int gate, int m_first, int M, int N,
                                               int n_first)
{
#pragma unroll
    for (int j = 0; j < 32; ++j) stage[j * 128 + channel] = __float2half(__uint_as_float(v[j]) * sc);
    asm volatile("bar.sync %0, 128;" ::"n"(kBarId) : "memory");
    uint4 res[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = tw + i * 128, row = idx >> 4, ch8 = idx & 15;
        res[i] = make_uint4(0u, 0u, 0u, 0u);
        if (residual != nullptr && m_first + row < M) {
            res[i] = *reinterpret_cast<const uint4*>(residual + (size_t)(m_first + row) * N + n_first + ch8 * 8);
        }
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int idx = tw + i * 128, row = idx >> 4, ch8 = idx & 15;
        if (m_first + row < M) {
            uint4 o = *reinterpret_cast<const uint4*>(stage + row * 128 + ch8 * 8);
            if (residual != nullptr) {
                __half2* oh = reinterpret_cast<__half2*>(&o);
                const __half2* rh = reinterpret_cast<const __half2*>(&res[i]);
                if (gate) {
                    // the second operand is the gate projection: this GEMM is the up projection of a gated FFN
#pragma unroll
                    for (int e = 0; e < 4; ++e) oh[e] = gated_silu2(rh[e], oh[e]);
                }
                else {
#pragma unroll
                    for (int e = 0; e < 4; ++e) oh[e] = __hadd2(oh[e], rh[e]);
                }
            }
            *reinterpret_cast<uint4*>(C + (size_t)(m_first + row) * N + n_first + ch8 * 8) = o;
        }
    }
}

template<int BN>
__global__ void __launch_bounds__(kTcThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint8_t* __restrict__ Bw, const __half* __restrict__ scale,
               __half* __restrict__ C, const __half* __restrict__ residual, int gate, int M, int N, int K)
{
    extern __shared__ __align__(1024) uint8_t tc_dyn[];
    __shared__ TcSmem sm;
    // the ring must start on a 1024-byte boundary for the swizzled tiles
    uint8_t* ring = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_dyn) + 1023) & ~(uintptr_t)1023);
    constexpr int kStageBytes = tc_stage_bytes(BN);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * 128;   // first output channel of the tile
    const int m0 = blockIdx.y * BN;    // first token of the tile
    const int KT = K / kTile;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kTcStages; ++s) {
            mbar_init(&sm.full[s], 1);
            mbar_init(&sm.ready[s], 4);
            mbar_init(&sm.empty[s], 1);
        }
        mbar_init(&sm.accum, 1);
        sm.abort = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        // tensor memory: BN fp32 columns x 128 lanes for the accumulator
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"((uint32_t)BN)
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
            // (ring positions are counters: this loop is one thread's chain of dependent instructions)
            int s = 0;
            uint32_t ph = 1;
            const uint8_t* w0 = Bw + (size_t)(n0 / kTile) * KT * kTileBytes;
            for (int kb = 0; kb < KT; ++kb, w0 += kTileBytes) {
                if (kb >= kTcStages && !tc_wait(&sm.empty[s], ph, &sm.abort)) break;
                uint8_t* st = ring + (size_t)s * kStageBytes;
                mbar_arrive_expect_tx(&sm.full[s], (uint32_t)(kTcW8Bytes + BN * 128));
                bulk_g2s(st, w0, kTileBytes, &sm.full[s]);
                bulk_g2s(st + kTileBytes, w0 + (size_t)KT * kTileBytes, kTileBytes, &sm.full[s]);
                tma_load_2d(st + kTcW8Bytes + kTcWhBytes, &tmap_x, kb * kTile, m0, &sm.full[s]);
                if (++s == kTcStages) {
                    s = 0;
                    ph ^= 1;
                }
            }
        }
    }
    else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(128, BN);
            const uint64_t a_desc0 = umma_desc_sw128(smem_u32(ring + kTcW8Bytes));
            const uint64_t b_desc0 = umma_desc_sw128(smem_u32(ring + kTcW8Bytes + kTcWhBytes));
            int s = 0;
            uint32_t ph = 0;
            for (int kb = 0; kb < KT; ++kb) {
                if (!tc_wait(&sm.full[s], ph, &sm.abort)) break;    // activations landed
                if (!tc_wait(&sm.ready[s], ph, &sm.abort)) break;   // fp16 weights written
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t a_desc = a_desc0 + (uint64_t)(s * (kStageBytes >> 4));
                const uint64_t b_desc = b_desc0 + (uint64_t)(s * (kStageBytes >> 4));
                // 16 reduction indices = 32 bytes along the swizzled row: +2 in 16-byte address units
                umma_f16(tmem, a_desc, b_desc, idesc, kb != 0);
                umma_f16(tmem, a_desc + 2, b_desc + 2, idesc, true);
                umma_f16(tmem, a_desc + 4, b_desc + 4, idesc, true);
                umma_f16(tmem, a_desc + 6, b_desc + 6, idesc, true);
                umma_commit(&sm.empty[s]);
                if (++s == kTcStages) {
                    s = 0;
                    ph ^= 1;
                }
            }
            umma_commit(&sm.accum);
        }
    }
    else {
        // ------------------------------------------------------------------ transform warps, then epilogue
        const int tw = threadIdx.x - 64;          // 0..127
        int s = 0;
        uint32_t ph = 0;
        for (int kb = 0; kb < KT; ++kb) {
            if (!tc_wait(&sm.full[s], ph, &sm.abort)) break;
            uint8_t* st = ring + (size_t)s * kStageBytes;
            const uint8_t* w8 = st;
            uint8_t* wh = st + kTcW8Bytes;
#pragma unroll
            for (int pass = 0; pass < 4; ++pass) {
                const int r = pass * 32 + (tw >> 2);   // channel row of the tile, 0..127
                const int qd = tw & 3;                 // 16-byte quarter of its 64 int8 values
                const uint4 raw = *reinterpret_cast<const uint4*>(w8 + r * 64 + qd * 16);
                uint4 o0, o1;
                cvt_u8x4_to_f16x4(raw.x, o0.x, o0.y);
                cvt_u8x4_to_f16x4(raw.y, o0.z, o0.w);
                cvt_u8x4_to_f16x4(raw.z, o1.x, o1.y);
                cvt_u8x4_to_f16x4(raw.w, o1.z, o1.w);
                uint8_t* row = wh + r * 128;
                *reinterpret_cast<uint4*>(row + (((2 * qd) ^ (r & 7)) << 4)) = o0;
                *reinterpret_cast<uint4*>(row + (((2 * qd + 1) ^ (r & 7)) << 4)) = o1;
            }
            // make the generic-proxy writes visible to the tensor core (async proxy), then signal
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.ready[s]);
            if (++s == kTcStages) {
                s = 0;
                ph ^= 1;
            }
        }

        // ---- epilogue: TMEM lane = channel, columns = tokens ----
        // every epilogue warp gets here (the waits are bounded); the barrier makes the abort decision uniform
        tc_wait(&sm.accum, 0, &sm.abort);
        asm volatile("bar.sync 1, 128;" ::: "memory");
        if (sm.abort == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const int lane_base = (warp & 3) * 32;        // the TMEM lanes this warp may read
            const float sc = __half2float(scale[n0 + lane_base + lane]);
            __half* stage = reinterpret_cast<__half*>(ring);
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (m0 + c0 >= M) break;
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)lane_base << 16) + (uint32_t)c0, v);
                epilogue_block(v, sc, stage + ((c0 >> 5) & 1) * kEpiStageHalves, lane_base + lane, tw, C, residual,
                               gate, m0 + c0, M, N, n0);
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)BN) : "memory");
    }
}

// ---------------------------------------------------------------------------------------------------
// Large-M variant: 256 channels x 256 tokens per output tile.  Two accumulators (one per 128-channel half)
// fill all 512 TMEM columns, and every activation tile fetched from L2 feeds twice as many MMAs as in the
// kernel above, which halves the L2 -> shared-memory traffic per flop.  The three data streams have their own
// rings so that each can run as far ahead as its buffer allows:
//   activations : 3 x 32 KiB, one 2-D TMA copy per k-block            (warp 0)
//   int8 weights: 4 x 16 KiB, four 4 KiB bulk copies per k-block      (warp 6)
//   fp16 weights: 2 x 32 KiB (k-block x two 128-channel halves), written by warps 2-5 / 7-10, read by tcgen05.mma
// One commit per k-block ("done", ring of 6 = lcm of the ring depths) releases the activation stage to its
// producer and the fp16 stage to the transform warps: the issuing thread pays for two waits, eight MMAs and
// one commit per k-block.
//
// Two ways to spread the tiles over the SMs:
//
// (a) Persistent CTAs (gridDim.z == 1), one per SM (fewer when there are fewer tiles): CTA i takes tiles i, i + G,
//     i + 2G, ... so that the CTAs of a wave walk the k-blocks in step: 16 CTAs want the same activation or
//     weight tile at about the same time (measured: out of step the k-loop runs 1.3x slower).  The rings and all
//     phase counters run on
//     across tiles: while the transform warps are busy with a tile's epilogue, the producers already fetch the
//     next tile's first k-blocks.  The epilogue's fp16 staging tiles live in the fp16 weight ring, which is idle
//     exactly then (all MMAs of the tile have completed, the next conversions come after).
//     Two ways of cutting the work so that no SM idles through the last, partial wave were built and measured
//     on 148 SMs, and dropped: (i) textbook stream-K (equal contiguous ranges of (tile, k-block) pairs, partial
//     accumulators handed on through a global scratch) ran 1.3x slower per k-block, because the CTAs no longer
//     read the same tiles at the same time (4096^2, M = 4096: 145 us against 109); (ii) whole tiles in waves and
//     only the left-over tiles cut along K into pieces that keep the k-blocks in step gained 0-3 % (4096 x 12288,
//     M = 4096: 328 us against 330; 11008 x 4096: 267 against 274) - exporting and importing 256 KiB accumulators
//     costs what the shorter wave saves.
//
// (b) Split-K over a thread-block cluster (gridDim.z = cluster size S = 2, 3 or 4) for shapes with fewer tiles
//     than SMs: the S CTAs of a cluster share one output tile (tile0 + blockIdx.x) and each walks 1/S of the
//     k-blocks.  The partial accumulators meet through distributed shared memory, never through global memory:
//     the tile's eight 32-token blocks are dealt out to the ranks (block b belongs to rank b % S), every CTA
//     stores its partial of a foreign block into the owner's shared memory (the operand rings are idle by then;
//     a warp's store instruction covers 512 contiguous bytes), and after one cluster barrier each owner adds
//     the S - 1 partials to its own accumulator in rank order and runs the usual epilogue for its blocks only.
// ---------------------------------------------------------------------------------------------------
constexpr int kTc2Threads = 352;   // X producer, MMA issuer, 4 + 4 transform/epilogue warps, W producer
constexpr int kTc2NX = 3, kTc2NW = 4, kTc2NH = 2, kTc2ND = 6;
constexpr int kTc2XBytes = 256 * 128, kTc2WBytes = 4 * kTileBytes, kTc2HBytes = 128 * 128;   // H: one half
constexpr int kTc2Smem = kTc2NX * kTc2XBytes + kTc2NW * kTc2WBytes + kTc2NH * 2 * kTc2HBytes;
constexpr int kTc2RedBlock = 256 * 128;               // one partial block: 256 channels x 32 tokens fp32
constexpr int kTc2StageBytes = 2 * 2 * kEpiStageHalves * 2;   // the epilogue's fp16 staging tiles (two per group)
// cluster mode: partial blocks received by one CTA (blocks owned, at most ceil(8 / S), x (S - 1) senders) follow
// the staging tiles at the start of the activation ring
static_assert(kTc2StageBytes + 6 * kTc2RedBlock <= kTc2Smem, "partials of S = 3 and S = 4 must fit behind the staging tiles");
static_assert(kTc2StageBytes <= kTc2NH * 2 * kTc2HBytes, "stream-K mode stages its output in the fp16 weight ring");

// Barrier of the 256 transform/epilogue threads of the 256 x 256 kernel that also ORs a predicate over them:
// every thread gets the same answer, so a decision taken on it cannot split the group before a later barrier.
__device__ __forceinline__ bool epi_bar_or(bool pred)
{
    uint32_t out;
    asm volatile(
        "{\n\t"
        ".reg .pred p, q;\n\t"
        "setp.ne.u32 q, %1, 0;\n\t"
        "bar.red.or.pred p, 3, 256, q;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(out)
        : "r"((uint32_t)pred)
        : "memory");
    return out != 0;
}

struct Tc2Smem {
    uint64_t x_full[kTc2NX];
    uint64_t w_full[kTc2NW], w_empty[kTc2NW];
    uint64_t h_ready[kTc2NH];     // both halves of a k-block are written (8 transform warps)
    uint64_t done[kTc2ND];        // the MMAs of a k-block have completed
    uint64_t accum;               // all MMAs of a segment have completed
    uint64_t acc_free;            // the 8 epilogue warps have read the segment's accumulators
    uint32_t tmem_base;
    volatile int abort;
};

// One CTA's share of the work: `nseg` segments, processed in order.
struct Tc2Seg {
    int tile, kb0, kb1;
    bool cluster;   // a k-range of a tile shared with the other CTAs of the cluster
};

struct Tc2Work {
    int KT, G, i, tile0, nseg, cluster_kb0, cluster_kb1, cluster_tile;

    __device__ Tc2Seg seg(int p) const
    {
        Tc2Seg s;
        if (cluster_tile >= 0) {
            s.tile = cluster_tile;
            s.kb0 = cluster_kb0;
            s.kb1 = cluster_kb1;
            s.cluster = true;
            return s;
        }
        s.tile = tile0 + p * G + i;
        s.kb0 = 0;
        s.kb1 = KT;
        s.cluster = false;
        return s;
    }
};

__global__ void __launch_bounds__(kTc2Threads, 1)
gemm_tc2_kernel(const __grid_constant__ CUtensorMap tmap_x, const uint8_t* __restrict__ Bw, const __half* __restrict__ scale,
                __half* __restrict__ C, const __half* __restrict__ residual, int gate, int M, int N, int K, int tile0,
                int tile_count)
{
    // This launch covers tiles [tile0, tile0 + tile_count) of the output, numbered row-major over (token tile,
    // channel tile).
    extern __shared__ __align__(1024) uint8_t tc_dyn[];
    __shared__ Tc2Smem sm;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(tc_dyn) + 1023) & ~(uintptr_t)1023);
    uint8_t* x_ring = base;                                   // 1024-byte aligned tiles (swizzled)
    uint8_t* h_ring = base + kTc2NX * kTc2XBytes;             // 1024-byte aligned tiles (swizzled)
    uint8_t* w_ring = h_ring + kTc2NH * 2 * kTc2HBytes;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int S = (int)gridDim.z, rank = (int)blockIdx.z;
    const int tiles_n = N / 256, tiles_m = (M + 255) / 256;

    Tc2Work wk;
    wk.KT = K / kTile;
    wk.G = (int)gridDim.x;
    wk.i = (int)blockIdx.x;
    wk.cluster_tile = -1;
    wk.cluster_kb0 = wk.cluster_kb1 = 0;
    wk.tile0 = tile0;
    if (S > 1) {
        // cluster mode: the cluster is the gridDim.z CTAs of tile tile0 + blockIdx.x
        wk.cluster_tile = tile0 + (int)blockIdx.x;
        wk.cluster_kb0 = (int)((long long)wk.KT * rank / S);
        wk.cluster_kb1 = (int)((long long)wk.KT * (rank + 1) / S);
        wk.nseg = 1;
    }
    else {
        wk.nseg = (tile_count - wk.i + wk.G - 1) / wk.G;   // tiles tile0 + i, tile0 + i + G, ...
    }
    (void)tiles_m;
    const int nseg = wk.nseg;

    pdl_launch_dependents();
    if (threadIdx.x == 0) {
        for (int s = 0; s < kTc2NX; ++s) mbar_init(&sm.x_full[s], 1);
        for (int s = 0; s < kTc2ND; ++s) mbar_init(&sm.done[s], 1);
        for (int s = 0; s < kTc2NW; ++s) {
            mbar_init(&sm.w_full[s], 1);
            mbar_init(&sm.w_empty[s], 8);
        }
        for (int s = 0; s < kTc2NH; ++s) mbar_init(&sm.h_ready[s], 8);
        mbar_init(&sm.accum, 1);
        mbar_init(&sm.acc_free, 8);
        sm.abort = 0;
        mbar_fence_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(512u)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;
    bool epi_live = false;   // cluster mode: this epilogue thread has a complete accumulator to reduce

    if (warp == 0) {
        // ------------------------------------------------------------------ activation producer
        if (lane == 0) {
            // (ring positions are counters: this loop is one thread's chain of dependent instructions)
            int s = 0, d = 0, it = 0;      // d: slot of done[] for k-block it - NX
            uint32_t phd = 0;
            bool ok = true;
            pdl_wait();            // the activations are the preceding kernel's output (the weights are not)
            for (int p = 0; p < nseg && ok; ++p) {
                const Tc2Seg sg = wk.seg(p);
                const int m0 = (sg.tile / tiles_n) * 256;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    if (it >= kTc2NX) {
                        if (!tc_wait(&sm.done[d], phd, &sm.abort)) {
                            ok = false;
                            break;
                        }
                        if (++d == kTc2ND) {
                            d = 0;
                            phd ^= 1;
                        }
                    }
                    mbar_arrive_expect_tx(&sm.x_full[s], (uint32_t)kTc2XBytes);
                    tma_load_2d(x_ring + (size_t)s * kTc2XBytes, &tmap_x, kb * kTile, m0, &sm.x_full[s]);
                    if (++s == kTc2NX) s = 0;
                }
            }
        }
    }
    else if (warp == 6) {
        // ------------------------------------------------------------------ int8 weight producer
        if (lane == 0) {
            int s = 0, it = 0;
            uint32_t ph = 1;
            bool ok = true;
            for (int p = 0; p < nseg && ok; ++p) {
                const Tc2Seg sg = wk.seg(p);
                const int n0 = (sg.tile % tiles_n) * 256;
                const uint8_t* w0 = Bw + ((size_t)(n0 / kTile) * wk.KT + sg.kb0) * kTileBytes;
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it, w0 += kTileBytes) {
                    if (it >= kTc2NW && !tc_wait(&sm.w_empty[s], ph, &sm.abort)) {
                        ok = false;
                        break;
                    }
                    mbar_arrive_expect_tx(&sm.w_full[s], (uint32_t)kTc2WBytes);
                    uint8_t* dst = w_ring + (size_t)s * kTc2WBytes;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        bulk_g2s(dst + i * kTileBytes, w0 + (size_t)i * wk.KT * kTileBytes, kTileBytes, &sm.w_full[s]);
                    }
                    if (++s == kTc2NW) {
                        s = 0;
                        ph ^= 1;
                    }
                }
            }
        }
    }
    else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(128, 256);
            const uint64_t b_desc0 = umma_desc_sw128(smem_u32(x_ring));
            const uint64_t a_desc0 = umma_desc_sw128(smem_u32(h_ring));
            int sx = 0, sd = 0, it = 0;
            uint32_t phx = 0;
            bool ok = true;
            for (int p = 0; p < nseg && ok; ++p) {
                const Tc2Seg sg = wk.seg(p);
                // the accumulators are overwritten: the epilogue of the previous segment must have read them
                if (p > 0 && !tc_wait(&sm.acc_free, (uint32_t)((p - 1) & 1), &sm.abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                    const int sh = it & 1;
                    if (!tc_wait(&sm.x_full[sx], phx, &sm.abort) ||
                        !tc_wait(&sm.h_ready[sh], (uint32_t)((it >> 1) & 1), &sm.abort)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint64_t b_desc = b_desc0 + (uint64_t)(sx * (kTc2XBytes >> 4));
                    const uint64_t a0 = a_desc0 + (uint64_t)(sh * (2 * kTc2HBytes >> 4));
                    const uint64_t a1 = a0 + (uint64_t)(kTc2HBytes >> 4);
                    const bool acc = kb != sg.kb0;
                    umma_f16(tmem, a0, b_desc, idesc, acc);
                    umma_f16(tmem, a0 + 2, b_desc + 2, idesc, true);
                    umma_f16(tmem, a0 + 4, b_desc + 4, idesc, true);
                    umma_f16(tmem, a0 + 6, b_desc + 6, idesc, true);
                    umma_f16(tmem + 256, a1, b_desc, idesc, acc);
                    umma_f16(tmem + 256, a1 + 2, b_desc + 2, idesc, true);
                    umma_f16(tmem + 256, a1 + 4, b_desc + 4, idesc, true);
                    umma_f16(tmem + 256, a1 + 6, b_desc + 6, idesc, true);
                    umma_commit(&sm.done[sd]);
                    if (++sd == kTc2ND) sd = 0;
                    if (++sx == kTc2NX) {
                        sx = 0;
                        phx ^= 1;
                    }
                }
                if (ok) umma_commit(&sm.accum);
            }
        }
    }
    else {
        // ------------------------------------------------------------------ transform warps, then epilogue
        // Two groups of four warps (2-5 and 7-10); group g owns the 128-channel half g of the tile: it converts
        // that half of every k-block and later runs that accumulator's epilogue.  One group alone could not
        // convert a k-block in the time the tensor core needs for it.
        const int grp = (warp >= 7) ? 1 : 0;
        const int tw = (warp - (grp ? 7 : 2)) * 32 + lane;  // 0..127 within the group
        const int lane_base = (warp & 3) * 32;              // the TMEM lanes this warp may read
        const int ch = grp * 128 + lane_base + lane;        // this thread's channel of the tile
        int sw = 0, d = 0, it = 0;     // d: slot of done[] for k-block it - NH
        uint32_t phw = 0, phd = 0;
        bool ok = true;
        for (int p = 0; p < nseg && ok; ++p) {
            const Tc2Seg sg = wk.seg(p);
            for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++it) {
                if (!tc_wait(&sm.w_full[sw], phw, &sm.abort)) {
                    ok = false;
                    break;
                }
                const uint8_t* w8 = w_ring + (size_t)sw * kTc2WBytes;
                const int sh = it & 1;
                if (it >= kTc2NH) {
                    if (!tc_wait(&sm.done[d], phd, &sm.abort)) {
                        ok = false;
                        break;
                    }
                    if (++d == kTc2ND) {
                        d = 0;
                        phd ^= 1;
                    }
                }
                uint8_t* wh = h_ring + (size_t)(sh * 2 + grp) * kTc2HBytes;
#pragma unroll
                for (int pass = 0; pass < 4; ++pass) {
                    const int r = pass * 32 + (tw >> 2);   // channel row of this half, 0..127
                    const int qd = tw & 3;
                    const uint4 raw = *reinterpret_cast<const uint4*>(w8 + (grp * 128 + r) * 64 + qd * 16);
                    uint4 o0, o1;
                    cvt_u8x4_to_f16x4(raw.x, o0.x, o0.y);
                    cvt_u8x4_to_f16x4(raw.y, o0.z, o0.w);
                    cvt_u8x4_to_f16x4(raw.z, o1.x, o1.y);
                    cvt_u8x4_to_f16x4(raw.w, o1.z, o1.w);
                    uint8_t* row = wh + r * 128;
                    *reinterpret_cast<uint4*>(row + (((2 * qd) ^ (r & 7)) << 4)) = o0;
                    *reinterpret_cast<uint4*>(row + (((2 * qd + 1) ^ (r & 7)) << 4)) = o1;
                }
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) {
                    mbar_arrive(&sm.h_ready[sh]);
                    mbar_arrive(&sm.w_empty[sw]);
                }
                if (++sw == kTc2NW) {
                    sw = 0;
                    phw ^= 1;
                }
            }
            if (!ok) break;

            // ---- end of the segment: every epilogue warp gets here (the waits are bounded); the OR-reducing
            // barrier gives all 256 epilogue threads the same answer, whoever saw the abort flag first ----
            tc_wait(&sm.accum, (uint32_t)(p & 1), &sm.abort);
            if (epi_bar_or(sm.abort != 0)) {
                ok = false;
                break;
            }
            if (sg.cluster) {   // cluster split: the epilogue follows the cluster barriers below
                epi_live = true;
                break;
            }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            pdl_wait();   // the output and the residual belong to the dependency chain
            const int n0 = (sg.tile % tiles_n) * 256, m0 = (sg.tile / tiles_n) * 256;
            {
                const float sc = __half2float(scale[n0 + ch]);
                __half* stage = reinterpret_cast<__half*>(h_ring) + grp * 2 * kEpiStageHalves;
                int blk = 0;
#pragma unroll 1
                for (int b = 0; b < 8; ++b, ++blk) {
                    const int c0 = 32 * b;
                    if (m0 + c0 >= M) break;
                    uint32_t v[32];
                    tmem_ld32(tmem + ((uint32_t)lane_base << 16) + (uint32_t)(grp * 256 + c0), v);
                    if (grp == 0) {
                        epilogue_block<1>(v, sc, stage + (blk & 1) * kEpiStageHalves, lane_base + lane, tw, C, residual, gate,
                                          m0 + c0, M, N, n0);
                    }
                    else {
                        epilogue_block<2>(v, sc, stage + (blk & 1) * kEpiStageHalves, lane_base + lane, tw, C, residual, gate,
                                          m0 + c0, M, N, n0 + 128);
                    }
                }
                // The staging tiles lie in this group's own part of the fp16 weight ring: its next conversions
                // must not start before every thread of the group has read its rows of the last tile.
                if (grp == 0) {
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                }
                else {
                    asm volatile("bar.sync 2, 128;" ::: "memory");
                }
            }
            // accumulators read: the next segment's MMAs may overwrite them
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.acc_free);
        }
    }

    if (S > 1) {
        // ---- cluster split: reduce the S partial accumulators through distributed shared memory, then the
        // epilogue: TMEM lane = channel within the half, columns = tokens; group g takes accumulator g ----
        const bool epi_warp = (warp >= 2 && warp <= 5) || (warp >= 7 && warp <= 10);
        const int grp = (warp >= 7) ? 1 : 0;
        const int tw = (warp - (grp ? 7 : 2)) * 32 + lane;   // 0..127 within the group
        const int lane_base = (warp & 3) * 32;
        const int ch = grp * 128 + lane_base + lane;          // this thread's channel of the tile
        const int n0 = (wk.cluster_tile % tiles_n) * 256, m0 = (wk.cluster_tile / tiles_n) * 256;
        uint8_t* red = base + kTc2StageBytes;
        // All CTAs of the cluster have completed their MMAs: their rings may be overwritten.
        cooperative_groups::this_cluster().sync();
        if (epi_warp && epi_live) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            for (int b = 0; b < 8; ++b) {
                if (m0 + 32 * b >= M) break;
                const int owner = b % S;
                if (owner == rank) continue;
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)lane_base << 16) + (uint32_t)(grp * 256 + 32 * b), v);
                // a partial block is laid out [4-token chunk][channel][16 bytes]: the 32 lanes of a warp store 512
                // contiguous bytes per instruction, and the owner reads them back the same way
                const int slot = (b / S) * (S - 1) + (rank < owner ? rank : rank - 1);
                const uint32_t local = smem_u32(red + (size_t)slot * kTc2RedBlock + (size_t)ch * 16);
                uint32_t remote;
                asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local), "r"((uint32_t)owner));
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    asm volatile("st.shared::cluster.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(remote + (uint32_t)(j * 256 * 16)),
                                 "r"(v[4 * j]), "r"(v[4 * j + 1]), "r"(v[4 * j + 2]), "r"(v[4 * j + 3])
                                 : "memory");
                }
            }
        }
        // the partials of this CTA's blocks have arrived
        cooperative_groups::this_cluster().sync();
        if (epi_warp && epi_live) {
            pdl_wait();   // the output (and the residual) belong to the dependency chain
            __half* stage = reinterpret_cast<__half*>(x_ring) + grp * 2 * kEpiStageHalves;
            const float sc = __half2float(scale[n0 + ch]);
            int blk = 0;
#pragma unroll 1
            for (int b = rank; b < 8; b += S, ++blk) {
                const int c0 = 32 * b;
                if (m0 + c0 >= M) break;
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)lane_base << 16) + (uint32_t)(grp * 256 + c0), v);
                for (int src = 0; src < S - 1; ++src) {
                    const uint8_t* p = red + (size_t)((b / S) * (S - 1) + src) * kTc2RedBlock + (size_t)ch * 16;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint4 q = *reinterpret_cast<const uint4*>(p + j * 256 * 16);
                        v[4 * j] = __float_as_uint(__uint_as_float(v[4 * j]) + __uint_as_float(q.x));
                        v[4 * j + 1] = __float_as_uint(__uint_as_float(v[4 * j + 1]) + __uint_as_float(q.y));
                        v[4 * j + 2] = __float_as_uint(__uint_as_float(v[4 * j + 2]) + __uint_as_float(q.z));
                        v[4 * j + 3] = __float_as_uint(__uint_as_float(v[4 * j + 3]) + __uint_as_float(q.w));
                    }
                }
                if (grp == 0) {
                    epilogue_block<1>(v, sc, stage + (blk & 1) * kEpiStageHalves, lane_base + lane, tw, C, residual, gate, m0 + c0, M,
                                      N, n0);
                }
                else {
                    epilogue_block<2>(v, sc, stage + (blk & 1) * kEpiStageHalves, lane_base + lane, tw, C, residual, gate, m0 + c0, M,
                                      N, n0 + 128);
                }
            }
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u) : "memory");
    }
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_tiled_fn()
{
    static EncodeTiledFn fn = nullptr;
    if (fn == nullptr) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<EncodeTiledFn>(p);
        }
    }
    return fn;
}

template<int BN>
int launch_tc(const CUtensorMap& map, const uint8_t* B, const __half* scale, __half* C, const __half* residual, int gate,
              int M, int N, int K, cudaStream_t stream)
{
    static bool attr_set[64] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    dev &= 63;
    const size_t smem = (size_t)kTcStages * tc_stage_bytes(BN) + 1024;
    if (!attr_set[dev]) {
        EET_CUDA(cudaFuncSetAttribute(gemm_tc_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    dim3 grid(N / 128, (M + BN - 1) / BN);
    gemm_tc_kernel<BN><<<grid, kTcThreads, smem, stream>>>(map, B, scale, C, residual, gate, M, N, K);
    EET_LAUNCH_CHECK();
    return 0;
}

}  // namespace

// Smallest M these kernels accept.  The dispatcher sends M <= 512 to the stream-K kernel first; only shapes
// that kernel does not take can arrive here with fewer tokens, and below 65 a one-tile-per-CTA kernel would
// leave most SMs idle, so the skinny kernel serves those.
constexpr int kTcMinM = 65;

// Clusters of `split` CTAs of the 256 x 256 kernel that can be resident at once (0: that cluster size cannot be
// launched), asked of the occupancy calculator once per device and size.
static int tc2_max_clusters(int split)
{
    static int cached[64][5] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    dev &= 63;
    if (cached[dev][split] == 0) {
        const size_t smem = (size_t)kTc2Smem + 1024;
        int n = 0;
        if (cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(1, 1, split);
            cfg.blockDim = dim3(kTc2Threads, 1, 1);
            cfg.dynamicSmemBytes = smem;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = split;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n, gemm_tc2_kernel, &cfg) != cudaSuccess) {
                (void)cudaGetLastError();
                n = 0;
            }
        }
        cached[dev][split] = n > 0 ? n : -1;
    }
    return cached[dev][split] > 0 ? cached[dev][split] : 0;
}

// Largest cluster size (4, 3, 2) over which the k-blocks of each of `tiles` tiles can be split: all clusters
// resident at once, at least four k-blocks per CTA; 0 if none.  (Clusters of 8 were measured too: the all-to-all
// of 7/8 of every accumulator costs more than the shorter k-loops save.)
static int tc2_cluster_size(int tiles, int K)
{
    const int KT = K / kTile;
    static const int sizes[3] = {4, 3, 2};
    for (int i = 0; i < 3; ++i) {
        const int sp = sizes[i];
        if (KT / sp >= 4 && tiles <= tc2_max_clusters(sp)) return sp;
    }
    return 0;
}

// How the 256 x 256 kernel would run this shape: 0 = not at all, 1 = whole tiles on persistent CTAs, 2/3/4 = the
// k-blocks of a tile split over a cluster of that size.  Whole tiles need most of the machine's worth of them
// (120); below that the largest split is taken that puts at least 96 CTAs to work, whose clusters are all
// resident at once and which still leaves each CTA four k-blocks.
int tc2_split(int M, int N, int K)
{
    if (N % 256 != 0 || M < kTcMinM) return 0;
    static int forced = -2;
    if (forced == -2) {
        const char* e = getenv("EET_TC2_SPLIT");
        forced = e ? atoi(e) : -1;
    }
    const long long tiles = (long long)(N / 256) * ((M + 255) / 256);
    if (forced == 0) return tiles >= 120 ? 1 : 0;
    if (tiles >= 120) return 1;
    const int sp = tc2_cluster_size((int)tiles, K);
    if (forced > 0) return (sp > 0 && K / kTile / forced >= 4 && tiles <= tc2_max_clusters(forced)) ? forced : 0;
    return (sp > 1 && tiles * sp >= 96) ? sp : 0;
}

bool gemm_tc_supported(int M, int N, int K)
{
    return M >= kTcMinM && N % 128 == 0 && K % 64 == 0;
}

int launch_gemm_tc(const __half* A, const uint8_t* B, const __half* scale, __half* C, const __half* residual, int gate,
                   int M, int N, int K, cudaStream_t stream)
{
    EET_CHECK(gemm_tc_supported(M, N, K), "tensor-core GEMM: needs M >= 65, N %% 128 == 0, K %% 64 == 0");
    EncodeTiledFn encode = encode_tiled_fn();
    EET_CHECK(encode != nullptr, "tensor-core GEMM: cuTensorMapEncodeTiled is not available from the driver");
    const int split = tc2_split(M, N, K);
    // token rows per activation tile: always 256 for the 256 x 256 kernel (rows past M read as zeros)
    const int bn = (split > 0 || M > 128) ? 256 : (M > 64 ? 128 : 64);
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)M};
    const cuuint64_t strides[1] = {(cuuint64_t)K * sizeof(__half)};
    const cuuint32_t box[2] = {64, (cuuint32_t)bn};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(A), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    EET_CHECK(rc == CUDA_SUCCESS, "tensor-core GEMM: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    // the 256 x 256 tiles pay off once there are enough of them to fill most of the machine - on a grid of
    // persistent CTAs, or with the k-blocks of a tile split over a cluster
    if (split > 0) {
        static bool attr_set2[64] = {};
        int dev = 0;
        EET_CUDA(cudaGetDevice(&dev));
        dev &= 63;
        const size_t smem = (size_t)kTc2Smem + 1024;
        if (!attr_set2[dev]) {
            EET_CUDA(cudaFuncSetAttribute(gemm_tc2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            attr_set2[dev] = true;
        }
        const int tiles = (N / 256) * ((M + 255) / 256);
        auto launch = [&](int tile0, int count, int grid_x, int cluster) -> cudaError_t {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3((unsigned)grid_x, 1, (unsigned)cluster);
            cfg.blockDim = dim3(kTc2Threads, 1, 1);
            cfg.dynamicSmemBytes = smem;
            cfg.stream = stream;
            cudaLaunchAttribute attr[2];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = 1;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = (unsigned)cluster;
            attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[1].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 2;
            return cudaLaunchKernelEx(&cfg, gemm_tc2_kernel, map, B, scale, C, residual, gate, M, N, K, tile0, count);
        };
        if (split > 1) {
            EET_CUDA(launch(0, tiles, tiles, split));
            return 0;
        }
        // Whole tiles on one persistent CTA per SM (fewer when there are fewer tiles).  When the last wave would
        // be at most half full, its tiles go to a second launch that splits each over a cluster instead: a
        // quarter or a third of the k-blocks per CTA rather than a full tile's worth on a fifth of the SMs.
        const int G = tiles < sm_count() ? tiles : sm_count();
        const int left = tiles % G;
        const int left_split = (left > 0 && 2 * left <= G) ? tc2_cluster_size(left, K) : 0;
        if (left_split > 1) {
            EET_CUDA(launch(0, tiles - left, G, 1));
            EET_CUDA(launch(tiles - left, left, left, left_split));
        }
        else {
            EET_CUDA(launch(0, tiles, G, 1));
        }
        return 0;
    }
    if (bn == 256) return launch_tc<256>(map, B, scale, C, residual, gate, M, N, K, stream);
    if (bn == 128) return launch_tc<128>(map, B, scale, C, residual, gate, M, N, K, stream);
    return launch_tc<64>(map, B, scale, C, residual, gate, M, N, K, stream);
}

}  // namespace eet
