// W8A16 GEMM for the batches between the decode kernel and the large prefill tiles (16 < M <= 512):
// sums[M,N] += A[M,K] (fp16) x q(B) (exact int8 values), B in the W8T64 layout.  Like the skinny kernel it only
// ADDS unscaled fp32 sums; scale, residual and rounding belong to whoever reads them.
//
// The reference serves these sizes with the same CUTLASS fpA_intB kernel as every other
// (fpA_intB_gemm_template.h:445-495, tile candidates cutlass_heuristic.cc:30-118): one CTA per 32..128 x 128
// output tile and no split-K on the hot call sites, i.e. 32-96 CTAs for N = 4096..12288.
//
// B200 design: stream-K over tcgen05.  A work unit is two consecutive 64-wide k-blocks (one at the odd end
// of K) of one 128-channel strip; the units are cut into as many equal, contiguous ranges as CTAs fit on
// the GPU (two per SM), so all SMs stream weights whatever N is, and a range that crosses a strip boundary
// simply ends one accumulation and starts the next.  Per CTA:
//   warp 0      weight producer: the int8 tiles of a unit (two 1-D bulk copies of up to 8 KiB), ring 3-5 deep;
//   warp 10     activation producer: the BN x 64 tiles of the unit's k-blocks (2-D tensor map, 128-byte
//               swizzle, rows past M read as zeros), ring 3-4 deep - L2 hits, but as slow as DRAM while the
//               weights stream;
//   warps 2-5   int8 -> fp16 (exact), one thread per channel: its 64 bytes of a k-block become 32 packed
//               half2 registers that go straight into TENSOR MEMORY (tcgen05.st, lane = channel), where the
//               MMA reads its A operand from - the fp16 weights never exist in shared memory, which carries
//               only the int8 bytes and the activations;
//   warp 1      tcgen05.mma M128 x BN x K16 with A from tensor memory, eight per unit, fp32 accumulators in
//               tensor memory too; two accumulator buffers alternate between consecutive strips;
//   warps 6-9   epilogue: tcgen05.ld (lane = channel), then red.global.add.f32 into sums - 32 lanes of a
//               warp hit 32 consecutive floats of one token row.
// The producer and issuer roles are single threads, i.e. chains of dependent instructions; what they do per
// unit (waits, address arithmetic, commits) bounds the kernel before any memory system does.  Hence units of
// two k-blocks, ring positions kept as counters, and waits that cost one try_wait when the phase is complete.
// Token tiles beyond the first (M > BN) are blockIdx.y: CTAs with the same blockIdx.x walk the same
// weights at the same time and share them through L2.
// Every wait is bounded (device status 2 on expiry) and the CTA frees its tensor memory on every path.
#include "common.cuh"
#include "kernels.h"

namespace eet {

namespace {

constexpr int kMidThreads = 352;
constexpr int kMidUnitK = 2;                         // k-blocks per unit
constexpr int kMidWStage = kMidUnitK * kTcW8Bytes;   // 16 KiB: [channel half][k-block][64 x 64 bytes]
constexpr int kMidACols = kMidUnitK * 32;            // TMEM columns of one fp16 weight buffer: 64 k as half2 each
constexpr int kMidNWMax = 6, kMidNXMax = 4, kMidNHMax = 4;

// (128-token tiles: the kernel alone runs as fast with four weight stages, but a call - this kernel followed by the
// finalize launch - measured 0.5-2.4 us shorter with five)
__host__ __device__ constexpr int mid_nw(int bn) { return bn == 64 ? 3 : (bn == 128 ? 5 : 4); }
__host__ __device__ constexpr int mid_nx(int bn) { return bn == 32 ? 4 : (bn == 256 ? 2 : 3); }
// accumulator buffers: two (the epilogue of a strip overlaps the next strip's MMAs) while they fit beside
// the fp16 weight buffers; one for 256-token tiles
__host__ __device__ constexpr int mid_acc_bufs(int bn) { return bn <= 128 ? 2 : 1; }
__host__ __device__ constexpr int mid_nh(int bn) { return bn == 32 ? 3 : (bn == 64 ? 2 : 4); }

__host__ __device__ constexpr int mid_smem_bytes(int bn)
{
    return mid_nw(bn) * kMidWStage + mid_nx(bn) * kMidUnitK * bn * 128;
}

// tensor-memory columns: two accumulators of BN columns, then the fp16 weight buffers
__host__ __device__ constexpr uint32_t mid_tmem_cols(int bn)
{
    return mid_acc_bufs(bn) * bn + mid_nh(bn) * kMidACols <= 256 ? 256u : 512u;
}

struct MidSmem {
    uint64_t w_full[kMidNWMax], w_empty[kMidNWMax];     // int8 tiles landed / read by the 4 transform warps
    uint64_t x_full[kMidNXMax], x_empty[kMidNXMax];     // activation tiles landed / their MMAs completed
    uint64_t h_ready[kMidNHMax], h_empty[kMidNHMax];    // fp16 weights written (4 warps) / their MMAs completed
    uint64_t acc_full[2];                               // all MMAs of a strip segment have completed
    uint64_t acc_empty[2];                              // the epilogue warps have read the accumulator buffer (4 warps)
    uint32_t tmem_base;
    volatile int abort;
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t (&v)[32])
{
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
        "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};\n" ::"r"(taddr),
        "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]), "r"(v[9]),
        "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]), "r"(v[16]), "r"(v[17]), "r"(v[18]),
        "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]), "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]),
        "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
        : "memory");
    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
}

// D[tmem] (+)= A[tmem] x B[smem]: the A operand (128 rows = lanes, 16 fp16 = 8 columns) comes from tensor memory
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, bool accumulate)
{
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t"
        "}\n" ::"r"(d_tmem),
        "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"((uint32_t)accumulate)
        : "memory");
}

__device__ __forceinline__ void red_add_f32(float* addr, float v)
{
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

template<int BN>
__global__ void __launch_bounds__(kMidThreads, BN <= 64 ? 2 : 1)
gemm_mid_kernel(const __grid_constant__ CUtensorMap tmap_x, GemmArgs a)
{
    extern __shared__ __align__(1024) uint8_t mid_dyn[];
    __shared__ MidSmem sm;
    uint8_t* base = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(mid_dyn) + 1023) & ~(uintptr_t)1023);
    constexpr int kMidNW = mid_nw(BN), kMidNX = mid_nx(BN), kMidNH = mid_nh(BN);
    constexpr int kXTile = BN * 128;                          // one k-block of activations
    constexpr int kXStage = kMidUnitK * kXTile;
    uint8_t* x_ring = base;                                   // 1024-byte aligned tiles (swizzled)
    uint8_t* w_ring = x_ring + kMidNX * kXStage;
    constexpr uint32_t kTmemCols = mid_tmem_cols(BN);
    constexpr int kAccBufs = mid_acc_bufs(BN);
    constexpr uint32_t kAColBase = kAccBufs * BN;             // first column of the fp16 weight buffers
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int KT = a.K / kTile;
    const int KP = (KT + kMidUnitK - 1) / kMidUnitK;          // units per strip
    const int strips1 = a.N / 128;                            // 128-channel strips of one matrix
    const long long U = (long long)strips1 * KP * (a.B2 ? 2 : 1);
    const int u0 = (int)(U * blockIdx.x / gridDim.x);
    const int u1 = (int)(U * (blockIdx.x + 1) / gridDim.x);
    const int m0 = blockIdx.y * BN;

    pdl_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMidNW; ++s) {
            mbar_init(&sm.w_full[s], 1);
            mbar_init(&sm.w_empty[s], 4);
        }
        for (int s = 0; s < kMidNX; ++s) {
            mbar_init(&sm.x_full[s], 1);
            mbar_init(&sm.x_empty[s], 1);
        }
        for (int s = 0; s < kMidNH; ++s) {
            mbar_init(&sm.h_ready[s], 4);
            mbar_init(&sm.h_empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&sm.acc_full[b], 1);
            mbar_init(&sm.acc_empty[b], 4);
        }
        sm.abort = 0;
        mbar_fence_init();
    }
    // ------------------------------------------------------------------ weight producer (thread 0)
    // Constant inputs: requested without waiting for the preceding kernel - and the first ring of requests
    // goes out before the block-wide barrier and the tensor-memory allocation, which nobody needs for it.
    int w_s = 0, w_fill = 0, w_u = u0;
    uint32_t w_ph = 1;   // parity of the previous round of slot w_s
    int w_strip = u0 / KP, w_kp = u0 - (u0 / KP) * KP;
    auto issue_w = [&]() {
        const int kb = w_kp * kMidUnitK;
        const uint32_t bytes = (uint32_t)min(kMidUnitK, KT - kb) * kTileBytes;   // per channel half
        const uint8_t* Bm = (w_strip < strips1) ? a.B : a.B2;
        const int st = (w_strip < strips1) ? w_strip : w_strip - strips1;
        const uint8_t* w0 = Bm + ((size_t)(2 * st) * KT + kb) * kTileBytes;
        uint8_t* dst = w_ring + (size_t)w_s * kMidWStage;
        mbar_arrive_expect_tx(&sm.w_full[w_s], 2 * bytes);
        bulk_g2s_stream(dst, w0, bytes, &sm.w_full[w_s]);
        bulk_g2s_stream(dst + kMidWStage / 2, w0 + (size_t)KT * kTileBytes, bytes, &sm.w_full[w_s]);
        ++w_fill;
        ++w_u;
        if (++w_s == kMidNW) {
            w_s = 0;
            w_ph ^= 1;
        }
        if (++w_kp == KP) {
            w_kp = 0;
            ++w_strip;
        }
    };
    if (threadIdx.x == 0) {
        while (w_fill < kMidNW && w_u < u1) issue_w();
    }
    if (warp == 1) {
        // tcgen05.alloc blocks until the columns are free.  With programmatic dependent launch a CTA of the NEXT
        // kernel can become resident beside a CTA of this one (shared memory permitting) and then waits here for
        // tensor memory; that cannot deadlock, because no CTA of an earlier kernel ever waits for a later one: it
        // runs to its dealloc.  (BN <= 64: 256 columns, two CTAs per SM; larger BN: 512 columns, and the shared-
        // memory footprint of 100+ KiB keeps a second TMEM-holding CTA of the same kernel off the SM.)
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&sm.tmem_base)),
                     "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem = sm.tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            while (w_u < u1) {
                if (!tc_wait(&sm.w_empty[w_s], w_ph, &sm.abort)) break;
                issue_w();
            }
        }
    }
    else if (warp == 10) {
        // ------------------------------------------------------------------ activation producer
        if (lane == 0) {
            pdl_wait();   // the activations are the preceding kernel's output
            int s = 0, fill = 0;
            uint32_t ph = 1;
            int kp = u0 % KP;
            for (int u = u0; u < u1; ++u) {
                if (fill >= kMidNX && !tc_wait(&sm.x_empty[s], ph, &sm.abort)) break;
                const int kb = kp * kMidUnitK;
                const bool two = kb + 1 < KT;
                uint8_t* dst = x_ring + (size_t)s * kXStage;
                mbar_arrive_expect_tx(&sm.x_full[s], (uint32_t)(two ? 2 * kXTile : kXTile));
                tma_load_2d(dst, &tmap_x, kb * kTile, m0, &sm.x_full[s]);
                if (two) tma_load_2d(dst + kXTile, &tmap_x, (kb + 1) * kTile, m0, &sm.x_full[s]);
                ++fill;
                if (++s == kMidNX) {
                    s = 0;
                    ph ^= 1;
                }
                if (++kp == KP) kp = 0;
            }
        }
    }
    else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc_f16(128, BN);
            const uint64_t b_desc0 = umma_desc_sw128(smem_u32(x_ring));
            const uint32_t a_tmem0 = tmem + kAColBase;
            int sx = 0, sh = 0, seg = 0;
            uint32_t phx = 0, phh = 0;
            bool ok = true;
            int strip_end = (u0 / KP + 1) * KP;   // first unit of the next strip
            const bool odd_tail = (KT & 1) != 0;  // the last unit of a strip then holds one k-block
            for (int u = u0; u < u1 && ok;) {
                const int u_end = min(u1, strip_end);
                const int buf = seg % kAccBufs;
                if (seg >= kAccBufs && !tc_wait(&sm.acc_empty[buf], (uint32_t)((seg / kAccBufs - 1) & 1), &sm.abort)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint32_t d_tmem = tmem + (uint32_t)(buf * BN);
                for (int uu = u; uu < u_end; ++uu) {
                    if (!tc_wait(&sm.x_full[sx], phx, &sm.abort) || !tc_wait(&sm.h_ready[sh], phh, &sm.abort)) {
                        ok = false;
                        break;
                    }
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    const uint32_t a_tmem = a_tmem0 + (uint32_t)(sh * kMidACols);
                    const uint64_t b_desc = b_desc0 + (uint64_t)(sx * (kXStage >> 4));
                    // 16 reduction indices per MMA: 8 columns of A, 32 bytes along the swizzled row of B
                    umma_f16_ts(d_tmem, a_tmem, b_desc, idesc, uu > u);
                    umma_f16_ts(d_tmem, a_tmem + 8, b_desc + 2, idesc, true);
                    umma_f16_ts(d_tmem, a_tmem + 16, b_desc + 4, idesc, true);
                    umma_f16_ts(d_tmem, a_tmem + 24, b_desc + 6, idesc, true);
                    if (!(odd_tail && uu + 1 == strip_end)) {
                        const uint64_t b2 = b_desc + (uint64_t)(kXTile >> 4);
                        umma_f16_ts(d_tmem, a_tmem + 32, b2, idesc, true);
                        umma_f16_ts(d_tmem, a_tmem + 40, b2 + 2, idesc, true);
                        umma_f16_ts(d_tmem, a_tmem + 48, b2 + 4, idesc, true);
                        umma_f16_ts(d_tmem, a_tmem + 56, b2 + 6, idesc, true);
                    }
                    umma_commit(&sm.h_empty[sh]);
                    umma_commit(&sm.x_empty[sx]);
                    if (++sx == kMidNX) {
                        sx = 0;
                        phx ^= 1;
                    }
                    if (++sh == kMidNH) {
                        sh = 0;
                        phh ^= 1;
                    }
                }
                if (ok) umma_commit(&sm.acc_full[buf]);
                u = u_end;
                strip_end += KP;
                ++seg;
            }
        }
    }
    else if (warp < 6) {
        // ------------------------------------------------------------------ transform warps
        // this thread's channel: TMEM lane = 32 * (warp % 4) + lane (the lanes a warp may access)
        const int r = (warp & 3) * 32 + lane;
        const int sxr = (lane >> 1) & 3;   // 16-byte chunks are read in XOR order: conflict-free for 64-byte rows
        const uint32_t row_off = (uint32_t)((r >> 6) * (kMidWStage / 2) + (r & 63) * 64);
        const uint32_t lane_addr = (uint32_t)((warp & 3) * 32) << 16;
        int sw = 0, sh = 0, fill = 0;
        uint32_t phw = 0, phh = 1;
        int kp = u0 % KP;
        for (int u = u0; u < u1; ++u) {
            if (!tc_wait(&sm.w_full[sw], phw, &sm.abort)) break;
            const int nk = (kp * kMidUnitK + 1 < KT) ? 2 : 1;
            const uint8_t* row = w_ring + (size_t)sw * kMidWStage + row_off;
            uint4 c[kMidUnitK][4];
#pragma unroll
            for (int kk = 0; kk < kMidUnitK; ++kk) {
                if (kk < nk) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        c[kk][j] = *reinterpret_cast<const uint4*>(row + kk * kTileBytes + ((j ^ sxr) << 4));
                    }
                }
            }
            // the int8 stage is free again as soon as the bytes are in registers
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.w_empty[sw]);
            bool live = true;
#pragma unroll
            for (int kk = 0; kk < kMidUnitK; ++kk) {
                if (kk < nk && live) {
                    // c[kk][j] holds chunk j ^ sxr: undo the permutation with two conditional swap stages
                    if (sxr & 1) {
                        uint4 t = c[kk][0]; c[kk][0] = c[kk][1]; c[kk][1] = t;
                        t = c[kk][2]; c[kk][2] = c[kk][3]; c[kk][3] = t;
                    }
                    if (sxr & 2) {
                        uint4 t = c[kk][0]; c[kk][0] = c[kk][2]; c[kk][2] = t;
                        t = c[kk][1]; c[kk][1] = c[kk][3]; c[kk][3] = t;
                    }
                    uint32_t h[32];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        cvt_u8x4_to_f16x4(c[kk][j].x, h[8 * j + 0], h[8 * j + 1]);
                        cvt_u8x4_to_f16x4(c[kk][j].y, h[8 * j + 2], h[8 * j + 3]);
                        cvt_u8x4_to_f16x4(c[kk][j].z, h[8 * j + 4], h[8 * j + 5]);
                        cvt_u8x4_to_f16x4(c[kk][j].w, h[8 * j + 6], h[8 * j + 7]);
                    }
                    if (kk == 0) {
                        if (fill >= kMidNH && !tc_wait(&sm.h_empty[sh], phh, &sm.abort)) live = false;
                        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    }
                    if (live) tmem_st32(tmem + lane_addr + kAColBase + (uint32_t)(sh * kMidACols + kk * 32), h);
                }
            }
            if (!live) break;
            asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
            __syncwarp();
            if (lane == 0) mbar_arrive(&sm.h_ready[sh]);
            ++fill;
            if (++sw == kMidNW) {
                sw = 0;
                phw ^= 1;
            }
            if (++sh == kMidNH) {
                sh = 0;
                phh ^= 1;
            }
            if (++kp == KP) kp = 0;
        }
    }
    else if (warp >= 10) {
        // (the other lanes of the activation producer's warp have nothing to do)
    }
    else {
        // ------------------------------------------------------------------ epilogue warps
        pdl_wait();   // the sums belong to the dependency chain
        const int lane_base = (warp & 3) * 32;   // the TMEM lanes this warp may read
        int seg = 0;
        for (int u = u0; u < u1; ++seg) {
            const int strip = u / KP;
            const int u_end = min(u1, (strip + 1) * KP);
            const int buf = seg % kAccBufs;
            // one lane polls (a segment lasts tens of microseconds: 128 spinning lanes would take issue
            // slots and shared-memory bandwidth from the threads that feed the tensor core)
            int got = 1;
            if (lane == 0) got = tc_wait(&sm.acc_full[buf], (uint32_t)((seg / kAccBufs) & 1), &sm.abort) ? 1 : 0;
            got = __shfl_sync(0xffffffffu, got, 0);
            if (!got) break;
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            float* sums = (strip < strips1) ? a.ws : a.ws2;
            const int n = ((strip < strips1) ? strip : strip - strips1) * 128 + lane_base + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                tmem_ld32(tmem + ((uint32_t)lane_base << 16) + (uint32_t)(buf * BN + c0), v);
                if (c0 + 32 >= BN) {
                    // everything of this buffer is in registers: hand it back before the global traffic
                    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&sm.acc_empty[buf]);
                }
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                    const int m = m0 + c0 + j;
                    if (m < a.M) red_add_f32(sums + (size_t)m * a.N + n, __uint_as_float(v[j]));
                }
            }
            u = u_end;
        }
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(kTmemCols) : "memory");
    }
}

template<int BN>
int launch_mid(const CUtensorMap& map, const GemmArgs& a, cudaStream_t stream)
{
    static bool attr_set[64] = {};
    int dev = 0;
    EET_CUDA(cudaGetDevice(&dev));
    dev &= 63;
    const size_t smem = (size_t)mid_smem_bytes(BN) + 1024;
    if (!attr_set[dev]) {
        EET_CUDA(cudaFuncSetAttribute(gemm_mid_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        attr_set[dev] = true;
    }
    const int m_tiles = (a.M + BN - 1) / BN;
    const long long U = (long long)(a.N / 128) * ((a.K / kTile + kMidUnitK - 1) / kMidUnitK) * (a.B2 ? 2 : 1);
    int grid_x = (BN <= 64 ? 2 : 1) * sm_count() / m_tiles;
    if (grid_x < 1) grid_x = 1;
    if (grid_x > U) grid_x = (int)U;
    EET_CUDA(launch_pdl(gemm_mid_kernel<BN>, dim3(grid_x, m_tiles), dim3(kMidThreads), smem, stream, map, a));
    return 0;
}

}  // namespace

bool gemm_mid_supported(int M, int N, int K)
{
    return M > 16 && M <= kMidMaxM && N % 128 == 0 && K % 64 == 0;
}

// Adds A[M,K] x q(B) (and, with B2, A x q(B2)) into the fp32 buffers a.ws (a.ws2), rows [0, M).
int launch_gemm_mid(const GemmArgs& a, cudaStream_t stream)
{
    EET_CHECK(gemm_mid_supported(a.M, a.N, a.K), "stream-K tensor-core GEMM: needs 16 < M <= %d, N %% 128 == 0, K %% 64 == 0",
              kMidMaxM);
    EncodeTiledFn encode = encode_tiled_fn();
    EET_CHECK(encode != nullptr, "stream-K tensor-core GEMM: cuTensorMapEncodeTiled is not available from the driver");
    static int force_bn = -1;
    if (force_bn < 0) {
        const char* e = getenv("EET_MID_BN");
        force_bn = e ? atoi(e) : 0;
    }
    // token tile: the smallest that holds M; above 128 tokens 256-token tiles (half the activation traffic
    // per flop, MMAs long enough to hide their issue cost) when every CTA still gets a decent run of units
    const long long units = (long long)(a.N / 128) * ((a.K / kTile + kMidUnitK - 1) / kMidUnitK) * (a.B2 ? 2 : 1);
    int bn = a.M <= 32 ? 32 : (a.M <= 64 ? 64 : 128);
    if (a.M > 128 && units >= 16LL * sm_count()) bn = 256;
    if (force_bn) bn = force_bn;
    CUtensorMap map;
    const cuuint64_t dims[2] = {(cuuint64_t)a.K, (cuuint64_t)a.M};
    const cuuint64_t strides[1] = {(cuuint64_t)a.K * sizeof(__half)};
    const cuuint32_t box[2] = {64, (cuuint32_t)bn};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult rc = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<__half*>(a.A), dims, strides, box, elem,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    EET_CHECK(rc == CUDA_SUCCESS, "stream-K tensor-core GEMM: cuTensorMapEncodeTiled failed with code %d", (int)rc);
    if (bn == 32) return launch_mid<32>(map, a, stream);
    if (bn == 64) return launch_mid<64>(map, a, stream);
    if (bn == 128) return launch_mid<128>(map, a, stream);
    return launch_mid<256>(map, a, stream);
}

}  // namespace eet
