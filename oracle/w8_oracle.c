/*
 * TEST INFRASTRUCTURE - CPU restatement of the reference's int8 weight-only quantizer and weight
 * packers.  Nothing the product ships may call into this file: only tests/, the smoke check and the
 * cpu_baseline / --impl reference legs of the benchmark load it, as the checker.
 *
 * Parity pin: every function here is compared bit for bit with the reference's own code compiled for
 * the host (oracle/_ref, built by the Makefile beside this file) and with golden vectors generated
 * from that build (tests/golden/).
 *
 * Restated reference code (paths inside the reference project):
 *   3rdparty/cutlass_kernels/cutlass_preprocessors.cc:581-678   symmetric_quantize
 *   3rdparty/cutlass_kernels/cutlass_preprocessors.cc:137-195   permute_B_rows_for_mixed_gemm
 *   3rdparty/cutlass_kernels/cutlass_preprocessors.cc:201-335   subbyte_transpose
 *   3rdparty/cutlass_kernels/cutlass_preprocessors.cc:432-495   interleave_column_major_tensor
 *   3rdparty/cutlass_kernels/cutlass_preprocessors.cc:337-358   add_bias_and_interleave_int8s_inplace
 *
 * Build with -fno-fast-math -ffp-contract=off: the rounding of every float operation matters.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

/* ---- IEEE binary16 <-> binary32, round to nearest even (what half(float) does on the host) ---- */
static float h2f(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1fu;
    uint32_t man = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        }
        else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while (!(man & 0x400u));
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | ((man & 0x3ffu) << 13);
        }
    }
    else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    }
    else {
        bits = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

static uint16_t f2h(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t ax = x & 0x7fffffffu;
    if (ax >= 0x7f800000u) { /* inf / nan */
        return (uint16_t)(sign | 0x7c00u | ((ax > 0x7f800000u) ? 0x200u : 0));
    }
    if (ax >= 0x477ff000u) { /* rounds to >= 65520 -> inf */
        return (uint16_t)(sign | 0x7c00u);
    }
    if (ax < 0x33000001u) { /* below half of the smallest subnormal (2^-25) or equal: rounds to 0 */
        return (uint16_t)sign;
    }
    int exp = (int)(ax >> 23) - 127;
    uint32_t man = (ax & 0x7fffffu) | 0x800000u;
    int shift;
    uint32_t hexp;
    if (exp < -14) { /* subnormal half */
        shift = 13 + (-14 - exp);
        hexp = 0;
    }
    else {
        shift = 13;
        hexp = (uint32_t)(exp + 15);
    }
    uint32_t q = man >> shift;
    uint32_t rem = man & ((1u << shift) - 1u);
    uint32_t halfway = 1u << (shift - 1);
    if (rem > halfway || (rem == halfway && (q & 1u))) {
        q++;
    }
    if (hexp == 0) {
        return (uint16_t)(sign | q); /* q may carry into the exponent field: that is correct */
    }
    /* q has the implicit bit at position 10 */
    uint32_t out = ((hexp - 1u) << 10) + q;
    return (uint16_t)(sign | out);
}

/* std::max(a, b) and std::min(a, b) exactly as libstdc++ defines them (NaN ordering matters:
 * cutlass_preprocessors.cc:627 and :647 rely on it). */
static float std_max(float a, float b)
{
    return (a < b) ? b : a;
}
static float std_min(float a, float b)
{
    return (b < a) ? b : a;
}

/*
 * symmetric_quantize for QuantType::INT8_WEIGHT_ONLY (cutlass_preprocessors.cc:581-678), without the
 * packing step at its end.
 *   weight        row-major [rows=K][cols=N], fp16 bits (is_fp32 = 0) or fp32 (is_fp32 = 1)
 *   q             row-major [K][N] int8, the "unprocessed" tensor
 *   scales        [N]; fp16 bits when the weight is fp16, fp32 when it is fp32
 *                 (fpA_intB_gemm_wrapper.cu:71,76-93)
 *   variant       0: the reference code - scale = amax * (1/128), clip to [-128, 127]  (:610,633,647)
 *                 1: amax / 127, clip to [-127, 127]  (not in the reference; the alternative the
 *                    benchmark description mentions)
 */
int oracle_symmetric_quantize_int8(const void* weight, int is_fp32, size_t rows, size_t cols, int8_t* q,
                                   void* scales, int variant)
{
    float* col_max = (float*)malloc(cols * sizeof(float));
    if (!col_max) {
        return 1;
    }
    const uint16_t* w16 = (const uint16_t*)weight;
    const float* w32 = (const float*)weight;
    for (size_t j = 0; j < cols; ++j) {
        col_max[j] = 0.f;
    }
    for (size_t i = 0; i < rows; ++i) { /* :623-628 */
        for (size_t j = 0; j < cols; ++j) {
            float w = is_fp32 ? w32[i * cols + j] : h2f(w16[i * cols + j]);
            col_max[j] = std_max(col_max[j], fabsf(w));
        }
    }
    const float range_scale = 1.f / 128.f; /* :610 */
    const float lo = variant ? -127.f : -128.f;
    for (size_t j = 0; j < cols; ++j) { /* :631-635 */
        col_max[j] = variant ? (col_max[j] / 127.f) : (col_max[j] * range_scale);
        if (is_fp32) {
            ((float*)scales)[j] = col_max[j];
        }
        else {
            ((uint16_t*)scales)[j] = f2h(col_max[j]);
        }
    }
    for (size_t i = 0; i < rows; ++i) { /* :638-649 */
        for (size_t j = 0; j < cols; ++j) {
            float w = is_fp32 ? w32[i * cols + j] : h2f(w16[i * cols + j]);
            float scaled = roundf(w / col_max[j]);
            q[i * cols + j] = (int8_t)std_max(lo, std_min(127.f, scaled));
        }
    }
    free(col_max);
    return 0;
}

/*
 * preprocess_weights_for_mixed_gemm for int8 and arch 75..89 (cutlass_preprocessors.cc:497-534) as a
 * single closed-form byte permutation:
 *   (1) rows permuted inside groups of 16 by 0 1 8 9 2 3 10 11 4 5 12 13 6 7 14 15      (:137-195)
 *   (2) transposed to [N][K]                                                            (:201-335)
 *   (3) pairs of columns interleaved in 64-row tiles, output seen as [N/2][2K]          (:432-495)
 *   (4) +128 and bytes 1<->2 swapped inside each aligned 4-byte word                    (:337-358)
 * Needs K % 64 == 0 and N % 64 == 0 like the reference; returns 1 otherwise.
 */
int oracle_ref_pack_int8(const int8_t* q, size_t K, size_t N, int8_t* packed)
{
    if (K % 64 || N % 64) {
        return 1;
    }
    for (size_t k = 0; k < K; ++k) {
        size_t t = k % 16;
        size_t src_k = (k - t) + 8 * ((t % 4) / 2) + (t % 2) + 2 * (t / 4);
        for (size_t n = 0; n < N; ++n) {
            size_t pos = (n / 2) * (2 * K) + 128 * (k / 64) + 64 * (n % 2) + (k % 64);
            size_t in_word = pos & 3u; /* step (4): swap byte 1 and byte 2 of each word */
            size_t dst = (pos & ~(size_t)3u) | (in_word == 1 ? 2 : (in_word == 2 ? 1 : in_word));
            packed[dst] = (int8_t)(uint8_t)((int)q[src_k * N + n] + 128);
        }
    }
    return 0;
}

/* Inverse of oracle_ref_pack_int8: recovers the row-major [K][N] int8 matrix from bytes packed by the
 * reference for sm75-89. */
int oracle_ref_unpack_int8(const int8_t* packed, size_t K, size_t N, int8_t* q)
{
    if (K % 64 || N % 64) {
        return 1;
    }
    for (size_t k = 0; k < K; ++k) {
        size_t t = k % 16;
        size_t src_k = (k - t) + 8 * ((t % 4) / 2) + (t % 2) + 2 * (t / 4);
        for (size_t n = 0; n < N; ++n) {
            size_t pos = (n / 2) * (2 * K) + 128 * (k / 64) + 64 * (n % 2) + (k % 64);
            size_t in_word = pos & 3u;
            size_t dst = (pos & ~(size_t)3u) | (in_word == 1 ? 2 : (in_word == 2 ? 1 : in_word));
            q[src_k * N + n] = (int8_t)((int)(uint8_t)packed[dst] - 128);
        }
    }
    return 0;
}

/*
 * The B200 layout this repository's kernels consume ("W8T64"): the matrix is cut into tiles of 64
 * output channels x 64 reduction indices; tiles are ordered [N/64][K/64]; inside a tile the byte for
 * (n, k) sits at (n % 64) * 64 + (k % 64); every byte is the quantized value + 128.  It replaces the
 * reference's sm75-89 layout (cutlass_preprocessors.cc:497-534) and has the same size, K*N bytes.
 */
int oracle_b200_pack_int8(const int8_t* q, size_t K, size_t N, uint8_t* packed)
{
    if (K % 64 || N % 64) {
        return 1;
    }
    const size_t kt_n = K / 64;
    for (size_t k = 0; k < K; ++k) {
        for (size_t n = 0; n < N; ++n) {
            size_t tile = (n / 64) * kt_n + (k / 64);
            packed[tile * 4096 + (n % 64) * 64 + (k % 64)] = (uint8_t)((int)q[k * N + n] + 128);
        }
    }
    return 0;
}

int oracle_b200_unpack_int8(const uint8_t* packed, size_t K, size_t N, int8_t* q)
{
    if (K % 64 || N % 64) {
        return 1;
    }
    const size_t kt_n = K / 64;
    for (size_t k = 0; k < K; ++k) {
        for (size_t n = 0; n < N; ++n) {
            size_t tile = (n / 64) * kt_n + (k / 64);
            q[k * N + n] = (int8_t)((int)packed[tile * 4096 + (n % 64) * 64 + (k % 64)] - 128);
        }
    }
    return 0;
}
