/* CPU restatement in plain C of the FP8 W8A16 reference arithmetic.
 * TEST INFRASTRUCTURE ONLY: built into oracle/c/libw8a16_ref.so, loaded by the
 * parity tests and by the benchmark's CPU-baseline leg; never by the package.
 *
 *  - ref_e4m3_to_fp16_bits : src/fp8_w8a16_sm70/fp8_dequant.cu:44-50
 *  - ref_dequant_block     : src/fp8_w8a16_sm70/fp8_dequant.cu:113-127
 *  - ref_linear_f32acc     : C[m,n] = sum_k A[m,k] * Wdq[n,k], fp32 accumulate,
 *                            the definition of correct used by
 *                            tests/test_phase5_matmul.py:88-175
 *
 * FP16 values travel as uint16_t bit patterns so that the file needs no
 * _Float16 support from the compiler.
 */
#include <stdint.h>
#include <string.h>
#include <math.h>

static float half_bits_to_float(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t out;
    if (exp == 0) {
        if (man == 0) {
            out = sign;
        } else {                       /* subnormal: renormalise */
            int e = -1;
            do { man <<= 1; ++e; } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            out = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 0x1F) {
        out = sign | 0x7F800000u | (man << 13);
    } else {
        out = sign | ((exp + 112u) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &out, 4);
    return f;
}

/* float -> FP16 bits, round to nearest even, subnormals kept. */
static uint16_t float_to_half_bits(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx >= 0x7F800000u) {                         /* inf / nan */
        if (absx == 0x7F800000u) return sign | 0x7C00u;
        uint16_t m = (uint16_t)((absx >> 13) & 0x3FFu);
        return sign | 0x7C00u | (m ? m : 0x200u);
    }
    if (absx >= 0x477FF000u) return sign | 0x7C00u;    /* rounds to >= 65520 -> inf */
    if (absx < 0x33000001u) return sign;               /* < 2^-25 (or == with tie to even 0) */
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x7FFFFFu) | 0x800000u;       /* 24-bit significand */
    int shift;
    uint32_t base;
    if (e < -14) { shift = 13 + (-14 - e); base = 0; } /* subnormal result */
    else         { shift = 13; base = (uint32_t)(e + 15) << 10; m &= 0x7FFFFFu; }
    uint32_t q = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (q & 1u))) q += 1u;
    return sign | (uint16_t)(base + q);                /* carry into exponent is correct */
}

uint16_t ref_e4m3_to_fp16_bits(uint8_t x) {
    uint16_t sign = (uint16_t)(x & 0x80u) << 8;
    uint16_t mag = (uint16_t)(x & 0x7Fu);
    float h = half_bits_to_float((uint16_t)(mag << 7)) * 256.0f;   /* exact in fp32 and in fp16 */
    uint16_t val = (mag == 0x7Fu) ? (uint16_t)0x7F80u : float_to_half_bits(h);
    return (uint16_t)(sign | val);
}

void ref_e4m3_table(uint16_t* out256) {
    for (int i = 0; i < 256; ++i) out256[i] = ref_e4m3_to_fp16_bits((uint8_t)i);
}

/* out[i,j] = RN16(cvt(W[i,j]) * S16[i/bh, j/bw]); scales given as FP16 bits. */
void ref_dequant_block(const uint8_t* w, const uint16_t* scales, uint16_t* out,
                       int64_t N, int64_t K, int block_h, int block_w) {
    int64_t Kb = (K + block_w - 1) / block_w;
    uint16_t tab[256];
    ref_e4m3_table(tab);
    for (int64_t i = 0; i < N; ++i) {
        const uint16_t* srow = scales + (i / block_h) * Kb;
        for (int64_t j = 0; j < K; ++j) {
            uint8_t b = w[i * K + j];
            if ((b & 0x7Fu) == 0x7Fu) { out[i * K + j] = tab[b]; continue; }
            float p = half_bits_to_float(tab[b]) * half_bits_to_float(srow[j / block_w]);
            out[i * K + j] = float_to_half_bits(p);   /* one rounding: product of two halves is exact in fp32 */
        }
    }
}

/* C[m,n] (float) = sum_k A[m,k] * Wdq[n,k]; A and Wdq as FP16 bits. */
void ref_linear_f32acc(const uint16_t* a, const uint16_t* wdq, float* c,
                       int64_t M, int64_t N, int64_t K) {
    for (int64_t m = 0; m < M; ++m) {
        for (int64_t n = 0; n < N; ++n) {
            float acc = 0.f;
            for (int64_t k = 0; k < K; ++k)
                acc += half_bits_to_float(a[m * K + k]) * half_bits_to_float(wdq[n * K + k]);
            c[m * N + n] = acc;
        }
    }
}
