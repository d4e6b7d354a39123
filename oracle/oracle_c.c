/*
 * CPU oracle, C restatement (OpenMP) of the cast / quantise rules.
 *
 * TEST INFRASTRUCTURE ONLY: the checker the CUDA kernels are compared against and
 * the timed CPU baseline.  Only the tests, the smoke check and the CPU-baseline /
 * reference legs of the benchmark may load it; the product library never does.
 *
 * NovaNN's dtype-conversion primitive is NumPy's ndarray.astype (call sites
 * novann/layers/linear/linear.py:81,96; novann/layers/convolutional/conv2d.py:159,188),
 * i.e. IEEE-754 round-to-nearest-even narrowing with overflow to infinity,
 * implemented in the third-party dependency NumPy 2.3.5 (pyproject.toml:10).  The
 * reference holds no bf16 / FP8 / FP4 code, so for those formats the rules are the
 * normative ones written next to each function ("parity unpinned" by the reference;
 * pinned in the tests against NumPy's own astype for fp16 and, where installed,
 * the ml_dtypes package for the others).  Everything is integer arithmetic on the
 * bit patterns so that no compiler or libm behaviour can leak into the result.
 *
 * Build: gcc -O2 -fopenmp -fno-fast-math -ffp-contract=off -shared -fPIC
 */
#include <stddef.h>
#include <stdint.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

static inline uint32_t f2u(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }
static inline float u2f(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }

/* RNE right shift of a non-negative integer by sh (0..63). */
static inline uint64_t rne_shift(uint64_t v, int sh) {
    if (sh <= 0) return v;
    if (sh > 62) return 0;
    uint64_t h = v >> sh;
    uint64_t r = v & ((1ull << sh) - 1);
    uint64_t half = 1ull << (sh - 1);
    if (r > half || (r == half && (h & 1))) h++;
    return h;
}

/*
 * Saturating RNE conversion of an fp32 magnitude (sign stripped, not NaN) to a tiny
 * float with `mbits` mantissa bits and exponent bias `bias`; `fmax_bits` is the
 * fp32 pattern of the largest finite value, `max_code` its code.
 */
static inline uint32_t small_from_abs(uint32_t a, int mbits, int bias, uint32_t fmax_bits,
                                      uint32_t max_code) {
    if (a >= fmax_bits) return max_code;
    uint32_t min_normal = (uint32_t)(127 + 1 - bias) << 23;
    if (a >= min_normal) {
        uint64_t v = (uint64_t)a - ((uint64_t)(127 - bias) << 23);
        return (uint32_t)rne_shift(v, 23 - mbits);
    }
    int e = (int)(a >> 23);
    uint64_t m = (a & 0x7FFFFFu) | 0x800000u;
    int sh = (150 + (1 - bias - mbits)) - e; /* value = m*2^(e-150); unit 2^(1-bias-mbits) */
    return (uint32_t)rne_shift(m, sh);
}

/* fp32 -> fp16, bit-identical to NumPy's astype(float16): RNE, overflow to inf,
 * NaN keeps sign and the top ten payload bits (0 payload -> 0x..01), not quieted. */
static inline uint16_t f32_to_f16_1(uint32_t u) {
    uint32_t sign = (u >> 16) & 0x8000u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) {
        uint32_t pay = (a >> 13) & 0x3FFu;
        return (uint16_t)(sign | 0x7C00u | (pay ? pay : 1u));
    }
    if (a >= 0x47800000u) return (uint16_t)(sign | 0x7C00u);
    uint32_t h;
    if (a >= 0x38800000u) {
        h = (uint32_t)rne_shift((uint64_t)a - 0x38000000u, 13);
        if (h > 0x7C00u) h = 0x7C00u;
    } else {
        int e = (int)(a >> 23);
        uint64_t m = (a & 0x7FFFFFu) | 0x800000u;
        h = (uint32_t)rne_shift(m, 126 - e);
    }
    return (uint16_t)(sign | h);
}

static inline uint32_t f16_to_f32_1(uint16_t hh) {
    uint32_t h = hh;
    uint32_t sign = (h & 0x8000u) << 16;
    uint32_t e = (h >> 10) & 0x1Fu, m = h & 0x3FFu;
    if (e == 0x1F) return sign | 0x7F800000u | (m << 13);
    if (e == 0) {
        if (m == 0) return sign;
        int s = 0;
        while (!(m & 0x400u)) { m <<= 1; s++; }
        return sign | ((uint32_t)(113 - s) << 23) | ((m & 0x3FFu) << 13);
    }
    return sign | ((e + 112) << 23) | (m << 13);
}

/* fp32 -> bf16: RNE on the low 16 bits (overflow to inf); any NaN -> sign|0x7fc0. */
static inline uint16_t f32_to_bf16_1(uint32_t u) {
    if ((u & 0x7FFFFFFFu) > 0x7F800000u) return (uint16_t)(((u >> 16) & 0x8000u) | 0x7FC0u);
    return (uint16_t)((u + 0x7FFFu + ((u >> 16) & 1u)) >> 16);
}

/* format ids shared with the CUDA library's header */
enum { FMT_E4M3 = 3, FMT_E5M2 = 4 };

/* FP8: E4M3 "fn" (bias 7, max 448=0x7e, NaN sign|0x7f); E5M2 (bias 15, max finite
 * 57344=0x7b, NaN sign|0x7e).  Saturating: |y| clamps to the max finite value. */
static inline uint8_t f32_to_fp8_1(uint32_t u, int fmt) {
    uint32_t s = (u >> 24) & 0x80u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (fmt == FMT_E4M3) {
        if (a > 0x7F800000u) return (uint8_t)(s | 0x7F);
        return (uint8_t)(s | small_from_abs(a, 3, 7, 0x43E00000u, 0x7E));
    }
    if (a > 0x7F800000u) return (uint8_t)(s | 0x7E);
    return (uint8_t)(s | small_from_abs(a, 2, 15, 0x47600000u, 0x7B));
}

/* FP4 E2M1 code points {0,.5,1,1.5,2,3,4,6}; sign in bit 3; +NaN -> 0x8, -NaN -> 0x0. */
static inline uint8_t f32_to_e2m1_1(uint32_t u) {
    uint32_t s = (u >> 28) & 0x8u;
    uint32_t a = u & 0x7FFFFFFFu;
    if (a > 0x7F800000u) return (uint8_t)(s ^ 0x8u);
    return (uint8_t)(s | small_from_abs(a, 1, 1, 0x40C00000u, 0x7));
}

/* exact fp32 pattern of an FP8 code; NaN codes -> sign|0x7fc00000 */
static inline uint32_t fp8_to_f32_1(uint8_t c, int fmt) {
    uint32_t sign = (uint32_t)(c & 0x80u) << 24;
    uint32_t a = c & 0x7Fu;
    int mbits = fmt == FMT_E4M3 ? 3 : 2, bias = fmt == FMT_E4M3 ? 7 : 15;
    if (fmt == FMT_E4M3 && a == 0x7F) return sign | 0x7FC00000u;
    if (fmt == FMT_E5M2 && a == 0x7C) return sign | 0x7F800000u;
    if (fmt == FMT_E5M2 && a > 0x7C) return sign | 0x7FC00000u;
    uint32_t e = a >> mbits, m = a & ((1u << mbits) - 1);
    if (e == 0) {
        if (m == 0) return sign;
        int s = 0;
        while (!(m & (1u << mbits))) { m <<= 1; s++; }
        return sign | ((uint32_t)(127 + 1 - bias - s) << 23) | ((m & ((1u << mbits) - 1)) << (23 - mbits));
    }
    return sign | ((e + 127 - bias) << 23) | (m << (23 - mbits));
}

static const float E2M1_VAL[16] = {0.f, .5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f,
                                   -0.f, -.5f, -1.f, -1.5f, -2.f, -3.f, -4.f, -6.f};

/* ------------------------------------------------------------------ array API */

void orc_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

int orc_max_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void orc_f32_to_f16(const float* x, uint16_t* out, size_t n) {
    const uint32_t* u = (const uint32_t*)x;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) out[i] = f32_to_f16_1(u[i]);
}

void orc_f16_to_f32(const uint16_t* h, float* out, size_t n) {
    uint32_t* o = (uint32_t*)out;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) o[i] = f16_to_f32_1(h[i]);
}

void orc_f32_to_bf16(const float* x, uint16_t* out, size_t n) {
    const uint32_t* u = (const uint32_t*)x;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) out[i] = f32_to_bf16_1(u[i]);
}

void orc_bf16_to_f32(const uint16_t* b, float* out, size_t n) {
    uint32_t* o = (uint32_t*)out;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) o[i] = (uint32_t)b[i] << 16;
}

/* fp64 -> fp32, bit-identical to NumPy's astype(float32) (the narrowing NovaNN's layers apply
 * to BatchNorm's float64 output, novann/layers/linear/linear.py:81): RNE on the 29 dropped
 * mantissa bits, subnormal results kept, overflow to inf; NaN keeps sign and the top 22
 * payload bits and comes out quiet. */
static inline uint32_t f64_to_f32_1(uint64_t u) {
    uint32_t sign = (uint32_t)(u >> 32) & 0x80000000u;
    uint64_t a = u & 0x7FFFFFFFFFFFFFFFull;
    if (a > 0x7FF0000000000000ull) return sign | 0x7FC00000u | (uint32_t)((a >> 29) & 0x3FFFFFu);
    if (a >= 0x47F0000000000000ull) return sign | 0x7F800000u;
    int e = (int)(a >> 52);
    if (e >= 897) {
        uint64_t h = rne_shift(a - (896ull << 52), 29);
        if (h > 0x7F800000ull) h = 0x7F800000ull;
        return sign | (uint32_t)h;
    }
    if (e == 0) return sign;
    uint64_t m = (a & ((1ull << 52) - 1)) | (1ull << 52);
    return sign | (uint32_t)rne_shift(m, 926 - e);
}

/* fp32 -> fp64: exact; NaN quiet, payload shifted left 29. */
static inline uint64_t f32_to_f64_1(uint32_t u) {
    uint64_t sign = (uint64_t)(u & 0x80000000u) << 32;
    uint32_t e = (u >> 23) & 0xFFu;
    uint64_t m = u & 0x7FFFFFu;
    if (e == 0xFF) return sign | 0x7FF0000000000000ull | (m << 29) | (m ? 0x0008000000000000ull : 0);
    if (e == 0) {
        if (m == 0) return sign;
        int s = 0;
        while (!(m & 0x800000u)) { m <<= 1; s++; }
        return sign | ((uint64_t)(897 - s) << 52) | ((m & 0x7FFFFFu) << 29);
    }
    return sign | ((uint64_t)(e + 896) << 52) | (m << 29);
}

void orc_f64_to_f32(const double* x, float* out, size_t n) {
    const uint64_t* u = (const uint64_t*)x;
    uint32_t* o = (uint32_t*)out;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) o[i] = f64_to_f32_1(u[i]);
}

void orc_f32_to_f64(const float* x, double* out, size_t n) {
    const uint32_t* u = (const uint32_t*)x;
    uint64_t* o = (uint64_t*)out;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) o[i] = f32_to_f64_1(u[i]);
}

/* max |x| with NaNs ignored; exact and order independent (integer max on the
 * magnitudes' bit patterns). */
float orc_amax_f32(const float* x, size_t n) {
    const uint32_t* u = (const uint32_t*)x;
    uint32_t best = 0;
#pragma omp parallel for schedule(static) reduction(max : best)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) {
        uint32_t a = u[i] & 0x7FFFFFFFu;
        if (a <= 0x7F800000u && a > best) best = a;
    }
    return u2f(best);
}

/* q_i = cvt_sat_rne(x_i * inv_scale): ONE fp32 multiply, then the conversion */
void orc_quantize_fp8(const float* x, uint8_t* q, size_t n, float inv_scale, int fmt) {
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) {
        float y = x[i] * inv_scale;
        q[i] = f32_to_fp8_1(f2u(y), fmt);
    }
}

/* x'_i = float(q_i) * scale; NaN codes -> canonical quiet NaN with the code's sign */
void orc_dequantize_fp8(const uint8_t* q, float* x, size_t n, float scale, int fmt) {
    uint32_t lut[256];
    for (int c = 0; c < 256; c++) lut[c] = fp8_to_f32_1((uint8_t)c, fmt);
    uint32_t* o = (uint32_t*)x;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t i = 0; i < (ptrdiff_t)n; i++) {
        uint32_t t = lut[q[i]];
        if ((t & 0x7FFFFFFFu) > 0x7F800000u) o[i] = t;
        else { float y = u2f(t) * scale; o[i] = f2u(y); }
    }
}

/* FP4 E2M1 with one fp32 scale per 32 consecutive elements of a row:
 * amax_b exact (NaN ignored); scale_b = amax_b/6; inv_b = amax_b>0 ? 6/amax_b : 0;
 * code = cvt_sat_rne_e2m1(float(x)*inv_b); byte j = code[2j] | code[2j+1]<<4. */
void orc_quantize_fp4_b32(const uint16_t* x, uint8_t* packed, float* scales, size_t rows,
                          size_t cols) {
    size_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t blk = 0; blk < (ptrdiff_t)(rows * nb); blk++) {
        const uint16_t* p = x + (size_t)blk * 32;
        uint32_t best = 0;
        for (int i = 0; i < 32; i++) {
            uint32_t a = ((uint32_t)p[i] << 16) & 0x7FFFFFFFu;
            if (a <= 0x7F800000u && a > best) best = a;
        }
        float amax = u2f(best);
        float scale = amax / 6.0f;
        float inv = amax > 0.0f ? 6.0f / amax : 0.0f;
        scales[blk] = scale;
        uint8_t* o = packed + (size_t)blk * 16;
        for (int i = 0; i < 16; i++) {
            float y0 = u2f((uint32_t)p[2 * i] << 16) * inv;
            float y1 = u2f((uint32_t)p[2 * i + 1] << 16) * inv;
            o[i] = (uint8_t)(f32_to_e2m1_1(f2u(y0)) | (f32_to_e2m1_1(f2u(y1)) << 4));
        }
    }
}

/* bf16_rne(e2m1_value(code) * scale_b) */
void orc_dequantize_fp4_b32(const uint8_t* packed, const float* scales, uint16_t* out,
                            size_t rows, size_t cols) {
    size_t nb = cols / 32;
#pragma omp parallel for schedule(static)
    for (ptrdiff_t blk = 0; blk < (ptrdiff_t)(rows * nb); blk++) {
        const uint8_t* p = packed + (size_t)blk * 16;
        float s = scales[blk];
        uint16_t* o = out + (size_t)blk * 32;
        for (int i = 0; i < 16; i++) {
            float y0 = E2M1_VAL[p[i] & 0xF] * s;
            float y1 = E2M1_VAL[p[i] >> 4] * s;
            o[2 * i] = f32_to_bf16_1(f2u(y0));
            o[2 * i + 1] = f32_to_bf16_1(f2u(y1));
        }
    }
}

/* scalar helpers for exhaustive single-code checks */
uint8_t orc_f32_bits_to_fp8(uint32_t u, int fmt) { return f32_to_fp8_1(u, fmt); }
uint8_t orc_f32_bits_to_e2m1(uint32_t u) { return f32_to_e2m1_1(u); }
uint32_t orc_fp8_to_f32_bits(uint8_t c, int fmt) { return fp8_to_f32_1(c, fmt); }
