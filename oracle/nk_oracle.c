/*
 *  TEST INFRASTRUCTURE ONLY. CPU restatement of NumKong v7.6.0's packed-contraction path, used as the
 *  checker for the CUDA kernels. Nothing the library ships imports, links or runs this file; only
 *  tests/, __graft_entry__.smoke() and bench.py's CPU-baseline leg do.
 *
 *  Parity status: PINNED. tests/test_oracle_pins.py checks every function below against
 *  (a) golden vectors generated from the reference's own kernels (tests/golden/, script committed
 *  beside them) and (b), when oracle/_ref/libnumkong.so is present, the reference library itself
 *  on fresh seeded inputs: bit-exact against its *_serial kernels wherever those are deterministic
 *  functions of the inputs (all dots, distances, norms), within a stated tolerance where the
 *  reference routes through run-time dispatched helpers (MaxSim refinement).
 *
 *  Each function cites the reference source it restates (paths inside the NumKong tree).
 *  Plain scalar C, compiled with -ffp-contract=off so no product is fused into a sum behind our back.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_API __attribute__((visibility("default")))

/* dtype codes, numerically nk_dtype_t (include/numkong/types.h:923-953) */
enum {
    ORC_I8 = 1 << 2, ORC_U8 = 1 << 6, ORC_F32 = 1 << 11, ORC_F16 = 1 << 12, ORC_BF16 = 1 << 13,
    ORC_E4M3 = 1 << 14, ORC_E5M2 = 1 << 15, ORC_E2M3 = 1 << 18, ORC_E3M2 = 1 << 19,
    ORC_I4 = 1 << 16, ORC_U4 = 1 << 17, /* two values per byte, low nibble first; depth counts values */
    ORC_U1 = 1 << 1,                    /* eight values per byte; depth counts bits */
    ORC_F64 = 1 << 10,
};
#define ORC_IS_INT(dt) ((dt) == ORC_I8 || (dt) == ORC_U8 || (dt) == ORC_I4 || (dt) == ORC_U4 || (dt) == ORC_U1)
#define ORC_IS_SIGNED_INT(dt) ((dt) == ORC_I8 || (dt) == ORC_I4)

static float bits_to_f32(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
static uint32_t f32_to_bits(float f) { uint32_t u; memcpy(&u, &f, 4); return u; }

/* ---- element decoders: value semantics of include/numkong/cast/serial.h ---------------------- */

/* bf16 is the upper half of an f32 (cast/serial.h:750-760). */
static float dec_bf16(const uint8_t *p) { return bits_to_f32(((uint32_t)p[0] << 16) | ((uint32_t)p[1] << 24)); }

/* IEEE binary16 (cast/serial.h:586-). */
static float dec_f16(const uint8_t *p) {
    uint32_t h = (uint32_t)p[0] | ((uint32_t)p[1] << 8);
    uint32_t sign = (h & 0x8000u) << 16, exp = (h >> 10) & 0x1fu, man = h & 0x3ffu;
    if (exp == 0) {
        float v = ldexpf((float)man, -24);
        return sign ? -v : v;
    }
    if (exp == 31) return bits_to_f32(sign | 0x7f800000u | (man << 13));
    return bits_to_f32(sign | ((exp + 112u) << 23) | (man << 13));
}

/* e4m3fn: bias 7, subnormals m/512, no infinities, NaN only at 0x7F / 0xFF (cast/serial.h:810-839). */
static float dec_e4m3(const uint8_t *p) {
    uint32_t b = p[0], exp = (b >> 3) & 0xfu, man = b & 7u;
    float v;
    if (exp == 15 && man == 7) return bits_to_f32(0x7fc00000u);
    if (exp == 0) v = ldexpf((float)man, -9);
    else v = ldexpf(1.0f + (float)man / 8.0f, (int)exp - 7);
    return (b & 0x80u) ? -v : v;
}

/* e5m2: the top byte of a binary16, inf/NaN included (cast/serial.h:1042-). */
static float dec_e5m2(const uint8_t *p) {
    uint8_t h[2] = {0, p[0]};
    return dec_f16(h);
}

/* e2m3: 0b00SEEMMM, bias 1, subnormals m/8, max 7.5, no inf/NaN (cast/serial.h:1318-1330). */
static float dec_e2m3(const uint8_t *p) {
    uint32_t b = p[0], exp = (b >> 3) & 3u, man = b & 7u;
    float v = exp == 0 ? (float)man / 8.0f : ldexpf(1.0f + (float)man / 8.0f, (int)exp - 1);
    return (b & 0x20u) ? -v : v;
}

/* e3m2: 0b00SEEEMM, bias 3, subnormals m/16, max 28, no inf/NaN (cast/serial.h:1455-1471). */
static float dec_e3m2(const uint8_t *p) {
    uint32_t b = p[0], exp = (b >> 2) & 7u, man = b & 3u;
    float v = exp == 0 ? (float)man / 16.0f : ldexpf(1.0f + (float)man / 4.0f, (int)exp - 3);
    return (b & 0x20u) ? -v : v;
}

static int elem_bytes(int dt) { return dt == ORC_F64 ? 8 : dt == ORC_F32 ? 4 : (dt == ORC_F16 || dt == ORC_BF16) ? 2 : 1; }

static float dec(int dt, const uint8_t *p) {
    switch (dt) {
    case ORC_BF16: return dec_bf16(p);
    case ORC_F16: return dec_f16(p);
    case ORC_E4M3: return dec_e4m3(p);
    case ORC_E5M2: return dec_e5m2(p);
    case ORC_E2M3: return dec_e2m3(p);
    case ORC_E3M2: return dec_e3m2(p);
    case ORC_I8: return (float)(int8_t)p[0];
    case ORC_U8: return (float)p[0];
    default: { float f; memcpy(&f, p, 4); return f; }
    }
}

ORC_API void orc_decode(int dt, const void *src, uint64_t count, float *dst) {
    const uint8_t *p = (const uint8_t *)src;
    int eb = elem_bytes(dt);
    for (uint64_t i = 0; i < count; ++i) dst[i] = dec(dt, p + i * eb);
}

/* ---- scalar helpers --------------------------------------------------------------------------- */

/* Bit-trick reciprocal square root with three Newton steps (include/numkong/scalar/serial.h:22-31). */
static float rsqrt_f32(float x) {
    float y = bits_to_f32(0x5F375A86u - (f32_to_bits(x) >> 1));
    y = y * (1.5f - 0.5f * x * y * y);
    y = y * (1.5f - 0.5f * x * y * y);
    y = y * (1.5f - 0.5f * x * y * y);
    return y;
}
/* scalar/serial.h:33 */
static float sqrt_f32(float x) { return x > 0 ? x * rsqrt_f32(x) : 0; }

/* scalar/serial.h:35-46: four Newton steps in f64 */
static double rsqrt_f64(double x) {
    uint64_t u; memcpy(&u, &x, 8);
    u = 0x5FE6EB50C7B537A9ull - (u >> 1);
    double y; memcpy(&y, &u, 8);
    for (int i = 0; i < 4; ++i) y = y * (1.5 - 0.5 * x * y * y);
    return y;
}
static double sqrt_f64(double x) { return x > 0 ? x * rsqrt_f64(x) : 0; }

ORC_API float orc_rsqrt_f32(float x) { return rsqrt_f32(x); }

/* ---- one dot product with the serial kernels' accumulation order ------------------------------
 * Sub-32-bit floats: four f32 lanes, lane (l mod 4) takes element l in order, lanes added 0+1+2+3
 * (include/numkong/dot/serial.h:341-374 f16, :376-404 through-f32, :406-439 bf16, :522-680 fp8/fp6).
 * f32: same with f64 lanes (dot/serial.h:305-335). i8/u8: two i64 lanes (even/odd), truncated to 32 bits
 * (dot/serial.h:445-479, :481-516). Zero padding of the packed depth adds exact zeros and is omitted.
 */
static float dot_f32lanes(int dt, const uint8_t *a, const uint8_t *b, uint64_t k) {
    int eb = elem_bytes(dt);
    float s[4] = {0, 0, 0, 0};
    for (uint64_t l = 0; l < k; ++l) s[l & 3] += dec(dt, a + l * eb) * dec(dt, b + l * eb);
    return s[0] + s[1] + s[2] + s[3];
}
static double dot_f64lanes(const uint8_t *a, const uint8_t *b, uint64_t k) {
    double s[4] = {0, 0, 0, 0};
    for (uint64_t l = 0; l < k; ++l) {
        float x, y; memcpy(&x, a + 4 * l, 4); memcpy(&y, b + 4 * l, 4);
        s[l & 3] += (double)x * y;
    }
    return s[0] + s[1] + s[2] + s[3];
}
/* 4-bit values: low nibble first, signed ones through (x ^ 8) - 8 (include/numkong/types.h:1551-1558). The depth is
 * rounded up to a whole byte, so both nibbles of the last byte always count (include/numkong/dot/serial.h:185-215). */
static int nibble(int dt, uint8_t byte, int high) {
    int x = high ? (byte >> 4) & 0xf : byte & 0xf;
    return dt == ORC_I4 ? (x ^ 8) - 8 : x;
}
/* f64 inputs: Dot2 - error-free product (FMA) and error-free sum (TwoSum), the errors gathered in a compensation term
 * (include/numkong/scalar/serial.h:128-136) - in two lanes, even and odd depth indices (dot/serial.h:274-296), folded by
 * the compensated lane reduction of include/numkong/reduce/serial.h:33-48. */
static void dot2(double *sum, double *compensation, double a, double b) {
    double product = a * b;
    double product_error = fma(a, b, -product);
    double running_sum = *sum + product;
    double recovered_addend = running_sum - *sum;
    double sum_error = (*sum - (running_sum - recovered_addend)) + (product - recovered_addend);
    *sum = running_sum;
    *compensation += sum_error + product_error;
}
static double dot_f64_dot2(const uint8_t *a, const uint8_t *b, uint64_t k) {
    double sums[2] = {0, 0}, comps[2] = {0, 0};
    for (uint64_t l = 0; l < k; ++l) {
        double x, y; memcpy(&x, a + 8 * l, 8); memcpy(&y, b + 8 * l, 8);
        dot2(&sums[l & 1], &comps[l & 1], x, y);
    }
    double running_sum = 0, accumulated_error = 0;
    for (int i = 0; i < 2; ++i) {
        double parts[2] = {sums[i], comps[i]};
        for (int p = 0; p < 2; ++p) {
            double tentative_sum = running_sum + parts[p];
            double virtual_addend = tentative_sum - running_sum;
            accumulated_error += (running_sum - (tentative_sum - virtual_addend)) + (parts[p] - virtual_addend);
            running_sum = tentative_sum;
        }
    }
    return running_sum + accumulated_error;
}
static int64_t dot_int(int dt, const uint8_t *a, const uint8_t *b, uint64_t k) {
    int64_t s = 0;
    if (dt == ORC_U1) { /* AND-popcount over whole bytes (include/numkong/dots/serial.h u1 instantiation, set/serial.h) */
        for (uint64_t l = 0; l < (k + 7) / 8; ++l) s += __builtin_popcount((unsigned)(a[l] & b[l]));
        return s;
    }
    if (dt == ORC_I4 || dt == ORC_U4) {
        for (uint64_t l = 0; l < (k + 1) / 2; ++l)
            s += (int64_t)nibble(dt, a[l], 0) * nibble(dt, b[l], 0) + (int64_t)nibble(dt, a[l], 1) * nibble(dt, b[l], 1);
        return s;
    }
    if (dt == ORC_I8) for (uint64_t l = 0; l < k; ++l) s += (int64_t)(int8_t)a[l] * (int8_t)b[l];
    else for (uint64_t l = 0; l < k; ++l) s += (int64_t)a[l] * b[l];
    return s;
}

/* C = A . B^T, overwriting C (include/numkong/dots/serial.h:520-1085; output types dot.h:633-654). */
ORC_API void orc_dots(int dt, const void *a, uint64_t a_stride, const void *b, uint64_t b_stride, void *c,
                      uint64_t c_stride, uint64_t m, uint64_t n, uint64_t k) {
    const uint8_t *ap = (const uint8_t *)a, *bp = (const uint8_t *)b;
    for (uint64_t i = 0; i < m; ++i) {
        uint8_t *row = (uint8_t *)c + i * c_stride;
        for (uint64_t j = 0; j < n; ++j) {
            const uint8_t *x = ap + i * a_stride, *y = bp + j * b_stride;
            if (ORC_IS_INT(dt)) ((int32_t *)row)[j] = (int32_t)dot_int(dt, x, y, k);
            else if (dt == ORC_F32) ((double *)row)[j] = dot_f64lanes(x, y, k);
            else if (dt == ORC_F64) ((double *)row)[j] = dot_f64_dot2(x, y, k);
            else ((float *)row)[j] = dot_f32lanes(dt, x, y, k);
        }
    }
}

/* ---- squared norms as the serial pack stores them ---------------------------------------------
 * Floats below 32 bits: compensated (Neumaier) f32 running sum of v*v
 * (include/numkong/reduce/serial.h:248-272 and siblings). f32: the same in f64. i8/u8: exact, truncated to u32
 * (dots/serial.h:159-170). Used for the norms appended by pack (dots/serial.h:326-332) and for the
 * per-query norm of the batched distances (dots/serial.h:2775-2778).
 */
static float sumsq_f32_neumaier(int dt, const uint8_t *x, uint64_t k) {
    int eb = elem_bytes(dt);
    float run = 0, comp = 0;
    for (uint64_t l = 0; l < k; ++l) {
        float v = dec(dt, x + l * eb), sq = v * v, t = run + sq;
        if (run >= sq) comp += (run - t) + sq; else comp += (sq - t) + run;
        run = t;
    }
    return run + comp;
}
ORC_API double orc_sumsq(int dt, const void *x, uint64_t k) {
    const uint8_t *p = (const uint8_t *)x;
    if (ORC_IS_INT(dt)) return (double)(uint32_t)(uint64_t)dot_int(dt, p, p, k);
    if (dt == ORC_F32 || dt == ORC_F64) {
        /* the same compensated sum carried in f64 (reduce/serial.h:50-92) */
        double run = 0, comp = 0;
        for (uint64_t l = 0; l < k; ++l) {
            double v;
            if (dt == ORC_F32) { float f; memcpy(&f, p + 4 * l, 4); v = f; } else memcpy(&v, p + 8 * l, 8);
            double sq = v * v, t = run + sq;
            if (run >= sq) comp += (run - t) + sq; else comp += (sq - t) + run;
            run = t;
        }
        return run + comp;
    }
    return (double)sumsq_f32_neumaier(dt, p, k);
}

/* ---- batched distances: GEMM, then the from-dot finalisers ------------------------------------
 * include/numkong/dots/serial.h:2756-2800 drives; formulas include/numkong/spatial/serial.h:257-350.
 * kind 0 = angular, 1 = euclidean. Output f32 (f64 for f32 inputs).
 */
static float angular_from_dot_f32(float dot, float an, float bn) {
    float product = an * bn;
    if (product > 0) {
        float r = 1.0f - dot * rsqrt_f32(product);
        return r > 0 ? r : 0;
    }
    return dot == 0 ? 0.0f : 1.0f;
}
static float euclidean_from_dot_f32(float dot, float an, float bn) {
    float d2 = an + bn - 2.0f * dot;
    return d2 > 0 ? sqrt_f32(d2) : 0.0f;
}
ORC_API void orc_spatials(int kind, int dt, const void *a, uint64_t a_stride, const void *b, uint64_t b_stride, void *c,
                          uint64_t c_stride, uint64_t m, uint64_t n, uint64_t k) {
    const uint8_t *ap = (const uint8_t *)a, *bp = (const uint8_t *)b;
    double *bn = (double *)malloc(sizeof(double) * (n ? n : 1));
    for (uint64_t j = 0; j < n; ++j) bn[j] = orc_sumsq(dt, bp + j * b_stride, k);
    for (uint64_t i = 0; i < m; ++i) {
        uint8_t *row = (uint8_t *)c + i * c_stride;
        const uint8_t *x = ap + i * a_stride;
        double an = orc_sumsq(dt, x, k);
        for (uint64_t j = 0; j < n; ++j) {
            const uint8_t *y = bp + j * b_stride;
            if (dt == ORC_F32 || dt == ORC_F64) {
                double dot = dt == ORC_F32 ? dot_f64lanes(x, y, k) : dot_f64_dot2(x, y, k), r;
                if (kind == 0) {
                    double product = an * bn[j];
                    if (product > 0) { r = 1.0 - dot * rsqrt_f64(product); r = r > 0 ? r : 0; }
                    else r = dot == 0 ? 0.0 : 1.0;
                } else {
                    double d2 = an + bn[j] - 2.0 * dot;
                    r = d2 > 0 ? sqrt_f64(d2) : 0.0;
                }
                ((double *)row)[j] = r;
            } else {
                float dot, fa, fb;
                if (ORC_IS_SIGNED_INT(dt)) { dot = (float)(int32_t)dot_int(dt, x, y, k); fa = (float)(int32_t)(uint32_t)an; fb = (float)(int32_t)(uint32_t)bn[j]; }
                else if (dt == ORC_U8 || dt == ORC_U4) { dot = (float)(uint32_t)dot_int(dt, x, y, k); fa = (float)(uint32_t)an; fb = (float)(uint32_t)bn[j]; }
                else { dot = dot_f32lanes(dt, x, y, k); fa = (float)an; fb = (float)bn[j]; }
                ((float *)row)[j] = kind == 0 ? angular_from_dot_f32(dot, fa, fb) : euclidean_from_dot_f32(dot, fa, fb);
            }
        }
    }
    free(bn);
}

/* ---- set distances of one-bit vectors --------------------------------------------------------------
 * include/numkong/sets/serial.h:19-39 drives (AND-popcount product, population counts as norms); formulas
 * include/numkong/set/serial.h:150-168. kind 0 = Hamming (u32 cells), 1 = Jaccard (f32 cells).
 */
ORC_API void orc_sets(int kind, const void *a, uint64_t a_stride, const void *b, uint64_t b_stride, void *c, uint64_t c_stride,
                      uint64_t m, uint64_t n, uint64_t k) {
    const uint8_t *ap = (const uint8_t *)a, *bp = (const uint8_t *)b;
    for (uint64_t i = 0; i < m; ++i) {
        const uint8_t *x = ap + i * a_stride;
        uint32_t pa = (uint32_t)dot_int(ORC_U1, x, x, k);
        uint8_t *row = (uint8_t *)c + i * c_stride;
        for (uint64_t j = 0; j < n; ++j) {
            const uint8_t *y = bp + j * b_stride;
            uint32_t pb = (uint32_t)dot_int(ORC_U1, y, y, k), dot = (uint32_t)dot_int(ORC_U1, x, y, k);
            if (kind == 0) ((uint32_t *)row)[j] = pa + pb - 2 * dot;
            else {
                float fdot = (float)dot, union_size = (float)pa + (float)pb - fdot;
                ((float *)row)[j] = union_size != 0 ? 1.0f - fdot / union_size : 0.0f;
            }
        }
    }
}

/* ---- in-place down-casts of a finished dots matrix ---------------------------------------------------
 * include/numkong/dots/serial.h:2707-2724 (f32 -> bf16, rounding of include/numkong/cast/serial.h:768-784) and
 * :2726-2754 (i32 -> i8 rescaled by 127 / (|a| |b|)). Rows are read `stride` bytes apart and written tightly packed
 * from the first byte of the same buffer, row by row, cell by cell, so a cell is always read before it is overwritten.
 */
ORC_API void orc_compact_bf16(void *c, uint64_t rows, uint64_t cols, uint64_t stride) {
    for (uint64_t i = 0; i < rows; ++i)
        for (uint64_t j = 0; j < cols; ++j) {
            uint32_t u; memcpy(&u, (const uint8_t *)c + i * stride + j * 4, 4);
            u += 0x7FFFu + ((u >> 16) & 1u);
            uint16_t h = (uint16_t)(u >> 16);
            memcpy((uint8_t *)c + (i * cols + j) * 2, &h, 2);
        }
}

ORC_API void orc_compact_i8(void *c, uint64_t rows, uint64_t cols, uint64_t stride, const int32_t *a_norms, const int32_t *b_norms) {
    for (uint64_t i = 0; i < rows; ++i) {
        float an = (float)a_norms[i], a_r = an > 0 ? 1.0f / sqrt_f32(an) : 0.0f;
        for (uint64_t j = 0; j < cols; ++j) {
            float bn = (float)b_norms[j], b_r = bn > 0 ? 1.0f / sqrt_f32(bn) : 0.0f;
            int32_t v; memcpy(&v, (const uint8_t *)c + i * stride + j * 4, 4);
            float scaled = (float)v * 127.0f * a_r * b_r;
            int32_t q = (int32_t)scaled;
            if (q < -128) q = -128;
            if (q > 127) q = 127;
            ((int8_t *)c)[i * cols + j] = (int8_t)q;
        }
    }
}

/* ---- MaxSim ------------------------------------------------------------------------------------
 * Inverse norm stored by pack: plain f32 running sum of v*v, then the bit-trick rsqrt, 0 for a zero
 * vector (include/numkong/maxsim/serial.h:122-141, :263).
 */
static float inverse_norm(int dt, const uint8_t *x, uint64_t k) {
    int eb = elem_bytes(dt);
    float s = 0;
    for (uint64_t l = 0; l < k; ++l) { float v = dec(dt, x + l * eb); s += v * v; }
    return s > 0 ? rsqrt_f32(s) : 0.0f;
}

/* Fused semantics of the tensor-engine back end (include/numkong/maxsim/sapphireamx.h:716-861), which the
 * CUDA kernel follows: for every query vector the FIRST document vector with the largest raw dot wins
 * (strict >, running maximum starts at the lowest finite f32); only the winner is normalised:
 * cosine = dot * inv|q| * inv|d|, angular = max(0, 1 - cosine); angulars are added in f64 and the sum is
 * returned (callers cast to f32 for bf16/f16). `best` (optional) receives the winning document indices.
 */
ORC_API double orc_maxsim_argmax_dot(int dt, const void *q, uint64_t q_stride, uint64_t nq, const void *d,
                                     uint64_t d_stride, uint64_t nd, uint64_t k, uint32_t *best) {
    const uint8_t *qp = (const uint8_t *)q, *dp = (const uint8_t *)d;
    float *inv_d = (float *)malloc(sizeof(float) * (nd ? nd : 1));
    for (uint64_t j = 0; j < nd; ++j) inv_d[j] = inverse_norm(dt, dp + j * d_stride, k);
    double total = 0;
    for (uint64_t i = 0; i < nq; ++i) {
        const uint8_t *x = qp + i * q_stride;
        uint32_t arg = 0;
        if (dt == ORC_F32) {
            /* f32 inputs keep the dot, the cosine and the angular in f64 (maxsim/serial.h:443-455). */
            double run = -1.7976931348623157e308;
            for (uint64_t j = 0; j < nd; ++j) {
                double dot = dot_f64lanes(x, dp + j * d_stride, k);
                if (dot > run) { run = dot; arg = (uint32_t)j; }
            }
            double angular = 1.0 - run * (double)inverse_norm(dt, x, k) * (double)inv_d[arg];
            total += angular < 0 ? 0 : angular;
        } else {
            float run = -3.402823466e+38f;
            for (uint64_t j = 0; j < nd; ++j) {
                float dot = dot_f32lanes(dt, x, dp + j * d_stride, k);
                if (dot > run) { run = dot; arg = (uint32_t)j; }
            }
            float cosine = run * inverse_norm(dt, x, k) * inv_d[arg];
            float angular = 1.0f - cosine;
            if (angular < 0) angular = 0;
            total += (double)angular;
        }
        if (best) best[i] = arg;
    }
    free(inv_d);
    return total;
}

/* Exhaustive definition the reference tests compare against (include/numkong/maxsim.hpp:82-110):
 * sum over queries of the minimum true angular distance, everything in f64. */
ORC_API double orc_maxsim_exhaustive(int dt, const void *q, uint64_t q_stride, uint64_t nq, const void *d,
                                     uint64_t d_stride, uint64_t nd, uint64_t k) {
    const uint8_t *qp = (const uint8_t *)q, *dp = (const uint8_t *)d;
    int eb = elem_bytes(dt);
    double total = 0;
    for (uint64_t i = 0; i < nq; ++i) {
        double best = 1.7976931348623157e308;
        for (uint64_t j = 0; j < nd; ++j) {
            double ab = 0, aa = 0, bb = 0;
            for (uint64_t l = 0; l < k; ++l) {
                double x = dec(dt, qp + i * q_stride + l * eb), y = dec(dt, dp + j * d_stride + l * eb);
                ab += x * y; aa += x * x; bb += y * y;
            }
            double ang;
            if (aa == 0 && bb == 0) ang = 0;
            else if (ab == 0) ang = 1;
            else { ang = 1.0 - ab / (sqrt(aa) * sqrt(bb)); if (ang < 0) ang = 0; }
            if (ang < best) best = ang;
        }
        total += best;
    }
    return total;
}

/* Serial back end of MaxSim (include/numkong/maxsim/serial.h:122-167 quantiser, :331-390 coarse argmax,
 * :392-424 refinement): per-vector symmetric i8 quantisation (scale = absmax/127, round half away from
 * zero), argmax of the i8 dot (strict >, first wins), winner re-scored with the full-precision dot. The
 * reference refines with its run-time dispatched 1-to-1 dot, so only the winners are bit-pinned; the
 * returned sum is compared with a tolerance. `best` receives the winners.
 */
ORC_API double orc_maxsim_coarse_i8(int dt, const void *q, uint64_t q_stride, uint64_t nq, const void *d,
                                    uint64_t d_stride, uint64_t nd, uint64_t k, uint32_t *best) {
    const uint8_t *qp = (const uint8_t *)q, *dp = (const uint8_t *)d;
    int eb = elem_bytes(dt);
    int8_t *qi = (int8_t *)malloc((nq ? nq : 1) * (k ? k : 1)), *di = (int8_t *)malloc((nd ? nd : 1) * (k ? k : 1));
    for (int side = 0; side < 2; ++side) {
        const uint8_t *src = side ? dp : qp;
        uint64_t cnt = side ? nd : nq, stride = side ? d_stride : q_stride;
        int8_t *dst = side ? di : qi;
        for (uint64_t v = 0; v < cnt; ++v) {
            float absmax = 0;
            for (uint64_t l = 0; l < k; ++l) { float x = fabsf(dec(dt, src + v * stride + l * eb)); if (x > absmax) absmax = x; }
            float scale = absmax / 127.0f;
            if (scale == 0) scale = 1.0f;
            for (uint64_t l = 0; l < k; ++l) {
                float s = dec(dt, src + v * stride + l * eb) / scale;
                int32_t z = s >= 0 ? (int32_t)(s + 0.5f) : (int32_t)(s - 0.5f);
                if (z > 127) z = 127;
                if (z < -127) z = -127;
                dst[v * k + l] = (int8_t)z;
            }
        }
    }
    double total = 0;
    for (uint64_t i = 0; i < nq; ++i) {
        int32_t run = INT32_MIN;
        uint32_t arg = 0;
        for (uint64_t j = 0; j < nd; ++j) {
            int32_t acc = 0;
            for (uint64_t l = 0; l < k; ++l) acc += (int32_t)qi[i * k + l] * (int32_t)di[j * k + l];
            if (acc > run) { run = acc; arg = (uint32_t)j; }
        }
        const uint8_t *x = qp + i * q_stride, *y = dp + arg * d_stride;
        if (dt == ORC_F32) {
            double angular = 1.0 - dot_f64lanes(x, y, k) * (double)inverse_norm(dt, x, k) * (double)inverse_norm(dt, y, k);
            total += angular < 0 ? 0 : angular;
        } else {
            float cosine = dot_f32lanes(dt, x, y, k) * inverse_norm(dt, x, k) * inverse_norm(dt, y, k);
            float angular = 1.0f - cosine;
            if (angular < 0) angular = 0;
            total += (double)angular;
        }
        if (best) best[i] = arg;
    }
    free(qi); free(di);
    return total;
}

/* ---- multi-threaded driver for the CPU-baseline timing (rows of A split across threads, as the
 * reference's callers do: README.md:199-212) is in Python (threads release the GIL inside ctypes). */

/* ---- bulk type conversion --------------------------------------------------------------------------
 * Restates nk_cast_serial (include/numkong/cast/serial.h:2250-2311): equal types are copied; two unsigned
 * integer types go through u64, two integer types with a signed one through i64, everything else through f64.
 * Values travel in batches of eight. Sub-byte conventions of the cast (cast/serial.h:1846-1871, :1966-1995):
 * u1 is most-significant-bit first, i4 / u4 keep the even index in the HIGH nibble - unlike the dots family.
 *
 * Narrowing rules restated:
 *   float -> f32: C cast of the f64 hub value; -> f16 / bf16 / e4m3 / e5m2 / e2m3 / e3m2: that f32, then round to
 *     nearest even onto the format's grid. e4m3 saturates at +-448 (infinity too) and keeps NaN as 0x7F | sign
 *     (cast/serial.h:866-943); e5m2 overflows to infinity, NaN is 0x7D | sign (:1108-1188); e2m3 / e3m2 saturate
 *     at +-7.5 / +-28, NaN included (:1340-1416, :1481-1560); f16 is IEEE (:669-741), bf16 too (:768-784).
 *   float -> integer: NaN gives 0, the value is clamped to the target range and rounded to nearest even
 *     (cast/serial.h:1583-1666). float -> i4 / u4: clamped, then truncated toward zero (:1973-1995); float -> u1:
 *     non-zero gives 1.
 *   integer -> integer: saturating; a u64 source that meets a signed type is first reinterpreted as i64
 *     (cast/serial.h:2043-2046), so values >= 2^63 come out as the target's minimum.
 * Pairs the reference leaves undefined (u1 -> signed integers; signed integers -> u4 / u1; complex types)
 * return 0 and write nothing. Tails: only whole result bytes that hold a converted value are written, missing
 * values of a partial sub-byte batch count as 0.
 */
enum { ORC_I16 = 1 << 3, ORC_I32 = 1 << 4, ORC_I64 = 1 << 5, ORC_U16 = 1 << 7, ORC_U32 = 1 << 8, ORC_U64 = 1 << 9 };
enum { FAMILY_NONE = 0, FAMILY_FLOAT, FAMILY_INT, FAMILY_UINT };

static int cast_family(int dt) {
    switch (dt) {
    case ORC_F64: case ORC_F32: case ORC_F16: case ORC_BF16: case ORC_E4M3: case ORC_E5M2: case ORC_E2M3: case ORC_E3M2: return FAMILY_FLOAT;
    case ORC_I4: case ORC_I8: case ORC_I16: case ORC_I32: case ORC_I64: return FAMILY_INT;
    case ORC_U1: case ORC_U4: case ORC_U8: case ORC_U16: case ORC_U32: case ORC_U64: return FAMILY_UINT;
    default: return FAMILY_NONE;
    }
}
static int cast_bits(int dt) {
    switch (dt) {
    case ORC_F64: case ORC_I64: case ORC_U64: return 64;
    case ORC_F32: case ORC_I32: case ORC_U32: return 32;
    case ORC_F16: case ORC_BF16: case ORC_I16: case ORC_U16: return 16;
    case ORC_I4: case ORC_U4: return 4;
    case ORC_U1: return 1;
    default: return cast_family(dt) == FAMILY_NONE ? 0 : 8;
    }
}

/* Round-to-nearest-even of an f32 onto a small binary format: `man_bits` fraction bits, exponent `bias`; returns the
 * magnitude code, possibly above the format's largest one (the caller applies the overflow rule). */
static uint32_t round_to_grid(uint32_t abs_bits, int man_bits, int bias) {
    int e = (int)(abs_bits >> 23) - 127, emin = 1 - bias;
    if ((abs_bits >> 23) == 0) return 0;                       /* f32 subnormals are far below every grid */
    uint32_t sig = 0x800000u | (abs_bits & 0x7fffffu);
    int shift = 23 - man_bits + (e < emin ? emin - e : 0);
    uint32_t r = 0;
    if (shift <= 24) {
        uint32_t rem = sig & ((1u << shift) - 1), half = 1u << (shift - 1);
        r = sig >> shift;
        if (rem > half || (rem == half && (r & 1))) ++r;
    }
    return ((uint32_t)(e < emin ? 0 : e - emin) << man_bits) + r;
}

static uint16_t enc_f16(float x) {
    uint32_t u = f32_to_bits(x), sign = (u >> 16) & 0x8000u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint16_t)(sign | 0x7e00u);
    if (a == 0x7f800000u || (int)(a >> 23) - 127 > 16) return (uint16_t)(sign | 0x7c00u);
    uint32_t code = round_to_grid(a, 10, 15);
    return (uint16_t)(sign | (code > 0x7c00u ? 0x7c00u : code));
}
static uint16_t enc_bf16(float x) {
    uint32_t u = f32_to_bits(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40u);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
static uint8_t enc_e4m3(float x) {
    uint32_t u = f32_to_bits(x), sign = (u >> 24) & 0x80u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7fu);
    if ((int)(a >> 23) - 127 > 9) return (uint8_t)(sign | 0x7eu);
    uint32_t code = round_to_grid(a, 3, 7);
    return (uint8_t)(sign | (code > 0x7eu ? 0x7eu : code));
}
static uint8_t enc_e5m2(float x) {
    uint32_t u = f32_to_bits(x), sign = (u >> 24) & 0x80u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return (uint8_t)(sign | 0x7du);
    if ((int)(a >> 23) - 127 > 16) return (uint8_t)(sign | 0x7cu);
    uint32_t code = round_to_grid(a, 2, 15);
    return (uint8_t)(sign | (code > 0x7cu ? 0x7cu : code));
}
static uint8_t enc_fp6(float x, int man_bits, int bias) {
    uint32_t u = f32_to_bits(x), sign = (u >> 26) & 0x20u, a = u & 0x7fffffffu;
    if ((int)(a >> 23) - 127 > 5) return (uint8_t)(sign | 0x1fu);   /* far above the range, infinities and NaN */
    uint32_t code = round_to_grid(a, man_bits, bias);
    return (uint8_t)(sign | (code > 0x1fu ? 0x1fu : code));
}

static double rint_even(double x) {  /* cast/serial.h:1583-1596, for |x| < 2^63 */
    double t = trunc(x), f = x - t;
    if (f > 0.5 || (f == 0.5 && fmod(t, 2.0) != 0.0)) return t + 1.0;
    if (f < -0.5 || (f == -0.5 && fmod(t, 2.0) != 0.0)) return t - 1.0;
    return t;
}
static double clamp_f64(double x, double lo, double hi) { return x > hi ? hi : (x < lo ? lo : x); }

static double load_f64(int dt, const uint8_t *p) {
    switch (dt) {
    case ORC_F64: { double v; memcpy(&v, p, 8); return v; }
    case ORC_I64: { int64_t v; memcpy(&v, p, 8); return (double)v; }
    case ORC_U64: { uint64_t v; memcpy(&v, p, 8); return (double)v; }
    case ORC_I32: { int32_t v; memcpy(&v, p, 4); return (double)v; }
    case ORC_U32: { uint32_t v; memcpy(&v, p, 4); return (double)v; }
    case ORC_I16: { int16_t v; memcpy(&v, p, 2); return (double)v; }
    case ORC_U16: { uint16_t v; memcpy(&v, p, 2); return (double)v; }
    default: return (double)dec(dt, p);   /* f32 and the small floats (through f32), i8, u8 */
    }
}
static void store_f64(int dt, double v, uint8_t *p) {
    float f = (float)v;
    switch (dt) {
    case ORC_F64: memcpy(p, &v, 8); break;
    case ORC_F32: memcpy(p, &f, 4); break;
    case ORC_F16: { uint16_t h = enc_f16(f); memcpy(p, &h, 2); } break;
    case ORC_BF16: { uint16_t h = enc_bf16(f); memcpy(p, &h, 2); } break;
    case ORC_E4M3: p[0] = enc_e4m3(f); break;
    case ORC_E5M2: p[0] = enc_e5m2(f); break;
    case ORC_E2M3: p[0] = enc_fp6(f, 3, 1); break;
    case ORC_E3M2: p[0] = enc_fp6(f, 2, 3); break;
    case ORC_I8: { int8_t o = v != v ? 0 : (int8_t)rint_even(clamp_f64(v, -128.0, 127.0)); memcpy(p, &o, 1); } break;
    case ORC_U8: { uint8_t o = v != v ? 0 : (uint8_t)rint_even(clamp_f64(v, 0.0, 255.0)); memcpy(p, &o, 1); } break;
    case ORC_I16: { int16_t o = v != v ? 0 : (int16_t)rint_even(clamp_f64(v, -32768.0, 32767.0)); memcpy(p, &o, 2); } break;
    case ORC_U16: { uint16_t o = v != v ? 0 : (uint16_t)rint_even(clamp_f64(v, 0.0, 65535.0)); memcpy(p, &o, 2); } break;
    case ORC_I32: { int32_t o = v != v ? 0 : (int32_t)rint_even(clamp_f64(v, -2147483648.0, 2147483647.0)); memcpy(p, &o, 4); } break;
    case ORC_U32: { uint32_t o = v != v ? 0 : (uint32_t)rint_even(clamp_f64(v, 0.0, 4294967295.0)); memcpy(p, &o, 4); } break;
    case ORC_I64: {  /* values at or beyond +-2^63 saturate (the reference leaves the upper end to the C cast) */
        int64_t o = v != v ? 0 : v >= 9223372036854775808.0 ? INT64_MAX : v <= -9223372036854775808.0 ? INT64_MIN : (int64_t)rint_even(v);
        memcpy(p, &o, 8);
    } break;
    case ORC_U64: {
        uint64_t o = v != v || v <= 0 ? 0 : v >= 18446744073709551616.0 ? UINT64_MAX
                     : (v < 9007199254740992.0 ? (uint64_t)rint_even(v) : (uint64_t)v);
        memcpy(p, &o, 8);
    } break;
    }
}
static int64_t load_i64(int dt, const uint8_t *p) {
    switch (dt) {
    case ORC_I64: case ORC_U64: { int64_t v; memcpy(&v, p, 8); return v; }   /* u64: reinterpreted */
    case ORC_I32: { int32_t v; memcpy(&v, p, 4); return v; }
    case ORC_U32: { uint32_t v; memcpy(&v, p, 4); return v; }
    case ORC_I16: { int16_t v; memcpy(&v, p, 2); return v; }
    case ORC_U16: { uint16_t v; memcpy(&v, p, 2); return v; }
    case ORC_I8: return (int8_t)p[0];
    default: return p[0];
    }
}
static int64_t clamp_i64(int64_t x, int64_t lo, int64_t hi) { return x > hi ? hi : (x < lo ? lo : x); }
static void store_i64(int dt, int64_t v, uint8_t *p) {
    switch (dt) {
    case ORC_I64: memcpy(p, &v, 8); break;
    case ORC_U64: { uint64_t o = v < 0 ? 0 : (uint64_t)v; memcpy(p, &o, 8); } break;
    case ORC_I32: { int32_t o = (int32_t)clamp_i64(v, INT32_MIN, INT32_MAX); memcpy(p, &o, 4); } break;
    case ORC_U32: { uint32_t o = (uint32_t)clamp_i64(v, 0, UINT32_MAX); memcpy(p, &o, 4); } break;
    case ORC_I16: { int16_t o = (int16_t)clamp_i64(v, INT16_MIN, INT16_MAX); memcpy(p, &o, 2); } break;
    case ORC_U16: { uint16_t o = (uint16_t)clamp_i64(v, 0, UINT16_MAX); memcpy(p, &o, 2); } break;
    case ORC_I8: { int8_t o = (int8_t)clamp_i64(v, INT8_MIN, INT8_MAX); memcpy(p, &o, 1); } break;
    case ORC_U8: p[0] = (uint8_t)clamp_i64(v, 0, UINT8_MAX); break;
    }
}
static uint64_t load_u64(int dt, const uint8_t *p) {
    switch (dt) {
    case ORC_U64: { uint64_t v; memcpy(&v, p, 8); return v; }
    case ORC_U32: { uint32_t v; memcpy(&v, p, 4); return v; }
    case ORC_U16: { uint16_t v; memcpy(&v, p, 2); return v; }
    default: return p[0];
    }
}
static void store_u64(int dt, uint64_t v, uint8_t *p) {
    switch (dt) {
    case ORC_U64: memcpy(p, &v, 8); break;
    case ORC_U32: { uint32_t o = v > UINT32_MAX ? UINT32_MAX : (uint32_t)v; memcpy(p, &o, 4); } break;
    case ORC_U16: { uint16_t o = v > UINT16_MAX ? UINT16_MAX : (uint16_t)v; memcpy(p, &o, 2); } break;
    case ORC_U8: p[0] = v > UINT8_MAX ? UINT8_MAX : (uint8_t)v; break;
    }
}

ORC_API int orc_cast(const void *from, int from_type, uint64_t n, void *to, int to_type) {
    const int from_family = cast_family(from_type), to_family = cast_family(to_type);
    const int from_bits = cast_bits(from_type), to_bits = cast_bits(to_type);
    if (!from_family || !to_family) return 0;
    if (from_type == to_type) { memcpy(to, from, (n * (uint64_t)from_bits + 7) / 8); return 1; }
    const int hub = (from_family == FAMILY_UINT && to_family == FAMILY_UINT) ? FAMILY_UINT
                    : (from_family != FAMILY_FLOAT && to_family != FAMILY_FLOAT) ? FAMILY_INT : FAMILY_FLOAT;
    if (hub == FAMILY_INT && (from_type == ORC_U1 || to_type == ORC_U4 || to_type == ORC_U1)) return 0;
    const uint8_t *src = (const uint8_t *)from;
    uint8_t *dst = (uint8_t *)to;
    for (uint64_t first = 0; first < n; first += 8) {
        const int count = n - first < 8 ? (int)(n - first) : 8;
        const uint8_t *s = src + first * (uint64_t)from_bits / 8;
        uint8_t *d = dst + first * (uint64_t)to_bits / 8;
        double f[8] = {0}; int64_t i[8] = {0}; uint64_t u[8] = {0};
        for (int l = 0; l < count; ++l) {
            int64_t small = 0;   /* value of a sub-byte source element */
            if (from_type == ORC_U1) small = (s[0] >> (7 - l)) & 1;
            else if (from_type == ORC_U4) small = (l & 1) ? (s[l / 2] & 0xF) : (s[l / 2] >> 4);
            else if (from_type == ORC_I4) { small = (l & 1) ? (s[l / 2] & 0xF) : (s[l / 2] >> 4); small = (small ^ 8) - 8; }
            if (from_bits < 8) f[l] = (double)small, i[l] = small, u[l] = (uint64_t)small;
            else if (hub == FAMILY_FLOAT) f[l] = load_f64(from_type, s + l * (from_bits / 8));
            else if (hub == FAMILY_INT) i[l] = load_i64(from_type, s + l * (from_bits / 8));
            else u[l] = load_u64(from_type, s + l * (from_bits / 8));
        }
        if (to_bits >= 8) {
            for (int l = 0; l < count; ++l) {
                uint8_t *cell = d + l * (to_bits / 8);
                if (hub == FAMILY_FLOAT) store_f64(to_type, f[l], cell);
                else if (hub == FAMILY_INT) store_i64(to_type, i[l], cell);
                else store_u64(to_type, u[l], cell);
            }
            continue;
        }
        uint8_t bytes[4] = {0, 0, 0, 0};
        for (int l = 0; l < count; ++l) {
            if (to_type == ORC_U1) bytes[0] |= (uint8_t)((hub == FAMILY_FLOAT ? f[l] != 0 : u[l] != 0) << (7 - l));
            else {
                int64_t v;
                if (to_type == ORC_I4) v = hub == FAMILY_FLOAT ? (int64_t)(int8_t)clamp_f64(f[l], -8.0, 7.0) : clamp_i64(i[l], -8, 7);
                else v = hub == FAMILY_FLOAT ? (int64_t)(uint8_t)clamp_f64(f[l], 0.0, 15.0) : (int64_t)(u[l] > 15 ? 15 : u[l]);
                bytes[l / 2] |= (uint8_t)((v & 0xF) << ((l & 1) ? 0 : 4));
            }
        }
        memcpy(d, bytes, ((uint64_t)count * (uint64_t)to_bits + 7) / 8);
    }
    return 1;
}

/* ---- moments: sum and sum of squares of a strided vector ----------------------------------------------
 * Restates nk_reduce_moments_<t>_serial (include/numkong/reduce/serial.h:52-416).
 *   f32 / f64: every value widened to f64, Neumaier-compensated running sums of the values and of their rounded
 *     squares, result = running + compensation (:52-94). f16 bf16 e4m3 e5m2 e2m3 e3m2: the same in f32 (:232-371).
 *   i8 u8 i16 u16 i4 u4 u1: plain 64-bit sums (:96-146, :373-416); sub-byte types count whole bytes, `stride`
 *     steps from byte to byte. i32 / i64: the sum is kept in 128 bits and saturated to i64 at the end; squares (for
 *     i64 saturated at 2^63 - 1) are added with unsigned saturation (:148-167, :182-205). u32 / u64: saturating
 *     unsigned sums of values and (saturated) squares (:169-180, :207-219).
 * `sum` and `sumsq` receive 8 bytes each: f64, or an f32 in the first four bytes, or i64 / u64.
 */
static uint64_t sat_add_u64(uint64_t a, uint64_t b) { return a + b < a ? UINT64_MAX : a + b; }
static uint64_t sat_square_u64(uint64_t a) { unsigned __int128 p = (unsigned __int128)a * a; return p > UINT64_MAX ? UINT64_MAX : (uint64_t)p; }

ORC_API int orc_moments(int dt, const void *data, uint64_t count, uint64_t stride, void *sum_out, void *sumsq_out) {
    const uint8_t *p = (const uint8_t *)data;
    if (dt == ORC_F64 || dt == ORC_F32) {
        double s = 0, sc = 0, q = 0, qc = 0;
        for (uint64_t i = 0; i < count; ++i, p += stride) {
            double v;
            if (dt == ORC_F64) memcpy(&v, p, 8); else { float f; memcpy(&f, p, 4); v = (double)f; }
            double t = s + v;
            if (fabs(s) >= fabs(v)) sc += (s - t) + v; else sc += (v - t) + s;
            s = t;
            double sq = v * v, tq = q + sq;
            if (q >= sq) qc += (q - tq) + sq; else qc += (sq - tq) + q;
            q = tq;
        }
        double rs = s + sc, rq = q + qc;
        memcpy(sum_out, &rs, 8); memcpy(sumsq_out, &rq, 8);
        return 1;
    }
    if (cast_family(dt) == FAMILY_FLOAT) {
        float s = 0, sc = 0, q = 0, qc = 0;
        for (uint64_t i = 0; i < count; ++i, p += stride) {
            float v = dec(dt, p), t = s + v;
            if (fabsf(s) >= fabsf(v)) sc += (s - t) + v; else sc += (v - t) + s;
            s = t;
            float sq = v * v, tq = q + sq;
            if (q >= sq) qc += (q - tq) + sq; else qc += (sq - tq) + q;
            q = tq;
        }
        float rs = s + sc, rq = q + qc;
        memset(sum_out, 0, 8); memset(sumsq_out, 0, 8);
        memcpy(sum_out, &rs, 4); memcpy(sumsq_out, &rq, 4);
        return 1;
    }
    if (dt == ORC_U1 || dt == ORC_I4 || dt == ORC_U4) {
        const uint64_t bytes = dt == ORC_U1 ? (count + 7) / 8 : (count + 1) / 2;
        int64_t s = 0; uint64_t q = 0;
        for (uint64_t i = 0; i < bytes; ++i, p += stride) {
            if (dt == ORC_U1) { int c = __builtin_popcount(p[0]); s += c; q += (uint64_t)c; continue; }
            int64_t lo = p[0] & 0xF, hi = p[0] >> 4;
            if (dt == ORC_I4) lo = (lo ^ 8) - 8, hi = (hi ^ 8) - 8;
            s += lo + hi; q += (uint64_t)(lo * lo) + (uint64_t)(hi * hi);
        }
        memcpy(sum_out, &s, 8); memcpy(sumsq_out, &q, 8);
        return 1;
    }
    if (cast_family(dt) == FAMILY_INT) {
        __int128 s = 0; uint64_t q = 0;
        for (uint64_t i = 0; i < count; ++i, p += stride) {
            int64_t v = load_i64(dt, p);
            s += v;
            if (dt == ORC_I64) { uint64_t a = v < 0 ? 0 - (uint64_t)v : (uint64_t)v, sq = sat_square_u64(a); q = sat_add_u64(q, sq > INT64_MAX ? INT64_MAX : sq); }
            else if (dt == ORC_I32) q = sat_add_u64(q, (uint64_t)(v * v));
            else q += (uint64_t)(v * v);
        }
        int64_t rs = (dt == ORC_I32 || dt == ORC_I64) ? (s > INT64_MAX ? INT64_MAX : s < INT64_MIN ? INT64_MIN : (int64_t)s) : (int64_t)s;
        memcpy(sum_out, &rs, 8); memcpy(sumsq_out, &q, 8);
        return 1;
    }
    if (cast_family(dt) == FAMILY_UINT) {
        uint64_t s = 0, q = 0;
        for (uint64_t i = 0; i < count; ++i, p += stride) {
            uint64_t v = load_u64(dt, p);
            if (dt == ORC_U32 || dt == ORC_U64) s = sat_add_u64(s, v), q = sat_add_u64(q, sat_square_u64(v));
            else s += v, q += v * v;
        }
        memcpy(sum_out, &s, 8); memcpy(sumsq_out, &q, 8);
        return 1;
    }
    return 0;
}
