/*
 *  TEST INFRASTRUCTURE ONLY. Compiled against the upstream NumKong headers where they lie (never copied):
 *  exports the header-only *_serial kernels of the packed-contraction path under ref_* names, so the tests
 *  can pin oracle/nk_oracle.c bit-for-bit against the reference's own scalar back end. Built by
 *  `make -C oracle ref` into oracle/_ref/libnkref_serial.so.
 */
#include <numkong/numkong.h>

#define REF_API __attribute__((visibility("default")))

#define REF_PACKED_FAMILY(T, IN, OUT, DOUT)                                                                          \
    REF_API nk_size_t ref_dots_packed_size_##T(nk_size_t n, nk_size_t k) { return nk_dots_packed_size_##T##_serial(n, k); } \
    REF_API void ref_dots_pack_##T(IN const *b, nk_size_t n, nk_size_t k, nk_size_t s, void *p) {                     \
        nk_dots_pack_##T##_serial(b, n, k, s, p);                                                                     \
    }                                                                                                                 \
    REF_API void ref_dots_packed_##T(IN const *a, void const *p, OUT *c, nk_size_t m, nk_size_t n, nk_size_t k,       \
                                     nk_size_t as, nk_size_t cs) {                                                    \
        nk_dots_packed_##T##_serial(a, p, c, m, n, k, as, cs);                                                        \
    }                                                                                                                 \
    REF_API void ref_angulars_packed_##T(IN const *a, void const *p, DOUT *c, nk_size_t m, nk_size_t n, nk_size_t k,  \
                                         nk_size_t as, nk_size_t cs) {                                                \
        nk_angulars_packed_##T##_serial(a, p, c, m, n, k, as, cs);                                                    \
    }                                                                                                                 \
    REF_API void ref_euclideans_packed_##T(IN const *a, void const *p, DOUT *c, nk_size_t m, nk_size_t n,             \
                                           nk_size_t k, nk_size_t as, nk_size_t cs) {                                 \
        nk_euclideans_packed_##T##_serial(a, p, c, m, n, k, as, cs);                                                  \
    }

REF_PACKED_FAMILY(i8, nk_i8_t, nk_i32_t, nk_f32_t)
REF_PACKED_FAMILY(u8, nk_u8_t, nk_u32_t, nk_f32_t)
REF_PACKED_FAMILY(bf16, nk_bf16_t, nk_f32_t, nk_f32_t)
REF_PACKED_FAMILY(f16, nk_f16_t, nk_f32_t, nk_f32_t)
REF_PACKED_FAMILY(e4m3, nk_e4m3_t, nk_f32_t, nk_f32_t)
REF_PACKED_FAMILY(e5m2, nk_e5m2_t, nk_f32_t, nk_f32_t)
REF_PACKED_FAMILY(e2m3, nk_e2m3_t, nk_f32_t, nk_f32_t)
REF_PACKED_FAMILY(e3m2, nk_e3m2_t, nk_f32_t, nk_f32_t)
REF_PACKED_FAMILY(f32, nk_f32_t, nk_f64_t, nk_f64_t)
REF_PACKED_FAMILY(i4, nk_i4x2_t, nk_i32_t, nk_f32_t)
REF_PACKED_FAMILY(u4, nk_u4x2_t, nk_u32_t, nk_f32_t)
REF_PACKED_FAMILY(f64, nk_f64_t, nk_f64_t, nk_f64_t)

/* one-bit vectors: AND-popcount product and the two set distances */
REF_API nk_size_t ref_dots_packed_size_u1(nk_size_t n, nk_size_t k) { return nk_dots_packed_size_u1_serial(n, k); }
REF_API void ref_dots_pack_u1(nk_u1x8_t const *b, nk_size_t n, nk_size_t k, nk_size_t s, void *p) { nk_dots_pack_u1_serial(b, n, k, s, p); }
REF_API void ref_dots_packed_u1(nk_u1x8_t const *a, void const *p, nk_u32_t *c, nk_size_t m, nk_size_t n, nk_size_t k, nk_size_t as, nk_size_t cs) {
    nk_dots_packed_u1_serial(a, p, c, m, n, k, as, cs);
}
REF_API void ref_hammings_packed_u1(nk_u1x8_t const *a, void const *p, nk_u32_t *c, nk_size_t m, nk_size_t n, nk_size_t k, nk_size_t as, nk_size_t cs) {
    nk_hammings_packed_u1_serial(a, p, c, m, n, k, as, cs);
}
REF_API void ref_jaccards_packed_u1(nk_u1x8_t const *a, void const *p, nk_f32_t *c, nk_size_t m, nk_size_t n, nk_size_t k, nk_size_t as, nk_size_t cs) {
    nk_jaccards_packed_u1_serial(a, p, c, m, n, k, as, cs);
}

/* in-place down-casts of a finished dots matrix (header-level helpers, not part of the dispatch table) */
REF_API void ref_dots_compact_bf16(void *c, nk_size_t rows, nk_size_t cols, nk_size_t stride) { nk_dots_compact_bf16_serial(c, rows, cols, stride); }
REF_API void ref_dots_compact_i8(void *c, nk_size_t rows, nk_size_t cols, nk_size_t stride, nk_i32_t const *an, nk_i32_t const *bn) {
    nk_dots_compact_i8_serial(c, rows, cols, stride, an, bn);
}

/* bulk type conversion, scalar back end */
REF_API void ref_cast(void const *from, int from_type, nk_size_t n, void *to, int to_type) { nk_cast_serial(from, (nk_dtype_t)from_type, n, to, (nk_dtype_t)to_type); }

/* moments (sum, sum of squares), scalar back end */
#define REF_MOMENTS(T, IN, SUM, SQ)                                                                                  \
    REF_API void ref_reduce_moments_##T(IN const *x, nk_size_t n, nk_size_t stride, SUM *s, SQ *q) {                 \
        nk_reduce_moments_##T##_serial(x, n, stride, s, q);                                                          \
    }
REF_MOMENTS(f64, nk_f64_t, nk_f64_t, nk_f64_t)
REF_MOMENTS(f32, nk_f32_t, nk_f64_t, nk_f64_t)
REF_MOMENTS(f16, nk_f16_t, nk_f32_t, nk_f32_t)
REF_MOMENTS(bf16, nk_bf16_t, nk_f32_t, nk_f32_t)
REF_MOMENTS(e4m3, nk_e4m3_t, nk_f32_t, nk_f32_t)
REF_MOMENTS(e5m2, nk_e5m2_t, nk_f32_t, nk_f32_t)
REF_MOMENTS(e2m3, nk_e2m3_t, nk_f32_t, nk_f32_t)
REF_MOMENTS(e3m2, nk_e3m2_t, nk_f32_t, nk_f32_t)
REF_MOMENTS(i8, nk_i8_t, nk_i64_t, nk_u64_t)
REF_MOMENTS(u8, nk_u8_t, nk_u64_t, nk_u64_t)
REF_MOMENTS(i16, nk_i16_t, nk_i64_t, nk_u64_t)
REF_MOMENTS(u16, nk_u16_t, nk_u64_t, nk_u64_t)
REF_MOMENTS(i32, nk_i32_t, nk_i64_t, nk_u64_t)
REF_MOMENTS(u32, nk_u32_t, nk_u64_t, nk_u64_t)
REF_MOMENTS(i64, nk_i64_t, nk_i64_t, nk_u64_t)
REF_MOMENTS(u64, nk_u64_t, nk_u64_t, nk_u64_t)
REF_MOMENTS(i4, nk_i4x2_t, nk_i64_t, nk_u64_t)
REF_MOMENTS(u4, nk_u4x2_t, nk_u64_t, nk_u64_t)
REF_MOMENTS(u1, nk_u1x8_t, nk_u64_t, nk_u64_t)

#define REF_MAXSIM_FAMILY(T, IN, OUT)                                                                                \
    REF_API nk_size_t ref_maxsim_packed_size_##T(nk_size_t n, nk_size_t k) { return nk_maxsim_packed_size_##T##_serial(n, k); } \
    REF_API void ref_maxsim_pack_##T(IN const *v, nk_size_t n, nk_size_t k, nk_size_t s, void *p) {                   \
        nk_maxsim_pack_##T##_serial(v, n, k, s, p);                                                                   \
    }                                                                                                                 \
    REF_API void ref_maxsim_packed_##T(void const *q, void const *d, nk_size_t nq, nk_size_t nd, nk_size_t k, OUT *r) { \
        nk_maxsim_packed_##T##_serial(q, d, nq, nd, k, r);                                                            \
    }

REF_MAXSIM_FAMILY(bf16, nk_bf16_t, nk_f32_t)
REF_MAXSIM_FAMILY(f16, nk_f16_t, nk_f32_t)
REF_MAXSIM_FAMILY(f32, nk_f32_t, nk_f64_t)

REF_API float ref_rsqrt_f32(float x) { return nk_f32_rsqrt_serial(x); }
REF_API void ref_sumsq_bf16(nk_bf16_t const *x, nk_size_t n, float *out) { float s; nk_reduce_moments_bf16_serial(x, n, 2, &s, out); }
REF_API void ref_sumsq_f16(nk_f16_t const *x, nk_size_t n, float *out) { float s; nk_reduce_moments_f16_serial(x, n, 2, &s, out); }
REF_API void ref_sumsq_e4m3(nk_e4m3_t const *x, nk_size_t n, float *out) { float s; nk_reduce_moments_e4m3_serial(x, n, 1, &s, out); }
