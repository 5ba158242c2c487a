/*
 *  TEST INFRASTRUCTURE ONLY. Compiled against the upstream NumKong headers where they lie (never copied):
 *  exports the x86 SIMD back ends of the packed 16-bit float kernels one by one, under refb_<backend>_* names,
 *  so the tests can measure the error of EVERY reference back end this CPU can run (the envelope the device
 *  kernels are held to), not only that of the one the dispatcher picks. Built by `make -C oracle ref` into
 *  oracle/_ref/libnkref_backends.so. The caller checks nk_capabilities() of the dispatch library before it calls
 *  a back end; the AMX one needs nk_configure_thread on the calling thread first.
 */
#include <numkong/numkong.h>

#define REFB_API __attribute__((visibility("default")))

#define REFB_FAMILY(BACKEND, T, IN)                                                                                   \
    REFB_API nk_size_t refb_##BACKEND##_dots_packed_size_##T(nk_size_t n, nk_size_t k) {                              \
        return nk_dots_packed_size_##T##_##BACKEND(n, k);                                                             \
    }                                                                                                                 \
    REFB_API void refb_##BACKEND##_dots_pack_##T(IN const *b, nk_size_t n, nk_size_t k, nk_size_t s, void *p) {       \
        nk_dots_pack_##T##_##BACKEND(b, n, k, s, p);                                                                  \
    }                                                                                                                 \
    REFB_API void refb_##BACKEND##_dots_packed_##T(IN const *a, void const *p, nk_f32_t *c, nk_size_t m, nk_size_t n, \
                                                   nk_size_t k, nk_size_t as, nk_size_t cs) {                         \
        nk_dots_packed_##T##_##BACKEND(a, p, c, m, n, k, as, cs);                                                     \
    }                                                                                                                 \
    REFB_API void refb_##BACKEND##_angulars_packed_##T(IN const *a, void const *p, nk_f32_t *c, nk_size_t m,          \
                                                       nk_size_t n, nk_size_t k, nk_size_t as, nk_size_t cs) {        \
        nk_angulars_packed_##T##_##BACKEND(a, p, c, m, n, k, as, cs);                                                 \
    }                                                                                                                 \
    REFB_API void refb_##BACKEND##_euclideans_packed_##T(IN const *a, void const *p, nk_f32_t *c, nk_size_t m,        \
                                                         nk_size_t n, nk_size_t k, nk_size_t as, nk_size_t cs) {      \
        nk_euclideans_packed_##T##_##BACKEND(a, p, c, m, n, k, as, cs);                                               \
    }

REFB_FAMILY(serial, bf16, nk_bf16_t)
REFB_FAMILY(serial, f16, nk_f16_t)
REFB_FAMILY(haswell, bf16, nk_bf16_t)
REFB_FAMILY(haswell, f16, nk_f16_t)
REFB_FAMILY(skylake, bf16, nk_bf16_t)
REFB_FAMILY(skylake, f16, nk_f16_t)
REFB_FAMILY(genoa, bf16, nk_bf16_t)
REFB_FAMILY(sapphireamx, bf16, nk_bf16_t)

REFB_API nk_u64_t refb_capabilities(void) { return nk_capabilities(); }
REFB_API int refb_configure_thread(nk_u64_t caps) { return nk_configure_thread(caps); }
