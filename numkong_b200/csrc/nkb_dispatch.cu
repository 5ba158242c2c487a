// Run-time kernel lookup for bindings that fetch function pointers instead of linking symbols
// (NumKong's Python and JavaScript modules do: python/matrix.c:430-437, javascript/numkong.c:398-463).
// Same contract as nk_find_kernel_punned (c/numkong.c:848-913): a known (kind, dtype) pair yields the
// entry point and a non-zero capability bit, anything else yields NULL and 0.
#include "../../include/numkong_b200.h"

namespace {

struct Entry {
    int kind;
    uint32_t dtype;
    void *fn;
};

#define NKB_PACKED_ENTRIES(T, DT)                                                                  \
    {'P', DT, (void *)&nk_dots_packed_size_##T}, {'Q', DT, (void *)&nk_dots_pack_##T},            \
    {'G', DT, (void *)&nk_dots_packed_##T}, {'N', DT, (void *)&nk_angulars_packed_##T},           \
    {'E', DT, (void *)&nk_euclideans_packed_##T}, {'y', DT, (void *)&nk_dots_symmetric_##T},      \
    {'n', DT, (void *)&nk_angulars_symmetric_##T}, {'D', DT, (void *)&nk_euclideans_symmetric_##T}
#define NKB_MAXSIM_ENTRIES(T, DT)                                                                  \
    {'L', DT, (void *)&nk_maxsim_packed_size_##T}, {'l', DT, (void *)&nk_maxsim_pack_##T},        \
    {'T', DT, (void *)&nk_maxsim_packed_##T}

const Entry kTable[] = {
    NKB_PACKED_ENTRIES(i8, NKB_DTYPE_I8),     NKB_PACKED_ENTRIES(u8, NKB_DTYPE_U8),
    NKB_PACKED_ENTRIES(bf16, NKB_DTYPE_BF16), NKB_PACKED_ENTRIES(f16, NKB_DTYPE_F16),
    NKB_PACKED_ENTRIES(e4m3, NKB_DTYPE_E4M3), NKB_PACKED_ENTRIES(e5m2, NKB_DTYPE_E5M2),
    NKB_PACKED_ENTRIES(e2m3, NKB_DTYPE_E2M3), NKB_PACKED_ENTRIES(e3m2, NKB_DTYPE_E3M2),
    NKB_PACKED_ENTRIES(f32, NKB_DTYPE_F32),   NKB_PACKED_ENTRIES(i4, NKB_DTYPE_I4),
    NKB_PACKED_ENTRIES(u4, NKB_DTYPE_U4),     NKB_PACKED_ENTRIES(f64, NKB_DTYPE_F64),
    {'P', NKB_DTYPE_U1, (void *)&nk_dots_packed_size_u1}, {'Q', NKB_DTYPE_U1, (void *)&nk_dots_pack_u1},
    {'G', NKB_DTYPE_U1, (void *)&nk_dots_packed_u1}, {'y', NKB_DTYPE_U1, (void *)&nk_dots_symmetric_u1},
    {'M', NKB_DTYPE_U1, (void *)&nk_hammings_packed_u1}, {'Y', NKB_DTYPE_U1, (void *)&nk_hammings_symmetric_u1},
    {'p', NKB_DTYPE_U1, (void *)&nk_jaccards_packed_u1}, {'Z', NKB_DTYPE_U1, (void *)&nk_jaccards_symmetric_u1},
    NKB_MAXSIM_ENTRIES(bf16, NKB_DTYPE_BF16), NKB_MAXSIM_ENTRIES(f16, NKB_DTYPE_F16),
    NKB_MAXSIM_ENTRIES(f32, NKB_DTYPE_F32),
    // Moments under kind 'R' (nk_kernel_reduce_moments_k, include/numkong/capabilities.h:225), one per element type, with the
    // numeric values of nk_dtype_t (types.h:923-953) for the integer widths the packed families do not use.
    {'R', NKB_DTYPE_F64, (void *)&nk_reduce_moments_f64},   {'R', NKB_DTYPE_F32, (void *)&nk_reduce_moments_f32},
    {'R', NKB_DTYPE_F16, (void *)&nk_reduce_moments_f16},   {'R', NKB_DTYPE_BF16, (void *)&nk_reduce_moments_bf16},
    {'R', NKB_DTYPE_E4M3, (void *)&nk_reduce_moments_e4m3}, {'R', NKB_DTYPE_E5M2, (void *)&nk_reduce_moments_e5m2},
    {'R', NKB_DTYPE_E2M3, (void *)&nk_reduce_moments_e2m3}, {'R', NKB_DTYPE_E3M2, (void *)&nk_reduce_moments_e3m2},
    {'R', NKB_DTYPE_I8, (void *)&nk_reduce_moments_i8},     {'R', NKB_DTYPE_U8, (void *)&nk_reduce_moments_u8},
    {'R', 1u << 3, (void *)&nk_reduce_moments_i16},         {'R', 1u << 7, (void *)&nk_reduce_moments_u16},
    {'R', 1u << 4, (void *)&nk_reduce_moments_i32},         {'R', 1u << 8, (void *)&nk_reduce_moments_u32},
    {'R', 1u << 5, (void *)&nk_reduce_moments_i64},         {'R', 1u << 9, (void *)&nk_reduce_moments_u64},
    {'R', NKB_DTYPE_I4, (void *)&nk_reduce_moments_i4},     {'R', NKB_DTYPE_U4, (void *)&nk_reduce_moments_u4},
    {'R', NKB_DTYPE_U1, (void *)&nk_reduce_moments_u1},
    // Bulk conversion under kind '-' with the "unknown" element type 0, which is how the reference's lookup reaches nk_cast
    // (nk_kernel_cast_k, capabilities.h:251; c/numkong.c:897).
    {'-', 0u, (void *)&nk_cast},
};

} // namespace

extern "C" NKB_API void nk_find_kernel_punned(int kind, uint32_t dtype, uint64_t viable_capabilities, void **kernel_output,
                                              uint64_t *capability_output) {
    void *fn = nullptr;
    if (viable_capabilities & NKB_CAPABILITY_B200)
        for (const Entry &e : kTable)
            if (e.kind == kind && e.dtype == dtype) { fn = e.fn; break; }
    if (kernel_output) *kernel_output = fn;
    if (capability_output) *capability_output = fn ? NKB_CAPABILITY_B200 : 0;
}
