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
