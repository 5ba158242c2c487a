/**
 *  @file numkong_b200.h
 *  @brief C ABI of libnumkong_b200.so: NumKong's packed-contraction entry points, executed on an
 *         NVIDIA B200 (sm_100a). Plain pointers and sizes only.
 *
 *  The `nk_*` functions below keep the exact names, argument order and argument meaning of
 *  NumKong v7.6.0, so a binding that resolves them by symbol (Rust `extern "C"`, Swift, cgo,
 *  ctypes) or through `nk_find_kernel_punned` needs no source change. The reference declaration
 *  each one stands in for is cited next to it (paths inside the NumKong tree).
 *
 *  Conventions kept from the reference:
 *   - row-major matrices, `C[i,j] = sum_l A[i,l] * B[j,l]`, all strides in BYTES (dots.h:60-72);
 *   - the caller owns every buffer; `packed_size` is a pure function of (width, depth);
 *   - the packed blob is opaque and position independent (it may be memcpy'd, moved, saved);
 *   - functions return void; on failure the output is filled with 0xFF bytes (c/numkong.c:78-81)
 *     and `nkb_last_error()` explains why; `packed_size` returns 0 for an unsupported call.
 *
 *  Pointer kinds: every pointer may be device memory, managed memory, pinned host memory or
 *  ordinary host memory, mixed freely. Device/managed operands are used in place and the call is
 *  asynchronous on the thread's stream (`nkb_set_stream`); when any operand lives in host memory
 *  the library stages it through device buffers it owns and the call returns with the result
 *  complete. A host-resident packed blob is uploaded once and its device copy is reused by later
 *  calls ("pack once, query many").
 *
 *  Element types: nk_bf16_t / nk_f16_t are 16-bit storage words, e4m3 / e5m2 / e2m3 / e3m2 one
 *  byte per value (FP6 as 0b00SEEMMM / 0b00SEEEMM, types.h:785-861). They are `void` here so the
 *  header stands alone; the dtype codes equal nk_dtype_t (types.h:923-953).
 */
#ifndef NUMKONG_B200_H_
#define NUMKONG_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#if defined(__GNUC__)
#define NKB_API __attribute__((visibility("default")))
#else
#define NKB_API
#endif

typedef uint64_t nk_size_t; /* types.h:854-856 */

/* dtype codes, numerically nk_dtype_t (types.h:923-953) */
#define NKB_DTYPE_U1 (1u << 1) /* eight values per byte; `depth` counts bits */
#define NKB_DTYPE_I8 (1u << 2)
#define NKB_DTYPE_U8 (1u << 6)
#define NKB_DTYPE_F64 (1u << 10)
#define NKB_DTYPE_F32 (1u << 11)
#define NKB_DTYPE_F16 (1u << 12)
#define NKB_DTYPE_BF16 (1u << 13)
#define NKB_DTYPE_E4M3 (1u << 14)
#define NKB_DTYPE_E5M2 (1u << 15)
#define NKB_DTYPE_I4 (1u << 16) /* two values per byte, low nibble first; `depth` counts values */
#define NKB_DTYPE_U4 (1u << 17)
#define NKB_DTYPE_E2M3 (1u << 18)
#define NKB_DTYPE_E3M2 (1u << 19)

/* ---- packed GEMM: size / pack / multiply ------------------------------------------------------
 * nk_dots_packed_size_<t>  replaces include/numkong/dots.h:177-201   (wrappers c/numkong.c:628-644)
 * nk_dots_pack_<t>         replaces include/numkong/dots.h:211-246   (wrappers c/numkong.c:646-665)
 * nk_dots_packed_<t>       replaces include/numkong/dots.h:259-296   (wrappers c/numkong.c:667-694)
 * Output cell type: i32 (i8), u32 (u8), f64 (f32), f32 otherwise (include/numkong/dot.h:633-654).
 * nk_angulars_packed_<t> / nk_euclideans_packed_<t> replace include/numkong/spatials.h:72-
 * (wrappers c/numkong.c:696-736); output f64 for f32 inputs, f32 otherwise (spatial.h:836-890).
 */
#define NKB_DECLARE_PACKED_FAMILY(T)                                                                                   \
    NKB_API nk_size_t nk_dots_packed_size_##T(nk_size_t width, nk_size_t depth);                                       \
    NKB_API void nk_dots_pack_##T(void const *b, nk_size_t width, nk_size_t depth, nk_size_t b_stride,                 \
                                  void *b_packed);                                                                     \
    NKB_API void nk_dots_packed_##T(void const *a, void const *b_packed, void *c, nk_size_t height, nk_size_t width,   \
                                    nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride);                          \
    NKB_API void nk_angulars_packed_##T(void const *a, void const *b_packed, void *c, nk_size_t height,                \
                                        nk_size_t width, nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride);     \
    NKB_API void nk_euclideans_packed_##T(void const *a, void const *b_packed, void *c, nk_size_t height,              \
                                          nk_size_t width, nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride);

NKB_DECLARE_PACKED_FAMILY(i8)
NKB_DECLARE_PACKED_FAMILY(u8)
NKB_DECLARE_PACKED_FAMILY(bf16)
NKB_DECLARE_PACKED_FAMILY(f16)
NKB_DECLARE_PACKED_FAMILY(e4m3)
NKB_DECLARE_PACKED_FAMILY(e5m2)
NKB_DECLARE_PACKED_FAMILY(e2m3)
NKB_DECLARE_PACKED_FAMILY(e3m2)
NKB_DECLARE_PACKED_FAMILY(f32)
NKB_DECLARE_PACKED_FAMILY(i4) /* include/numkong/dots.h:197,239,289; both nibbles of the last byte count (dot/serial.h:185-215) */
NKB_DECLARE_PACKED_FAMILY(u4)
NKB_DECLARE_PACKED_FAMILY(f64) /* f64 cells; dots accumulate with the reference's two-lane Dot2 (dot/serial.h:274-303): bit-identical */

/* ---- symmetric products A x A^T and the distance matrices built on them ----------------------------
 * nk_dots_symmetric_<t>        replaces include/numkong/dots.h:309-359      (wrappers c/numkong.c:673-686)
 * nk_angulars_symmetric_<t> / nk_euclideans_symmetric_<t> replace include/numkong/spatials.h:77-
 * (generator include/numkong/dots/serial.h:2802-2872). Only rows [row_start, row_start + row_count) are touched and of
 * those only the cells with column >= row; the rest of `result` is left as it was. Dots put the squared norm on the
 * diagonal, the distances put 0 there. Cell types as for the packed family.
 */
#define NKB_DECLARE_SYMMETRIC_FAMILY(T)                                                                                \
    NKB_API void nk_dots_symmetric_##T(void const *vectors, nk_size_t vectors_count, nk_size_t depth, nk_size_t stride, \
                                       void *result, nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count); \
    NKB_API void nk_angulars_symmetric_##T(void const *vectors, nk_size_t vectors_count, nk_size_t depth,              \
                                           nk_size_t stride, void *result, nk_size_t result_stride,                    \
                                           nk_size_t row_start, nk_size_t row_count);                                  \
    NKB_API void nk_euclideans_symmetric_##T(void const *vectors, nk_size_t vectors_count, nk_size_t depth,            \
                                             nk_size_t stride, void *result, nk_size_t result_stride,                  \
                                             nk_size_t row_start, nk_size_t row_count);

NKB_DECLARE_SYMMETRIC_FAMILY(i8)
NKB_DECLARE_SYMMETRIC_FAMILY(u8)
NKB_DECLARE_SYMMETRIC_FAMILY(bf16)
NKB_DECLARE_SYMMETRIC_FAMILY(f16)
NKB_DECLARE_SYMMETRIC_FAMILY(e4m3)
NKB_DECLARE_SYMMETRIC_FAMILY(e5m2)
NKB_DECLARE_SYMMETRIC_FAMILY(e2m3)
NKB_DECLARE_SYMMETRIC_FAMILY(e3m2)
NKB_DECLARE_SYMMETRIC_FAMILY(f32)
NKB_DECLARE_SYMMETRIC_FAMILY(i4)
NKB_DECLARE_SYMMETRIC_FAMILY(u4)
NKB_DECLARE_SYMMETRIC_FAMILY(f64)

/* ---- one-bit vectors: AND-popcount products and the set distances built on them -----------------------
 * nk_dots_packed_size_u1 / nk_dots_pack_u1 / nk_dots_packed_u1 / nk_dots_symmetric_u1 replace
 * include/numkong/dots.h:201,245,295,357 (u32 cells); nk_hammings_* and nk_jaccards_* replace include/numkong/sets.h:69-117:
 * Hamming = |a| + |b| - 2 |a & b| (u32 cells), Jaccard = 1 - |a & b| / |a | b| (f32 cells, 0 for two empty sets). The
 * blob packed by nk_dots_pack_u1 serves all three; every bit of the last byte counts when `depth` stops inside it.
 */
NKB_API nk_size_t nk_dots_packed_size_u1(nk_size_t width, nk_size_t depth);
NKB_API void nk_dots_pack_u1(void const *b, nk_size_t width, nk_size_t depth, nk_size_t b_stride, void *b_packed);
NKB_API void nk_dots_packed_u1(void const *a, void const *b_packed, void *c, nk_size_t height, nk_size_t width,
                               nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride);
NKB_API void nk_dots_symmetric_u1(void const *vectors, nk_size_t vectors_count, nk_size_t depth, nk_size_t stride,
                                  void *result, nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count);
NKB_API void nk_hammings_packed_u1(void const *v, void const *q_packed, void *result, nk_size_t rows, nk_size_t cols,
                                   nk_size_t d, nk_size_t v_stride_in_bytes, nk_size_t r_stride_in_bytes);
NKB_API void nk_hammings_symmetric_u1(void const *vectors, nk_size_t vectors_count, nk_size_t d, nk_size_t stride,
                                      void *result, nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count);
NKB_API void nk_jaccards_packed_u1(void const *v, void const *q_packed, void *result, nk_size_t rows, nk_size_t cols,
                                   nk_size_t d, nk_size_t v_stride_in_bytes, nk_size_t r_stride_in_bytes);
NKB_API void nk_jaccards_symmetric_u1(void const *vectors, nk_size_t vectors_count, nk_size_t d, nk_size_t stride,
                                      void *result, nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count);

/* ---- In-place down-casts of a finished dots matrix -----------------------------------------------
 * replace the header-level helpers include/numkong/dots/serial.h:2707-2754 (nk_dots_compact_bf16_serial,
 * nk_dots_compact_i8_serial; AMX twins dots/sapphireamx.h:1301, :1834). The matrix `c` (rows `c_stride_in_bytes`
 * apart) is overwritten from its first byte with the tightly packed result: row r starts at byte
 * r * column_count * sizeof(out).
 *   bf16: every f32 cell rounded to nearest even.
 *   i8:   every i32 cell c[i][j] * 127 / sqrt(a_squared_norms[i] * b_squared_norms[j]), computed in f32 with the
 *         reference's own reciprocal square root, truncated toward zero, clamped to [-128, 127]; 0 when a norm is 0.
 * Host or device pointers (the norm vectors too). */
NKB_API void nk_dots_compact_bf16(void *c, nk_size_t row_count, nk_size_t column_count, nk_size_t c_stride_in_bytes);
NKB_API void nk_dots_compact_i8(void *c, nk_size_t row_count, nk_size_t column_count, nk_size_t c_stride_in_bytes,
                                int32_t const *a_squared_norms, int32_t const *b_squared_norms);

/* ---- Bulk type conversion ----------------------------------------------------------------------------
 * replaces nk_cast (include/numkong/cast.h:55, dispatch c/numkong.c:770) with the rules of nk_cast_serial
 * (include/numkong/cast/serial.h:2250-2311): `n` values of `from_type` become `n` values of `to_type`; every real
 * scalar type of nk_dtype_t (f64 f32 f16 bf16 e4m3 e5m2 e2m3 e3m2, i8..i64, u8..u64, i4 u4 u1). Floats round to
 * nearest even (e4m3 / e2m3 / e3m2 saturate, e5m2 and f16 overflow to infinity), integers saturate, float -> integer
 * rounds to nearest even after clamping, NaN -> 0. u1 is most-significant-bit first and i4 / u4 keep the even index in
 * the high nibble here. Host or device pointers. Pairs the reference leaves undefined (u1 -> signed integer, signed
 * integer -> u4 / u1, complex types) set the error text and write nothing. */
NKB_API void nk_cast(void const *from, uint32_t from_type, nk_size_t n, void *to, uint32_t to_type);

/* ---- Moments: sum and sum of squares of a strided vector -------------------------------------------------
 * replace nk_reduce_moments_<t> (include/numkong/reduce.h:120-279, scalar back end reduce/serial.h:52-416): `count`
 * values `stride_bytes` apart (sub-byte types: whole bytes, the stride steps from byte to byte). Integers are exact,
 * with the reference's saturation rules for 32 / 64-bit types; floats are summed in f64 and rounded once to the
 * result type. `data` and the two result pointers may each be host or device memory. */
NKB_API void nk_reduce_moments_f64(double const *data, nk_size_t count, nk_size_t stride_bytes, double *sum, double *sumsq);
NKB_API void nk_reduce_moments_f32(float const *data, nk_size_t count, nk_size_t stride_bytes, double *sum, double *sumsq);
NKB_API void nk_reduce_moments_f16(void const *data, nk_size_t count, nk_size_t stride_bytes, float *sum, float *sumsq);
NKB_API void nk_reduce_moments_bf16(void const *data, nk_size_t count, nk_size_t stride_bytes, float *sum, float *sumsq);
NKB_API void nk_reduce_moments_e4m3(void const *data, nk_size_t count, nk_size_t stride_bytes, float *sum, float *sumsq);
NKB_API void nk_reduce_moments_e5m2(void const *data, nk_size_t count, nk_size_t stride_bytes, float *sum, float *sumsq);
NKB_API void nk_reduce_moments_e2m3(void const *data, nk_size_t count, nk_size_t stride_bytes, float *sum, float *sumsq);
NKB_API void nk_reduce_moments_e3m2(void const *data, nk_size_t count, nk_size_t stride_bytes, float *sum, float *sumsq);
NKB_API void nk_reduce_moments_i8(int8_t const *data, nk_size_t count, nk_size_t stride_bytes, int64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_u8(uint8_t const *data, nk_size_t count, nk_size_t stride_bytes, uint64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_i16(int16_t const *data, nk_size_t count, nk_size_t stride_bytes, int64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_u16(uint16_t const *data, nk_size_t count, nk_size_t stride_bytes, uint64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_i32(int32_t const *data, nk_size_t count, nk_size_t stride_bytes, int64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_u32(uint32_t const *data, nk_size_t count, nk_size_t stride_bytes, uint64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_i64(int64_t const *data, nk_size_t count, nk_size_t stride_bytes, int64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_u64(uint64_t const *data, nk_size_t count, nk_size_t stride_bytes, uint64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_i4(void const *data, nk_size_t count, nk_size_t stride_bytes, int64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_u4(void const *data, nk_size_t count, nk_size_t stride_bytes, uint64_t *sum, uint64_t *sumsq);
NKB_API void nk_reduce_moments_u1(void const *data, nk_size_t count, nk_size_t stride_bytes, uint64_t *sum, uint64_t *sumsq);

/* ---- MaxSim late interaction -------------------------------------------------------------------
 * replaces include/numkong/maxsim.h:72-114 (wrappers c/numkong.c:738-765). Both sides are packed
 * with the same function. result: f32 for bf16/f16, f64 for f32 (maxsim.h:350-357):
 *   sum_i max(0, 1 - (max_j q_i . d_j) / (|q_i| |d_j*|)),  j* = first argmax of the raw dot.
 */
#define NKB_DECLARE_MAXSIM_FAMILY(T)                                                                                   \
    NKB_API nk_size_t nk_maxsim_packed_size_##T(nk_size_t vector_count, nk_size_t depth);                              \
    NKB_API void nk_maxsim_pack_##T(void const *vectors, nk_size_t vector_count, nk_size_t depth, nk_size_t stride,    \
                                    void *packed);                                                                     \
    NKB_API void nk_maxsim_packed_##T(void const *query_packed, void const *document_packed, nk_size_t query_count,    \
                                      nk_size_t document_count, nk_size_t depth, void *result);

NKB_DECLARE_MAXSIM_FAMILY(bf16)
NKB_DECLARE_MAXSIM_FAMILY(f16)
NKB_DECLARE_MAXSIM_FAMILY(f32)

/* ---- run-time lookup ---------------------------------------------------------------------------
 * replaces nk_find_kernel_punned (c/numkong.c:848-913) for the kernel kinds of this path:
 * 'P' packed size, 'Q' pack, 'G' dots_packed, 'N' angulars_packed, 'E' euclideans_packed,
 * 'L' / 'l' / 'T' MaxSim size / pack / compute, 'y' / 'n' / 'D' the symmetric family, 'M' / 'Y' / 'p' / 'Z' the set
 * distances of one-bit vectors, 'R' moments per element type, '-' with element type 0 the bulk conversion
 * (capabilities.h:225-251). Unknown combinations give
 * *kernel_output = NULL and *capability_output = 0, which callers already treat as "no kernel".
 */
#define NKB_CAPABILITY_B200 (1ull << 40)
NKB_API void nk_find_kernel_punned(int kind, uint32_t dtype, uint64_t viable_capabilities, void **kernel_output,
                                   uint64_t *capability_output);
NKB_API uint64_t nk_capabilities(void);            /* c/numkong.c:832-843: here NKB_CAPABILITY_B200 or 0 */
NKB_API int nk_configure_thread(uint64_t caps);    /* capabilities.h:909: nothing to set up per thread here; returns 1 */

/* ---- results too large to return whole (no counterpart in the reference) -----------------------
 * Each of these equals "call the reference function, then reduce": the tests check them that way.
 *
 * nkb_<metric>s_packed_topk_<t>: for every row of A the `top` (<= 1024) nearest rows of the packed
 *   matrix, ascending by distance, ties by lower id: distances[height x top] f32, ids[height x top] i64
 *   (= id_base + row index inside the packed matrix; unused slots hold +inf / -1). Equivalent to
 *   nk_<metric>s_packed_<t> followed by a per-row selection, without ever storing height x width values.
 * nkb_maxsims_packed_<t>: all-pairs MaxSim. `q_packed` / `d_packed` hold the token vectors of all queries /
 *   all documents back to back (one nk_maxsim_pack_<t> call each); q_offsets[n_queries+1] and
 *   d_offsets[n_documents+1] (u64, ascending, starting at 0) delimit them; every document needs at least
 *   one vector. scores[q * score_stride/4 + d] receives what nk_maxsim_packed_<t> returns for that pair.
 *   For the duration of the call the documents are copied onto 32-token boundaries (every document's last vector repeated
 *   up to the next multiple of 32: the same scores, bit for bit, and a scan without document boundaries inside its
 *   32-column chunks); the copy lives in the calling thread's staging memory (about 1.1 x the packed documents, kept for the
 *   next call and returned by nkb_release_caches()) and is skipped when it would take more than half of the free device
 *   memory. (Allocating it per call was measured: a stream-ordered allocation of 10 GB per call costs more than the call.)
 * nkb_topk_smallest_f32: per row of a score matrix, the `top` smallest values and their columns + id_base.
 */
#define NKB_DECLARE_TOPK_FAMILY(T)                                                                                     \
    NKB_API void nkb_angulars_packed_topk_##T(void const *a, void const *b_packed, nk_size_t height, nk_size_t width,  \
                                              nk_size_t depth, nk_size_t a_stride, nk_size_t top, void *distances,     \
                                              void *ids, nk_size_t id_base);                                           \
    NKB_API void nkb_euclideans_packed_topk_##T(void const *a, void const *b_packed, nk_size_t height, nk_size_t width, \
                                                nk_size_t depth, nk_size_t a_stride, nk_size_t top, void *distances,   \
                                                void *ids, nk_size_t id_base);
NKB_DECLARE_TOPK_FAMILY(f16)
NKB_DECLARE_TOPK_FAMILY(bf16)

#define NKB_DECLARE_MAXSIMS_FAMILY(T)                                                                                  \
    NKB_API void nkb_maxsims_packed_##T(void const *q_packed, void const *q_offsets, nk_size_t n_queries,              \
                                        void const *d_packed, void const *d_offsets, nk_size_t n_documents,            \
                                        nk_size_t depth, void *scores, nk_size_t score_stride);
NKB_DECLARE_MAXSIMS_FAMILY(bf16)
NKB_DECLARE_MAXSIMS_FAMILY(f16)

NKB_API void nkb_topk_smallest_f32(void const *scores, nk_size_t rows, nk_size_t cols, nk_size_t stride, nk_size_t top,
                                   nk_size_t id_base, void *out_values, void *out_ids);
/* nkb_merge_topk: the cross-shard step of a sharded search. `values` (f32) and `ids` (i64) hold `parts` nearest-k lists
 * per row, laid out [part][row][top] - what a gather of every shard's nkb_*_topk_* result delivers; slots with id < 0 are
 * empty. out_values[rows x top] / out_ids[rows x top] receive the `top` smallest per row ordered by (value, id) (-0 before
 * +0, as in every selection of this library), empty
 * slots as +inf / -1. parts * top (rounded up to a power of two) may not exceed 16384. Host or device pointers. */
NKB_API void nkb_merge_topk(void const *values, void const *ids, nk_size_t parts, nk_size_t rows, nk_size_t top,
                            void *out_values, void *out_ids);

/* nkb_dots_packed_columns: nk_dots_packed_<t> (element type by its code) restricted to the columns
 * [first_column, first_column + column_count) of the result, i.e. to that range of packed rows; first_column must be a
 * multiple of 256. `c` points at cell (0, 0) of the full height x width result, of which only those columns are written.
 * For callers that receive the packed matrix piecewise (a broadcast in column blocks: the packed rows of a block are one
 * contiguous byte range of the blob, 256 rows = 256 * depth_padded bytes from offset 128 on) and want to multiply the
 * blocks that have arrived while the others are still on their way. No counterpart in the reference. */
NKB_API void nkb_dots_packed_columns(uint32_t dtype, void const *a, void const *b_packed, void *c, nk_size_t height,
                                     nk_size_t width, nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride,
                                     nk_size_t first_column, nk_size_t column_count);

/* ---- batched angular distances without any device allocation -----------------------------------
 * No counterpart in the reference (which never allocates because it runs on the caller's CPU buffers).
 *
 * Same result as nk_angulars_packed_<t>, for callers that must not trigger cudaMalloc: code inside a stream
 * capture, latency-critical serving loops, hosts whose pool allocator owns the whole device heap. The scratch the
 * regular path allocates (one f32 squared norm per row of A, plus the error word of the pipeline waits) lives in
 * fixed device arrays inside this library instead: 256 KiB + 256 B per GPU, held from library load to process exit.
 *
 *  - `dtype` is one of NKB_DTYPE_{BF16,F16,E4M3,E5M2,I8,U8}; c receives height x width f32.
 *  - height <= NKB_NOALLOC_MAX_ROWS; larger calls are refused (split them by rows of A).
 *  - a, b_packed and c must be device or managed memory; a and b_packed 16-byte aligned, a_stride a multiple of 16
 *    (nothing can be staged or re-strided without allocating).
 *  - Returns 0 when the work was enqueued on the calling thread's stream, a non-zero code (and nkb_last_error())
 *    when the call was refused; nothing is written to c in that case.
 *  - The first call on each GPU looks up the device addresses of the fixed arrays and clears the error word with a
 *    synchronous memset; make that first call (any small problem) before starting a stream capture.
 *  - All calls on one GPU share the fixed arrays: the norms are rewritten by every call, so two calls that overlap
 *    on the GPU (different streams or threads) race; run them in stream order.
 *  - A bounded pipeline wait that gives up inside such a call leaves its code in the fixed error word; nkb_synchronize()
 *    returns it (and clears it) without allocating anything, so check its return value after synchronising.
 */
#define NKB_NOALLOC_MAX_ROWS 65536
NKB_API int nkb_angulars_packed_noalloc(uint32_t dtype, void const *a, void const *b_packed, void *c, nk_size_t height,
                                        nk_size_t width, nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride);

/* ---- additions (no counterpart in the reference) -------------------------------------------- */
/** Last error of the calling thread, "" when the last call succeeded. The string stays valid until the next call. */
NKB_API char const *nkb_last_error(void);
/** Stream (a cudaStream_t) the calling thread's next calls are enqueued on. NULL selects the default stream. The library's
 *  per-thread staging buffers pass from one call to the next, so a switch puts the new stream behind the work this thread
 *  already enqueued on the old one (an event wait on the device; the host does not block). */
NKB_API void nkb_set_stream(void *cuda_stream);
/** Waits for the calling thread's stream and returns the device error word: 0, or 0x80000000 | site << 16 | block of the
 *  first bounded pipeline wait that gave up on this GPU since the last report (sites: 1 loader waiting for a free stage,
 *  2 / 3 MMA issuer waiting for a drained accumulator / a loaded stage, 4 epilogue waiting for a finished accumulator,
 *  5 / 6 the issuer's / loader's final drain, 7 epilogue waiting for the other half of a tile whose depth two CTA pairs
 *  share, 8 nkb_peer_barrier waiting for another GPU - the low bits then name that peer). Covers the regular entry points
 *  and nkb_angulars_packed_noalloc alike,
 *  allocates nothing, and clears the word it reports: the failure belongs to the calls enqueued before this
 *  synchronisation (their results are not valid), later calls start clean. Calls with a host-resident operand do this
 *  check themselves and fill their output with 0xFF. */
NKB_API uint32_t nkb_synchronize(void);
/** Shortens (or restores) the limit of the kernels' bounded waits. `site` as listed under nkb_synchronize, 0 = all sites;
 *  `nanoseconds` 0 = the default of 2 s, larger values are capped there. Process-wide; for tests of the give-up path and
 *  for callers that would rather fail fast than wait two seconds for a pipeline that will never move. */
NKB_API void nkb_set_wait_limit_ns(int site, uint64_t nanoseconds);
/** Test hook: stores `value` in the current GPU's error word as a wait that gave up would (which = 0: the word of the
 *  regular entry points, created if need be; 1: the fixed word of nkb_angulars_packed_noalloc, which must have run on this
 *  GPU before). Returns 0 on success. Nothing on the device fails. */
NKB_API int nkb_test_set_error_word(int which, uint32_t value);
/** Number of host-resident packed blobs whose device copies are cached right now (all GPUs). */
NKB_API uint64_t nkb_cached_blob_count(void);
/** Kernels launched by this library in this process so far (for launch accounting in benchmarks). */
NKB_API uint64_t nkb_launch_count(void);
/** Tuning word for tests and A/B measurements; 0 = the library chooses everything. Bits 0-7 force a GEMM tile configuration
 *  (1: 128 x 256 tiles per CTA, 2: 128 x 128, 3: CTA pairs on 256 x 256 tiles, 4: the four-stage 128 x 256 kernel, 5: CTA
 *  pairs with the depth of the last tiles split between pairs - the one setting under which a row's bits depend on how many
 *  rows are multiplied with it); bits 8-15 are the accumulation span (nkb_set_accumulation_span writes them); bits 16-23 the
 *  number of query tiles of the all-pairs MaxSim that walk a document segment side by side (0: eight); bit 24 keeps that call
 *  on the caller's document layout instead of the copy on 32-token boundaries. Process-wide. */
NKB_API void nkb_set_gemm_variant(int variant);
/** Accuracy / speed trade of the floating-point tensor-core products. The tensor cores truncate when they add into their
 *  f32 accumulators, so the depth is cut into spans of `stages` x 128 bytes that are added with round-to-nearest in
 *  registers. 0 (default): chosen by type and depth so that the error stays within that of the reference's own kernels on the
 *  same inputs: sqrt(depth)/16 stages for bf16 (6 at depth 8192), sqrt(depth)/11 for f16 (8 at depth 8192), 16 stages for the
 *  8-bit floats, 32 for e2m3. Every read-out of a span keeps the tensor cores waiting for about 256 cycles (a stage takes
 *  512), so longer spans are faster (16 stages at depth 8192: about +5 %) and less accurate in proportion (bf16, same-sign
 *  data, depth 8192: 2.8 units in the last place at 6 stages, 14.5 at 16; the reference's scalar kernel 2.9). f16 products
 *  carry 22 significant bits and lose some in every tensor-core addition: on same-sign f16 data even 1-stage spans leave
 *  1.8 - 2.2 units where the reference has 0.6 - 3.0. Integer products are exact and ignore the setting. Process-wide. */
NKB_API void nkb_set_accumulation_span(int stages);
/** SMs the persistent GEMM kernels may occupy; 0 (default) = all. These kernels put one CTA on every SM for as long as they
 *  run, so a collective that should progress at the same time on another stream (its kernel needs a few SMs of its own)
 *  only does so when some are left free: a caller that overlaps a broadcast of the packed matrix with the products of the
 *  parts that have arrived sets e.g. 132 of 148 for those products and 0 again afterwards. Process-wide. */
NKB_API void nkb_set_sm_budget(int sms);
/** One-to-all delivery of `bytes` bytes (a packed matrix, typically) through the NVSwitch: `multicast_dst` is the MULTICAST
 *  address of a buffer that exists on every GPU of the group (an NVLink multicast mapping, e.g. the `multicast_ptr` of a
 *  torch.distributed._symmetric_memory buffer, plus the offset inside it); `src` is ordinary device memory of the calling
 *  GPU. Every 16 bytes are issued once with `multimem.st` and written into all GPUs' copies by the switch, the sender's
 *  included, so the sender's link carries the data once whatever the number of receivers (a ring broadcast forwards it hop by
 *  hop). Enqueued on the calling thread's stream; the caller orders the receivers behind it (a barrier across the group on
 *  their streams). Addresses and size must be multiples of 16. `blocks` = CTAs to use (0: 64). Stands where the reference's
 *  callers hand "the full packed B" to every worker (README.md:199-212). Returns 0, or non-zero with nkb_last_error() set.
 *  An address that is not a multicast mapping is undefined behaviour, as for any store through a bad pointer. */
NKB_API int nkb_multicast_store(void *multicast_dst, void const *src, nk_size_t bytes, int blocks);
/** Barrier between the GPUs of a group, enqueued on the calling thread's stream: work enqueued behind it on any of them
 *  starts only after every GPU has reached it - e.g. after the sender's nkb_multicast_store has finished. `peer_flags` is a
 *  HOST array of `world` device addresses: entry p is GPU p's flag buffer (at least `world` 32-bit words, zero before the
 *  first barrier, used for nothing else) as mapped into this process - the `buffer_ptrs` of a symmetric-memory buffer.
 *  Every GPU writes `epoch` into its own slot of every peer's buffer and waits until all slots of its own buffer have reached
 *  `epoch`; callers pass 1, 2, 3, ... in step on all GPUs. The wait is bounded like every other wait of this library (site 8,
 *  nkb_set_wait_limit_ns): when a peer does not show up the kernel records the error word and returns, nkb_synchronize()
 *  reports it, and what was ordered behind the barrier must be treated as not ordered. `world` <= 16. */
NKB_API int nkb_peer_barrier(void *const *peer_flags, int world, int rank, uint32_t epoch);
/** How e2m3 / e3m2 operands reach the tensor cores: 1 (default) = packed 6-bit operands with the native
 *  e2m3 / e3m2 MMA formats, 0 = recoded to the e4m3 code of the same value (exact as well). Applies to later pack AND multiply calls;
 *  a blob packed under one setting must be multiplied under the same one. */
NKB_API void nkb_set_fp6_native(int native);
/** Packed rows handled per panel by the distance top-k (rounded up to 256); 0 = sized from the scratch budget. */
NKB_API void nkb_set_topk_panel_rows(nk_size_t rows);
/** How the distance top-k selects. 1 (default): for k <= 128 and at least 8,192 packed rows only the first 2,048 packed
 *  rows are materialised; the rest go through a GEMM whose epilogue stores nothing but values below each row's current
 *  k-th smallest (at most 512 per row and panel, a row that overflows sends the whole call to the materialising path;
 *  the filtered path synchronises with its stream before returning). 0: always materialise panels. >= 256: filter with
 *  that many bootstrap rows whenever the packed matrix is larger (testing). Results are identical in every mode. */
NKB_API void nkb_set_topk_filter(int mode);
/** Number of top-k calls redone on the materialising path after a candidate list overflowed (process-wide). */
NKB_API nk_size_t nkb_topk_filter_fallbacks(void);
/** Drops the cached device copies of host-resident packed blobs and the staging buffers of the calling thread. */
NKB_API void nkb_release_caches(void);

#ifdef __cplusplus
}
#endif
#endif /* NUMKONG_B200_H_ */
