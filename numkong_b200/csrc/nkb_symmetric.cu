// Symmetric products C = A x A^T and the distance matrices built on them.
//
// Replaces NumKong's nk_dots_symmetric_<t> (include/numkong/dots.h:309-359, generator
// include/numkong/dots/serial.h:2039-2440) and nk_angulars_symmetric_<t> / nk_euclideans_symmetric_<t>
// (include/numkong/spatials.h:77-, generator include/numkong/dots/serial.h:2802-2872). Contract kept:
//   * only rows [row_start, row_start + row_count) of the result are touched, and of those only the cells
//     on or above the diagonal (column >= row); everything below the diagonal is left as the caller had it;
//   * dots: the diagonal holds the squared norm; distances: the diagonal is 0 and cell (i, j), j > i, is
//     the batched formula applied to dot(i, j), |a_i|^2, |a_j|^2;
//   * disjoint row ranges may be computed by different threads into the same result matrix.
//
// The rows at and after the first wanted column are packed into a scratch blob on the device (same kernels as
// nk_dots_pack_<t>), then the packed GEMM runs in its triangular mode: tiles wholly below the diagonal are
// never scheduled and the stores are masked per cell.
#include <cstdio>
#include <cstring>
#include "nkb_internal.h"
#include "nkb_host.h"
#include "../../include/numkong_b200.h"

namespace nkb {
namespace {

void symmetric_impl(uint32_t dt, int epilogue, const void *vectors, uint64_t count, uint64_t depth, uint64_t stride,
                    void *result, uint64_t result_stride, uint64_t row_start, uint64_t row_count) {
    clear_error();
    if (count == 0 || row_count == 0 || row_start >= count) return;
    const uint64_t row_end = row_start + row_count < count ? row_start + row_count : count;
    const uint64_t m = row_end - row_start;
    const uint32_t out_bytes = dot_out_bytes(dt);
    const MemKind v_kind = classify(vectors), r_kind = classify(result);
    // First packed column: the 256-row block that holds row_start (nothing to its left is wanted).
    const uint64_t col0 = row_start / kRowPad * kRowPad;
    const uint64_t cols = count - col0;
    uint8_t *touched = result ? static_cast<uint8_t *>(result) + row_start * result_stride + col0 * out_bytes : nullptr;
    auto fail = [&]() {
        // Error convention of the reference: 0xFF bytes - here only over the cells this call owns (column >= row).
        if (!touched) return;
        for (uint64_t i = 0; i < m && r_kind == kMemHost; ++i) {
            uint8_t *row = static_cast<uint8_t *>(result) + (row_start + i) * result_stride;
            std::memset(row + (row_start + i) * out_bytes, 0xFF, (count - row_start - i) * out_bytes);
        }
    };
    if (!dtype_supported(dt) || !vectors || !result) { set_error("symmetric: unsupported element type or null pointer%s", ""); fail(); return; }
    if (depth == 0) { set_error("symmetric: depth must be positive%s", ""); fail(); return; }
    if (result_stride < count * out_bytes || result_stride % out_bytes) { set_error("symmetric: bad result stride%s", ""); fail(); return; }
    if (stride < source_row_bytes(dt, depth) && count > 1) { set_error("symmetric: stride is smaller than a vector%s", ""); fail(); return; }
    cudaStream_t stream = current_stream();
    unsigned int *err = device_error_word();
    if (!err) { set_error("could not allocate the device error word%s", ""); fail(); return; }

    const uint64_t row_bytes = source_row_bytes(dt, depth);
    const uint32_t op_dt = operand_dtype(dt);          // 4-bit rows are expanded to i8 / u8 on the device
    const uint64_t op_depth = operand_depth(dt, depth);
    const int piece_mode = piece_mode_for(dt);
    bool ok = true;
    // ---- column operand: rows [col0, count) packed into a scratch blob
    const PackedGeometry g = packed_geometry(dt, cols, depth);
    uint8_t *blob = static_cast<uint8_t *>(scratch(kSlotAux, g.total_bytes));
    if (!blob) { fail(); return; }
    const uint8_t *col_src = static_cast<const uint8_t *>(vectors) + col0 * stride;
    uint64_t col_pitch = stride;
    if (v_kind == kMemHost) {
        void *stage = scratch(kSlotAux2, cols * row_bytes + 16);
        ok = stage && cuda_ok(cudaMemcpy2DAsync(stage, row_bytes, col_src, stride < row_bytes ? row_bytes : stride, row_bytes, cols,
                                                cudaMemcpyHostToDevice, stream), "upload of vectors");
        col_src = static_cast<const uint8_t *>(stage);
        col_pitch = row_bytes;
    }
    if (ok) {
        ok = cuda_ok(launch_pack_payload(dt, col_src, cols, depth, col_pitch, blob + g.payload_offset, g.rows_padded,
                                         g.depth_padded_bytes, piece_mode_for(dt), stream), "pack kernel");
        g_launches++;
    }
    if (ok) {
        ok = cuda_ok(launch_row_sumsq(dt, col_src, cols, depth, col_pitch, blob + g.norms_offset, false, false, stream), "norm kernel");
        g_launches++;
    }
    // ---- row operand: rows [row_start, row_end). They already sit in the staged / caller's device copy.
    const uint8_t *a_src = col_src + (row_start - col0) * col_pitch;
    uint64_t a_pitch = 0;
    const void *a_raw = ok ? resident_matrix(a_src, kMemDevice, m, row_bytes, col_pitch, kSlotA, is_subbyte(dt) ? piece_mode : kPieceNone, &a_pitch) : nullptr;
    if (!a_raw) { fail(); return; }
    void *a_norms = nullptr;
    if (epilogue != kEpiDot) {
        a_norms = scratch(kSlotNorms, m * 8);
        ok = a_norms && cuda_ok(launch_row_sumsq(op_dt, a_raw, m, op_depth, a_pitch, a_norms, !is_cuda_core_dtype(dt), false, stream), "row norm kernel");
        g_launches++;
    }
    const void *a_dev = a_raw;
    if (ok && piece_mode != kPieceNone && !is_subbyte(dt)) {
        // FP6 rows are rewritten for the tensor cores: in place when they already live in this thread's staging buffer.
        void *dst = const_cast<void *>(a_raw);
        uint64_t dst_pitch = a_pitch;
        if (a_raw == static_cast<const void *>(a_src)) {
            dst_pitch = round_up(row_bytes, 16);
            dst = scratch(kSlotA, m * dst_pitch + 16);
            if (!dst) { fail(); return; }
        }
        ok = cuda_ok(launch_restride(a_raw, m, row_bytes, a_pitch, dst, dst_pitch, piece_mode, stream), "operand rewrite kernel");
        g_launches++;
        a_dev = dst;
        a_pitch = dst_pitch;
    }
    // ---- result: in place when it is device memory with aligned cells; otherwise a staged copy that starts out as the
    // caller's current cells, so that the cells this call does not own travel back unchanged.
    uint8_t *c_dev = touched;
    uint64_t c_pitch = result_stride;
    const uint64_t c_row_bytes = cols * out_bytes;
    const bool direct = r_kind == kMemDevice && (reinterpret_cast<uintptr_t>(touched) % out_bytes) == 0;
    if (ok && !direct) {
        c_pitch = round_up(c_row_bytes, 16);
        c_dev = static_cast<uint8_t *>(scratch(kSlotC, m * c_pitch));
        if (!c_dev) { fail(); return; }
        ok = cuda_ok(cudaMemcpy2DAsync(c_dev, c_pitch, touched, result_stride, c_row_bytes, m,
                                       r_kind == kMemHost ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToDevice, stream), "upload of result cells");
    }
    const int32_t tri_diag = (int32_t)(row_start - col0);
    if (ok && dt == kF32) {
        ok = cuda_ok(launch_gemm_f32(epilogue, static_cast<const float *>(a_dev), a_pitch, reinterpret_cast<const float *>(blob + g.payload_offset),
                                     g.depth_padded_bytes, reinterpret_cast<const double *>(blob + g.norms_offset),
                                     static_cast<const double *>(a_norms), reinterpret_cast<double *>(c_dev), c_pitch, m, cols, depth, stream,
                                     tri_diag), "f32 GEMM kernel");
        g_launches++;
    } else if (ok && dt == kF64) {
        ok = cuda_ok(launch_gemm_f64(epilogue, static_cast<const double *>(a_dev), a_pitch, reinterpret_cast<const double *>(blob + g.payload_offset),
                                     g.depth_padded_bytes, reinterpret_cast<const double *>(blob + g.norms_offset),
                                     static_cast<const double *>(a_norms), reinterpret_cast<double *>(c_dev), c_pitch, m, cols, depth, stream,
                                     tri_diag), "f64 GEMM kernel");
        g_launches++;
    } else if (ok) {
        GemmArgs args;
        args.dtype = op_dt; args.epilogue = epilogue; args.a = a_dev; args.a_stride = a_pitch;
        args.b_payload = blob + g.payload_offset; args.b_norms = blob + g.norms_offset; args.a_norms = static_cast<const float *>(a_norms);
        args.c = c_dev; args.c_stride = c_pitch; args.m = m; args.n = cols; args.k = op_depth;
        args.depth_padded_bytes = g.depth_padded_bytes; args.error_word = err; args.variant = current_variant();
        args.tri_diag = tri_diag;
        ok = cuda_ok(launch_gemm_tc(args, stream), "tensor-core GEMM kernel");
        g_launches++;
    }
    if (ok && !direct)
        ok = cuda_ok(cudaMemcpy2DAsync(touched, result_stride, c_dev, c_pitch, c_row_bytes, m,
                                       r_kind == kMemHost ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice, stream), "download of result");
    if (ok && (v_kind == kMemHost || r_kind == kMemHost)) {
        ok = cuda_ok(cudaStreamSynchronize(stream), "symmetric call");
        if (ok) {
            uint32_t w = read_device_error();
            if (w) { char buf[64]; std::snprintf(buf, sizeof buf, "0x%08x", w); set_error("a pipeline wait inside the GEMM kernel gave up (error word %s)", buf); ok = false; }
        }
    }
    if (!ok) fail();
}

} // namespace
} // namespace nkb

using namespace nkb;

extern "C" {

#define NKB_DEFINE_SYMMETRIC(T, DT)                                                                                         \
    NKB_API void nk_dots_symmetric_##T(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride, void *result, \
                                       nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count) {                 \
        symmetric_impl(DT, kEpiDot, vectors, count, depth, stride, result, result_stride, row_start, row_count);            \
    }                                                                                                                       \
    NKB_API void nk_angulars_symmetric_##T(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride,         \
                                           void *result, nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count) { \
        symmetric_impl(DT, kEpiAngular, vectors, count, depth, stride, result, result_stride, row_start, row_count);        \
    }                                                                                                                       \
    NKB_API void nk_euclideans_symmetric_##T(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride,       \
                                             void *result, nk_size_t result_stride, nk_size_t row_start,                   \
                                             nk_size_t row_count) {                                                         \
        symmetric_impl(DT, kEpiEuclidean, vectors, count, depth, stride, result, result_stride, row_start, row_count);      \
    }

NKB_DEFINE_SYMMETRIC(i8, kI8)
NKB_DEFINE_SYMMETRIC(u8, kU8)
NKB_DEFINE_SYMMETRIC(f32, kF32)
NKB_DEFINE_SYMMETRIC(f16, kF16)
NKB_DEFINE_SYMMETRIC(bf16, kBF16)
NKB_DEFINE_SYMMETRIC(e4m3, kE4M3)
NKB_DEFINE_SYMMETRIC(e5m2, kE5M2)
NKB_DEFINE_SYMMETRIC(e2m3, kE2M3)
NKB_DEFINE_SYMMETRIC(e3m2, kE3M2)
NKB_DEFINE_SYMMETRIC(i4, kI4)
NKB_DEFINE_SYMMETRIC(u4, kU4)
NKB_DEFINE_SYMMETRIC(f64, kF64)

// One-bit vectors (include/numkong/dots.h:357, include/numkong/sets.h:84-117).
NKB_API void nk_dots_symmetric_u1(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride, void *result,
                                  nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count) {
    symmetric_impl(kU1, kEpiDot, vectors, count, depth, stride, result, result_stride, row_start, row_count);
}
NKB_API void nk_hammings_symmetric_u1(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride, void *result,
                                      nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count) {
    symmetric_impl(kU1, kEpiHamming, vectors, count, depth, stride, result, result_stride, row_start, row_count);
}
NKB_API void nk_jaccards_symmetric_u1(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride, void *result,
                                      nk_size_t result_stride, nk_size_t row_start, nk_size_t row_count) {
    symmetric_impl(kU1, kEpiJaccard, vectors, count, depth, stride, result, result_stride, row_start, row_count);
}

} // extern "C"
