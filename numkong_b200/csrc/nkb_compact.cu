// In-place down-casts of a finished dots matrix ("compact" helpers of the dots family).
//
// Replaces NumKong's nk_dots_compact_bf16_serial (include/numkong/dots/serial.h:2707-2724: every f32 cell becomes
// bf16, round to nearest even) and nk_dots_compact_i8_serial (include/numkong/dots/serial.h:2726-2754: every i32 cell
// is rescaled to c * 127 / (|a_i| |b_j|) from the two vectors' squared norms, truncated toward zero and clamped to
// [-128, 127]). Both read rows that are `c_stride_in_bytes` apart and write the result TIGHTLY packed at the start
// of the same buffer (row r of the result starts at byte r * columns * sizeof(out)).
//
// HBM bound: 4 bytes read and 2 (or 1) written per cell. The work is done in place, without a second matrix:
// result row r lands inside source rows < r (for r >= 1), so rows are converted in waves [H,2H), [2H,4H), [4H,8H)
// - one launch per wave; inside a wave no block writes what another block of the same or a later wave still has
// to read, because the bytes written by rows [R, 2R) end where source row R begins. The head [0, H), H = rows / 8,
// which holds the self-overlapping row 0, goes through a small staging buffer instead.
#include <cstdio>
#include <cstring>
#include "nkb_internal.h"
#include "nkb_host.h"
#include "../../include/numkong_b200.h"

namespace nkb {
namespace {

struct ToBf16 {
    using Out = uint16_t;
    // Round to nearest even on the bit pattern (include/numkong/cast/serial.h:768-784); a NaN stays a quiet NaN.
    __device__ __forceinline__ Out operator()(uint32_t bits, uint32_t, uint32_t) const {
        if ((bits & 0x7fffffffu) > 0x7f800000u) return (Out)((bits >> 16) | 0x40u);
        return (Out)((bits + 0x7fffu + ((bits >> 16) & 1u)) >> 16);
    }
};

struct ToI8 {
    using Out = int8_t;
    const float *row_factors, *column_factors;  // 1 / sqrt(norm), or 0 for an empty vector
    __device__ __forceinline__ Out operator()(uint32_t bits, uint32_t row, uint32_t column) const {
        // Same operations in the same order as the reference: ((c * 127) * 1/|a|) * 1/|b|, then C's float -> int cast.
        float v = __fmul_rn(__fmul_rn(__fmul_rn((float)(int32_t)bits, 127.0f), row_factors[row]), column_factors[column]);
        int q = __float2int_rz(v);
        q = q < -128 ? -128 : (q > 127 ? 127 : q);
        return (Out)q;
    }
};

// 1 / sqrt of a squared norm exactly as the reference computes it (include/numkong/scalar/serial.h:22-33):
// bit-trick seed, three Newton steps, sqrt(x) = x * rsqrt(x), then an IEEE division. Every operation is a separate
// round-to-nearest f32 operation, as in a build of the reference without fused multiply-add.
__global__ void compact_factors_kernel(const int32_t *__restrict__ squared_norms, float *__restrict__ factors, uint32_t count) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    const float number = (float)squared_norms[i];
    float factor = 0.0f;
    if (number > 0.0f) {
        float y = __uint_as_float(0x5F375A86u - (__float_as_uint(number) >> 1));
        const float half = __fmul_rn(0.5f, number);
#pragma unroll
        for (int step = 0; step < 3; ++step) y = __fmul_rn(y, __fsub_rn(1.5f, __fmul_rn(__fmul_rn(half, y), y)));
        factor = __fdiv_rn(1.0f, __fmul_rn(number, y));
    }
    factors[i] = factor;
}

// Converts rows [row_begin, row_begin + items / chunks_per_row) of the source matrix into tightly packed rows of
// `destination` (row r of the source becomes row r - row_begin + destination_row). A block converts 2048 consecutive
// cells of one row per step; kVec = 4 reads 16 bytes per thread and needs 16-byte aligned rows and columns % 4 == 0.
template <typename Convert, int kVec>
__global__ void __launch_bounds__(256)
compact_rows_kernel(const uint8_t *source_matrix, uint64_t stride, typename Convert::Out *destination, uint32_t columns,
                    uint32_t row_begin, uint32_t destination_row, uint32_t chunks_per_row, uint64_t work_items, Convert convert) {
    using Out = typename Convert::Out;
    constexpr int kChunk = 2048, kPer = kChunk / (256 * kVec);
    for (uint64_t item = blockIdx.x; item < work_items; item += gridDim.x) {
        const uint32_t local_row = (uint32_t)(item / chunks_per_row);
        const uint32_t row = row_begin + local_row;
        const uint32_t first = (uint32_t)(item % chunks_per_row) * kChunk;
        const uint8_t *source = source_matrix + (uint64_t)row * stride;
        Out *out_row = destination + (uint64_t)(destination_row + local_row) * columns;
        if constexpr (kVec == 4) {
            uint4 cells[kPer];
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const uint32_t column = first + (i * 256u + threadIdx.x) * 4u;
                cells[i] = column < columns ? *reinterpret_cast<const uint4 *>(source + (uint64_t)column * 4) : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const uint32_t column = first + (i * 256u + threadIdx.x) * 4u;
                if (column >= columns) continue;
                const Out o0 = convert(cells[i].x, row, column), o1 = convert(cells[i].y, row, column + 1);
                const Out o2 = convert(cells[i].z, row, column + 2), o3 = convert(cells[i].w, row, column + 3);
                if constexpr (sizeof(Out) == 2) {
                    *reinterpret_cast<uint2 *>(out_row + column) = make_uint2((uint32_t)(uint16_t)o0 | ((uint32_t)(uint16_t)o1 << 16),
                                                                              (uint32_t)(uint16_t)o2 | ((uint32_t)(uint16_t)o3 << 16));
                } else {
                    *reinterpret_cast<uint32_t *>(out_row + column) = (uint32_t)(uint8_t)o0 | ((uint32_t)(uint8_t)o1 << 8) |
                                                                      ((uint32_t)(uint8_t)o2 << 16) | ((uint32_t)(uint8_t)o3 << 24);
                }
            }
        } else {
            uint32_t bits[kPer];
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const uint32_t column = first + i * 256u + threadIdx.x;
                bits[i] = column < columns ? reinterpret_cast<const uint32_t *>(source)[column] : 0u;
            }
#pragma unroll
            for (int i = 0; i < kPer; ++i) {
                const uint32_t column = first + i * 256u + threadIdx.x;
                if (column < columns) out_row[column] = convert(bits[i], row, column);
            }
        }
    }
}

template <typename Convert>
bool launch_rows(const uint8_t *source, uint64_t stride, typename Convert::Out *destination, uint64_t columns, uint64_t row_begin,
                 uint64_t row_end, uint64_t destination_row, bool vectors, Convert convert, cudaStream_t stream) {
    const uint32_t chunks_per_row = (uint32_t)((columns + 2047) / 2048);
    const uint64_t items = (row_end - row_begin) * chunks_per_row;
    const unsigned grid = (unsigned)(items < 148ull * 16 ? items : 148ull * 16);
    if (vectors)
        compact_rows_kernel<Convert, 4><<<grid, 256, 0, stream>>>(source, stride, destination, (uint32_t)columns, (uint32_t)row_begin,
                                                                  (uint32_t)destination_row, chunks_per_row, items, convert);
    else
        compact_rows_kernel<Convert, 1><<<grid, 256, 0, stream>>>(source, stride, destination, (uint32_t)columns, (uint32_t)row_begin,
                                                                  (uint32_t)destination_row, chunks_per_row, items, convert);
    g_launches++;
    return cuda_ok(cudaGetLastError(), "compact kernel");
}

// The whole matrix, in place. The first eighth of the rows (the "head", which holds row 0 - the one row whose result
// overlaps its own source) is converted into a staging buffer and copied back; the rest follows in doubling waves.
template <typename Convert>
bool compact_on_device(uint8_t *c, uint64_t rows, uint64_t columns, uint64_t stride, Convert convert, cudaStream_t stream) {
    using Out = typename Convert::Out;
    const bool vectors = columns % 4 == 0 && stride % 16 == 0 && reinterpret_cast<uintptr_t>(c) % 16 == 0;
    const uint64_t head = (rows + 7) / 8;
    Out *staging = static_cast<Out *>(scratch(kSlotAux2, head * columns * sizeof(Out)));
    if (!staging) return false;
    bool ok = launch_rows(c, stride, staging, columns, 0, head, 0, vectors, convert, stream) &&
              cuda_ok(cudaMemcpyAsync(c, staging, head * columns * sizeof(Out), cudaMemcpyDeviceToDevice, stream), "compact: head copy");
    for (uint64_t begin = head; ok && begin < rows; begin *= 2)
        ok = launch_rows(c, stride, reinterpret_cast<Out *>(c), columns, begin, begin * 2 < rows ? begin * 2 : rows, begin, vectors,
                         convert, stream);
    return ok;
}

void compact_impl(bool to_i8, void *c, uint64_t rows, uint64_t columns, uint64_t stride, const int32_t *a_norms,
                  const int32_t *b_norms) {
    clear_error();
    if (rows == 0 || columns == 0) return;
    const uint64_t out_bytes = to_i8 ? 1 : 2;
    const MemKind kind = classify(c);
    auto fail = [&]() {
        if (c && kind == kMemHost) std::memset(c, 0xFF, rows * columns * out_bytes);
        else if (c) cudaMemsetAsync(c, 0xFF, rows * columns * out_bytes, current_stream());
    };
    if (!c || (to_i8 && (!a_norms || !b_norms))) { set_error("dots_compact: null pointer%s", ""); return; }
    if (stride % 4 || (stride < columns * 4 && rows > 1) || rows > 0xffffffffull || columns > 0xffffffffull) {
        set_error("dots_compact: the stride must be a multiple of 4 bytes and hold a row%s", "");
        fail();
        return;
    }
    cudaStream_t stream = current_stream();
    const uint64_t span = (rows - 1) * stride + columns * 4;  // bytes of the source matrix, first to last cell
    uint8_t *dev = static_cast<uint8_t *>(c);
    bool ok = true;
    if (kind == kMemHost) {
        dev = static_cast<uint8_t *>(scratch(kSlotC, span));
        if (!dev) { fail(); return; }
        ok = cuda_ok(cudaMemcpyAsync(dev, c, span, cudaMemcpyHostToDevice, stream), "upload of the matrix");
    }
    if (ok && to_i8) {
        float *factors = static_cast<float *>(scratch(kSlotNorms, (rows + columns) * sizeof(float)));
        int32_t *staged = nullptr;
        const int32_t *an = a_norms, *bn = b_norms;
        const bool a_host = classify(a_norms) == kMemHost, b_host = classify(b_norms) == kMemHost;
        if (a_host || b_host) {
            staged = static_cast<int32_t *>(scratch(kSlotAux, (rows + columns) * sizeof(int32_t)));
            ok = staged != nullptr;
            if (ok && a_host) { ok = cuda_ok(cudaMemcpyAsync(staged, a_norms, rows * 4, cudaMemcpyHostToDevice, stream), "upload of norms"); an = staged; }
            if (ok && b_host) { ok = cuda_ok(cudaMemcpyAsync(staged + rows, b_norms, columns * 4, cudaMemcpyHostToDevice, stream), "upload of norms"); bn = staged + rows; }
        }
        ok = ok && factors;
        if (ok) {
            compact_factors_kernel<<<(unsigned)((rows + 255) / 256), 256, 0, stream>>>(an, factors, (uint32_t)rows);
            compact_factors_kernel<<<(unsigned)((columns + 255) / 256), 256, 0, stream>>>(bn, factors + rows, (uint32_t)columns);
            g_launches += 2;
            ok = compact_on_device(dev, rows, columns, stride, ToI8{factors, factors + rows}, stream);
        }
    } else if (ok) {
        ok = compact_on_device(dev, rows, columns, stride, ToBf16{}, stream);
    }
    if (ok && kind == kMemHost) {
        ok = cuda_ok(cudaMemcpyAsync(c, dev, rows * columns * out_bytes, cudaMemcpyDeviceToHost, stream), "download of the result") &&
             cuda_ok(cudaStreamSynchronize(stream), "compact");
    }
    if (!ok) fail();
}

} // namespace
} // namespace nkb

extern "C" {

NKB_API void nk_dots_compact_bf16(void *c, size_t row_count, size_t column_count, size_t c_stride_in_bytes) {
    nkb::compact_impl(false, c, row_count, column_count, c_stride_in_bytes, nullptr, nullptr);
}

NKB_API void nk_dots_compact_i8(void *c, size_t row_count, size_t column_count, size_t c_stride_in_bytes,
                                const int32_t *a_squared_norms, const int32_t *b_squared_norms) {
    nkb::compact_impl(true, c, row_count, column_count, c_stride_in_bytes, a_squared_norms, b_squared_norms);
}

} // extern "C"
