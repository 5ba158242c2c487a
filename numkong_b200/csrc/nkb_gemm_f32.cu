// f32 x f32 -> f64 and f64 x f64 -> f64 packed GEMMs on CUDA cores.
//
// f32: inputs stay f32 in memory, every product and the whole accumulation run in f64, the result is stored as f64.
// This is NumKong's contract for nk_dots_packed_f32 (f64 lane sums, include/numkong/dot/serial.h:305-335; f64 output,
// include/numkong/dots.h:276-277), which no tensor-core kind can meet, so it uses DFMA.
//
// f64: NumKong accumulates with Dot2 (error-free product through FMA, error-free sum through TwoSum, errors gathered
// in a compensation term; include/numkong/scalar/serial.h:128-136) in two lanes - even and odd depth indices
// (include/numkong/dot/serial.h:274-303) - and folds the lanes with include/numkong/reduce/serial.h:33-48. The kernel
// below performs exactly those IEEE operations in exactly that order (explicit round-to-nearest intrinsics keep the
// compiler from contracting or re-associating them), so its dots equal the reference's scalar kernel bit for bit.
//
// The angular / euclidean epilogues follow include/numkong/spatial/serial.h:281-302 in f64.
#include "nkb_internal.h"

namespace nkb {

namespace {

constexpr int kDepth = 16;  // depth slice per shared-memory stage (even, so lane parity = parity inside the slice)

// Accumulator of one output cell.
template <typename In>
struct Cell;
template <>
struct Cell<float> {  // one f64 running sum (the reference's four f32 lanes summed in f64 differ only in rounding order)
    double sum = 0.0;
    __device__ __forceinline__ void add(double a, double b, int) { sum = fma(a, b, sum); }
    __device__ __forceinline__ double total() const { return sum; }
};
template <>
struct Cell<double> {  // two Dot2 lanes
    double sums[2] = {0.0, 0.0}, compensations[2] = {0.0, 0.0};
    __device__ __forceinline__ void add(double a, double b, int lane) {
        const double product = __dmul_rn(a, b);
        const double product_error = __fma_rn(a, b, -product);
        const double running_sum = __dadd_rn(sums[lane], product);
        const double recovered_addend = __dsub_rn(running_sum, sums[lane]);
        const double sum_error = __dadd_rn(__dsub_rn(sums[lane], __dsub_rn(running_sum, recovered_addend)),
                                           __dsub_rn(product, recovered_addend));
        sums[lane] = running_sum;
        compensations[lane] = __dadd_rn(compensations[lane], __dadd_rn(sum_error, product_error));
    }
    __device__ __forceinline__ double total() const {
        double running_sum = 0.0, accumulated_error = 0.0;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
            const double values[2] = {sums[i], compensations[i]};
#pragma unroll
            for (int part = 0; part < 2; ++part) {
                const double tentative_sum = __dadd_rn(running_sum, values[part]);
                const double virtual_addend = __dsub_rn(tentative_sum, running_sum);
                accumulated_error = __dadd_rn(accumulated_error,
                                              __dadd_rn(__dsub_rn(running_sum, __dsub_rn(tentative_sum, virtual_addend)),
                                                        __dsub_rn(values[part], virtual_addend)));
                running_sum = tentative_sum;
            }
        }
        return __dadd_rn(running_sum, accumulated_error);
    }
};

// Register tile of one thread: kTR x kTC output cells, spread with a stride of 16 over the block tile so that a warp's
// shared-memory reads are broadcasts (rows) or consecutive words (columns) and its stores to C are contiguous.
template <typename In> struct TileShape;
template <> struct TileShape<float> { static constexpr int kTR = 8, kTC = 8; };    // 64 f64 accumulators
template <> struct TileShape<double> { static constexpr int kTR = 2, kTC = 4; };   // 8 Dot2 cells = 32 doubles (4 x 4 cells: 220 registers, slower)

template <int kEpi, typename In>
__global__ void __launch_bounds__(256)
gemm_fp64_kernel(const uint8_t *__restrict__ a, uint64_t a_stride, const In *__restrict__ b, uint64_t b_stride_elems,
                 const double *__restrict__ b_norms, const double *__restrict__ a_norms, uint8_t *__restrict__ c,
                 uint64_t c_stride, uint32_t m, uint32_t n, uint32_t k, int32_t tri_diag) {
    constexpr int kTR = TileShape<In>::kTR, kTC = TileShape<In>::kTC;
    constexpr int kTileRows = 16 * kTR, kTileCols = 16 * kTC;
    // Triangular mode (A x A^T): only cells with column >= row + tri_diag are wanted; blocks wholly below that line leave.
    if (tri_diag >= 0 && (blockIdx.x + 1) * kTileCols <= blockIdx.y * kTileRows + (uint32_t)tri_diag) return;
    // Operands are widened to f64 once, on their way into shared memory.
    __shared__ double a_s[kDepth][kTileRows + 2];
    __shared__ double b_s[kDepth][kTileCols + 2];
    const uint32_t m0 = blockIdx.y * kTileRows, n0 = blockIdx.x * kTileCols;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    Cell<In> acc[kTR][kTC];

    // The next depth slice travels from global memory into registers while the current one is being multiplied.
    constexpr int kAPer = kTileRows * kDepth / 256, kBPer = kTileCols * kDepth / 256;
    In a_next[kAPer], b_next[kBPer];
    auto fetch = [&](uint32_t k0) {
#pragma unroll
        for (int t = 0; t < kAPer; ++t) {
            const int idx = threadIdx.x + t * 256, r = idx >> 4, d = idx & 15;
            a_next[t] = (m0 + r < m && k0 + d < k)
                            ? *reinterpret_cast<const In *>(a + (uint64_t)(m0 + r) * a_stride + (uint64_t)(k0 + d) * sizeof(In)) : In(0);
        }
#pragma unroll
        for (int t = 0; t < kBPer; ++t) {
            const int idx = threadIdx.x + t * 256, r = idx >> 4, d = idx & 15;
            b_next[t] = (n0 + r < n && k0 + d < k) ? b[(uint64_t)(n0 + r) * b_stride_elems + k0 + d] : In(0);
        }
    };
    auto stash = [&]() {
#pragma unroll
        for (int t = 0; t < kAPer; ++t) {
            const int idx = threadIdx.x + t * 256;
            a_s[idx & 15][idx >> 4] = (double)a_next[t];
        }
#pragma unroll
        for (int t = 0; t < kBPer; ++t) {
            const int idx = threadIdx.x + t * 256;
            b_s[idx & 15][idx >> 4] = (double)b_next[t];
        }
    };
    fetch(0);
    stash();
    __syncthreads();
    for (uint32_t k0 = 0; k0 < k; k0 += kDepth) {
        const bool more = k0 + kDepth < k;
        if (more) fetch(k0 + kDepth);
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            double av[kTR], bv[kTC];
#pragma unroll
            for (int i = 0; i < kTR; ++i) av[i] = a_s[d][ty + 16 * i];
#pragma unroll
            for (int j = 0; j < kTC; ++j) bv[j] = b_s[d][tx + 16 * j];
#pragma unroll
            for (int i = 0; i < kTR; ++i)
#pragma unroll
                for (int j = 0; j < kTC; ++j) acc[i][j].add(av[i], bv[j], d & 1);
        }
        __syncthreads();
        if (more) {
            stash();
            __syncthreads();
        }
    }

#pragma unroll
    for (int i = 0; i < kTR; ++i) {
        const uint32_t row = m0 + ty + 16 * i;
        if (row >= m) continue;
        double *c_row = reinterpret_cast<double *>(c + (uint64_t)row * c_stride);
        double an = 0.0;
        if constexpr (kEpi != kEpiDot) an = a_norms[row];
#pragma unroll
        for (int j = 0; j < kTC; ++j) {
            const uint32_t col = n0 + tx + 16 * j;
            if (col >= n || (tri_diag >= 0 && col < row + (uint32_t)tri_diag)) continue;
            double v = acc[i][j].total();
            if constexpr (kEpi == kEpiAngular) {
                double product = an * b_norms[col];
                if (product > 0.0) {
                    double r = 1.0 - v / sqrt(product);
                    v = r > 0.0 ? r : 0.0;
                } else v = (v == 0.0) ? 0.0 : 1.0;
            } else if constexpr (kEpi == kEpiEuclidean) {
                double d2 = an + b_norms[col] - 2.0 * v;
                v = d2 > 0.0 ? sqrt(d2) : 0.0;
            }
            if (kEpi != kEpiDot && tri_diag >= 0 && col == row + (uint32_t)tri_diag) v = 0.0;  // distance to itself
            c_row[col] = v;
        }
    }
}

template <typename In>
cudaError_t launch_fp64(int epilogue, const void *a, uint64_t a_stride, const void *b, uint64_t b_stride, const double *b_norms,
                        const double *a_norms, double *c, uint64_t c_stride, uint64_t m, uint64_t n, uint64_t k,
                        cudaStream_t stream, int32_t tri_diag) {
    if (m == 0 || n == 0) return cudaSuccess;
    if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull) return cudaErrorInvalidValue;
    constexpr int kTileRows = 16 * TileShape<In>::kTR, kTileCols = 16 * TileShape<In>::kTC;
    dim3 grid((unsigned)((n + kTileCols - 1) / kTileCols), (unsigned)((m + kTileRows - 1) / kTileRows));
    if (grid.y > 65535) return cudaErrorInvalidValue;
    const uint8_t *ab = static_cast<const uint8_t *>(a);
    const In *bp = static_cast<const In *>(b);
    uint8_t *cb = reinterpret_cast<uint8_t *>(c);
    const uint64_t bse = b_stride / sizeof(In);
    switch (epilogue) {
    case kEpiDot:
        gemm_fp64_kernel<kEpiDot, In><<<grid, 256, 0, stream>>>(ab, a_stride, bp, bse, b_norms, a_norms, cb, c_stride, (uint32_t)m, (uint32_t)n, (uint32_t)k, tri_diag);
        break;
    case kEpiAngular:
        gemm_fp64_kernel<kEpiAngular, In><<<grid, 256, 0, stream>>>(ab, a_stride, bp, bse, b_norms, a_norms, cb, c_stride, (uint32_t)m, (uint32_t)n, (uint32_t)k, tri_diag);
        break;
    case kEpiEuclidean:
        gemm_fp64_kernel<kEpiEuclidean, In><<<grid, 256, 0, stream>>>(ab, a_stride, bp, bse, b_norms, a_norms, cb, c_stride, (uint32_t)m, (uint32_t)n, (uint32_t)k, tri_diag);
        break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

} // namespace

cudaError_t launch_gemm_f32(int epilogue, const float *a, uint64_t a_stride, const float *b, uint64_t b_stride,
                            const double *b_norms, const double *a_norms, double *c, uint64_t c_stride, uint64_t m,
                            uint64_t n, uint64_t k, cudaStream_t stream, int32_t tri_diag) {
    return launch_fp64<float>(epilogue, a, a_stride, b, b_stride, b_norms, a_norms, c, c_stride, m, n, k, stream, tri_diag);
}

cudaError_t launch_gemm_f64(int epilogue, const double *a, uint64_t a_stride, const double *b, uint64_t b_stride,
                            const double *b_norms, const double *a_norms, double *c, uint64_t c_stride, uint64_t m,
                            uint64_t n, uint64_t k, cudaStream_t stream, int32_t tri_diag) {
    return launch_fp64<double>(epilogue, a, a_stride, b, b_stride, b_norms, a_norms, c, c_stride, m, n, k, stream, tri_diag);
}

} // namespace nkb
