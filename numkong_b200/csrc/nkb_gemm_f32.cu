// f32 x f32 -> f64 packed GEMM on CUDA cores: inputs stay f32 in memory, every product and
// the whole accumulation run in f64, the result is stored as f64. This is NumKong's contract for
// nk_dots_packed_f32 (f64 lane sums, include/numkong/dot/serial.h:305-335; f64 output,
// include/numkong/dots.h:276-277), which no tensor-core kind can meet, so it uses DFMA.
// The angular / euclidean epilogues follow include/numkong/spatial/serial.h:281-302 in f64.
#include "nkb_internal.h"

namespace nkb {

namespace {

constexpr int kTile = 64;   // output tile edge
constexpr int kDepth = 16;  // depth slice per shared-memory stage

template <int kEpi>
__global__ void __launch_bounds__(256)
gemm_f32_kernel(const uint8_t *__restrict__ a, uint64_t a_stride, const float *__restrict__ b, uint64_t b_stride_elems,
                const double *__restrict__ b_norms, const double *__restrict__ a_norms, uint8_t *__restrict__ c,
                uint64_t c_stride, uint32_t m, uint32_t n, uint32_t k, int32_t tri_diag) {
    // Triangular mode (A x A^T): only cells with column >= row + tri_diag are wanted; blocks wholly below that line leave.
    if (tri_diag >= 0 && (blockIdx.x + 1) * kTile <= blockIdx.y * kTile + (uint32_t)tri_diag) return;
    __shared__ float a_s[kDepth][kTile + 1];
    __shared__ float b_s[kDepth][kTile + 1];
    const uint32_t m0 = blockIdx.y * kTile, n0 = blockIdx.x * kTile;
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16 threads, 4 x 4 outputs each
    double acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;

    for (uint32_t k0 = 0; k0 < k; k0 += kDepth) {
        // 64 rows x 16 depth values per operand = 1024 values, 4 per thread.
#pragma unroll
        for (int t = 0; t < 4; ++t) {
            int idx = threadIdx.x + t * 256;
            int r = idx >> 4, d = idx & 15;
            float av = 0.0f, bv = 0.0f;
            if (m0 + r < m && k0 + d < k)
                av = *reinterpret_cast<const float *>(a + (uint64_t)(m0 + r) * a_stride + (uint64_t)(k0 + d) * 4);
            if (n0 + r < n && k0 + d < k) bv = b[(uint64_t)(n0 + r) * b_stride_elems + k0 + d];
            a_s[d][r] = av;
            b_s[d][r] = bv;
        }
        __syncthreads();
#pragma unroll
        for (int d = 0; d < kDepth; ++d) {
            double av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) av[i] = (double)a_s[d][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) bv[j] = (double)b_s[d][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fma(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }

#pragma unroll
    for (int i = 0; i < 4; ++i) {
        uint32_t row = m0 + ty * 4 + i;
        if (row >= m) continue;
        double *c_row = reinterpret_cast<double *>(c + (uint64_t)row * c_stride);
        double an = 0.0;
        if constexpr (kEpi != kEpiDot) an = a_norms[row];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            uint32_t col = n0 + tx * 4 + j;
            if (col >= n || (tri_diag >= 0 && col < row + (uint32_t)tri_diag)) continue;
            double v = acc[i][j];
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

} // namespace

cudaError_t launch_gemm_f32(int epilogue, const float *a, uint64_t a_stride, const float *b, uint64_t b_stride,
                            const double *b_norms, const double *a_norms, double *c, uint64_t c_stride, uint64_t m,
                            uint64_t n, uint64_t k, cudaStream_t stream, int32_t tri_diag) {
    if (m == 0 || n == 0) return cudaSuccess;
    if (m > 0x7fffffffull || n > 0x7fffffffull || k > 0x7fffffffull) return cudaErrorInvalidValue;
    dim3 grid((unsigned)((n + kTile - 1) / kTile), (unsigned)((m + kTile - 1) / kTile));
    if (grid.y > 65535) return cudaErrorInvalidValue;
    const uint8_t *ab = reinterpret_cast<const uint8_t *>(a);
    uint8_t *cb = reinterpret_cast<uint8_t *>(c);
    const uint64_t bse = b_stride / 4;
    switch (epilogue) {
    case kEpiDot:
        gemm_f32_kernel<kEpiDot><<<grid, 256, 0, stream>>>(ab, a_stride, b, bse, b_norms, a_norms, cb, c_stride, (uint32_t)m, (uint32_t)n, (uint32_t)k, tri_diag);
        break;
    case kEpiAngular:
        gemm_f32_kernel<kEpiAngular><<<grid, 256, 0, stream>>>(ab, a_stride, b, bse, b_norms, a_norms, cb, c_stride, (uint32_t)m, (uint32_t)n, (uint32_t)k, tri_diag);
        break;
    case kEpiEuclidean:
        gemm_f32_kernel<kEpiEuclidean><<<grid, 256, 0, stream>>>(ab, a_stride, b, bse, b_norms, a_norms, cb, c_stride, (uint32_t)m, (uint32_t)n, (uint32_t)k, tri_diag);
        break;
    default: return cudaErrorInvalidValue;
    }
    return cudaGetLastError();
}

} // namespace nkb
