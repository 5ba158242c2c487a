// Bandwidth-bound helpers around the GEMM: the B pre-packer, row norms and a re-striding copy.
//
// launch_pack_payload replaces the copy loop of NumKong's nk_dots_pack_<t>
// (include/numkong/dots/serial.h:286-333): instead of a padded row-major copy it writes B
// directly in the shared-memory image tcgen05.mma consumes (see PackedHeader).
// launch_row_sumsq replaces the nk_reduce_moments_<t> calls that append per-row squared norms
// (include/numkong/dots/serial.h:114-180, 326-332) and the per-query norm pass of the batched
// distances (include/numkong/dots/serial.h:2775-2778); with `inverse` it produces the
// 1/sqrt(sumsq) MaxSim stores (include/numkong/maxsim/serial.h:263).
#include "nkb_internal.h"
#include "nkb_decode.cuh"

namespace nkb {

namespace {

// 16 bytes from a possibly unaligned, possibly short source. Bytes at and past `valid` read as zero.
__device__ __forceinline__ uint4 load16_guarded(const uint8_t *src, int64_t valid) {
    if (valid >= 16 && (reinterpret_cast<uintptr_t>(src) & 15u) == 0) return *reinterpret_cast<const uint4 *>(src);
    uint32_t w[4] = {0, 0, 0, 0};
    if (valid > 16) valid = 16;
    for (int i = 0; i < valid; ++i) w[i >> 2] |= (uint32_t)src[i] << ((i & 3) * 8);
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// ---- FP6 operands -------------------------------------------------------------------------------
// NumKong stores e2m3 / e3m2 one value per byte (0b00SEEMMM / 0b00SEEEMM, include/numkong/types.h:803-814).
// tcgen05.mma kind::f8f6f4 does not read that layout, so every 16-byte piece (16 values) is rewritten on
// its way to the tensor cores, in the packer for B and in a copy pass for A. Two rewrites exist:
//   kPieceFp6ToE4M3  each value becomes the e4m3 code of exactly the same number (both 6-bit formats
//                    embed in e4m3: at most 3 mantissa bits, exponents within range), MMA runs as e4m3;
//   kPieceFp6Pack    the 16 six-bit codes are packed back to back into 12 bytes followed by 4 bytes of
//                    padding (the 16-byte-aligned 6-bit operand layout), MMA runs with the native
//                    e2m3 / e3m2 operand formats.
// Zero codes map to zero either way, so zero padding commutes with the rewrite.
__device__ __forceinline__ uint32_t e2m3_to_e4m3(uint32_t c) {
    const uint32_t sign = (c & 0x20u) << 2, e = (c >> 3) & 3u, m = c & 7u;
    if (e == 0) {
        if (m == 0) return sign;
        const uint32_t p = 31u - __clz(m);               // m/8 = 2^(p-3) * (m / 2^p)
        return sign | ((p + 4u) << 3) | ((m << (3u - p)) & 7u);
    }
    return sign | ((e + 6u) << 3) | m;                   // (1 + m/8) * 2^(e-1)
}
__device__ __forceinline__ uint32_t e3m2_to_e4m3(uint32_t c) {
    const uint32_t sign = (c & 0x20u) << 2, e = (c >> 2) & 7u, m = c & 3u;
    if (e == 0) {
        if (m == 0) return sign;
        const uint32_t p = 31u - __clz(m);               // m/16 = 2^(p-4) * (m / 2^p)
        return sign | ((p + 3u) << 3) | ((m << (3u - p)) & 7u);
    }
    return sign | ((e + 4u) << 3) | (m << 1);            // (1 + m/4) * 2^(e-3)
}

// 4-bit operands: the low 8 bytes of `v` hold 16 nibbles, low nibble first; each becomes one i8 (sign extended through
// (x ^ 8) - 8, include/numkong/types.h:1556-1558) or u8.
__device__ __forceinline__ uint4 expand_nibbles(uint4 v, bool is_signed) {
    const uint32_t src[2] = {v.x, v.y};
    uint32_t out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t two_bytes = (src[w >> 1] >> ((w & 1) * 16)) & 0xffffu;
        // nibbles n0..n3 of these two bytes -> bytes 0..3 of the output word
        uint32_t spread = (two_bytes & 0xfu) | ((two_bytes & 0xf0u) << 4) | ((two_bytes & 0xf00u) << 8) | ((two_bytes & 0xf000u) << 12);
        if (is_signed) spread |= ((spread >> 3) & 0x01010101u) * 0xF0u;  // nibbles 8..15 are -8..-1: fill the byte's upper half
        out[w] = spread;
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

// One-bit operands: the low 2 bytes of `v` hold 16 bits, least significant first; each becomes a byte 0 / 1. (Any fixed
// bit order gives the same AND-popcount as long as both operands use it.)
__device__ __forceinline__ uint4 expand_bits(uint4 v) {
    uint32_t out[4];
#pragma unroll
    for (int w = 0; w < 4; ++w) {
        const uint32_t four = (v.x >> (4 * w)) & 0xfu;
        out[w] = (four & 1u) | ((four & 2u) << 7) | ((four & 4u) << 14) | ((four & 8u) << 21);
    }
    return make_uint4(out[0], out[1], out[2], out[3]);
}

__device__ __forceinline__ uint4 transform_piece(uint4 v, int mode) {
    if (mode == kPieceNone) return v;
    if (mode == kPieceI4ToI8 || mode == kPieceU4ToU8) return expand_nibbles(v, mode == kPieceI4ToI8);
    if (mode == kPieceU1ToU8) return expand_bits(v);
    uint32_t w[4] = {v.x, v.y, v.z, v.w};
    if (mode == kPieceE2M3ToE4M3 || mode == kPieceE3M2ToE4M3) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            uint32_t out = 0;
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                uint32_t c = (w[i] >> (8 * b)) & 0x3fu;
                out |= (mode == kPieceE2M3ToE4M3 ? e2m3_to_e4m3(c) : e3m2_to_e4m3(c)) << (8 * b);
            }
            w[i] = out;
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
    // kPieceFp6Pack: value i occupies bits [6i, 6i+6) of the first 96 bits.
    unsigned long long lo = 0, hi = 0;  // lo: bits 0..63, hi: bits 64..95
#pragma unroll
    for (int i = 0; i < 16; ++i) {
        unsigned long long c = (w[i >> 2] >> (8 * (i & 3))) & 0x3fu;
        const int bit = 6 * i;
        if (bit < 64) {
            lo |= c << bit;
            if (bit > 58) hi |= c >> (64 - bit);
        } else hi |= c << (bit - 64);
    }
    return make_uint4((uint32_t)lo, (uint32_t)(lo >> 32), (uint32_t)hi, 0u);
}

// One thread per 16-byte piece of the payload.
template <bool kSwizzled>
__global__ void pack_payload_kernel(const uint8_t *__restrict__ b, uint64_t rows, uint64_t row_bytes, uint64_t stride,
                                    uint4 *__restrict__ payload, uint64_t pieces, uint32_t kblocks, int piece_mode) {
    for (uint64_t o = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; o < pieces; o += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t row, byte_off;
        if constexpr (kSwizzled) {
            uint64_t chunk = o >> 10;            // 1024 pieces per 16 KiB chunk
            uint32_t within = (uint32_t)(o & 1023u);
            uint32_t r = within >> 3;            // row inside the chunk
            uint32_t pos = within & 7u;          // stored piece position
            uint32_t piece = pos ^ (r & 7u);     // logical piece of the 128-byte span
            uint64_t row_block = chunk / kblocks;
            uint64_t kb = chunk % kblocks;
            row = row_block * kChunkRows + r;
            byte_off = kb * kChunkRowBytes + piece * 16u;
        } else {
            uint64_t pieces_per_row = (uint64_t)kblocks * (kChunkRowBytes / 16);
            row = o / pieces_per_row;
            byte_off = (o % pieces_per_row) * 16u;
        }
        // Expanding modes produce a 16-byte piece from 8 (nibbles) or 2 (bits) source bytes.
        const int shift = piece_mode_shift(piece_mode);
        const uint64_t src_off = byte_off >> shift;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (row < rows && src_off < row_bytes) {
            int64_t valid = (int64_t)(row_bytes - src_off);
            if (valid > (16 >> shift)) valid = 16 >> shift;
            v = load16_guarded(b + row * stride + src_off, valid);
        }
        payload[o] = transform_piece(v, piece_mode);
    }
}

// `src` and `dst` may be the same buffer (in-place rewrite with equal pitches), hence no __restrict__.
__global__ void restride_kernel(const uint8_t *src, uint64_t rows, uint64_t row_bytes, uint64_t src_stride,
                                uint4 *dst, uint64_t dst_pieces_per_row, int piece_mode) {
    uint64_t total = rows * dst_pieces_per_row;
    for (uint64_t o = blockIdx.x * (uint64_t)blockDim.x + threadIdx.x; o < total; o += (uint64_t)gridDim.x * blockDim.x) {
        uint64_t row = o / dst_pieces_per_row;
        uint64_t byte_off = (o % dst_pieces_per_row) * 16u;
        const int shift = piece_mode_shift(piece_mode);
        const uint64_t src_off = byte_off >> shift;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (src_off < row_bytes) {
            int64_t valid = (int64_t)(row_bytes - src_off);
            if (valid > (16 >> shift)) valid = 16 >> shift;
            v = load16_guarded(src + row * src_stride + src_off, valid);
        }
        dst[o] = transform_piece(v, piece_mode);
    }
}

template <uint32_t kDtype>
struct SumSq {
    using Acc = double;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) {
        float v = decode<kDtype>(p);
        acc += (double)v * (double)v;
    }
};
template <>
struct SumSq<kF64> {
    using Acc = double;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) {
        double v;
        memcpy(&v, p, 8);
        acc += v * v;
    }
};
template <>
struct SumSq<kI8> {
    using Acc = unsigned long long;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) {
        int v = (int8_t)*p;
        acc += (unsigned long long)(v * v);
    }
};
template <>
struct SumSq<kU8> {
    using Acc = unsigned long long;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) {
        unsigned v = *p;
        acc += (unsigned long long)(v * v);
    }
};

// 4-bit rows: one "element" of the loop below is a byte holding two values.
template <>
struct SumSq<kI4> {
    using Acc = unsigned long long;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) {
        const int lo = (int)((*p & 0xfu) ^ 8u) - 8, hi = (int)((*p >> 4) ^ 8u) - 8;
        acc += (unsigned long long)(lo * lo + hi * hi);
    }
};
template <>
struct SumSq<kU4> {
    using Acc = unsigned long long;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) {
        const unsigned lo = *p & 0xfu, hi = *p >> 4;
        acc += (unsigned long long)(lo * lo + hi * hi);
    }
};

template <>
struct SumSq<kU1> {  // a bit squared is the bit: the "norm" of a bit row is its population count
    using Acc = unsigned long long;
    static __device__ __forceinline__ void add(Acc &acc, const uint8_t *p) { acc += (unsigned long long)__popc((unsigned)*p); }
};

// One warp per row; 16-byte vector loads, four per lane in flight, when the row start allows it.
template <uint32_t kDtype>
__global__ void row_sumsq_kernel(const uint8_t *__restrict__ x, uint64_t rows, uint64_t depth, uint64_t stride,
                                 void *__restrict__ out, int out_mode /*0 native, 1 f32*/, int inverse) {
    constexpr uint32_t eb = kDtype == kF64 ? 8 : kDtype == kF32 ? 4 : (kDtype == kF16 || kDtype == kBF16) ? 2 : 1;
    constexpr uint32_t per16 = 16 / eb;
    using Acc = typename SumSq<kDtype>::Acc;
    const int lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t row = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < rows; row += warps) {
        const uint8_t *p = x + row * stride;
        Acc acc = 0;
        uint64_t done = 0;
        if ((reinterpret_cast<uintptr_t>(p) & 15u) == 0) {
            const uint64_t vecs = depth / per16;
            const uint4 *pv = reinterpret_cast<const uint4 *>(p);
            uint64_t v = lane;
            // Four independent 16-byte loads per lane in flight (2 KiB per warp): one load at a time left the kernel waiting
            // on memory latency at two thirds of the copy rate.
            for (; v + 96 < vecs; v += 128) {
                uint4 q[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) q[u] = __ldg(pv + v + 32 * u);
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const uint8_t *qb = reinterpret_cast<const uint8_t *>(&q[u]);
#pragma unroll
                    for (uint32_t e = 0; e < per16; ++e) SumSq<kDtype>::add(acc, qb + e * eb);
                }
            }
            for (; v < vecs; v += 32) {
                uint4 q = __ldg(pv + v);
                const uint8_t *qb = reinterpret_cast<const uint8_t *>(&q);
#pragma unroll
                for (uint32_t e = 0; e < per16; ++e) SumSq<kDtype>::add(acc, qb + e * eb);
            }
            done = vecs * per16;
        }
        for (uint64_t i = done + lane; i < depth; i += 32) {
            uint8_t tmp[8];
            for (uint32_t bidx = 0; bidx < eb; ++bidx) tmp[bidx] = p[i * eb + bidx];
            SumSq<kDtype>::add(acc, tmp);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) {
            if constexpr (kDtype == kI8 || kDtype == kU8 || kDtype == kI4 || kDtype == kU4 || kDtype == kU1) {
                if (inverse) {
                    float s = (float)acc;
                    static_cast<float *>(out)[row] = s > 0.0f ? (float)(1.0 / sqrt((double)s)) : 0.0f;
                } else if (out_mode == 1) static_cast<float *>(out)[row] = (float)(uint32_t)acc;
                else static_cast<uint32_t *>(out)[row] = (uint32_t)acc;
            } else if constexpr (kDtype == kF32 || kDtype == kF64) {
                if (inverse) static_cast<float *>(out)[row] = acc > 0.0 ? (float)(1.0 / sqrt(acc)) : 0.0f;  // MaxSim keeps f32 inverse norms
                else static_cast<double *>(out)[row] = acc;
            } else {
                float s = (float)acc;
                if (inverse) static_cast<float *>(out)[row] = s > 0.0f ? (float)(1.0 / sqrt((double)s)) : 0.0f;
                else static_cast<float *>(out)[row] = s;
            }
        }
    }
}

inline int grid_for(uint64_t work_items, int block, int cap = 148 * 16) {
    uint64_t g = (work_items + block - 1) / block;
    if (g < 1) g = 1;
    if (g > (uint64_t)cap) g = cap;
    return (int)g;
}

} // namespace

cudaError_t launch_row_sumsq(uint32_t dt, const void *x, uint64_t rows, uint64_t depth, uint64_t stride_bytes,
                             void *out, bool as_f32, bool inverse, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const int block = 256;
    const int grid = grid_for(rows * 32, block);
    const uint8_t *p = static_cast<const uint8_t *>(x);
    const int mode = as_f32 ? 1 : 0, inv = inverse ? 1 : 0;
    if (is_subbyte(dt)) depth = source_row_bytes(dt, depth);  // the kernel walks bytes, several values each
#define NKB_CASE(DT) case DT: row_sumsq_kernel<DT><<<grid, block, 0, stream>>>(p, rows, depth, stride_bytes, out, mode, inv); break
    switch (dt) {
        NKB_CASE(kI8); NKB_CASE(kU8); NKB_CASE(kF32); NKB_CASE(kF16); NKB_CASE(kBF16);
        NKB_CASE(kE4M3); NKB_CASE(kE5M2); NKB_CASE(kE2M3); NKB_CASE(kE3M2); NKB_CASE(kI4); NKB_CASE(kU4); NKB_CASE(kU1); NKB_CASE(kF64);
    default: return cudaErrorInvalidValue;
    }
#undef NKB_CASE
    return cudaGetLastError();
}

cudaError_t launch_pack_payload(uint32_t dt, const void *b, uint64_t rows, uint64_t depth, uint64_t stride_bytes,
                                void *payload, uint64_t rows_padded, uint64_t depth_padded_bytes, int piece_mode,
                                cudaStream_t stream) {
    const uint64_t pieces = rows_padded * depth_padded_bytes / 16;
    const uint32_t kblocks = (uint32_t)(depth_padded_bytes / kChunkRowBytes);
    const int block = 256;
    const int grid = grid_for(pieces, block, 148 * 32);
    const uint64_t row_bytes = source_row_bytes(dt, depth);
    if (is_cuda_core_dtype(dt))
        pack_payload_kernel<false><<<grid, block, 0, stream>>>(static_cast<const uint8_t *>(b), rows, row_bytes, stride_bytes,
                                                               static_cast<uint4 *>(payload), pieces, kblocks, kPieceNone);
    else
        pack_payload_kernel<true><<<grid, block, 0, stream>>>(static_cast<const uint8_t *>(b), rows, row_bytes, stride_bytes,
                                                              static_cast<uint4 *>(payload), pieces, kblocks, piece_mode);
    return cudaGetLastError();
}

cudaError_t launch_restride(const void *src, uint64_t rows, uint64_t row_bytes, uint64_t src_stride, void *dst,
                            uint64_t dst_stride, int piece_mode, cudaStream_t stream) {
    if (rows == 0) return cudaSuccess;
    const uint64_t per_row = dst_stride / 16;
    const int block = 256;
    const int grid = grid_for(rows * per_row, block, 148 * 32);
    restride_kernel<<<grid, block, 0, stream>>>(static_cast<const uint8_t *>(src), rows, row_bytes, src_stride,
                                                static_cast<uint4 *>(dst), per_row, piece_mode);
    return cudaGetLastError();
}

} // namespace nkb
