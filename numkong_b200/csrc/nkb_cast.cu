// Bulk type conversion on the device: nk_cast(from, from_type, n, to, to_type).
//
// Replaces NumKong's nk_cast (include/numkong/cast.h:55, dispatch c/numkong.c:770) with the rules of its scalar
// back end nk_cast_serial (include/numkong/cast/serial.h:2250-2311):
//   * equal types are copied; two unsigned integer types meet in u64, two integer types of which one is signed meet in
//     i64 (a u64 source is reinterpreted, cast/serial.h:2043-2046), every other pair meets in f64;
//   * values travel in batches of eight; u1 is most-significant-bit first and i4 / u4 keep the even index in the HIGH
//     nibble (cast/serial.h:1846-1871, :1966-1995) - the dots family uses the opposite order;
//   * narrowing to a float type goes through f32 and then rounds to nearest even onto the target's grid: e4m3
//     saturates at +-448 and keeps NaN (cast/serial.h:866-943), e5m2 overflows to infinity (:1108-1188), e2m3 / e3m2
//     saturate at +-7.5 / +-28, NaN included (:1340-1416, :1481-1560), f16 and bf16 are IEEE (:669-741, :768-784);
//   * narrowing to an integer: NaN gives 0, the value is clamped to the target's range and rounded to nearest even
//     (cast/serial.h:1583-1666); to i4 / u4: clamped and truncated toward zero; to u1: non-zero gives 1;
//   * integer to integer saturates.
// Pairs the reference leaves undefined (u1 to a signed integer, a signed integer to u4 / u1, complex types) are
// refused: the error text is set and nothing is written. A partial last batch writes only the bytes that hold
// converted values; the missing values of a partial sub-byte batch count as 0. NaN payloads are not preserved.
//
// HBM bound. General kernel: one thread converts one batch - it reads the batch's `from_bits` bytes (1 to 64) with
// 16-byte accesses where the pointers allow, decodes into eight 64-bit hub registers, encodes, and writes `to_bits`
// bytes. Pairs of types of at most 32 bits with a float among them (the quantisation pairs: f32 / f16 / bf16 / fp8 /
// fp6 / i8 / u8) take a kernel compiled for the pair, with f32 in the middle and fully coalesced 16-byte vectors.
#include <cstdio>
#include <cstring>
#include <cuda_fp16.h>
#include "nkb_internal.h"
#include "nkb_decode.cuh"
#include "nkb_host.h"
#include "../../include/numkong_b200.h"

namespace nkb {
namespace {

// Element types of the cast beyond those of the packed path (numerically nk_dtype_t, include/numkong/types.h:923-953).
enum CastDtype : uint32_t { kI16 = 1u << 3, kI32 = 1u << 4, kI64 = 1u << 5, kU16 = 1u << 7, kU32 = 1u << 8, kU64 = 1u << 9 };
enum Family : int { kFamilyNone = 0, kFamilyFloat = 1, kFamilyInt = 2, kFamilyUint = 3 };

__host__ __device__ constexpr int cast_family(uint32_t dt) {
    switch (dt) {
    case kF64: case kF32: case kF16: case kBF16: case kE4M3: case kE5M2: case kE2M3: case kE3M2: return kFamilyFloat;
    case kI4: case kI8: case kI16: case kI32: case kI64: return kFamilyInt;
    case kU1: case kU4: case kU8: case kU16: case kU32: case kU64: return kFamilyUint;
    default: return kFamilyNone;
    }
}
__host__ __device__ constexpr int cast_bits(uint32_t dt) {
    switch (dt) {
    case kF64: case kI64: case kU64: return 64;
    case kF32: case kI32: case kU32: return 32;
    case kF16: case kBF16: case kI16: case kU16: return 16;
    case kI4: case kU4: return 4;
    case kU1: return 1;
    default: return cast_family(dt) == kFamilyNone ? 0 : 8;
    }
}

// ---- small float formats ----

// Round to nearest even of a finite f32 magnitude onto a binary format with `man_bits` fraction bits and exponent
// `bias`; returns the magnitude code, possibly above the format's largest (the caller applies the overflow rule).
__device__ __forceinline__ uint32_t round_to_grid(uint32_t abs_bits, int man_bits, int bias) {
    const int e = (int)(abs_bits >> 23) - 127, emin = 1 - bias;
    if ((abs_bits >> 23) == 0) return 0;  // f32 subnormals lie far below every grid
    const uint32_t sig = 0x800000u | (abs_bits & 0x7fffffu);
    const int shift = 23 - man_bits + (e < emin ? emin - e : 0);
    uint32_t r = 0;
    if (shift <= 24) {
        const uint32_t rem = sig & ((1u << shift) - 1u), half = 1u << (shift - 1);
        r = sig >> shift;
        if (rem > half || (rem == half && (r & 1u))) ++r;
    }
    return ((uint32_t)(e < emin ? 0 : e - emin) << man_bits) + r;
}

__device__ __forceinline__ uint32_t encode_f16(float x) { return __half_as_ushort(__float2half_rn(x)); }
__device__ __forceinline__ uint32_t encode_bf16(float x) {
    const uint32_t u = __float_as_uint(x);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (u >> 16) | 0x40u;
    return (u + 0x7fffu + ((u >> 16) & 1u)) >> 16;
}
__device__ __forceinline__ uint32_t encode_e4m3(float x) {
    const uint32_t u = __float_as_uint(x), sign = (u >> 24) & 0x80u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return sign | 0x7fu;
    const uint32_t code = round_to_grid(a, 3, 7);
    return sign | (code > 0x7eu ? 0x7eu : code);
}
__device__ __forceinline__ uint32_t encode_e5m2(float x) {
    const uint32_t u = __float_as_uint(x), sign = (u >> 24) & 0x80u, a = u & 0x7fffffffu;
    if (a > 0x7f800000u) return sign | 0x7du;
    const uint32_t code = round_to_grid(a, 2, 15);
    return sign | (code > 0x7cu ? 0x7cu : code);
}
__device__ __forceinline__ uint32_t encode_fp6(float x, int man_bits, int bias) {
    const uint32_t u = __float_as_uint(x), sign = (u >> 26) & 0x20u, a = u & 0x7fffffffu;
    const uint32_t code = round_to_grid(a, man_bits, bias);  // infinities and NaN land far above the range
    return sign | (code > 0x1fu ? 0x1fu : code);
}

// ---- integers out of the f64 hub ----
__device__ __forceinline__ long long f64_to_signed(double v, double lo, double hi) {
    if (v != v) return 0;
    return __double2ll_rn(v > hi ? hi : (v < lo ? lo : v));  // round to nearest even; saturates at +-2^63
}
__device__ __forceinline__ unsigned long long f64_to_unsigned(double v, double hi) {
    if (v != v || v <= 0.0) return 0;
    return __double2ull_rn(v > hi ? hi : v);                 // saturates at 2^64 - 1
}
__device__ __forceinline__ long long clamp_ll(long long v, long long lo, long long hi) { return v > hi ? hi : (v < lo ? lo : v); }

// ---- raw batch access: 16 words hold the up to 64 bytes of one batch ----
__device__ __forceinline__ uint32_t raw_byte(const uint32_t (&raw)[16], int l) { return (raw[l >> 2] >> (8 * (l & 3))) & 0xffu; }
__device__ __forceinline__ uint32_t raw_half(const uint32_t (&raw)[16], int l) { return (raw[l >> 1] >> (16 * (l & 1))) & 0xffffu; }
__device__ __forceinline__ unsigned long long raw_quad(const uint32_t (&raw)[16], int l) {
    return (unsigned long long)raw[2 * l] | ((unsigned long long)raw[2 * l + 1] << 32);
}
__device__ __forceinline__ void put_byte(uint32_t (&raw)[16], int l, uint32_t v) { raw[l >> 2] |= (v & 0xffu) << (8 * (l & 3)); }
__device__ __forceinline__ void put_half(uint32_t (&raw)[16], int l, uint32_t v) { raw[l >> 1] |= (v & 0xffffu) << (16 * (l & 1)); }
__device__ __forceinline__ void put_quad(uint32_t (&raw)[16], int l, unsigned long long v) {
    raw[2 * l] = (uint32_t)v;
    raw[2 * l + 1] = (uint32_t)(v >> 32);
}
// Sub-byte source element l of a batch (cast conventions: u1 most significant bit first, even nibble high).
__device__ __forceinline__ long long raw_small(const uint32_t (&raw)[16], uint32_t dt, int l) {
    if (dt == kU1) return (raw[0] >> (7 - l)) & 1u;
    const uint32_t nibble = (raw_byte(raw, l >> 1) >> ((l & 1) ? 0 : 4)) & 0xfu;
    return dt == kI4 ? (long long)((int)(nibble ^ 8u) - 8) : (long long)nibble;
}

template <int kHub>
__global__ void __launch_bounds__(256)
cast_kernel(const uint8_t *__restrict__ from, uint8_t *__restrict__ to, uint64_t n, uint32_t from_type, uint32_t to_type,
            bool from_vectors, bool to_vectors) {
    const uint64_t batch = (uint64_t)blockIdx.x * 256 + threadIdx.x;
    if (batch * 8 >= n) return;
    const int count = n - batch * 8 < 8 ? (int)(n - batch * 8) : 8;
    const int from_bits = cast_bits(from_type), to_bits = cast_bits(to_type);  // = bytes of a full batch
    const uint8_t *src = from + batch * from_bits;
    uint8_t *dst = to + batch * to_bits;

    uint32_t raw[16];
#pragma unroll
    for (int w = 0; w < 16; ++w) raw[w] = 0;
    if (count == 8 && from_vectors) {
        if (from_bits == 1) raw[0] = src[0];
        else if (from_bits == 4) raw[0] = *reinterpret_cast<const uint32_t *>(src);
        else if (from_bits == 8) { const uint2 v = *reinterpret_cast<const uint2 *>(src); raw[0] = v.x, raw[1] = v.y; }
        else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (q * 16 < from_bits) {
                    const uint4 v = reinterpret_cast<const uint4 *>(src)[q];
                    raw[4 * q] = v.x, raw[4 * q + 1] = v.y, raw[4 * q + 2] = v.z, raw[4 * q + 3] = v.w;
                }
        }
    } else {
        const int bytes = (count * from_bits + 7) / 8;
#pragma unroll
        for (int i = 0; i < 64; ++i)
            if (i < bytes) raw[i >> 2] |= (uint32_t)src[i] << (8 * (i & 3));
    }

    // ---- decode into the hub
    double f[8];
    long long s[8];
    unsigned long long u[8];
#pragma unroll
    for (int l = 0; l < 8; ++l) f[l] = 0.0, s[l] = 0, u[l] = 0;
    if (from_bits < 8) {
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            const long long v = raw_small(raw, from_type, l);
            if constexpr (kHub == kFamilyFloat) f[l] = (double)v;
            else if constexpr (kHub == kFamilyInt) s[l] = v;
            else u[l] = (unsigned long long)v;
        }
    } else if constexpr (kHub == kFamilyFloat) {
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            switch (from_type) {
            case kF64: f[l] = __longlong_as_double((long long)raw_quad(raw, l)); break;
            case kF32: f[l] = (double)__uint_as_float(raw[l]); break;
            case kF16: f[l] = (double)decode_bits<kF16>(raw_half(raw, l)); break;
            case kBF16: f[l] = (double)decode_bits<kBF16>(raw_half(raw, l)); break;
            case kE4M3: f[l] = (double)decode_bits<kE4M3>(raw_byte(raw, l)); break;
            case kE5M2: f[l] = (double)decode_bits<kE5M2>(raw_byte(raw, l)); break;
            case kE2M3: f[l] = (double)decode_bits<kE2M3>(raw_byte(raw, l)); break;
            case kE3M2: f[l] = (double)decode_bits<kE3M2>(raw_byte(raw, l)); break;
            case kI64: f[l] = (double)(long long)raw_quad(raw, l); break;
            case kU64: f[l] = (double)raw_quad(raw, l); break;
            case kI32: f[l] = (double)(int)raw[l]; break;
            case kU32: f[l] = (double)raw[l]; break;
            case kI16: f[l] = (double)(short)raw_half(raw, l); break;
            case kU16: f[l] = (double)raw_half(raw, l); break;
            case kI8: f[l] = (double)(signed char)raw_byte(raw, l); break;
            default: f[l] = (double)raw_byte(raw, l); break;
            }
        }
    } else if constexpr (kHub == kFamilyInt) {
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            switch (from_type) {
            case kI64: case kU64: s[l] = (long long)raw_quad(raw, l); break;  // u64: reinterpreted, as the reference does
            case kI32: s[l] = (int)raw[l]; break;
            case kU32: s[l] = raw[l]; break;
            case kI16: s[l] = (short)raw_half(raw, l); break;
            case kU16: s[l] = raw_half(raw, l); break;
            case kI8: s[l] = (signed char)raw_byte(raw, l); break;
            default: s[l] = raw_byte(raw, l); break;
            }
        }
    } else {
#pragma unroll
        for (int l = 0; l < 8; ++l) {
            switch (from_type) {
            case kU64: u[l] = raw_quad(raw, l); break;
            case kU32: u[l] = raw[l]; break;
            case kU16: u[l] = raw_half(raw, l); break;
            default: u[l] = raw_byte(raw, l); break;
            }
        }
    }

    // ---- encode
    uint32_t out[16];
#pragma unroll
    for (int w = 0; w < 16; ++w) out[w] = 0;
#pragma unroll
    for (int l = 0; l < 8; ++l) {
        if (l >= count) break;
        if (to_bits < 8) {
            if (to_type == kU1) {
                const bool set = kHub == kFamilyFloat ? f[l] != 0.0 : u[l] != 0;
                out[0] |= (uint32_t)set << (7 - l);
            } else {
                long long v;
                if (to_type == kI4) v = kHub == kFamilyFloat ? (long long)__double2int_rz(f[l] > 7.0 ? 7.0 : (f[l] < -8.0 ? -8.0 : f[l])) : clamp_ll(s[l], -8, 7);
                else v = kHub == kFamilyFloat ? (long long)__double2int_rz(f[l] > 15.0 ? 15.0 : (f[l] < 0.0 ? 0.0 : f[l])) : (long long)(u[l] > 15 ? 15 : u[l]);
                out[l >> 3] |= ((uint32_t)v & 0xfu) << (8 * ((l >> 1) & 3) + ((l & 1) ? 0 : 4));
            }
        } else if constexpr (kHub == kFamilyFloat) {
            const float narrow = __double2float_rn(f[l]);
            switch (to_type) {
            case kF64: put_quad(out, l, (unsigned long long)__double_as_longlong(f[l])); break;
            case kF32: out[l] = __float_as_uint(narrow); break;
            case kF16: put_half(out, l, encode_f16(narrow)); break;
            case kBF16: put_half(out, l, encode_bf16(narrow)); break;
            case kE4M3: put_byte(out, l, encode_e4m3(narrow)); break;
            case kE5M2: put_byte(out, l, encode_e5m2(narrow)); break;
            case kE2M3: put_byte(out, l, encode_fp6(narrow, 3, 1)); break;
            case kE3M2: put_byte(out, l, encode_fp6(narrow, 2, 3)); break;
            case kI64: put_quad(out, l, (unsigned long long)f64_to_signed(f[l], -9223372036854775808.0, 9223372036854775808.0)); break;
            case kU64: put_quad(out, l, f64_to_unsigned(f[l], 18446744073709551616.0)); break;
            case kI32: out[l] = (uint32_t)f64_to_signed(f[l], -2147483648.0, 2147483647.0); break;
            case kU32: out[l] = (uint32_t)f64_to_unsigned(f[l], 4294967295.0); break;
            case kI16: put_half(out, l, (uint32_t)f64_to_signed(f[l], -32768.0, 32767.0)); break;
            case kU16: put_half(out, l, (uint32_t)f64_to_unsigned(f[l], 65535.0)); break;
            case kI8: put_byte(out, l, (uint32_t)f64_to_signed(f[l], -128.0, 127.0)); break;
            default: put_byte(out, l, (uint32_t)f64_to_unsigned(f[l], 255.0)); break;
            }
        } else if constexpr (kHub == kFamilyInt) {
            switch (to_type) {
            case kI64: put_quad(out, l, (unsigned long long)s[l]); break;
            case kU64: put_quad(out, l, s[l] < 0 ? 0ull : (unsigned long long)s[l]); break;
            case kI32: out[l] = (uint32_t)clamp_ll(s[l], -2147483648ll, 2147483647ll); break;
            case kU32: out[l] = (uint32_t)clamp_ll(s[l], 0, 4294967295ll); break;
            case kI16: put_half(out, l, (uint32_t)clamp_ll(s[l], -32768, 32767)); break;
            case kU16: put_half(out, l, (uint32_t)clamp_ll(s[l], 0, 65535)); break;
            case kI8: put_byte(out, l, (uint32_t)clamp_ll(s[l], -128, 127)); break;
            default: put_byte(out, l, (uint32_t)clamp_ll(s[l], 0, 255)); break;
            }
        } else {
            switch (to_type) {
            case kU64: put_quad(out, l, u[l]); break;
            case kU32: out[l] = u[l] > 4294967295ull ? 4294967295u : (uint32_t)u[l]; break;
            case kU16: put_half(out, l, u[l] > 65535ull ? 65535u : (uint32_t)u[l]); break;
            default: put_byte(out, l, u[l] > 255ull ? 255u : (uint32_t)u[l]); break;
            }
        }
    }

    if (count == 8 && to_vectors) {
        if (to_bits == 1) dst[0] = (uint8_t)out[0];
        else if (to_bits == 4) *reinterpret_cast<uint32_t *>(dst) = out[0];
        else if (to_bits == 8) *reinterpret_cast<uint2 *>(dst) = make_uint2(out[0], out[1]);
        else {
#pragma unroll
            for (int q = 0; q < 4; ++q)
                if (q * 16 < to_bits) reinterpret_cast<uint4 *>(dst)[q] = make_uint4(out[4 * q], out[4 * q + 1], out[4 * q + 2], out[4 * q + 3]);
        }
    } else {
        const int bytes = (count * to_bits + 7) / 8;
#pragma unroll
        for (int i = 0; i < 64; ++i)
            if (i < bytes) dst[i] = (uint8_t)(out[i >> 2] >> (8 * (i & 3)));
    }
}

// ---- fast path: both types at most 32 bits wide and at least one of them a float ------------------------------------
// Such a pair never needs more than f32 in the middle: every source value is exactly an f32, and the reference narrows
// the f64 hub value to f32 before it encodes a small float anyway; for the 8-bit integer targets clamping and rounding
// an f32 gives what clamping and rounding its f64 image gives. With both types known at compile time a thread moves one
// 16-byte vector of the wider type per step and every access of a warp is contiguous.
// Two f32 values to two 8-bit codes with the conversion unit (round to nearest even, saturating to the largest finite
// value): low byte = first value. The reference's rules that differ from the instruction's are patched per value:
// a NaN keeps its sign (0x7F / 0x7D / largest value), and e5m2 overflows to infinity from the rounding boundary 61440 on.
#define NKB_HW_PAIR(NAME, FORMAT)                                                                          \
    __device__ __forceinline__ uint32_t NAME(float first, float second) {                                  \
        unsigned short packed;                                                                             \
        asm("cvt.rn.satfinite." FORMAT ".f32 %0, %1, %2;" : "=h"(packed) : "f"(second), "f"(first));      \
        return packed;                                                                                     \
    }
NKB_HW_PAIR(hw_pair_e4m3, "e4m3x2")
NKB_HW_PAIR(hw_pair_e5m2, "e5m2x2")
NKB_HW_PAIR(hw_pair_e2m3, "e2m3x2")
NKB_HW_PAIR(hw_pair_e3m2, "e3m2x2")
#undef NKB_HW_PAIR

__device__ __forceinline__ uint32_t patch_e4m3(uint32_t code, float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x7fffffffu) > 0x7f800000u ? ((u >> 24) & 0x80u) | 0x7fu : code;
}
__device__ __forceinline__ uint32_t patch_e5m2(uint32_t code, float x) {
    const uint32_t u = __float_as_uint(x), a = u & 0x7fffffffu, sign = (u >> 24) & 0x80u;
    return a > 0x7f800000u ? sign | 0x7du : (a >= 0x47700000u ? sign | 0x7cu : code);
}
__device__ __forceinline__ uint32_t patch_fp6(uint32_t code, float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x7fffffffu) > 0x7f800000u ? ((u >> 26) & 0x20u) | 0x1fu : code;
}

template <uint32_t kType> struct Scalar32;
template <> struct Scalar32<kF32> {
    static constexpr int kBytes = 4;
    static __device__ __forceinline__ float decode(uint32_t b) { return __uint_as_float(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return __float_as_uint(x); }
    static __device__ __forceinline__ uint32_t encode2(float a, float) { return encode(a); }
};
template <> struct Scalar32<kF16> {
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ float decode(uint32_t b) { return decode_bits<kF16>(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return encode_f16(x); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) { return encode(a) | (encode(b) << (8 * kBytes)); }
};
template <> struct Scalar32<kBF16> {
    static constexpr int kBytes = 2;
    static __device__ __forceinline__ float decode(uint32_t b) { return decode_bits<kBF16>(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return encode_bf16(x); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) { return encode(a) | (encode(b) << (8 * kBytes)); }
};
template <> struct Scalar32<kE4M3> {
    static constexpr int kBytes = 1;
    static __device__ __forceinline__ float decode(uint32_t b) { return decode_bits<kE4M3>(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return encode_e4m3(x); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) {
        const uint32_t packed = hw_pair_e4m3(a, b);
        return patch_e4m3(packed & 0xffu, a) | (patch_e4m3(packed >> 8, b) << 8);
    }
};
template <> struct Scalar32<kE5M2> {
    static constexpr int kBytes = 1;
    static __device__ __forceinline__ float decode(uint32_t b) { return decode_bits<kE5M2>(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return encode_e5m2(x); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) {
        const uint32_t packed = hw_pair_e5m2(a, b);
        return patch_e5m2(packed & 0xffu, a) | (patch_e5m2(packed >> 8, b) << 8);
    }
};
template <> struct Scalar32<kE2M3> {
    static constexpr int kBytes = 1;
    static __device__ __forceinline__ float decode(uint32_t b) { return decode_bits<kE2M3>(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return encode_fp6(x, 3, 1); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) {
        const uint32_t packed = hw_pair_e2m3(a, b);
        return patch_fp6(packed & 0xffu, a) | (patch_fp6(packed >> 8, b) << 8);
    }
};
template <> struct Scalar32<kE3M2> {
    static constexpr int kBytes = 1;
    static __device__ __forceinline__ float decode(uint32_t b) { return decode_bits<kE3M2>(b); }
    static __device__ __forceinline__ uint32_t encode(float x) { return encode_fp6(x, 2, 3); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) {
        const uint32_t packed = hw_pair_e3m2(a, b);
        return patch_fp6(packed & 0xffu, a) | (patch_fp6(packed >> 8, b) << 8);
    }
};
template <> struct Scalar32<kI8> {
    static constexpr int kBytes = 1;
    static __device__ __forceinline__ float decode(uint32_t b) { return (float)(signed char)b; }
    static __device__ __forceinline__ uint32_t encode(float x) { return x != x ? 0u : (uint32_t)__float2int_rn(fminf(fmaxf(x, -128.0f), 127.0f)) & 0xffu; }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) { return encode(a) | (encode(b) << (8 * kBytes)); }
};
template <> struct Scalar32<kU8> {
    static constexpr int kBytes = 1;
    static __device__ __forceinline__ float decode(uint32_t b) { return (float)(b & 0xffu); }
    static __device__ __forceinline__ uint32_t encode(float x) { return x != x ? 0u : (uint32_t)__float2int_rn(fminf(fmaxf(x, 0.0f), 255.0f)); }
    static __device__ __forceinline__ uint32_t encode2(float a, float b) { return encode(a) | (encode(b) << (8 * kBytes)); }
};

template <int kBytes>
__device__ __forceinline__ uint32_t vector_element(const uint32_t (&words)[4], int j) {
    if constexpr (kBytes == 4) return words[j];
    else if constexpr (kBytes == 2) return (words[j >> 1] >> (16 * (j & 1))) & 0xffffu;
    else return (words[j >> 2] >> (8 * (j & 3))) & 0xffu;
}
template <int kBytes>
__device__ __forceinline__ void set_vector_element(uint32_t (&words)[4], int j, uint32_t v) {
    if constexpr (kBytes == 4) words[j] = v;
    else if constexpr (kBytes == 2) words[j >> 1] |= (v & 0xffffu) << (16 * (j & 1));
    else words[j >> 2] |= (v & 0xffu) << (8 * (j & 3));
}
template <int kVectorBytes>
__device__ __forceinline__ void load_vector(const uint8_t *p, uint32_t (&words)[4]) {
    if constexpr (kVectorBytes == 16) { const uint4 v = *reinterpret_cast<const uint4 *>(p); words[0] = v.x, words[1] = v.y, words[2] = v.z, words[3] = v.w; }
    else if constexpr (kVectorBytes == 8) { const uint2 v = *reinterpret_cast<const uint2 *>(p); words[0] = v.x, words[1] = v.y; }
    else words[0] = *reinterpret_cast<const uint32_t *>(p);
}
template <int kVectorBytes>
__device__ __forceinline__ void store_vector(uint8_t *p, const uint32_t (&words)[4]) {
    if constexpr (kVectorBytes == 16) *reinterpret_cast<uint4 *>(p) = make_uint4(words[0], words[1], words[2], words[3]);
    else if constexpr (kVectorBytes == 8) *reinterpret_cast<uint2 *>(p) = make_uint2(words[0], words[1]);
    else *reinterpret_cast<uint32_t *>(p) = words[0];
}

template <uint32_t kFrom, uint32_t kTo>
__global__ void __launch_bounds__(256) cast_pair_kernel(const uint8_t *__restrict__ from, uint8_t *__restrict__ to, uint64_t n) {
    using In = Scalar32<kFrom>;
    using Out = Scalar32<kTo>;
    constexpr int kWide = In::kBytes > Out::kBytes ? In::kBytes : Out::kBytes;
    constexpr int kNarrow = In::kBytes < Out::kBytes ? In::kBytes : Out::kBytes;
    // Values per vector: the wider side moves 16 bytes, unless that leaves the narrower side under 4 bytes.
    constexpr int kVec = (16 / kWide) * kNarrow >= 4 ? 16 / kWide : 4 / kNarrow;
    static_assert(kVec * kWide <= 16 && kVec * kNarrow >= 4, "vector shape");
    const uint64_t vectors = n / kVec;
    for (uint64_t i = (uint64_t)blockIdx.x * 256 + threadIdx.x; i < vectors; i += (uint64_t)gridDim.x * 256) {
        uint32_t in_words[4] = {0, 0, 0, 0}, out_words[4] = {0, 0, 0, 0};
        load_vector<kVec * In::kBytes>(from + i * (kVec * In::kBytes), in_words);
        if constexpr (Out::kBytes == 4) {
#pragma unroll
            for (int j = 0; j < kVec; ++j) out_words[j] = Out::encode(In::decode(vector_element<In::kBytes>(in_words, j)));
        } else {  // two values per step: the 8-bit float formats convert in pairs
#pragma unroll
            for (int j = 0; j < kVec; j += 2) {
                const uint32_t two = Out::encode2(In::decode(vector_element<In::kBytes>(in_words, j)),
                                                  In::decode(vector_element<In::kBytes>(in_words, j + 1)));
                if constexpr (Out::kBytes == 2) out_words[j >> 1] = two;
                else out_words[j >> 2] |= two << (16 * ((j >> 1) & 1));
            }
        }
        store_vector<kVec * Out::kBytes>(to + i * (kVec * Out::kBytes), out_words);
    }
    // ragged end: fewer than kVec values, one thread each
    const uint64_t done = vectors * kVec;
    if (blockIdx.x == 0 && threadIdx.x < n - done) {
        const uint64_t e = done + threadIdx.x;
        // Whole-element accesses (the launch checked that both buffers are aligned to a vector). Storing the two bytes of
        // a fresh binary16 conversion one by one came out wrong on sm_100a with nvcc 12.9: the low byte held the VALUE
        // converted to an integer.
        uint32_t bits;
        if constexpr (In::kBytes == 4) bits = reinterpret_cast<const uint32_t *>(from)[e];
        else if constexpr (In::kBytes == 2) bits = reinterpret_cast<const uint16_t *>(from)[e];
        else bits = from[e];
        const uint32_t code = Out::encode(In::decode(bits));
        if constexpr (Out::kBytes == 4) reinterpret_cast<uint32_t *>(to)[e] = code;
        else if constexpr (Out::kBytes == 2) reinterpret_cast<uint16_t *>(to)[e] = (uint16_t)code;
        else to[e] = (uint8_t)code;
    }
}

template <uint32_t kFrom, uint32_t kTo>
bool launch_pair(const uint8_t *from, uint8_t *to, uint64_t n, cudaStream_t stream) {
    if constexpr (kFrom == kTo || ((kFrom == kI8 || kFrom == kU8) && (kTo == kI8 || kTo == kU8))) return false;
    else {
        using In = Scalar32<kFrom>;
        using Out = Scalar32<kTo>;
        constexpr int kWide = In::kBytes > Out::kBytes ? In::kBytes : Out::kBytes;
        constexpr int kNarrow = In::kBytes < Out::kBytes ? In::kBytes : Out::kBytes;
        constexpr int kVec = (16 / kWide) * kNarrow >= 4 ? 16 / kWide : 4 / kNarrow;
        if (reinterpret_cast<uintptr_t>(from) % (kVec * In::kBytes) || reinterpret_cast<uintptr_t>(to) % (kVec * Out::kBytes)) return false;
        const uint64_t vectors = n / kVec, wanted = (vectors + 255) / 256;
        const unsigned grid = (unsigned)(wanted < 1 ? 1 : (wanted > 148ull * 32 ? 148ull * 32 : wanted));
        cast_pair_kernel<kFrom, kTo><<<grid, 256, 0, stream>>>(from, to, n);
        return true;
    }
}
template <uint32_t kFrom>
bool launch_pair_to(uint32_t to_type, const uint8_t *from, uint8_t *to, uint64_t n, cudaStream_t stream) {
    switch (to_type) {
    case kF32: return launch_pair<kFrom, kF32>(from, to, n, stream);
    case kF16: return launch_pair<kFrom, kF16>(from, to, n, stream);
    case kBF16: return launch_pair<kFrom, kBF16>(from, to, n, stream);
    case kE4M3: return launch_pair<kFrom, kE4M3>(from, to, n, stream);
    case kE5M2: return launch_pair<kFrom, kE5M2>(from, to, n, stream);
    case kE2M3: return launch_pair<kFrom, kE2M3>(from, to, n, stream);
    case kE3M2: return launch_pair<kFrom, kE3M2>(from, to, n, stream);
    case kI8: return launch_pair<kFrom, kI8>(from, to, n, stream);
    case kU8: return launch_pair<kFrom, kU8>(from, to, n, stream);
    default: return false;
    }
}
// Launches the compile-time pair kernel when there is one for (from_type, to_type) and the pointers allow vectors.
bool launch_fast_pair(uint32_t from_type, uint32_t to_type, const uint8_t *from, uint8_t *to, uint64_t n, cudaStream_t stream) {
    switch (from_type) {
    case kF32: return launch_pair_to<kF32>(to_type, from, to, n, stream);
    case kF16: return launch_pair_to<kF16>(to_type, from, to, n, stream);
    case kBF16: return launch_pair_to<kBF16>(to_type, from, to, n, stream);
    case kE4M3: return launch_pair_to<kE4M3>(to_type, from, to, n, stream);
    case kE5M2: return launch_pair_to<kE5M2>(to_type, from, to, n, stream);
    case kE2M3: return launch_pair_to<kE2M3>(to_type, from, to, n, stream);
    case kE3M2: return launch_pair_to<kE3M2>(to_type, from, to, n, stream);
    case kI8: return launch_pair_to<kI8>(to_type, from, to, n, stream);
    case kU8: return launch_pair_to<kU8>(to_type, from, to, n, stream);
    default: return false;
    }
}

void cast_impl(const void *from, uint32_t from_type, uint64_t n, void *to, uint32_t to_type) {
    clear_error();
    if (n == 0) return;
    const int from_family = cast_family(from_type), to_family = cast_family(to_type);
    if (!from_family || !to_family) { set_error("cast: element type is not a real scalar type%s", ""); return; }
    if (!from || !to) { set_error("cast: null pointer%s", ""); return; }
    const int hub = (from_family == kFamilyUint && to_family == kFamilyUint) ? kFamilyUint
                    : (from_family != kFamilyFloat && to_family != kFamilyFloat) ? kFamilyInt : kFamilyFloat;
    if (from_type != to_type && hub == kFamilyInt && (from_type == kU1 || to_type == kU4 || to_type == kU1)) {
        set_error("cast: the reference defines no conversion between these two integer types%s", "");
        return;
    }
    const uint64_t from_bytes = (n * (uint64_t)cast_bits(from_type) + 7) / 8, to_bytes = (n * (uint64_t)cast_bits(to_type) + 7) / 8;
    const MemKind from_kind = classify(from), to_kind = classify(to);
    cudaStream_t stream = current_stream();
    bool ok = true;
    const uint8_t *src = static_cast<const uint8_t *>(from);
    uint8_t *dst = static_cast<uint8_t *>(to);
    if (from_type == to_type) {  // a copy, whatever sides the two buffers are on
        ok = cuda_ok(cudaMemcpyAsync(to, from, from_bytes, cudaMemcpyDefault, stream), "cast: copy");
        if (ok && (from_kind == kMemHost || to_kind == kMemHost)) ok = cuda_ok(cudaStreamSynchronize(stream), "cast");
        return;
    }
    if (from_kind == kMemHost) {
        uint8_t *staged = static_cast<uint8_t *>(scratch(kSlotA, from_bytes));
        ok = staged && cuda_ok(cudaMemcpyAsync(staged, from, from_bytes, cudaMemcpyHostToDevice, stream), "cast: upload");
        src = staged;
    }
    if (ok && to_kind == kMemHost) {
        dst = static_cast<uint8_t *>(scratch(kSlotC, to_bytes));
        ok = dst != nullptr;
    }
    if (ok) {
        auto aligned = [](const void *p, int batch_bytes) { return reinterpret_cast<uintptr_t>(p) % (batch_bytes < 16 ? batch_bytes : 16) == 0; };
        const bool from_vectors = aligned(src, cast_bits(from_type)), to_vectors = aligned(dst, cast_bits(to_type));
        const uint64_t batches = (n + 7) / 8, blocks = (batches + 255) / 256;
        if (blocks > 0x7fffffffull) { set_error("cast: too many values for one call%s", ""); return; }
        if (launch_fast_pair(from_type, to_type, src, dst, n, stream)) {}
        else if (hub == kFamilyFloat) cast_kernel<kFamilyFloat><<<(unsigned)blocks, 256, 0, stream>>>(src, dst, n, from_type, to_type, from_vectors, to_vectors);
        else if (hub == kFamilyInt) cast_kernel<kFamilyInt><<<(unsigned)blocks, 256, 0, stream>>>(src, dst, n, from_type, to_type, from_vectors, to_vectors);
        else cast_kernel<kFamilyUint><<<(unsigned)blocks, 256, 0, stream>>>(src, dst, n, from_type, to_type, from_vectors, to_vectors);
        g_launches++;
        ok = cuda_ok(cudaGetLastError(), "cast kernel");
    }
    if (ok && to_kind == kMemHost)
        ok = cuda_ok(cudaMemcpyAsync(to, dst, to_bytes, cudaMemcpyDeviceToHost, stream), "cast: download") &&
             cuda_ok(cudaStreamSynchronize(stream), "cast");
    if (!ok && to_kind == kMemHost) std::memset(to, 0xFF, to_bytes);
}

} // namespace
} // namespace nkb

extern "C" NKB_API void nk_cast(const void *from, uint32_t from_type, size_t n, void *to, uint32_t to_type) {
    nkb::cast_impl(from, from_type, n, to, to_type);
}
