// Exact device-side decoders of NumKong's storage types to f32
// (value semantics of include/numkong/cast/serial.h:586-1471; bit layouts include/numkong/types.h:785-861).
#pragma once
#include <cstdint>
#include <cuda_fp16.h>
#include "nkb_internal.h"

namespace nkb {

__device__ __forceinline__ float half_bits_to_float(uint16_t bits) {
    return __half2float(__ushort_as_half(bits));
}

// Register form: the code sits in the low bits of a word (higher bits are ignored).
template <uint32_t kDtype>
__device__ __forceinline__ float decode_bits(uint32_t bits);

template <>
__device__ __forceinline__ float decode_bits<kF32>(uint32_t bits) { return __uint_as_float(bits); }
template <>
__device__ __forceinline__ float decode_bits<kBF16>(uint32_t bits) { return __uint_as_float(bits << 16); }
template <>
__device__ __forceinline__ float decode_bits<kF16>(uint32_t bits) { return half_bits_to_float((uint16_t)bits); }
// e5m2 is the top byte of an IEEE half.
template <>
__device__ __forceinline__ float decode_bits<kE5M2>(uint32_t bits) { return half_bits_to_float((uint16_t)((bits & 0xffu) << 8)); }
// e4m3 (bias 7, no infinities, NaN only at S.1111.111): drop sign and the 7 magnitude bits into a half's
// sign / exponent / mantissa fields and rescale by 2^(15-7); half subnormals reproduce e4m3 subnormals exactly.
template <>
__device__ __forceinline__ float decode_bits<kE4M3>(uint32_t bits) {
    if ((bits & 0x7fu) == 0x7fu) return __uint_as_float(((bits & 0x80u) << 24) | 0x7fc00000u);
    return half_bits_to_float((uint16_t)(((bits & 0x80u) << 8) | ((bits & 0x7fu) << 7))) * 256.0f;
}
// e2m3: 0b00SEEMMM, bias 1, no infinities or NaN.
template <>
__device__ __forceinline__ float decode_bits<kE2M3>(uint32_t bits) {
    return half_bits_to_float((uint16_t)(((bits & 0x20u) << 10) | ((bits & 0x1fu) << 7))) * 16384.0f;
}
// e3m2: 0b00SEEEMM, bias 3, no infinities or NaN.
template <>
__device__ __forceinline__ float decode_bits<kE3M2>(uint32_t bits) {
    return half_bits_to_float((uint16_t)(((bits & 0x20u) << 10) | ((bits & 0x1fu) << 8))) * 4096.0f;
}
template <>
__device__ __forceinline__ float decode_bits<kI8>(uint32_t bits) { return (float)(int8_t)bits; }
template <>
__device__ __forceinline__ float decode_bits<kU8>(uint32_t bits) { return (float)(bits & 0xffu); }

// Memory form: little-endian bytes at `p`.
template <uint32_t kDtype>
__device__ __forceinline__ float decode(const uint8_t *p) {
    if constexpr (kDtype == kF32) return decode_bits<kF32>((uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24));
    else if constexpr (kDtype == kBF16 || kDtype == kF16) return decode_bits<kDtype>((uint32_t)p[0] | ((uint32_t)p[1] << 8));
    else return decode_bits<kDtype>(p[0]);
}

} // namespace nkb
