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

template <uint32_t kDtype>
__device__ __forceinline__ float decode(const uint8_t *p);

template <>
__device__ __forceinline__ float decode<kF32>(const uint8_t *p) {
    uint32_t b = (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
    return __uint_as_float(b);
}
template <>
__device__ __forceinline__ float decode<kBF16>(const uint8_t *p) {
    return __uint_as_float(((uint32_t)p[0] << 16) | ((uint32_t)p[1] << 24));
}
template <>
__device__ __forceinline__ float decode<kF16>(const uint8_t *p) {
    return half_bits_to_float((uint16_t)(p[0] | (p[1] << 8)));
}
// e5m2 is the top byte of an IEEE half.
template <>
__device__ __forceinline__ float decode<kE5M2>(const uint8_t *p) {
    return half_bits_to_float((uint16_t)(p[0] << 8));
}
// e4m3 (bias 7, no infinities, NaN only at S.1111.111): drop the 7 magnitude bits into a half's
// exponent/mantissa fields and rescale by 2^(15-7); half subnormals reproduce e4m3 subnormals exactly.
template <>
__device__ __forceinline__ float decode<kE4M3>(const uint8_t *p) {
    uint32_t b = p[0];
    if ((b & 0x7fu) == 0x7fu) return __uint_as_float(0x7fc00000u);
    float mag = half_bits_to_float((uint16_t)((b & 0x7fu) << 7)) * 256.0f;
    return (b & 0x80u) ? -mag : mag;
}
// e2m3: 0b00SEEMMM, bias 1, no infinities or NaN.
template <>
__device__ __forceinline__ float decode<kE2M3>(const uint8_t *p) {
    uint32_t b = p[0];
    float mag = half_bits_to_float((uint16_t)((b & 0x1fu) << 7)) * 16384.0f;
    return (b & 0x20u) ? -mag : mag;
}
// e3m2: 0b00SEEEMM, bias 3, no infinities or NaN.
template <>
__device__ __forceinline__ float decode<kE3M2>(const uint8_t *p) {
    uint32_t b = p[0];
    float mag = half_bits_to_float((uint16_t)((b & 0x1fu) << 8)) * 4096.0f;
    return (b & 0x20u) ? -mag : mag;
}
template <>
__device__ __forceinline__ float decode<kI8>(const uint8_t *p) { return (float)(int8_t)p[0]; }
template <>
__device__ __forceinline__ float decode<kU8>(const uint8_t *p) { return (float)p[0]; }

} // namespace nkb
