// Sum and sum of squares of a strided vector on the device: nk_reduce_moments_<t>(data, count, stride, &sum, &sumsq).
//
// Replaces NumKong's nk_reduce_moments_<t> (include/numkong/reduce.h:120-279; scalar back end
// include/numkong/reduce/serial.h:52-416) for the nineteen real scalar types. Result types as there: f64 for f32 /
// f64, f32 for the 16-bit and smaller floats, i64 + u64 for signed integers, u64 + u64 for unsigned ones.
//   * Integers are exact and follow the reference's overflow rules: 8 / 16-bit and sub-byte types add in 64 bits;
//     i32 / i64 keep the sum in 128 bits and saturate it to i64 at the end; their squares (an i64 square saturates
//     at 2^63 - 1, a u64 square at 2^64 - 1) and the u32 / u64 sums are added with unsigned saturation - adding
//     non-negative terms with saturation gives min(true total, 2^64 - 1) in any order, so 128-bit partial sums that
//     are saturated once at the end give the same bits.
//   * Sub-byte types count whole bytes (the count is rounded up), `stride` steps from byte to byte.
//   * Floats: the reference runs a compensated (Neumaier) serial sum in the result type, which is the correctly
//     rounded sum to within an ulp. Here every thread adds in f64 (f64 inputs: compensated TwoSum in f64; squares
//     rounded to f64 first as the reference does), partial sums are combined in a fixed order in f64, and the total
//     is rounded once to the result type: deterministic, and within an ulp of the reference except under heavy
//     cancellation, where both are within ~2^-50 of the sum of magnitudes.
//
// HBM bound: one pass over the data by up to 148 x 8 blocks, per-block partials in a staging buffer, a one-block
// kernel that folds them and writes the two results, which travel to the host when the result pointers are host memory.
#include <cstdio>
#include <cstring>
#include <type_traits>
#include <cuda_fp16.h>
#include "nkb_internal.h"
#include "nkb_decode.cuh"
#include "nkb_host.h"
#include "../../include/numkong_b200.h"

namespace nkb {
namespace {

enum MomentsDtype : uint32_t { kI16 = 1u << 3, kI32 = 1u << 4, kI64 = 1u << 5, kU16 = 1u << 7, kU32 = 1u << 8, kU64 = 1u << 9 };

// 128-bit accumulator (two's complement when used for signed sums).
struct Wide {
    unsigned long long lo = 0, hi = 0;
    __device__ __forceinline__ void add_unsigned(unsigned long long v) {
        lo += v;
        hi += lo < v;
    }
    __device__ __forceinline__ void add_signed(long long v) {
        const unsigned long long u = (unsigned long long)v;
        lo += u;
        hi += (unsigned long long)(lo < u) + (unsigned long long)(v >> 63);
    }
    __device__ __forceinline__ void add(const Wide &o) {
        lo += o.lo;
        hi += o.hi + (lo < o.lo);
    }
};

// Four 64-bit words per partial result: what they hold depends on the type's family.
//   floats:   [0] sum, [1] sum compensation, [2] sum of squares, [3] its compensation (f64 bit patterns)
//   integers: [0],[1] = 128-bit sum, [2],[3] = 128-bit sum of squares
struct Partial { unsigned long long w[4]; };

template <uint32_t kType> struct Moments;

// ---- floats: f64 running sums ----
struct FloatState {
    double sum = 0.0, sum_error = 0.0, squares = 0.0, squares_error = 0.0;
    __device__ __forceinline__ void combine(const FloatState &o) {
        // TwoSum keeps what the f64 addition of two partial sums drops
        double t = sum + o.sum, v = t - sum;
        sum_error += ((sum - (t - v)) + (o.sum - v)) + o.sum_error;
        sum = t;
        t = squares + o.squares, v = t - squares;
        squares_error += ((squares - (t - v)) + (o.squares - v)) + o.squares_error;
        squares = t;
    }
    __device__ __forceinline__ Partial pack() const {
        Partial p;
        p.w[0] = (unsigned long long)__double_as_longlong(sum), p.w[1] = (unsigned long long)__double_as_longlong(sum_error);
        p.w[2] = (unsigned long long)__double_as_longlong(squares), p.w[3] = (unsigned long long)__double_as_longlong(squares_error);
        return p;
    }
    static __device__ __forceinline__ FloatState unpack(const Partial &p) {
        FloatState s;
        s.sum = __longlong_as_double((long long)p.w[0]), s.sum_error = __longlong_as_double((long long)p.w[1]);
        s.squares = __longlong_as_double((long long)p.w[2]), s.squares_error = __longlong_as_double((long long)p.w[3]);
        return s;
    }
};
template <int kBytesPerValue, bool kCompensated>
struct FloatMoments {
    using State = FloatState;
    static constexpr int kBytes = kBytesPerValue;
    static constexpr bool kIsFloat = true;
    static __device__ __forceinline__ void add_value(State &s, double v) {
        if constexpr (kCompensated) {
            double t = s.sum + v, u = t - s.sum;
            s.sum_error += (s.sum - (t - u)) + (v - u);
            s.sum = t;
            const double sq = __dmul_rn(v, v);
            t = s.squares + sq, u = t - s.squares;
            s.squares_error += (s.squares - (t - u)) + (sq - u);
            s.squares = t;
        } else {
            s.sum += v;
            s.squares = fma(v, v, s.squares);
        }
    }
};
template <> struct Moments<kF64> : FloatMoments<8, true> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, __longlong_as_double((long long)bits)); }
};
template <> struct Moments<kF32> : FloatMoments<4, false> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, (double)__uint_as_float((uint32_t)bits)); }
};
template <> struct Moments<kF16> : FloatMoments<2, false> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, (double)decode_bits<kF16>((uint32_t)bits)); }
};
template <> struct Moments<kBF16> : FloatMoments<2, false> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, (double)decode_bits<kBF16>((uint32_t)bits)); }
};
// The sixteen values of a vector of e4m3 / e2m3 / e3m2 add up EXACTLY in f32 (values are multiples of 2^-9 / 2^-3 / 2^-4
// and sixteen of them stay below 2^13 / 2^7 / 2^9), and so do their squares for the two 6-bit formats. e4m3 squares span
// 36 bits, so they are added in two classes: |v| < 2 (multiples of 2^-18 below 4: exact over the sixteen values) and
// |v| >= 2 (multiples of 2^-4 up to 2^17.6: exact over the four values of a word). Only these partial sums go through
// f64 additions. Two codes are decoded at a time: their bits are moved into a binary16 pair (value / kScale), which
// converts to f32 exactly; the power-of-two scale is applied to the partial sums.
struct E4M3Format {
    static constexpr float kScale = 256.0f;
    static __device__ __forceinline__ uint32_t half_pair(uint32_t x) { return (x & 0x80008000u) | ((x >> 1) & 0x3f803f80u); }
    static __device__ __forceinline__ float decode(uint32_t c) { return decode_bits<kE4M3>(c); }
};
struct E2M3Format {
    static constexpr float kScale = 16384.0f;
    static __device__ __forceinline__ uint32_t half_pair(uint32_t x) { return ((x & 0x20002000u) << 2) | ((x >> 1) & 0x0f800f80u); }
    static __device__ __forceinline__ float decode(uint32_t c) { return decode_bits<kE2M3>(c); }
};
struct E3M2Format {
    static constexpr float kScale = 4096.0f;
    static __device__ __forceinline__ uint32_t half_pair(uint32_t x) { return ((x & 0x20002000u) << 2) | (x & 0x1f001f00u); }
    static __device__ __forceinline__ float decode(uint32_t c) { return decode_bits<kE3M2>(c); }
};
// Codes 2p and 2p+1 of a word as f32 values divided by kScale.
template <typename Format>
__device__ __forceinline__ float2 scaled_pair(uint32_t word, int p) {
    const uint32_t x = __byte_perm(word, 0u, p ? 0x3424u : 0x1404u);  // the two codes in the high bytes of the two halves
    const uint32_t bits = Format::half_pair(x);
    return __half22float2(*reinterpret_cast<const __half2 *>(&bits));
}

template <> struct Moments<kE4M3> : FloatMoments<1, false> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, (double)E4M3Format::decode((uint32_t)bits)); }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        float total = 0.0f, small_squares = 0.0f, large_squares[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        uint32_t nan_bytes = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            nan_bytes |= ((w[i] & 0x7f7f7f7fu) + 0x01010101u) & 0x80808080u;  // a byte of 0x7F / 0xFF is the format's NaN
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const float2 v = scaled_pair<E4M3Format>(w[i], p);
                const uint32_t large_bits = w[i] >> (16 * p);                  // bit 6 of a code: exponent field >= 8, |v| >= 2
                const float large_x = (large_bits & 0x40u) ? v.x : 0.0f, large_y = (large_bits & 0x4000u) ? v.y : 0.0f;
                const float small_x = v.x - large_x, small_y = v.y - large_y;
                total += v.x, total += v.y;
                small_squares = fmaf(small_x, small_x, small_squares), small_squares = fmaf(small_y, small_y, small_squares);
                large_squares[i] = fmaf(large_x, large_x, large_squares[i]), large_squares[i] = fmaf(large_y, large_y, large_squares[i]);
            }
        }
        if (nan_bytes) total = __uint_as_float(0x7fc00000u), small_squares = total;
        constexpr double kScale = E4M3Format::kScale, kScaleSquared = kScale * kScale;
        s.sum += (double)total * kScale;
        s.squares += (double)small_squares * kScaleSquared;
#pragma unroll
        for (int i = 0; i < 4; ++i) s.squares += (double)large_squares[i] * kScaleSquared;
    }
};
// An e5m2 code is the high byte of a binary16 value: two codes become a binary16 pair with one byte permutation and are
// then added in f64 in the same order as the one-by-one path (the sums are the same bits; squares of e5m2 values span 60
// binades, so no f32 partial sum of them is exact).
template <> struct Moments<kE5M2> : FloatMoments<1, false> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, (double)decode_bits<kE5M2>((uint32_t)bits)); }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const uint32_t bits = __byte_perm(w[i], 0u, p ? 0x3424u : 0x1404u);  // the two codes in the high bytes of the two halves
                const float2 v = __half22float2(*reinterpret_cast<const __half2 *>(&bits));
                add_value(s, (double)v.x);
                add_value(s, (double)v.y);
            }
    }
};
template <typename Format>
struct Fp6Moments : FloatMoments<1, false> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { add_value(s, (double)Format::decode((uint32_t)bits)); }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        float total = 0.0f, squares = 0.0f;
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
            for (int p = 0; p < 2; ++p) {
                const float2 v = scaled_pair<Format>(w[i], p);
                total += v.x, total += v.y;
                squares = fmaf(v.x, v.x, squares), squares = fmaf(v.y, v.y, squares);
            }
        constexpr double kScale = Format::kScale;
        s.sum += (double)total * kScale;
        s.squares += (double)squares * (kScale * kScale);
    }
};
template <> struct Moments<kE2M3> : Fp6Moments<E2M3Format> {};
template <> struct Moments<kE3M2> : Fp6Moments<E3M2Format> {};

// ---- integers ----
struct IntState {
    Wide sum, squares;
    __device__ __forceinline__ void combine(const IntState &o) { sum.add(o.sum), squares.add(o.squares); }
    __device__ __forceinline__ Partial pack() const {
        Partial p;
        p.w[0] = sum.lo, p.w[1] = sum.hi, p.w[2] = squares.lo, p.w[3] = squares.hi;
        return p;
    }
    static __device__ __forceinline__ IntState unpack(const Partial &p) {
        IntState s;
        s.sum.lo = p.w[0], s.sum.hi = p.w[1], s.squares.lo = p.w[2], s.squares.hi = p.w[3];
        return s;
    }
};
template <int kBytesPerValue>
struct IntMoments {
    using State = IntState;
    static constexpr int kBytes = kBytesPerValue;
    static constexpr bool kIsFloat = false;
};
template <> struct Moments<kI8> : IntMoments<1> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { const long long v = (signed char)bits; s.sum.add_signed(v), s.squares.add_unsigned((unsigned long long)(v * v)); }
    // sixteen values at once with the byte dot-product instruction; the 32-bit partial sums cannot overflow
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        int total = 0, squares = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) total = __dp4a((int)w[i], 0x01010101, total), squares = __dp4a((int)w[i], (int)w[i], squares);
        s.sum.add_signed(total), s.squares.add_unsigned((unsigned long long)(unsigned)squares);
    }
};
template <> struct Moments<kU8> : IntMoments<1> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { const unsigned long long v = bits & 0xffu; s.sum.add_unsigned(v), s.squares.add_unsigned(v * v); }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        uint32_t total = 0, squares = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) total = __dp4a(w[i], 0x01010101u, total), squares = __dp4a(w[i], w[i], squares);
        s.sum.add_unsigned(total), s.squares.add_unsigned(squares);
    }
};
template <> struct Moments<kI16> : IntMoments<2> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { const long long v = (short)bits; s.sum.add_signed(v), s.squares.add_unsigned((unsigned long long)(v * v)); }
    // eight values: their sum fits 32 bits, the sum of their squares (each at most 2^30) fits 64
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        int total = 0;
        unsigned long long squares = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int low = (short)(w[i] & 0xffffu), high = (int)w[i] >> 16;
            total += low + high;
            squares += (unsigned long long)(unsigned)(low * low) + (unsigned long long)(unsigned)(high * high);
        }
        s.sum.add_signed(total), s.squares.add_unsigned(squares);
    }
};
template <> struct Moments<kU16> : IntMoments<2> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { const unsigned long long v = bits & 0xffffu; s.sum.add_unsigned(v), s.squares.add_unsigned(v * v); }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        uint32_t total = 0;
        unsigned long long squares = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t low = w[i] & 0xffffu, high = w[i] >> 16;
            total += low + high;
            squares += (unsigned long long)(low * low) + (unsigned long long)(high * high);
        }
        s.sum.add_unsigned(total), s.squares.add_unsigned(squares);
    }
};
template <> struct Moments<kI32> : IntMoments<4> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { const long long v = (int)bits; s.sum.add_signed(v), s.squares.add_unsigned((unsigned long long)(v * v)); }
};
template <> struct Moments<kU32> : IntMoments<4> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) { const unsigned long long v = bits & 0xffffffffu; s.sum.add_unsigned(v), s.squares.add_unsigned(v * v); }
};
template <> struct Moments<kI64> : IntMoments<8> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) {
        const long long v = (long long)bits;
        const unsigned long long a = v < 0 ? 0ull - (unsigned long long)v : (unsigned long long)v;
        const unsigned long long square = (__umul64hi(a, a) || a * a > 0x7fffffffffffffffull) ? 0x7fffffffffffffffull : a * a;
        s.sum.add_signed(v), s.squares.add_unsigned(square);
    }
};
template <> struct Moments<kU64> : IntMoments<8> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) {
        s.sum.add_unsigned(bits), s.squares.add_unsigned(__umul64hi(bits, bits) ? 0xffffffffffffffffull : bits * bits);
    }
};
// Sub-byte types: a byte holds two nibbles or eight bits, every one of them counts.
template <> struct Moments<kU4> : IntMoments<1> {
    static __device__ __forceinline__ void nibble_sums(uint32_t word, uint32_t &total, uint32_t &squares) {
        const uint32_t lo = word & 0x0f0f0f0fu, hi = (word >> 4) & 0x0f0f0f0fu;
        total = __dp4a(lo, 0x01010101u, __dp4a(hi, 0x01010101u, total));
        squares = __dp4a(lo, lo, __dp4a(hi, hi, squares));
    }
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) {
        uint32_t total = 0, squares = 0;
        nibble_sums((uint32_t)bits & 0xffu, total, squares);
        s.sum.add_unsigned(total), s.squares.add_unsigned(squares);
    }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        uint32_t total = 0, squares = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) nibble_sums(w[i], total, squares);
        s.sum.add_unsigned(total), s.squares.add_unsigned(squares);
    }
};
template <> struct Moments<kI4> : IntMoments<1> {
    // A signed nibble n is (n ^ 8) - 8 = m - 8 with m in [0, 15]: sum = S1 - 8 k, squares = S2 - 16 S1 + 64 k over k nibbles.
    static __device__ __forceinline__ void finish(State &s, uint32_t s1, uint32_t s2, int nibbles) {
        s.sum.add_signed((long long)s1 - 8 * nibbles);
        s.squares.add_unsigned((unsigned long long)((long long)s2 - 16ll * s1 + 64ll * nibbles));
    }
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) {
        uint32_t s1 = 0, s2 = 0;
        Moments<kU4>::nibble_sums(((uint32_t)bits & 0xffu) ^ 0x88u, s1, s2);
        finish(s, s1, s2, 2);
    }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        uint32_t s1 = 0, s2 = 0;
#pragma unroll
        for (int i = 0; i < 4; ++i) Moments<kU4>::nibble_sums(w[i] ^ 0x88888888u, s1, s2);
        finish(s, s1, s2, 32);
    }
};
template <> struct Moments<kU1> : IntMoments<1> {
    static __device__ __forceinline__ void add(State &s, unsigned long long bits) {
        const unsigned long long ones = (unsigned long long)__popc((uint32_t)bits & 0xffu);
        s.sum.add_unsigned(ones), s.squares.add_unsigned(ones);
    }
    static __device__ __forceinline__ void add_vector(State &s, const uint32_t (&w)[4]) {
        const unsigned long long ones = (unsigned long long)(__popc(w[0]) + __popc(w[1]) + __popc(w[2]) + __popc(w[3]));
        s.sum.add_unsigned(ones), s.squares.add_unsigned(ones);
    }
};

template <typename T, typename = void> struct HasVectorPath : std::false_type {};
template <typename T> struct HasVectorPath<T, std::void_t<decltype(&T::add_vector)>> : std::true_type {};

template <typename State>
__device__ __forceinline__ State shuffle_down(const State &s, int delta) {
    Partial p = s.pack(), q;
#pragma unroll
    for (int w = 0; w < 4; ++w) q.w[w] = __shfl_down_sync(0xffffffffu, p.w[w], delta);
    return State::unpack(q);
}

// Folds the block's 256 thread states in a fixed order; thread 0 returns the total.
template <typename State>
__device__ __forceinline__ State block_fold(State mine) {
    __shared__ Partial warp_totals[8];
#pragma unroll
    for (int delta = 16; delta > 0; delta >>= 1) mine.combine(shuffle_down(mine, delta));
    if ((threadIdx.x & 31) == 0) warp_totals[threadIdx.x >> 5] = mine.pack();
    __syncthreads();
    if (threadIdx.x == 0)
        for (int w = 1; w < 8; ++w) mine.combine(State::unpack(warp_totals[w]));
    return mine;
}

// `units` = number of storage elements (values, or bytes for sub-byte types). Contiguous data is read as 16-byte
// vectors between an unaligned head and a ragged tail; strided data element by element.
template <uint32_t kType>
__global__ void __launch_bounds__(256)
moments_partial_kernel(const uint8_t *__restrict__ data, uint64_t units, uint64_t stride, Partial *__restrict__ partials) {
    using M = Moments<kType>;
    constexpr int kBytes = M::kBytes;
    typename M::State state;
    const uint64_t thread = (uint64_t)blockIdx.x * 256 + threadIdx.x, threads = (uint64_t)gridDim.x * 256;
    auto add_at = [&](uint64_t unit) {
        const uint8_t *p = data + unit * stride;
        unsigned long long bits;
        if constexpr (kBytes == 8) bits = *reinterpret_cast<const unsigned long long *>(p);
        else if constexpr (kBytes == 4) bits = *reinterpret_cast<const uint32_t *>(p);
        else if constexpr (kBytes == 2) bits = *reinterpret_cast<const uint16_t *>(p);
        else bits = *p;
        M::add(state, bits);
    };
    if (stride != (uint64_t)kBytes) {
        for (uint64_t unit = thread; unit < units; unit += threads) add_at(unit);
    } else {
        // head: up to the first 16-byte boundary
        const uint64_t misaligned = reinterpret_cast<uintptr_t>(data) & 15u;
        uint64_t head = misaligned ? (16 - misaligned) / kBytes : 0;
        if (head > units) head = units;
        const uint64_t vectors = (units - head) * kBytes / 16, per_vector = 16 / kBytes;
        if (thread < head) add_at(thread);
        const uint4 *base = reinterpret_cast<const uint4 *>(data + head * kBytes);
        for (uint64_t v = thread; v < vectors; v += threads) {
            const uint4 q = base[v];
            const uint32_t words[4] = {q.x, q.y, q.z, q.w};
            if constexpr (HasVectorPath<M>::value) {
                M::add_vector(state, words);
            } else if constexpr (kBytes == 8) {
                M::add(state, (unsigned long long)words[0] | ((unsigned long long)words[1] << 32));
                M::add(state, (unsigned long long)words[2] | ((unsigned long long)words[3] << 32));
            } else {
#pragma unroll
                for (int e = 0; e < 16 / kBytes; ++e) {
                    const int per_word = 4 / kBytes;
                    M::add(state, (words[e / per_word] >> (8 * kBytes * (e % per_word))) & (kBytes == 4 ? 0xffffffffu : (1u << (8 * kBytes)) - 1u));
                }
            }
        }
        const uint64_t done = head + vectors * per_vector;
        if (thread < units - done) add_at(done + thread);
    }
    state = block_fold(state);
    if (threadIdx.x == 0) partials[blockIdx.x] = state.pack();
}

// One block: folds the per-block partials in index order and writes the two results (8 bytes each).
template <uint32_t kType>
__global__ void __launch_bounds__(256) moments_finish_kernel(const Partial *__restrict__ partials, uint32_t count, unsigned long long *results) {
    using M = Moments<kType>;
    typename M::State state;
    for (uint32_t i = threadIdx.x; i < count; i += 256) state.combine(M::State::unpack(partials[i]));
    state = block_fold(state);
    if (threadIdx.x != 0) return;
    if constexpr (M::kIsFloat) {
        const double sum = state.sum + state.sum_error, squares = state.squares + state.squares_error;
        if constexpr (kType == kF64 || kType == kF32) {
            results[0] = (unsigned long long)__double_as_longlong(sum), results[1] = (unsigned long long)__double_as_longlong(squares);
        } else {
            results[0] = __float_as_uint(__double2float_rn(sum)), results[1] = __float_as_uint(__double2float_rn(squares));
        }
    } else {
        const Wide s = state.sum, q = state.squares;
        constexpr bool kSigned = kType == kI8 || kType == kI16 || kType == kI32 || kType == kI64 || kType == kI4;
        constexpr bool kSaturates = kType == kI32 || kType == kI64 || kType == kU32 || kType == kU64;
        if constexpr (!kSaturates) results[0] = s.lo, results[1] = q.lo;
        else {
            if constexpr (kSigned) {
                const unsigned long long sign_fill = (unsigned long long)((long long)s.lo >> 63);
                results[0] = s.hi == sign_fill ? s.lo : ((long long)s.hi >= 0 ? 0x7fffffffffffffffull : 0x8000000000000000ull);
            } else results[0] = s.hi ? 0xffffffffffffffffull : s.lo;
            results[1] = q.hi ? 0xffffffffffffffffull : q.lo;
        }
    }
}

template <uint32_t kType>
void moments_impl(const void *data, uint64_t count, uint64_t stride, void *sum_out, void *squares_out, int result_bytes) {
    clear_error();
    using M = Moments<kType>;
    constexpr int per_unit = kType == kU1 ? 8 : (kType == kI4 || kType == kU4) ? 2 : 1;
    const uint64_t units = (count + per_unit - 1) / per_unit;
    unsigned long long host_results[2] = {0, 0};
    auto deliver = [&](const unsigned long long *device_results, cudaStream_t stream) {
        bool ok = true;
        void *outs[2] = {sum_out, squares_out};
        bool any_host = false;
        for (int i = 0; i < 2 && ok; ++i) {
            if (classify(outs[i]) == kMemHost) any_host = true;
            else if (device_results) ok = cuda_ok(cudaMemcpyAsync(outs[i], device_results + i, result_bytes, cudaMemcpyDeviceToDevice, stream), "moments: result");
            else ok = cuda_ok(cudaMemsetAsync(outs[i], 0, result_bytes, stream), "moments: result");
        }
        if (ok && any_host) {
            if (device_results)
                ok = cuda_ok(cudaMemcpyAsync(host_results, device_results, 16, cudaMemcpyDeviceToHost, stream), "moments: result") &&
                     cuda_ok(cudaStreamSynchronize(stream), "moments");
            for (int i = 0; i < 2 && ok; ++i)
                if (classify(outs[i]) == kMemHost) std::memcpy(outs[i], &host_results[i], result_bytes);
        }
        return ok;
    };
    if (!sum_out || !squares_out) { set_error("reduce_moments: null result pointer%s", ""); return; }
    cudaStream_t stream = current_stream();
    if (units == 0) { deliver(nullptr, stream); return; }
    if (!data) { set_error("reduce_moments: null pointer%s", ""); return; }
    if (stride < (uint64_t)M::kBytes && units > 1) { set_error("reduce_moments: the stride is smaller than a value%s", ""); return; }
    if (M::kBytes > 1 && (reinterpret_cast<uintptr_t>(data) % M::kBytes || stride % M::kBytes)) { set_error("reduce_moments: data and stride must be aligned to the value size%s", ""); return; }
    const uint8_t *src = static_cast<const uint8_t *>(data);
    uint64_t device_stride = stride;
    bool ok = true;
    if (classify(data) == kMemHost) {  // staged tightly packed
        uint8_t *staged = static_cast<uint8_t *>(scratch(kSlotA, units * M::kBytes));
        if (!staged) ok = false;
        else if (stride == (uint64_t)M::kBytes || units == 1)
            ok = cuda_ok(cudaMemcpyAsync(staged, data, units * M::kBytes, cudaMemcpyHostToDevice, stream), "moments: upload");
        else
            ok = cuda_ok(cudaMemcpy2DAsync(staged, M::kBytes, data, stride, M::kBytes, units, cudaMemcpyHostToDevice, stream), "moments: upload");
        src = staged;
        device_stride = M::kBytes;
    }
    const uint64_t wanted = (units * M::kBytes / 16 + 255) / 256 + 1;
    const unsigned blocks = (unsigned)(wanted < 148ull * 8 ? wanted : 148ull * 8);
    Partial *partials = static_cast<Partial *>(scratch(kSlotAux, (blocks + 1) * sizeof(Partial)));
    ok = ok && partials;
    if (ok) {
        unsigned long long *results = reinterpret_cast<unsigned long long *>(partials + blocks);
        moments_partial_kernel<kType><<<blocks, 256, 0, stream>>>(src, units, device_stride, partials);
        moments_finish_kernel<kType><<<1, 256, 0, stream>>>(partials, blocks, results);
        g_launches += 2;
        ok = cuda_ok(cudaGetLastError(), "moments kernels") && deliver(results, stream);
    }
    if (!ok) {
        if (classify(sum_out) == kMemHost) std::memset(sum_out, 0xFF, result_bytes);
        if (classify(squares_out) == kMemHost) std::memset(squares_out, 0xFF, result_bytes);
    }
}

} // namespace
} // namespace nkb

#define NKB_DEFINE_MOMENTS(T, CODE, IN, SUM, SQ)                                                                         \
    extern "C" NKB_API void nk_reduce_moments_##T(IN const *data, size_t count, size_t stride_bytes, SUM *sum, SQ *sumsq) { \
        nkb::moments_impl<CODE>(data, count, stride_bytes, sum, sumsq, (int)sizeof(SUM));                                 \
    }
NKB_DEFINE_MOMENTS(f64, nkb::kF64, double, double, double)
NKB_DEFINE_MOMENTS(f32, nkb::kF32, float, double, double)
NKB_DEFINE_MOMENTS(f16, nkb::kF16, void, float, float)
NKB_DEFINE_MOMENTS(bf16, nkb::kBF16, void, float, float)
NKB_DEFINE_MOMENTS(e4m3, nkb::kE4M3, void, float, float)
NKB_DEFINE_MOMENTS(e5m2, nkb::kE5M2, void, float, float)
NKB_DEFINE_MOMENTS(e2m3, nkb::kE2M3, void, float, float)
NKB_DEFINE_MOMENTS(e3m2, nkb::kE3M2, void, float, float)
NKB_DEFINE_MOMENTS(i8, nkb::kI8, int8_t, int64_t, uint64_t)
NKB_DEFINE_MOMENTS(u8, nkb::kU8, uint8_t, uint64_t, uint64_t)
NKB_DEFINE_MOMENTS(i16, nkb::kI16, int16_t, int64_t, uint64_t)
NKB_DEFINE_MOMENTS(u16, nkb::kU16, uint16_t, uint64_t, uint64_t)
NKB_DEFINE_MOMENTS(i32, nkb::kI32, int32_t, int64_t, uint64_t)
NKB_DEFINE_MOMENTS(u32, nkb::kU32, uint32_t, uint64_t, uint64_t)
NKB_DEFINE_MOMENTS(i64, nkb::kI64, int64_t, int64_t, uint64_t)
NKB_DEFINE_MOMENTS(u64, nkb::kU64, uint64_t, uint64_t, uint64_t)
NKB_DEFINE_MOMENTS(i4, nkb::kI4, void, int64_t, uint64_t)
NKB_DEFINE_MOMENTS(u4, nkb::kU4, void, uint64_t, uint64_t)
NKB_DEFINE_MOMENTS(u1, nkb::kU1, void, uint64_t, uint64_t)
