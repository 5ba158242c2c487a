// Packed GEMM C = A * B^T on the 5th-generation tensor cores (tcgen05), with the
// dot / angular / euclidean epilogues fused into the TMEM read-out.
//
// Replaces the depth loops of NumKong's nk_dots_packed_<t> (include/numkong/dots/serial.h:520-1085,
// AMX form include/numkong/dots/sapphireamx.h:981-) and the second pass of
// nk_angulars_packed_<t> / nk_euclideans_packed_<t> (include/numkong/dots/serial.h:2756-2800).
//
// One persistent CTA per SM, ten warps:
//   warp 0      producer: TMA tiled loads of A (128-byte swizzle) and untiled bulk copies of the
//               pre-swizzled B chunks into a multi-stage shared-memory ring (mbarrier full/empty pairs)
//   warp 1      allocates TMEM and issues tcgen05.mma from one thread; accumulators live in TMEM,
//               two of them, so reading one out overlaps the MMAs that fill the other
//   warps 2..9  epilogue: tcgen05.ld of their 32-lane quarter and column half, f32/i32 summation of the
//               accumulation spans in registers, finalisation, global stores
#include <atomic>
#include <cmath>
#include <mutex>
#include <type_traits>
#include "nkb_internal.h"
#include "nkb_ptx.cuh"

namespace nkb {

namespace {

constexpr int kBM = 128;          // rows of A per tile = TMEM lanes
constexpr int kBKBytes = 128;     // bytes of depth per pipeline stage (one swizzle span)
constexpr int kUmmaKBytes = 32;   // bytes of depth one tcgen05.mma consumes
constexpr int kEpilogueWarps = 8;
constexpr int kThreads = 64 + 32 * kEpilogueWarps;
constexpr int kGroupM = 8;        // tile rasterisation: walk 8 row-tiles before moving to the next column-tile

struct GemmDev {
    const uint8_t *b_payload;
    const void *b_norms;
    const float *a_norms;
    uint8_t *c;
    uint64_t c_stride;
    uint32_t m, n;
    uint32_t kblocks;             // depth_padded_bytes / 128
    uint32_t elems_per_kblock;    // 128 / element bytes
    uint32_t tiles_m, tiles_n;
    uint32_t idesc;
    uint32_t int_mode;            // 0 float accumulators, 1 signed i32, 2 unsigned u32
    uint32_t flush_kblocks;       // stages per accumulation span (see the MMA issuer)
    unsigned int *error_word;
    uint32_t wait_us[kWaitSites];  // limit of every bounded wait, by wait site (microseconds)
    // Triangular mode (A x A^T): >= 0 keeps only cells with column >= row + tri_diag (the diagonal itself reads 0 under a
    // distance epilogue), tiles wholly below that line are never computed; -1 = plain rectangular product.
    int32_t tri_diag;
    // Candidate filter of the distance epilogues (see GemmArgs); `candidates == nullptr` means "store the tile".
    const uint32_t *threshold_bits;
    uint32_t *candidate_counts;
    uint2 *candidates;
    uint32_t candidate_capacity;
    uint32_t column_id_base;
    // Split mode of the CTA-pair kernel (see PairWork): hand-over flags of this launch and the value that marks them set.
    uint32_t *split_flags;   // nullptr = whole tiles
    uint32_t split_epoch;
};

// Epilogue scratch after the barriers: column factors (2 x 256 f32) + eight staging blocks of 32 rows x (W + 4) words,
// W = columns a warp stages per round (16, or 64 in the three-stage variant that has the room for it).
constexpr int epi_smem_bytes(int stage_cols) { return 2 * 256 * 4 + 8 * 32 * (stage_cols + 4) * 4; }
constexpr int kEpiSmemBytesDecl = epi_smem_bytes(16);
// Short depths make the kernel store bound (C leaves at ~2.3 TB/s with 64-byte row pieces). Three stages are enough
// to feed such problems and free the shared memory for 64-column staging: 256-byte row pieces per store instruction.
constexpr int stage_cols_for(int bn, int stages) { return bn == 256 && stages == 3 ? 64 : 16; }
constexpr uint32_t kShortDepthBlocks = 4;  // depths up to 4 x 128 bytes take the three-stage, wide-store variant (measured: 2.2 x faster dots at depth 128, a few % slower at depth 768)

template <int kBN, int kStages>
struct SmemPlan {
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBBytes = kBN * kBKBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierOffset = kStages * kStageBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kStageCols = stage_cols_for(kBN, kStages);
    static constexpr int kTotal = kBarrierOffset + kBarrierBytes + epi_smem_bytes(kStageCols) + 1024;  // + slack for manual 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t &mt, uint32_t &nt) {
    uint32_t per_group = kGroupM * tiles_n;
    uint32_t group = tile / per_group;
    uint32_t first_m = group * kGroupM;
    uint32_t group_rows = min(tiles_m - first_m, (uint32_t)kGroupM);
    uint32_t in_group = tile % per_group;
    mt = first_m + in_group % group_rows;
    nt = in_group / group_rows;
    // Odd groups walk the column tiles backwards: the packed rows the previous group touched last are still in L2 when the
    // next group begins with them.
    if (group & 1u) nt = tiles_n - 1u - nt;
}

// True when no cell of a tile (first row, one past its last column) survives the triangular mask. Every warp role asks
// the same question for the same tile, so skipped tiles move no barrier.
__device__ __forceinline__ bool tile_skipped(int32_t tri_diag, uint32_t first_row, uint32_t end_col) {
    return tri_diag >= 0 && end_col <= first_row + (uint32_t)tri_diag;
}

// ---- epilogue helpers shared by the single-CTA and the CTA-pair kernels ---------------------------------
// Shared memory after the barriers: per-tile column factors (two tiles deep) and one 32 x 16 staging block per
// epilogue warp (row pitch 20 words keeps 16-byte vector accesses aligned and nearly conflict-free).
constexpr int kEpiColfBytes = 2 * 256 * 4;
constexpr int kEpiStagePitch = 20;
constexpr int kEpiStageWords = 32 * kEpiStagePitch;
constexpr int kEpiSmemBytes = kEpiColfBytes + kEpilogueWarps * kEpiStageWords * 4;
static_assert(kEpiSmemBytes == kEpiSmemBytesDecl, "epilogue scratch size");

__device__ __forceinline__ float rsqrt_refined(float x) {
    float r = rsqrtf(x);
    return r * (1.5f - 0.5f * x * r * r);
}
__device__ __forceinline__ float sqrt_approx(float x) {
    float r;
    asm("sqrt.approx.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(kEpilogueWarps * 32) : "memory"); }
// The same barrier, returning the OR of `flag` over the epilogue threads.
__device__ __forceinline__ bool epilogue_barrier_any(bool flag) {
    uint32_t any;
    asm volatile("{\n\t.reg .pred in, out;\n\tsetp.ne.u32 in, %1, 0;\n\tbar.red.or.pred out, 1, %2, in;\n\tselp.u32 %0, 1, 0, out;\n\t}"
                 : "=r"(any) : "r"((uint32_t)flag), "n"(kEpilogueWarps * 32) : "memory");
    return any != 0;
}

// Column factor of one packed row for the distance epilogues: 1/|b| (0 for a zero row) for angular, |b|^2 for euclidean.
template <int kEpi>
__device__ __forceinline__ float column_factor(const GemmDev &p, uint32_t col) {
    if (col >= p.n) return 0.0f;
    float bn = p.int_mode == 0 ? __ldg(reinterpret_cast<const float *>(p.b_norms) + col)
                               : (float)__ldg(reinterpret_cast<const uint32_t *>(p.b_norms) + col);
    if constexpr (kEpi == kEpiAngular) return bn > 0.0f ? rsqrt_refined(bn) : 0.0f;
    return bn;
}

// True for a row or column factor that rules out the shortcuts of the distance epilogues. Angular: a zero factor calls for
// the zero-norm rule. Both: a factor that is not finite (an Inf or NaN element, a squared norm that overflowed) goes with
// dots that are not finite either, and only the full formula maps those the way the storing path does. With every
// factor of a tile finite, every dot of the tile is finite too: |dot| <= |a||b| <= max(|a|^2, |b|^2).
template <int kEpi>
__device__ __forceinline__ bool special_factor(float f) {
    if constexpr (kEpi == kEpiAngular) return !(f > 0.0f && f < __uint_as_float(0x7f800000u));
    else if constexpr (kEpi == kEpiEuclidean) return !(fabsf(f) < __uint_as_float(0x7f800000u));
    else return false;
}

// One finalised distance. Never NaN and never below -0: a NaN dot or factor falls out of fmaxf as 0.
//   kFloat       the accumulator holds f32 bits (known at compile time for the float kinds; the integer kinds read `int_mode`)
//   kZeroRule    apply the zero-norm rule of the angular distance; callers switch it off for a tile whose row and column
//                factors are all non-zero and finite, which is nearly every tile
template <int kEpi, bool kFloat, bool kZeroRule = true>
__device__ __forceinline__ float distance_value(uint32_t raw, uint32_t int_mode, float row_factor, float col_factor) {
    float dot;
    if constexpr (kFloat) dot = __uint_as_float(raw);
    else dot = int_mode == 1 ? (float)(int32_t)raw : (float)raw;
    if constexpr (kEpi == kEpiAngular) {
        float r = fmaxf(fmaf(-(dot * row_factor), col_factor, 1.0f), 0.0f);
        if constexpr (kZeroRule)
            if (row_factor == 0.0f || col_factor == 0.0f) r = dot == 0.0f ? 0.0f : 1.0f;
        return r;
    } else {
        return sqrt_approx(fmaxf(fmaf(-2.0f, dot, row_factor + col_factor), 0.0f));
    }
}

// Bits of one finalised output cell for every epilogue but the raw dot. The set distances (one-bit inputs: `raw` is the
// AND-popcount, the factors are the two population counts, exact in f32 below 2^24) follow
// include/numkong/set/serial.h:150-168: Hamming = |a| + |b| - 2 |a & b| in u32, Jaccard = 1 - |a & b| / (|a| + |b| - |a & b|)
// in f32 with the reference's operation order (0 for two empty sets).
template <int kEpi, bool kFloat, bool kZeroRule = true>
__device__ __forceinline__ uint32_t cell_bits(uint32_t raw, uint32_t int_mode, float row_factor, float col_factor) {
    if constexpr (kEpi == kEpiHamming) {
        return __float2uint_rn(row_factor) + __float2uint_rn(col_factor) - 2u * raw;
    } else if constexpr (kEpi == kEpiJaccard) {
        const float dot = (float)raw;
        const float union_size = row_factor + col_factor - dot;
        return __float_as_uint(union_size != 0.0f ? 1.0f - __fdiv_rn(dot, union_size) : 0.0f);
    } else {
        return __float_as_uint(distance_value<kEpi, kFloat, kZeroRule>(raw, int_mode, row_factor, col_factor));
    }
}

// Filter mode of the distance epilogues: nothing is stored; the values of this thread's row that lie below the row's
// threshold are appended to the row's candidate list (in no particular order; a count beyond the capacity tells the
// consumer that values were dropped). Distances are >= -0 and never NaN, so the signed integer order of their bit
// patterns is their numeric order (with -0 before +0, as the selection kernels order them) and one integer compare per
// value decides. Pass 1 only builds a bit mask; a row then reserves all its slots with ONE atomic (a per-value atomic
// would put its round trip on the critical path of every hit), and pass 2 recomputes and writes the few hits.
template <int kEpi, int kCols, bool kFloat>
__device__ __forceinline__ void filter_tile(uint32_t (&acc)[kCols], const GemmDev &p, uint32_t my_row, uint32_t col_base,
                                            float row_factor, const float *colf, uint32_t *stage, int lane, bool zero_factors) {
    static_assert(kCols % 32 == 0, "whole mask words");
    const int threshold = my_row < p.m ? (int)__ldg(p.threshold_bits + my_row) : (int)0x80000000;
    uint32_t mask[kCols / 32];
    auto build_masks = [&](auto zero_rule) {
#pragma unroll
        for (int w = 0; w < kCols / 32; ++w) {
            uint32_t bits = 0;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float4 f = *reinterpret_cast<const float4 *>(colf + w * 32 + c * 4);
                const float cf[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float r = distance_value<kEpi, kFloat, decltype(zero_rule)::value>(acc[w * 32 + c * 4 + j], p.int_mode, row_factor, cf[j]);
                    bits |= (uint32_t)((int)__float_as_uint(r) < threshold) << (c * 4 + j);
                }
            }
            // Columns past the end of the packed matrix are padding.
            const uint32_t first = col_base + w * 32;
            const uint32_t valid = first >= p.n ? 0u : (p.n - first >= 32u ? 0xffffffffu : (1u << (p.n - first)) - 1u);
            mask[w] = bits & valid;
        }
    };
    // Float kinds: a two- or three-instruction prefilter per value instead of the full distance, decided by a sign bit that
    // a funnel shift collects (columns are walked downwards so that bit i ends up standing for column i). The bound is
    // moved so far that the roundings behind the exact distance cannot hide a value below the threshold; the few extra
    // values that pass are weeded out when pass 2 recomputes the exact distance.
    //   angular (no zero factor in sight): r < threshold needs dot * col_factor > (1 - threshold) / row_factor; the bound is
    //     lowered by 2^-18 relative to 1 + |1 - threshold|; the sign of fma(-dot, col_factor, bound) decides.
    //   euclidean: r < threshold needs |b|^2 - 2 dot < threshold^2 - |a|^2 up to 2^-21 (|a|^2 + |b|^2), and a column that
    //     passes has |b|^2 <= 4 max(|a|^2, threshold^2) (triangle inequality), so the bound is raised by
    //     2^-18 * 9 max(|a|^2, threshold^2) and threshold^2 by 2^-16; the sign of fma(-2, dot, |b|^2) - bound decides.
    bool prefiltered = false;
    if constexpr ((kEpi == kEpiAngular || kEpi == kEpiEuclidean) && kFloat) {
        if (!zero_factors) {  // no zero and no non-finite factor in sight: every dot of the tile is finite
            prefiltered = true;
            constexpr bool kAngular = kEpi == kEpiAngular;
            const float pass_all = __uint_as_float(kAngular ? 0xff800000u : 0x7f800000u);
            const float pass_none = __uint_as_float(kAngular ? 0x7f800000u : 0xff800000u);
            float bound;
            if (my_row >= p.m) bound = pass_none;
            else if (threshold == 0x7fffffff) bound = pass_all;  // no threshold yet
            else if constexpr (kAngular) {
                const float b = 1.0f - __int_as_float(threshold), w = __frcp_rn(row_factor);
                bound = fmaf(b, w, -(fabsf(b) + 1.0f) * w * 0x1p-18f);
            } else {
                const float t = __int_as_float(threshold), t2 = t * t;
                bound = fmaf(t2, 1.0f + 0x1p-16f, -row_factor) + 9.0f * fmaxf(row_factor, t2) * 0x1p-18f;
            }
#pragma unroll
            for (int w = 0; w < kCols / 32; ++w) {
                uint32_t bits = 0;
#pragma unroll
                for (int c = 7; c >= 0; --c) {
                    const float4 f = *reinterpret_cast<const float4 *>(colf + w * 32 + c * 4);
                    const float cf[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
                    for (int j = 3; j >= 0; --j) {
                        const float dot = __uint_as_float(acc[w * 32 + c * 4 + j]);
                        const float decision = kAngular ? fmaf(-dot, cf[j], bound) : fmaf(-2.0f, dot, cf[j]) - bound;
                        bits = __funnelshift_l(__float_as_uint(decision), bits, 1);
                    }
                }
                const uint32_t first = col_base + w * 32;
                const uint32_t valid = first >= p.n ? 0u : (p.n - first >= 32u ? 0xffffffffu : (1u << (p.n - first)) - 1u);
                mask[w] = bits & valid;
            }
        }
    }
    if (!prefiltered) {
        if constexpr (kEpi == kEpiAngular && kFloat) build_masks(std::true_type{});  // only reached with a special factor in sight
        else if (zero_factors) build_masks(std::true_type{});
        else build_masks(std::false_type{});
    }
    uint32_t hits = 0;
#pragma unroll
    for (int w = 0; w < kCols / 32; ++w) hits += __popc(mask[w]);
    if (!__any_sync(0xffffffffu, hits != 0)) return;
    uint32_t slot = 0;
    if (hits) slot = atomicAdd(p.candidate_counts + my_row, hits);
    uint2 *list = p.candidates + (uint64_t)my_row * p.candidate_capacity;
    // Pass 2, 16 columns at a time: a thread with hits parks the 16 accumulators in its own row of the warp's staging
    // block (shared memory can be indexed by a run-time value, registers cannot) and walks the set bits.
    uint32_t *mine = stage + lane * kEpiStagePitch;
#pragma unroll
    for (int c = 0; c < kCols / 16; ++c) {
        uint32_t m16 = (mask[c / 2] >> ((c & 1) * 16)) & 0xffffu;
        if (m16 == 0) continue;
#pragma unroll
        for (int q = 0; q < 4; ++q)
            *reinterpret_cast<uint4 *>(mine + q * 4) =
                make_uint4(acc[c * 16 + q * 4], acc[c * 16 + q * 4 + 1], acc[c * 16 + q * 4 + 2], acc[c * 16 + q * 4 + 3]);
        while (m16) {
            const int j = __ffs((int)m16) - 1;
            m16 &= m16 - 1;
            const float r = distance_value<kEpi, kFloat>(mine[j], p.int_mode, row_factor, colf[c * 16 + j]);
            // A value the prefilter let through although it is not below the threshold keeps its reserved slot as +infinity,
            // which the selection sorts behind everything else.
            const uint32_t value = (int)__float_as_uint(r) < threshold ? __float_as_uint(r) : 0x7f800000u;
            if (slot < p.candidate_capacity) list[slot] = make_uint2(value, col_base + c * 16 + j + p.column_id_base);
            ++slot;
        }
    }
}

// Finalises and stores this thread's row x kCols accumulators. Values go through the warp's staging block 16 columns at a
// time so that each store instruction writes 8 rows x 64 contiguous bytes instead of 32 rows x 16 bytes.
//   row_base  first of the 32 rows this warp owns;  col_base  first of this thread's kCols columns
//   colf      this tile's column factors in shared memory, indexed by column inside the tile;  colf_off  col_base inside the tile
// Angular: max(0, 1 - dot/(|a||b|)), and for a zero norm 0 when the dot is 0 else 1 (include/numkong/spatial/serial.h:257-269).
// Euclidean: sqrt(max(0, |a|^2 + |b|^2 - 2 dot)) (include/numkong/spatial/serial.h:272-278).
//   zero_cols  some column factor of this tile is special (see special_factor: a zero vector or padding past the last column
//              under the angular epilogue, a norm that is not finite under either)
//   kAccum     (raw dots only) add the values to what the cells already hold instead of overwriting them: the second half of a
//              tile whose depth was split between two CTA pairs
template <int kEpi, int kCols, int kW, bool kFloat, bool kAccum = false>
__device__ __forceinline__ void store_tile(uint32_t (&acc)[kCols], const GemmDev &p, uint32_t row_base, uint32_t col_base,
                                           uint32_t *stage, const float *colf, uint32_t colf_off, int lane, bool zero_cols) {
    static_assert(!kAccum || kEpi == kEpiDot, "only raw dots can be added up across depth ranges");
    auto plus = [](uint32_t x, uint32_t y) { return kFloat ? __float_as_uint(__uint_as_float(x) + __uint_as_float(y)) : x + y; };
    constexpr int kPitch = kW + 4;          // words per staged row (keeps 16-byte accesses aligned and conflict-free)
    constexpr int kQuads = kW / 4;          // 16-byte pieces per staged row
    constexpr int kRowsPerStore = 32 / kQuads;
    static_assert(kCols % kW == 0 && (kW == 16 || kW == 32 || kW == 64), "staging width");
    const uint32_t my_row = row_base + lane;
    float row_factor = 0.0f;
    if constexpr (kEpi != kEpiDot) {
        float an = my_row < p.m ? p.a_norms[my_row] : 0.0f;
        row_factor = kEpi == kEpiAngular ? (an > 0.0f ? rsqrt_refined(an) : 0.0f) : an;
    }
    // The angular zero-norm rule is only compiled into the path taken when this row or some column of the tile has a zero factor.
    // The predicate is uniform over the warp: the store loop below synchronises the warp.
    const bool zero_factors = (kEpi == kEpiAngular || kEpi == kEpiEuclidean) &&
                              (zero_cols || __any_sync(0xffffffffu, special_factor<kEpi>(row_factor)));
    if constexpr (kEpi == kEpiAngular || kEpi == kEpiEuclidean) {
        if (p.candidates != nullptr) {
            filter_tile<kEpi, kCols, kFloat>(acc, p, my_row, col_base, row_factor, colf + colf_off, stage, lane, zero_factors);
            return;
        }
    }
    auto emit = [&](auto zero_rule) {
#pragma unroll
    for (int c = 0; c < kCols / kW; ++c) {
        const uint32_t col0 = col_base + c * kW;
        if (col0 >= p.n) break;  // same for the whole warp
#pragma unroll
        for (int q = 0; q < kQuads; ++q) {
            uint32_t out[4];
            float4 f = make_float4(0.f, 0.f, 0.f, 0.f);
            if constexpr (kEpi != kEpiDot) f = *reinterpret_cast<const float4 *>(colf + colf_off + c * kW + q * 4);
            const float cf[4] = {f.x, f.y, f.z, f.w};
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const uint32_t raw = acc[c * kW + q * 4 + j];
                if constexpr (kEpi == kEpiDot) out[j] = raw;
                else out[j] = cell_bits<kEpi, kFloat, decltype(zero_rule)::value>(raw, p.int_mode, row_factor, cf[j]);
            }
            *reinterpret_cast<uint4 *>(stage + lane * kPitch + q * 4) = make_uint4(out[0], out[1], out[2], out[3]);
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < kQuads; ++it) {
            const uint32_t r = it * kRowsPerStore + (uint32_t)lane / kQuads, q = (uint32_t)lane % kQuads;
            uint4 v = *reinterpret_cast<const uint4 *>(stage + r * kPitch + q * 4);
            const uint32_t row = row_base + r, col = col0 + q * 4;
            // Triangular mode: the first column this row keeps (0 when the product is rectangular).
            const uint32_t keep_from = p.tri_diag >= 0 ? row + (uint32_t)p.tri_diag : 0u;
            if (row < p.m && col < p.n && col + 4 > keep_from) {
                uint32_t *dst = reinterpret_cast<uint32_t *>(p.c + (uint64_t)row * p.c_stride) + col;
                if (col + 4 <= p.n && col >= keep_from + (kEpi != kEpiDot ? 1u : 0u) && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
                    if constexpr (kAccum) {
                        const uint4 old = *reinterpret_cast<const uint4 *>(dst);
                        v = make_uint4(plus(v.x, old.x), plus(v.y, old.y), plus(v.z, old.z), plus(v.w, old.w));
                    }
                    // Streaming store: result cells are written once and not read here again, so they should be the first
                    // lines L2 gives up - ahead of the operand chunks that other tiles are about to ask for.
                    __stcs(reinterpret_cast<uint4 *>(dst), v);
                } else {
                    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j)
                        if (col + j < p.n && col + j >= keep_from) {
                            if constexpr (kAccum) dst[j] = plus(w[j], dst[j]);
                            else dst[j] = (kEpi != kEpiDot && p.tri_diag >= 0 && col + j == keep_from) ? 0u : w[j];  // distance to itself
                        }
                }
            }
        }
        __syncwarp();
    }
    };
    if (kEpi == kEpiAngular && zero_factors) emit(std::true_type{});
    else emit(std::false_type{});
}

template <int kKind, int kBN, int kStages, int kEpi>
// Ten warps land three deep on some SM sub-partitions (16 K registers each), which caps a thread at 168
// registers: 128 accumulators + 16 loaded values + addressing fits.
__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const __grid_constant__ CUtensorMap a_map, const GemmDev p) {
    using Plan = SmemPlan<kBN, kStages>;
    constexpr int kTmemCols = 2 * kBN;        // two accumulator buffers
    constexpr int kColsPerThread = kBN / 2;   // each epilogue thread owns one row x half the tile's columns
    static_assert(kTmemCols == 256 || kTmemCols == 512, "TMEM allocation must be a power of two");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));

    const uint32_t bar_base = smem_base + Plan::kBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + Plan::kBarrierOffset + 8 * (2 * kStages + 4));
    const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 5);  // the MMA issuer's "all my MMAs have retired"

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;

    if (threadIdx.x == 0) {
        prefetch_tensormap(&a_map);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full_bar(a), 1);
            mbar_init(tmem_empty_bar(a), kEpilogueWarps * 32);
        }
        mbar_init(drain_bar, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        tmem_relinquish<1>();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, issued = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t mt, nt;
                tile_coords(tile, p.tiles_m, p.tiles_n, mt, nt);
                if (tile_skipped(p.tri_diag, mt * kBM, (nt + 1) * kBN)) continue;
                const uint8_t *b_tile = p.b_payload + (uint64_t)nt * (kBN / kChunkRows) * p.kblocks * kChunkBytes;
                for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, 1, p.error_word, p.wait_us[1])) { ok = false; break; }
                    uint32_t a_dst = smem_base + stage * Plan::kStageBytes;
                    uint32_t b_dst = a_dst + Plan::kABytes;
                    mbar_expect_tx(full_bar(stage), Plan::kStageBytes);
                    tma_load_2d(a_dst, &a_map, (int)(kb * p.elems_per_kblock), (int)(mt * kBM), full_bar(stage));
#pragma unroll
                    for (int j = 0; j < kBN / (int)kChunkRows; ++j)
                        bulk_load(b_dst + j * kChunkBytes, b_tile + ((uint64_t)j * p.kblocks + kb) * kChunkBytes,
                                  kChunkBytes, full_bar(stage));
                    ++issued;
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // The consumer has stopped. Copies this thread issued may still be in flight, and shared memory must not
                // be released under them: wait (bounded) until the `full` barrier of every stage issued last has
                // counted its bytes. Stages the MMA issuer already took return at once.
                int s = stage;
                uint32_t ph = phase;
                for (uint32_t i = 0; i < issued && i < (uint32_t)kStages; ++i) {
                    if (s == 0) { s = kStages; ph ^= 1u; }
                    --s;
                    if (!mbar_wait(full_bar(s), ph, 6, p.error_word, p.wait_us[6])) break;
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer
        // The depth is cut into spans of `flush_kblocks` stages. Each span accumulates in one of the two
        // TMEM buffers and is handed to the epilogue warps, which add the spans up in registers with
        // round-to-nearest f32 adds. The tensor cores truncate when they accumulate; short spans keep
        // that error at the level of NumKong's own f32 kernels. Integer kinds use a single span.
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            uint32_t seq = 0;  // spans issued so far, across tiles
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t mt, nt;
                tile_coords(tile, p.tiles_m, p.tiles_n, mt, nt);
                if (tile_skipped(p.tri_diag, mt * kBM, (nt + 1) * kBN)) continue;
                for (uint32_t kb0 = 0; kb0 < p.kblocks && ok; kb0 += p.flush_kblocks, ++seq) {
                    const uint32_t buf = seq & 1u;
                    const uint32_t buf_phase = (seq >> 1) & 1u;
                    if (!mbar_wait(tmem_empty_bar(buf), buf_phase ^ 1u, 2, p.error_word, p.wait_us[2])) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * kBN;
                    const uint32_t kb1 = min(kb0 + p.flush_kblocks, p.kblocks);
                    for (uint32_t kb = kb0; kb < kb1; ++kb) {
                        if (!mbar_wait(full_bar(stage), phase, 3, p.error_word, p.wait_us[3])) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t a_src = smem_base + stage * Plan::kStageBytes;
                        const uint64_t a_desc = make_smem_desc_sw128(a_src);
                        const uint64_t b_desc = make_smem_desc_sw128(a_src + Plan::kABytes);
#pragma unroll
                        for (int k = 0; k < kBKBytes / kUmmaKBytes; ++k) {
                            // Stepping 32 bytes along depth inside the 128-byte swizzle span = +2 in the (addr >> 4) field.
                            umma<kKind, 1>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, ((kb - kb0) | (uint32_t)k) != 0u);
                        }
                        umma_commit(empty_bar(stage));  // frees the stage once these MMAs have read it
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) umma_commit(tmem_full_bar(buf));
                }
            }
            // TMEM and shared memory are released after the block-wide barrier below; no MMA may still be running then.
            // On the regular path the epilogue's last wait already implies that; after a wait that gave up nothing
            // does, so the issuer always waits (bounded) for its own last MMAs.
            umma_commit(drain_bar);
            mbar_wait(drain_bar, 0u, 5, p.error_word, p.wait_us[5]);
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        const uint32_t quarter = warp & 3u;               // TMEM lanes this warp may read: 32*quarter .. +31
        const uint32_t half = (uint32_t)(warp - 2) >> 2;  // which half of the tile's columns
        float *colf = reinterpret_cast<float *>(smem_gen + Plan::kBarrierOffset + Plan::kBarrierBytes);
        uint32_t *epi_stage = reinterpret_cast<uint32_t *>(smem_gen + Plan::kBarrierOffset + Plan::kBarrierBytes + kEpiColfBytes) +
                              (warp - 2) * 32 * (Plan::kStageCols + 4);
        uint32_t seq = 0, local_tile = 0;
        bool ok = true;
        // After a wait has given up (`ok` false) the epilogue warps stop waiting and stop touching TMEM but still walk every
        // tile: they share a named barrier per tile, and a warp that left early would strand the others inside it.
        for (uint32_t tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            uint32_t mt, nt;
            tile_coords(tile, p.tiles_m, p.tiles_n, mt, nt);
            if (tile_skipped(p.tri_diag, mt * kBM, (nt + 1) * kBN)) continue;
            bool zero_cols = false;
            if constexpr (kEpi != kEpiDot) {
                // One column factor per epilogue thread, shared by all rows of the tile (double-buffered by tile parity).
                const uint32_t e = threadIdx.x - 64u;
                const float factor = e < (uint32_t)kBN ? column_factor<kEpi>(p, nt * kBN + e) : 1.0f;
                colf[(local_tile & 1u) * 256 + e] = factor;
                zero_cols = epilogue_barrier_any(special_factor<kEpi>(factor));
            }
            uint32_t acc[kColsPerThread];
#pragma unroll
            for (int j = 0; j < kColsPerThread; ++j) acc[j] = 0u;
            for (uint32_t kb0 = 0; kb0 < p.kblocks && ok; kb0 += p.flush_kblocks, ++seq) {
                const uint32_t buf = seq & 1u;
                const uint32_t buf_phase = (seq >> 1) & 1u;
                if (!mbar_wait(tmem_full_bar(buf), buf_phase, 4, p.error_word, p.wait_us[4])) { ok = false; break; }
                tc_fence_after_sync();
                if (kb0 == 0) {
                    // First span of a tile: nothing to add to, so every load goes straight into the accumulators and all of
                    // them are in flight before the one wait.
#pragma unroll
                    for (int c = 0; c < kColsPerThread / 16; ++c)
                        tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + buf * kBN + half * kColsPerThread + c * 16,
                                      *reinterpret_cast<uint32_t(*)[16]>(&acc[c * 16]));
#pragma unroll
                    for (int c = 0; c < kColsPerThread / 32; ++c) tmem_ld_wait_for(*reinterpret_cast<uint32_t(*)[32]>(&acc[c * 32]));
                } else {
                    // Later spans are added to the running sums eight columns at a time, two loads deep: while the values of
                    // one load are added, the next load is on its way from TMEM (no more registers than one 16-column load).
                    const uint32_t span_addr = tmem_base + ((quarter * 32u) << 16) + buf * kBN + half * kColsPerThread;
                    uint32_t va[8], vb[8];
                    auto add8 = [&](int c8, const uint32_t (&v)[8]) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if constexpr (kKind == kKindI8) acc[c8 * 8 + j] += v[j];
                            else acc[c8 * 8 + j] = __float_as_uint(__uint_as_float(acc[c8 * 8 + j]) + __uint_as_float(v[j]));
                        }
                    };
                    tmem_ld_32x8(span_addr, va);
#pragma unroll
                    for (int c8 = 0; c8 < kColsPerThread / 8; c8 += 2) {
                        tmem_ld_wait_for(va);
                        tmem_ld_32x8(span_addr + (c8 + 1) * 8, vb);
                        add8(c8, va);
                        tmem_ld_wait_for(vb);
                        if (c8 + 2 < kColsPerThread / 8) tmem_ld_32x8(span_addr + (c8 + 2) * 8, va);
                        add8(c8 + 1, vb);
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(tmem_empty_bar(buf));
            }
            if (!ok) continue;  // nothing valid to store; the next tile's barrier is still met
            store_tile<kEpi, kColsPerThread, Plan::kStageCols, kKind != kKindI8>(acc, p, mt * kBM + quarter * 32u, nt * kBN + half * kColsPerThread,
                                                                                  epi_stage, colf + (local_tile & 1u) * 256, half * kColsPerThread, lane, zero_cols);
            ++local_tile;
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 cta_group::2): two CTAs on neighbouring SMs share one 256 x 256 output tile. Each
// CTA loads its own 128 rows of A and HALF of the B tile (128 packed rows); the MMA issued by the leader CTA
// reads B from both CTAs' shared memory, so every SM fetches 32 KiB per stage instead of 48 KiB, and each CTA
// accumulates its 128 x 256 half in its own TMEM. No multicast: every CTA issues its own loads.
//   - loads of both CTAs complete on the LEADER's `full` barrier (pair-form TMA);
//   - the leader's tcgen05.commit releases a stage / publishes an accumulator in BOTH CTAs;
//   - epilogue warps of both CTAs report a drained accumulator to the leader's `tmem_empty` barrier.
constexpr int kPairStages = 6;
constexpr int kPairBN = 256;
constexpr int kPairStageBytes = kBM * kBKBytes + (kPairBN / 2) * kBKBytes;  // 16 KiB of A + 16 KiB of B per CTA
constexpr int kPairBarrierOffset = kPairStages * kPairStageBytes;
constexpr int kPairSmemTotal = kPairBarrierOffset + 256 + kEpiSmemBytesDecl + 1024;

// The work of one CTA pair. Whole-tile mode (the default): tiles pair, pair + P, pair + 2 P, ... Split mode (opt-in, see
// launch_pair for why it is not the default): the pipeline stages of all tiles
// are numbered tile by tile and dealt out in P equal contiguous shares, so that every pair is busy for the same time even when
// the tiles do not fill a whole number of waves (1024 x 8192 makes 128 tiles for 74 pairs: 1.73 waves, 2 with whole tiles). A
// share may begin in the middle of one tile and end in the middle of another. Shares are at least one tile long (the launcher
// sees to that), so a tile is shared by at most two pairs: the one whose share BEGINS inside it computes the later depth range
// first thing and stores it as a partial result; the one whose share ENDS inside it computes the earlier depth range last and
// adds it to the stored partial (a + b = b + a: the result does not depend on timing). Flags in global memory order the two.
struct PairWork {
    uint32_t tile, k0, k1;  // current item: depth stages [k0, k1) of `tile`
    uint32_t next_tile, stride, num_tiles, kblocks;
    uint64_t unit, unit_end;
    bool split;
    __device__ PairWork(const GemmDev &p, uint32_t pair, uint32_t num_pairs, uint32_t tiles)
        : tile(0), k0(0), k1(0), next_tile(pair), stride(num_pairs), num_tiles(tiles), kblocks(p.kblocks), unit(0), unit_end(0),
          split(p.split_flags != nullptr) {
        if (split) {
            const uint64_t total = (uint64_t)tiles * kblocks;
            unit = total * pair / num_pairs;
            unit_end = total * (pair + 1) / num_pairs;
        }
    }
    __device__ bool next() {
        if (!split) {
            if (next_tile >= num_tiles) return false;
            tile = next_tile; k0 = 0; k1 = kblocks;
            next_tile += stride;
            return true;
        }
        if (unit >= unit_end) return false;
        tile = (uint32_t)(unit / kblocks);
        k0 = (uint32_t)(unit - (uint64_t)tile * kblocks);
        const uint64_t left = unit_end - unit;
        k1 = left < (uint64_t)(kblocks - k0) ? k0 + (uint32_t)left : kblocks;
        unit += k1 - k0;
        return true;
    }
};

// Sixteen flags per shared tile, one per epilogue warp of the pair that stored the partial result.
__device__ __forceinline__ void publish_partial(uint32_t *flag, uint32_t epoch) {
    __threadfence();
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(flag), "r"(epoch) : "memory");
}
// All lanes of a warp call this; returns false (recording wait site 7) when the flags do not show up within the limit.
__device__ __forceinline__ bool await_partial(const uint32_t *flags, uint32_t epoch, int lane, unsigned int *error_word, uint32_t limit_us) {
    const uint64_t start = global_timer_ns();
    while (true) {
        uint32_t v = epoch;
        if (lane < 2 * kEpilogueWarps) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + lane) : "memory");
        if (__all_sync(0xffffffffu, v == epoch)) return true;
        const bool expired = __shfl_sync(0xffffffffu, (uint32_t)(global_timer_ns() - start > (uint64_t)limit_us * 1000ull), 0) != 0;
        if (expired) {
            if (lane == 0) atomicCAS(error_word, 0u, (7u << 16) | (blockIdx.x & 0xffffu) | 0x80000000u);
            return false;
        }
        __nanosleep(200);
    }
}

template <int kKind, int kEpi>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap a_map, const __grid_constant__ CUtensorMap b_map, const GemmDev p) {
    constexpr int kBN = kPairBN;
    constexpr int kStages = kPairStages;
    constexpr int kTmemCols = 2 * kBN;
    constexpr int kColsPerThread = kBN / 2;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kPairBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kStages + s); };
    auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kStages + a); };
    auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kStages + 2 + a); };
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kPairBarrierOffset + 8 * (2 * kStages + 4));
    const uint32_t drain_bar = bar_base + 8u * (2 * kStages + 5);  // leader only: "all MMAs of the pair have retired"

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_ctarank();           // 0 = leader
    const uint32_t pair = blockIdx.x >> 1;
    const uint32_t num_pairs = gridDim.x >> 1;
    const uint32_t num_tiles = p.tiles_m * p.tiles_n;  // 256 x 256 tiles

    if (threadIdx.x == 0) {
        prefetch_tensormap(&a_map);
        prefetch_tensormap(&b_map);
        for (int s = 0; s < kStages; ++s) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(tmem_full_bar(a), 1);
            mbar_init(tmem_empty_bar(a), 2 * kEpilogueWarps);  // one arrival per epilogue warp of both CTAs
        }
        mbar_init(drain_bar, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<2>(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        tmem_relinquish<2>();
    }
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();  // the peer's barriers must exist before anything is signalled across the pair
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------------------------------------ producer (both CTAs)
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, issued = 0;
            bool ok = true;
            for (PairWork work(p, pair, num_pairs, num_tiles); ok && work.next();) {
                uint32_t mt, nt;
                tile_coords(work.tile, p.tiles_m, p.tiles_n, mt, nt);
                if (tile_skipped(p.tri_diag, mt * 256u, (nt + 1) * kBN)) continue;
                const uint32_t a_row = mt * 256u + rank * 128u;
                const uint64_t b_chunk0 = ((uint64_t)nt * 2u + rank) * p.kblocks;  // this CTA's half of the B tile
                for (uint32_t kb = work.k0; kb < work.k1; ++kb) {
                    if (!mbar_wait<true>(empty_bar(stage), phase ^ 1u, 1, p.error_word, p.wait_us[1])) { ok = false; break; }
                    const uint32_t a_dst = smem_base + stage * kPairStageBytes;
                    const uint32_t b_dst = a_dst + kBM * kBKBytes;
                    const uint32_t leader_full = map_to_cta(full_bar(stage), 0);
                    if (rank == 0) mbar_expect_tx(full_bar(stage), 2 * kPairStageBytes);
                    tma_load_2d_pair(a_dst, &a_map, (int)(kb * p.elems_per_kblock), (int)a_row, leader_full);
                    tma_load_2d_pair(b_dst, &b_map, 0, (int)((b_chunk0 + kb) * kChunkRows), leader_full);
                    ++issued;
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // See the single-CTA kernel. Both CTAs' copies count on the LEADER's `full` barriers, so the leader can
                // wait for them; the follower cannot read a remote barrier and sleeps instead - its last copy was issued
                // at least one wait limit ago, and neither CTA retires before the cluster barrier at the end.
                if (rank == 0) {
                    int s = stage;
                    uint32_t ph = phase;
                    for (uint32_t i = 0; i < issued && i < (uint32_t)kStages; ++i) {
                        if (s == 0) { s = kStages; ph ^= 1u; }
                        --s;
                        if (!mbar_wait<true>(full_bar(s), ph, 6, p.error_word, p.wait_us[6])) break;
                    }
                } else {
                    for (int i = 0; i < 1000; ++i) __nanosleep(1000);
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------ MMA issuer (leader CTA only)
        if (lane == 0 && rank == 0) {
            int stage = 0;
            uint32_t phase = 0, seq = 0;
            bool ok = true;
            for (PairWork work(p, pair, num_pairs, num_tiles); ok && work.next();) {
                uint32_t mt, nt;
                tile_coords(work.tile, p.tiles_m, p.tiles_n, mt, nt);
                if (tile_skipped(p.tri_diag, mt * 256u, (nt + 1) * kBN)) continue;
                for (uint32_t kb0 = work.k0; kb0 < work.k1 && ok; kb0 += p.flush_kblocks, ++seq) {
                    const uint32_t buf = seq & 1u, buf_phase = (seq >> 1) & 1u;
                    if (!mbar_wait<true>(tmem_empty_bar(buf), buf_phase ^ 1u, 2, p.error_word, p.wait_us[2])) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * kBN;
                    const uint32_t kb1 = min(kb0 + p.flush_kblocks, work.k1);
                    for (uint32_t kb = kb0; kb < kb1; ++kb) {
                        if (!mbar_wait<true>(full_bar(stage), phase, 3, p.error_word, p.wait_us[3])) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t a_src = smem_base + stage * kPairStageBytes;
                        const uint64_t a_desc = make_smem_desc_sw128(a_src);
                        const uint64_t b_desc = make_smem_desc_sw128(a_src + kBM * kBKBytes);
#pragma unroll
                        for (int k = 0; k < kBKBytes / kUmmaKBytes; ++k)
                            umma<kKind, 2>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, ((kb - kb0) | (uint32_t)k) != 0u);
                        umma_commit_pair(empty_bar(stage), 3);  // frees the stage in both CTAs
                        if (++stage == kStages) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) umma_commit_pair(tmem_full_bar(buf), 3);
                }
            }
            // As in the single-CTA kernel: wait (bounded) for the pair's last MMAs before either CTA passes the final cluster barrier.
            umma_commit_pair(drain_bar, 1);
            mbar_wait<true>(drain_bar, 0u, 5, p.error_word, p.wait_us[5]);
        }
    } else {
        // ------------------------------------------------------------ epilogue (both CTAs): rows of this CTA's half
        const uint32_t quarter = warp & 3u;
        const uint32_t half = (uint32_t)(warp - 2) >> 2;
        float *colf = reinterpret_cast<float *>(smem_gen + kPairBarrierOffset + 256);
        uint32_t *epi_stage = reinterpret_cast<uint32_t *>(smem_gen + kPairBarrierOffset + 256 + kEpiColfBytes) + (warp - 2) * kEpiStageWords;
        uint32_t seq = 0, local_tile = 0;
        bool ok = true;
        for (PairWork work(p, pair, num_pairs, num_tiles); work.next();) {  // keeps walking after a failed wait, see above
            uint32_t mt, nt;
            tile_coords(work.tile, p.tiles_m, p.tiles_n, mt, nt);
            if (tile_skipped(p.tri_diag, mt * 256u, (nt + 1) * kBN)) continue;
            bool zero_cols = false;
            if constexpr (kEpi != kEpiDot) {
                const uint32_t e = threadIdx.x - 64u;
                const float factor = column_factor<kEpi>(p, nt * kBN + e);
                colf[(local_tile & 1u) * 256 + e] = factor;
                zero_cols = epilogue_barrier_any(special_factor<kEpi>(factor));
            }
            uint32_t acc[kColsPerThread];
#pragma unroll
            for (int j = 0; j < kColsPerThread; ++j) acc[j] = 0u;
            for (uint32_t kb0 = work.k0; kb0 < work.k1 && ok; kb0 += p.flush_kblocks, ++seq) {
                const uint32_t buf = seq & 1u, buf_phase = (seq >> 1) & 1u;
                if (!mbar_wait<true>(tmem_full_bar(buf), buf_phase, 4, p.error_word, p.wait_us[4])) { ok = false; break; }
                tc_fence_after_sync();
                if (kb0 == work.k0) {
                    // First span of a tile: nothing to add to, so every load goes straight into the accumulators and all of
                    // them are in flight before the one wait.
#pragma unroll
                    for (int c = 0; c < kColsPerThread / 16; ++c)
                        tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + buf * kBN + half * kColsPerThread + c * 16,
                                      *reinterpret_cast<uint32_t(*)[16]>(&acc[c * 16]));
#pragma unroll
                    for (int c = 0; c < kColsPerThread / 32; ++c) tmem_ld_wait_for(*reinterpret_cast<uint32_t(*)[32]>(&acc[c * 32]));
                } else {
                    // Later spans are added to the running sums eight columns at a time, two loads deep: while the values of
                    // one load are added, the next load is on its way from TMEM (no more registers than one 16-column load).
                    const uint32_t span_addr = tmem_base + ((quarter * 32u) << 16) + buf * kBN + half * kColsPerThread;
                    uint32_t va[8], vb[8];
                    auto add8 = [&](int c8, const uint32_t (&v)[8]) {
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            if constexpr (kKind == kKindI8) acc[c8 * 8 + j] += v[j];
                            else acc[c8 * 8 + j] = __float_as_uint(__uint_as_float(acc[c8 * 8 + j]) + __uint_as_float(v[j]));
                        }
                    };
                    tmem_ld_32x8(span_addr, va);
#pragma unroll
                    for (int c8 = 0; c8 < kColsPerThread / 8; c8 += 2) {
                        tmem_ld_wait_for(va);
                        tmem_ld_32x8(span_addr + (c8 + 1) * 8, vb);
                        add8(c8, va);
                        tmem_ld_wait_for(vb);
                        if (c8 + 2 < kColsPerThread / 8) tmem_ld_32x8(span_addr + (c8 + 2) * 8, va);
                        add8(c8 + 1, vb);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive_cluster_addr(map_to_cta(tmem_empty_bar(buf), 0));
            }
            if (!ok) continue;
            if constexpr (kEpi == kEpiDot) {
                if (work.k1 < p.kblocks) {
                    // The earlier depth range of a tile shared with the next pair, which stored the later range long ago (it was
                    // that pair's first item, this is our last): wait for its sixteen warps' flags, then add to what they stored.
                    if (!await_partial(p.split_flags + (uint64_t)pair * (2 * kEpilogueWarps), p.split_epoch, lane, p.error_word, p.wait_us[7])) {
                        ok = false;
                        continue;
                    }
                    store_tile<kEpi, kColsPerThread, 16, kKind != kKindI8, true>(acc, p, mt * 256u + rank * 128u + quarter * 32u, nt * kBN + half * kColsPerThread,
                                                                                 epi_stage, colf + (local_tile & 1u) * 256, half * kColsPerThread, lane, zero_cols);
                    ++local_tile;
                    continue;
                }
            }
            store_tile<kEpi, kColsPerThread, 16, kKind != kKindI8>(acc, p, mt * 256u + rank * 128u + quarter * 32u, nt * kBN + half * kColsPerThread,
                                                                   epi_stage, colf + (local_tile & 1u) * 256, half * kColsPerThread, lane, zero_cols);
            ++local_tile;
            if constexpr (kEpi == kEpiDot) {
                if (work.k0 > 0) {
                    // The later depth range of a tile shared with the previous pair: tell it that this warp's cells are in place.
                    __syncwarp();
                    if (lane == 0) publish_partial(p.split_flags + (uint64_t)(pair - 1) * (2 * kEpilogueWarps) + rank * kEpilogueWarps + (warp - 2), p.split_epoch);
                }
            }
        }
    }

    // Neither CTA may retire while its partner can still read its shared memory or signal its barriers.
    tc_fence_before_sync();
    __syncwarp();
    cluster_sync_all();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<2>(tmem_base, kTmemCols);
    }
}

struct KindInfo {
    int kind;
    uint32_t c_fmt, ab_fmt;
    CUtensorMapDataType tma_type;
    uint32_t int_mode;
};

bool kind_info(uint32_t dt, KindInfo &ki) {
    switch (dt) {
    case kBF16: ki = {kKindF16, 1, 1, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 0}; return true;
    case kF16: ki = {kKindF16, 1, 0, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 0}; return true;
    case kE4M3: ki = {kKindF8F6F4, 1, 0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 0}; return true;
    case kE5M2: ki = {kKindF8F6F4, 1, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 0}; return true;
    // FP6 operands arrive already rewritten (see transform_piece): as e4m3 codes, or packed for the native formats.
    case kE2M3: ki = {kKindF8F6F4, 1, fp6_native() ? 3u : 0u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 0}; return true;
    case kE3M2: ki = {kKindF8F6F4, 1, fp6_native() ? 4u : 0u, CU_TENSOR_MAP_DATA_TYPE_UINT8, 0}; return true;
    case kI8: ki = {kKindI8, 2, 1, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1}; return true;
    case kU8: ki = {kKindI8, 2, 0, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2}; return true;
    default: return false;
    }
}

int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (cached[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        cached[dev] = n > 0 ? n : 148;
    }
    return cached[dev];
}

template <int kKind, int kBN, int kStages, int kEpi>
cudaError_t launch_one(const CUtensorMap &map, const GemmDev &dev, cudaStream_t stream) {
    using Plan = SmemPlan<kBN, kStages>;
    auto kernel = gemm_tc_kernel<kKind, kBN, kStages, kEpi>;
    static bool configured[64] = {false};
    int d = 0;
    cudaGetDevice(&d);
    if (d >= 0 && d < 64 && !configured[d]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan::kTotal);
        if (e != cudaSuccess) return e;
        configured[d] = true;
    }
    uint32_t tiles = dev.tiles_m * dev.tiles_n;
    uint32_t sms = (uint32_t)device_sm_count();
    if (sm_budget() > 0 && (uint32_t)sm_budget() < sms) sms = (uint32_t)sm_budget();
    uint32_t grid = tiles < sms ? tiles : sms;
    kernel<<<grid, kThreads, Plan::kTotal, stream>>>(map, dev);
    return cudaGetLastError();
}

template <int kKind, int kEpi>
cudaError_t launch_by_tile(int bn, bool wide_store, const CUtensorMap &map, const GemmDev &dev, cudaStream_t stream) {
    if (bn == 256 && wide_store) return launch_one<kKind, 256, 3, kEpi>(map, dev, stream);
    if (bn == 256) return launch_one<kKind, 256, 4, kEpi>(map, dev, stream);
    return launch_one<kKind, 128, 6, kEpi>(map, dev, stream);
}

template <int kKind>
cudaError_t launch_by_epilogue(int epi, int bn, bool wide_store, const CUtensorMap &map, const GemmDev &dev, cudaStream_t stream) {
    switch (epi) {
    case kEpiDot: return launch_by_tile<kKind, kEpiDot>(bn, wide_store, map, dev, stream);
    case kEpiAngular: return launch_by_tile<kKind, kEpiAngular>(bn, wide_store, map, dev, stream);
    case kEpiEuclidean: return launch_by_tile<kKind, kEpiEuclidean>(bn, wide_store, map, dev, stream);
    case kEpiHamming:  // the set distances exist for one-bit inputs only, which run on the integer kind
        if constexpr (kKind == kKindI8) return launch_by_tile<kKind, kEpiHamming>(bn, wide_store, map, dev, stream);
        else return cudaErrorInvalidValue;
    case kEpiJaccard:
        if constexpr (kKind == kKindI8) return launch_by_tile<kKind, kEpiJaccard>(bn, wide_store, map, dev, stream);
        else return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
}

// Hand-over flags of the split mode: a ring of 64 launches x 128 pairs x 16 flags per GPU, allocated on the first launch
// that splits and never cleared - every launch marks its flags with its own number. Only raw-dot products split, so the
// entry points that promise not to allocate (distance epilogues) never come here.
constexpr uint32_t kSplitRing = 64, kSplitPairsMax = 128, kSplitFlagsPerLaunch = kSplitPairsMax * 2 * kEpilogueWarps;
std::atomic<uint32_t> g_split_epoch{0};
uint32_t *split_flag_ring() {
    static std::mutex mutex;
    static uint32_t *ring[64] = {nullptr};
    int d = 0;
    cudaGetDevice(&d);
    if (d < 0 || d >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mutex);
    if (!ring[d]) {
        void *ptr = nullptr;
        const size_t bytes = (size_t)kSplitRing * kSplitFlagsPerLaunch * sizeof(uint32_t);
        if (cudaMalloc(&ptr, bytes) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        if (cudaMemset(ptr, 0, bytes) != cudaSuccess) { cudaGetLastError(); cudaFree(ptr); return nullptr; }
        ring[d] = static_cast<uint32_t *>(ptr);
    }
    return ring[d];
}

// `split`: 0 = whole tiles (the default for every shape), 2 = split the depth between pairs whenever the shape allows it
// (nkb_set_gemm_variant(5)). Splitting by itself whenever whole tiles leave pairs idle was measured and withdrawn: at
// 1024 x 8192 x 8192 (bf16) 135 us against 114 us with whole tiles, at 2048 rows 272 against 221 - pairs that start at
// different depths no longer fetch the same A and B chunks at the same time, and the L2 sharing that the lock-step sweep
// gives is worth more than the idle tail of the last wave. It would also make the bits of a row depend on how many rows
// are multiplied with it, which the reference's row-slicing callers may not see.
template <int kKind, int kEpi>
cudaError_t launch_pair(const CUtensorMap &a_map, const CUtensorMap &b_map, GemmDev dev, cudaStream_t stream, int split) {
    auto kernel = gemm_tc_pair_kernel<kKind, kEpi>;
    static int max_pairs[64] = {0};
    int d = 0;
    cudaGetDevice(&d);
    if (d < 0 || d >= 64) d = 0;
    if (max_pairs[d] == 0) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kPairSmemTotal);
        if (e != cudaSuccess) return e;
        // How many CTA pairs can be resident at once (pairs must sit on SMs that can form a cluster).
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(2 * device_sm_count());
        cfg.blockDim = dim3(kThreads);
        cfg.dynamicSmemBytes = kPairSmemTotal;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        int n = 0;
        if (cudaOccupancyMaxActiveClusters(&n, kernel, &cfg) != cudaSuccess || n <= 0) { cudaGetLastError(); n = device_sm_count() / 2; }
        max_pairs[d] = n;
    }
    uint32_t tiles = dev.tiles_m * dev.tiles_n;
    uint32_t most = (uint32_t)max_pairs[d];
    if (sm_budget() > 1 && (uint32_t)sm_budget() / 2 < most) most = (uint32_t)sm_budget() / 2;
    uint32_t pairs = tiles < most ? tiles : most;
    dev.split_flags = nullptr;
    dev.split_epoch = 0;
    if (kEpi == kEpiDot && split != 0 && dev.tri_diag < 0 && tiles > pairs && pairs <= kSplitPairsMax) {
        // Every share is at least one tile long (tiles > pairs), so no tile is shared by more than two pairs.
        if (split == 2) {
            uint32_t *ring = split_flag_ring();
            if (ring) {
                uint32_t epoch = g_split_epoch.fetch_add(1) + 1;
                if (epoch == 0) epoch = g_split_epoch.fetch_add(1) + 1;  // 0 is what untouched flags hold
                dev.split_flags = ring + (size_t)(epoch % kSplitRing) * kSplitFlagsPerLaunch;
                dev.split_epoch = epoch;
            }
        }
    }
    kernel<<<2 * pairs, kThreads, kPairSmemTotal, stream>>>(a_map, b_map, dev);
    return cudaGetLastError();
}

template <int kKind>
cudaError_t launch_pair_by_epilogue(int epi, const CUtensorMap &a_map, const CUtensorMap &b_map, const GemmDev &dev, cudaStream_t stream, int split) {
    switch (epi) {
    case kEpiDot: return launch_pair<kKind, kEpiDot>(a_map, b_map, dev, stream, split);
    case kEpiAngular: return launch_pair<kKind, kEpiAngular>(a_map, b_map, dev, stream, 0);
    case kEpiEuclidean: return launch_pair<kKind, kEpiEuclidean>(a_map, b_map, dev, stream, 0);
    case kEpiHamming:
        if constexpr (kKind == kKindI8) return launch_pair<kKind, kEpiHamming>(a_map, b_map, dev, stream, 0);
        else return cudaErrorInvalidValue;
    case kEpiJaccard:
        if constexpr (kKind == kKindI8) return launch_pair<kKind, kEpiJaccard>(a_map, b_map, dev, stream, 0);
        else return cudaErrorInvalidValue;
    default: return cudaErrorInvalidValue;
    }
}

} // namespace

// The tensor cores truncate (toward zero) when they add products into their f32 accumulators, so one long accumulation
// chain drifts: measured on B200, a bf16 chain of 8192 values is off by 3.7e-7 .. 7.8e-7 of sum |a||b|, ten times the error
// of NumKong's own f32 kernels. The depth is therefore cut into spans; each span is accumulated in TMEM, read out, and the
// spans are added in registers with round-to-nearest. A read-out keeps the tensor cores off TMEM for the ~256 cycles it
// lasts, so spans are made as long as the reference's own error allows. Measured against every x86 back end of the
// reference (scalar, Haswell, Skylake, Genoa, Sapphire Rapids AMX) on the same inputs, error as |c - exact| / sum |a||b|,
// max / mean, 64 values per stage:
//   bf16, N(0,1):           depth 1024: reference 4.0e-8 / 4.3e-9, here 2 stages 5.0e-8 / 4.8e-9, 3 stages 6.3e-8 / 6.5e-9
//                           depth 8192: reference 5.1e-8 / 5.1e-9, here 6 stages 3.2e-8 / 4.9e-9, 8 stages 4.6e-8 / 6.6e-9
//   bf16, all-positive:     depth 1024: reference 3.6e-7 / 7.2e-8, here 3 stages 2.7e-7 / 7.0e-8, 4 stages 3.7e-7 / 1.6e-7
//                           depth 8192: reference 1.5e-6 / 2.7e-7, here 6 stages 5.8e-7 / 2.6e-7, 8 stages 7.9e-7 / 4.9e-7
//   f16, N(0,1):            depth 1024: reference 1.0e-7 / 1.05e-8, here 3 stages 9.5e-8 / 1.0e-8, 4 stages 9.4e-8 / 1.3e-8
//                           depth 8192: reference 7.6e-8 / 1.07e-8, here 8 stages 6.1e-8 / 8.9e-9, 12 stages 8.1e-8 / 1.3e-8
// Both follow span ~ sqrt(depth): bf16 sqrt(depth)/16 stages (4 sqrt(depth) values), f16 sqrt(depth)/11 stages. (bf16 products
// carry 16 significant bits and survive the alignment to an accumulator up to 2^8 times larger untouched, which is why its
// all-positive error has a knee at 256 values; f16 products carry 22 bits and lose some from the first stage on: on
// all-positive f16 data even one-stage spans leave 1.8 units in the last place where the reference has 0.6 - 1.1.)
// The 8- and 6-bit floats sit ten times lower and level off at 1e-8: 16 stages (measured at depth 8192: the error of the
// reference's own kernels; 32 stages double it on wide-range inputs). e2m3 products are multiples of 2^-6 of at most 56.25,
// so 4660 of them add up exactly in f32 whatever the inputs: 32 stages (4096 values).
uint32_t default_accumulation_span(uint32_t dtype, uint64_t depth) {
    if (dtype == kE2M3) return 32u;
    if (dtype != kBF16 && dtype != kF16) return 16u;
    const double stages = sqrt((double)depth) / (dtype == kBF16 ? 16.0 : 11.0);
    uint32_t span = (uint32_t)(stages + 0.5);
    if (span < 1u) span = 1u;
    if (span > 16u) span = 16u;
    return span;
}

EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void *ptr = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(ptr);
    }
    return fn;
}

cudaError_t launch_gemm_tc(const GemmArgs &args, cudaStream_t stream) {
    KindInfo ki;
    if (!kind_info(args.dtype, ki)) return cudaErrorInvalidValue;
    if (args.m == 0 || args.n == 0) return cudaSuccess;
    if (args.m > 0x7fffffffull || args.n > 0x7fffffffull || args.k > 0x7fffffffull) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(args.a) & 15u) || (args.a_stride & 15u)) return cudaErrorMisalignedAddress;

    const uint32_t eb = dtype_bytes(args.dtype);
    // Tile configuration: 3 = CTA pairs sharing 256 x 256 tiles, 1 = 128 x 256 per CTA, 2 = 128 x 128 per CTA.
    const uint64_t chunk_rows_total = round_up(args.n, kRowPad) * (args.depth_padded_bytes / kBKBytes);
    // Measured on B200 at 8192^3 the pair kernel is 5-10 % faster (bf16 1440 vs 1368, i8 3090 vs 2802 Tops), and at
    // 8192 x 8192 it leads from 8 stages of depth on (bf16 depth 512: 817 vs 790, 2048: 1290 vs 1213; i8 depth 1024:
    // 1377 vs 1300, 4096: 2610 vs 2270; i8 at 4 stages: 720 vs 830, the other way round). With the filtering distance
    // epilogue at depth 768 the two are level. So pairs are used from 8 stages on when there is at least one
    // 256 x 256 tile per CTA pair.
    const uint64_t pair_tiles = ((args.m + 255) / 256) * ((args.n + 255) / 256);
    const bool pair_by_shape = (args.variant & 0xff) == 0 && args.depth_padded_bytes / kBKBytes >= 8 &&
                               pair_tiles >= (uint64_t)device_sm_count() / 2;
    // Variant 5 = CTA pairs with the depth split between pairs whenever the shape allows; variant 3 = CTA pairs, whole tiles.
    const bool use_pair = ((args.variant & 0xff) == 3 || (args.variant & 0xff) == 5 || pair_by_shape) && chunk_rows_total < 0x7fffffffull;
    const int split = (args.variant & 0xff) == 5 ? 2 : 0;
    int bn = 256;
    if ((args.variant & 0xff) == 1 || (args.variant & 0xff) == 4) bn = 256;
    else if ((args.variant & 0xff) == 2) bn = 128;
    else {
        uint64_t tiles256 = ((args.m + kBM - 1) / kBM) * ((args.n + 255) / 256);
        if (args.n <= 128 || tiles256 < (uint64_t)device_sm_count()) bn = 128;
    }

    // Variant 4 forces the four-stage 128 x 256 kernel (A/B comparisons); otherwise short depths take the wide-store one.
    const bool wide_store = (args.variant & 0xff) != 4 && args.depth_padded_bytes / kBKBytes <= kShortDepthBlocks;

    EncodeTiledFn encode = get_encode_tiled();
    if (!encode) return cudaErrorNotSupported;
    CUtensorMap map;
    cuuint64_t dims[2] = {args.k, args.m};
    cuuint64_t strides[1] = {args.a_stride};
    cuuint32_t box[2] = {kBKBytes / eb, (cuuint32_t)kBM};
    cuuint32_t elem_strides[2] = {1, 1};
    CUresult r = encode(&map, ki.tma_type, 2, const_cast<void *>(args.a), dims, strides, box, elem_strides,
                        CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                        CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;

    GemmDev dev;
    dev.b_payload = static_cast<const uint8_t *>(args.b_payload);
    dev.b_norms = args.b_norms;
    dev.a_norms = args.a_norms;
    dev.c = static_cast<uint8_t *>(args.c);
    dev.c_stride = args.c_stride;
    dev.m = (uint32_t)args.m;
    dev.n = (uint32_t)args.n;
    dev.kblocks = (uint32_t)(args.depth_padded_bytes / kBKBytes);
    dev.elems_per_kblock = kBKBytes / eb;
    dev.tiles_m = (uint32_t)((args.m + kBM - 1) / kBM);
    dev.tiles_n = (uint32_t)((args.n + bn - 1) / bn);
    dev.idesc = make_idesc(ki.c_fmt, ki.ab_fmt, kBM, bn);
    dev.int_mode = ki.int_mode;
    // Integers are exact in one span; floats take the span the element type and depth call for unless one is forced.
    const uint32_t forced_flush = ((uint32_t)args.variant >> 8) & 0xffu;  // nkb_set_accumulation_span
    const uint32_t auto_flush = default_accumulation_span(args.dtype, args.k);
    dev.flush_kblocks = ki.kind == kKindI8 ? dev.kblocks : (forced_flush ? forced_flush : auto_flush);
    if (dev.flush_kblocks == 0) dev.flush_kblocks = 1;
    dev.error_word = args.error_word;
    wait_limits_us(dev.wait_us);
    dev.tri_diag = args.tri_diag;
    const bool filtering = args.candidates != nullptr && args.epilogue != kEpiDot;
    dev.threshold_bits = filtering ? args.threshold_bits : nullptr;
    dev.candidate_counts = filtering ? args.candidate_counts : nullptr;
    dev.candidates = filtering ? args.candidates : nullptr;
    dev.candidate_capacity = args.candidate_capacity;
    dev.column_id_base = args.column_id_base;
    dev.split_flags = nullptr;
    dev.split_epoch = 0;

    if (use_pair) {
        // The packed payload seen as rows of 128 bytes: one 16 KiB chunk = 128 consecutive rows, copied verbatim
        // (the swizzle is already in the data).
        CUtensorMap b_map;
        cuuint64_t b_dims[2] = {kBKBytes, chunk_rows_total};
        cuuint64_t b_strides[1] = {kBKBytes};
        cuuint32_t b_box[2] = {kBKBytes, kChunkRows};
        r = encode(&b_map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void *>(args.b_payload), b_dims, b_strides, b_box,
                   elem_strides, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
        dev.tiles_m = (uint32_t)((args.m + 255) / 256);
        dev.tiles_n = (uint32_t)((args.n + 255) / 256);
        dev.idesc = make_idesc(ki.c_fmt, ki.ab_fmt, 256, 256);
        switch (ki.kind) {
        case kKindF16: return launch_pair_by_epilogue<kKindF16>(args.epilogue, map, b_map, dev, stream, split);
        case kKindF8F6F4: return launch_pair_by_epilogue<kKindF8F6F4>(args.epilogue, map, b_map, dev, stream, split);
        default: return launch_pair_by_epilogue<kKindI8>(args.epilogue, map, b_map, dev, stream, split);
        }
    }
    switch (ki.kind) {
    case kKindF16: return launch_by_epilogue<kKindF16>(args.epilogue, bn, wide_store, map, dev, stream);
    case kKindF8F6F4: return launch_by_epilogue<kKindF8F6F4>(args.epilogue, bn, wide_store, map, dev, stream);
    default: return launch_by_epilogue<kKindI8>(args.epilogue, bn, wide_store, map, dev, stream);
    }
}

} // namespace nkb
