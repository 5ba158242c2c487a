// Internal declarations shared by the translation units of libnumkong_b200.so:
// dtype codes (numerically equal to NumKong's nk_dtype_t, include/numkong/types.h:923-953),
// the packed-blob header, and the launchers each .cu file provides.
#pragma once
#include <cstddef>
#include <cstdint>
#include <cuda.h>
#include <cuda_runtime.h>

namespace nkb {

enum Dtype : uint32_t {
    kU1 = 1u << 1,    // eight one-bit values per byte (include/numkong/types.h:925)
    kI8 = 1u << 2,
    kU8 = 1u << 6,
    kF64 = 1u << 10,
    kF32 = 1u << 11,
    kF16 = 1u << 12,
    kBF16 = 1u << 13,
    kE4M3 = 1u << 14,
    kE5M2 = 1u << 15,
    kI4 = 1u << 16,   // two signed 4-bit values per byte, low nibble first (include/numkong/types.h:1551-1558)
    kU4 = 1u << 17,   // two unsigned 4-bit values per byte
    kE2M3 = 1u << 18,
    kE3M2 = 1u << 19,
};

// What the accumulators are turned into before they are stored.
// Hamming / Jaccard (u1 only) turn the AND-popcount "dot" and the two population counts into a set distance
// (include/numkong/set/serial.h:150-168).
enum Epilogue : int { kEpiDot = 0, kEpiAngular = 1, kEpiEuclidean = 2, kEpiHamming = 3, kEpiJaccard = 4 };

constexpr uint32_t kMagicDots = 0x32424B4Eu;    // "NKB2"
constexpr uint32_t kMagicMaxsim = 0x4D424B4Eu;  // "NKBM"
constexpr uint32_t kHeaderBytes = 128;
constexpr uint32_t kChunkRows = 128;            // rows per pre-swizzled chunk
constexpr uint32_t kChunkRowBytes = 128;        // bytes of depth per chunk row (one swizzle span)
constexpr uint32_t kChunkBytes = kChunkRows * kChunkRowBytes;  // 16 KiB
constexpr uint32_t kRowPad = 256;               // rows are padded to a multiple of this

// 128-byte header at the start of every packed blob. The blob is position independent:
// it holds offsets only, so callers may memcpy, move or serialise it freely.
//
// Tensor-core dtypes: the payload is a grid of 16 KiB chunks ordered [row_block][depth_block];
// a chunk is 128 rows x 128 bytes of depth in exactly the shared-memory image tcgen05.mma
// reads for a K-major, 128-byte-swizzled operand (row r at (r/8)*1024 + (r%8)*128, its
// 16-byte piece c stored at piece position c ^ (r%8)). One untiled bulk copy brings a
// chunk into shared memory with no further rearrangement.
// f32: the payload is plain row-major f32 with rows padded to `depth_padded_bytes`.
// After the payload: one norm per row (squared norm for dots blobs, inverse norm for MaxSim blobs).
struct PackedHeader {
    uint32_t magic;
    uint32_t dtype;
    uint32_t element_bytes;
    uint32_t norm_bytes;
    uint64_t rows;                // n (vectors)
    uint64_t depth;               // k (logical dimensions)
    uint64_t rows_padded;         // multiple of 256
    uint64_t depth_padded_bytes;  // multiple of 128
    uint64_t payload_offset;
    uint64_t norms_offset;
    uint64_t total_bytes;
    uint64_t nonce;               // changes with every pack call; keys the device-side cache of host blobs
    uint64_t reserved[6];
};
static_assert(sizeof(PackedHeader) == 128, "header must be 128 bytes");

inline uint32_t dtype_bytes(uint32_t dt) {
    switch (dt) {
    case kF64: return 8;
    case kF32: return 4;
    case kF16: case kBF16: return 2;
    default: return 1;
    }
}
// Bytes of one stored norm: u32 for integers, f64 for f32 / f64, f32 otherwise.
inline uint32_t norm_bytes(uint32_t dt) { return (dt == kF32 || dt == kF64) ? 8 : 4; }
// Bytes of one output cell of dots_packed: f64 for f32 / f64 inputs, 4 bytes otherwise.
inline uint32_t dot_out_bytes(uint32_t dt) { return (dt == kF32 || dt == kF64) ? 8 : 4; }
// f32 and f64 inputs run on CUDA cores with f64 results; their packed payload is plain row-major.
inline bool is_cuda_core_dtype(uint32_t dt) { return dt == kF32 || dt == kF64; }
inline bool dtype_supported(uint32_t dt) {
    switch (dt) {
    case kI8: case kU8: case kF32: case kF16: case kBF16: case kE4M3: case kE5M2: case kE2M3: case kE3M2: case kI4: case kU4: case kU1: case kF64: return true;
    default: return false;
    }
}

inline uint64_t round_up(uint64_t x, uint64_t m) { return (x + m - 1) / m * m; }

// Every mbarrier wait inside the tensor-core kernels is bounded. Wait sites (the number a wait that gave up leaves in the
// error word, 0x80000000 | site << 16 | block):
//   1 producer waits for a free pipeline stage          2 MMA issuer waits for a drained accumulator
//   3 MMA issuer waits for a loaded stage               4 epilogue waits for a finished accumulator
//   5 MMA issuer waits for its last MMAs before leaving 6 producer waits for its last copies before leaving
//   7 epilogue waits for the partial tile another CTA pair stored (depth split between pairs)
//   8 a GPU waits for the other GPUs of its group at nkb_peer_barrier (the low 16 bits then name the missing peer)
#ifndef NKB_WAIT_LIMIT_NS
#define NKB_WAIT_LIMIT_NS 2000000000ull  // 2 s
#endif
constexpr uint32_t kDefaultWaitLimitUs = (uint32_t)(NKB_WAIT_LIMIT_NS / 1000ull);
constexpr int kWaitSites = 9;

// Sub-byte types: `depth` counts values (nibbles for i4 / u4, bits for u1), a row occupies ceil(depth / per_byte) bytes,
// and - like the reference's kernels (include/numkong/dot/serial.h:185-215) - every value of the last byte takes part
// even when `depth` stops inside it. On the device such a row is expanded to one i8 / u8 per value, so everything after
// the packer and the operand staging sees i8 / u8.
inline uint32_t values_per_byte(uint32_t dt) { return dt == kU1 ? 8u : (dt == kI4 || dt == kU4) ? 2u : 0u; }  // 0: not sub-byte
inline bool is_subbyte(uint32_t dt) { return values_per_byte(dt) != 0; }
inline uint64_t source_row_bytes(uint32_t dt, uint64_t depth) {
    const uint32_t per = values_per_byte(dt);
    return per ? (depth + per - 1) / per : depth * dtype_bytes(dt);
}
inline uint32_t operand_dtype(uint32_t dt) { return dt == kI4 ? kI8 : (dt == kU4 || dt == kU1) ? kU8 : dt; }
inline uint64_t operand_depth(uint32_t dt, uint64_t depth) {
    const uint32_t per = values_per_byte(dt);
    return per ? (depth + per - 1) / per * per : depth;
}

#ifdef __CUDACC__
// Order-preserving integer key of an f32 for selection: a < b  <=>  key(a) < key(b); every NaN shares the last key
// but one (0xffffffff stays free as "no value").
__device__ __forceinline__ uint32_t selection_key(float f) {
    const uint32_t u = __float_as_uint(f);
    if ((u & 0x7fffffffu) > 0x7f800000u) return 0xfffffffeu;
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float selection_value(uint32_t key) {
    return __uint_as_float((key & 0x80000000u) ? (key & 0x7fffffffu) : ~key);
}
#endif

struct PackedGeometry {
    uint64_t rows_padded, depth_padded_bytes, payload_offset, norms_offset, total_bytes;
};
inline PackedGeometry packed_geometry(uint32_t dt, uint64_t rows, uint64_t depth) {
    PackedGeometry g;
    g.rows_padded = round_up(rows ? rows : 1, kRowPad);
    g.depth_padded_bytes = round_up((depth ? operand_depth(dt, depth) : 1) * dtype_bytes(dt), kChunkRowBytes);
    g.payload_offset = kHeaderBytes;
    g.norms_offset = g.payload_offset + g.rows_padded * g.depth_padded_bytes;
    g.total_bytes = g.norms_offset + round_up(rows * norm_bytes(dt), 128);
    return g;
}

// ---- launchers (all asynchronous on `stream`; return a cudaError_t from the launch) ----

// Sum of squares of every row. `out` is f32 (float dtypes), u32 (i8/u8) or f64 (f32 input);
// `as_f32` forces an f32 result for integers (the batched-distance epilogues read f32 norms).
// `inverse` stores 1/sqrt(sumsq) (0 for a zero row) instead, as MaxSim blobs do.
cudaError_t launch_row_sumsq(uint32_t dt, const void *x, uint64_t rows, uint64_t depth, uint64_t stride_bytes,
                             void *out, bool as_f32, bool inverse, cudaStream_t stream);

// Rewrites applied to each 16-byte piece of an FP6 operand on its way to the tensor cores.
enum PieceMode : int { kPieceNone = 0, kPieceE2M3ToE4M3 = 1, kPieceE3M2ToE4M3 = 2, kPieceFp6Pack = 3,
                       kPieceI4ToI8 = 4, kPieceU4ToU8 = 5, kPieceU1ToU8 = 6 };
// The expanding modes write a 16-byte piece from 16 >> shift source bytes (8 for nibbles, 2 for bits).
#ifdef __CUDACC__
__host__ __device__
#endif
inline int piece_mode_shift(int mode) { return mode == kPieceU1ToU8 ? 3 : (mode == kPieceI4ToI8 || mode == kPieceU4ToU8) ? 1 : 0; }
// How FP6 operands are fed to tcgen05.mma: 0 = recoded to e4m3 (exact), 1 = native 6-bit operand formats.
int fp6_native();
inline int piece_mode_for(uint32_t dt) {
    if (dt == kI4) return kPieceI4ToI8;
    if (dt == kU4) return kPieceU4ToU8;
    if (dt == kU1) return kPieceU1ToU8;
    if (dt != kE2M3 && dt != kE3M2) return kPieceNone;
    if (fp6_native()) return kPieceFp6Pack;
    return dt == kE2M3 ? kPieceE2M3ToE4M3 : kPieceE3M2ToE4M3;
}

// Writes the pre-swizzled chunk grid (or padded row-major f32) of a packed blob.
cudaError_t launch_pack_payload(uint32_t dt, const void *b, uint64_t rows, uint64_t depth, uint64_t stride_bytes,
                                void *payload, uint64_t rows_padded, uint64_t depth_padded_bytes, int piece_mode,
                                cudaStream_t stream);

// Copies a strided matrix into a 16-byte-aligned, 16-byte-pitched scratch copy (for TMA),
// applying `piece_mode` to every 16-byte piece. `row_bytes` counts SOURCE bytes (a half / an eighth of the written bytes for
// the expanding modes).
cudaError_t launch_restride(const void *src, uint64_t rows, uint64_t row_bytes, uint64_t src_stride,
                            void *dst, uint64_t dst_stride, int piece_mode, cudaStream_t stream);

struct GemmArgs {
    uint32_t dtype;
    int epilogue;                 // Epilogue
    const void *a;                // device, 16-byte aligned, stride multiple of 16
    uint64_t a_stride;
    const void *b_payload;        // device, chunk grid
    const void *b_norms;          // device (epilogue != dot)
    const float *a_norms;         // device f32 (epilogue != dot)
    void *c;
    uint64_t c_stride;
    uint64_t m, n, k;
    uint64_t depth_padded_bytes;
    unsigned int *error_word;     // device
    int variant;                  // 0 = default for the shape; otherwise forces a tile configuration (testing/tuning)
    // Triangular mode for A x A^T: >= 0 stores only the cells with column >= row + tri_diag (rows and columns counted from
    // the first row of `a` / first packed row), writes 0 on that diagonal under a distance epilogue, and skips the tiles
    // that lie wholly below it. -1 = rectangular.
    int32_t tri_diag = -1;
    // Candidate filter (distance epilogues only). When `candidates` is set nothing is written to `c`: every value below
    // its row's threshold is appended to that row's candidate list as (f32 bits of the distance, column + column_id_base).
    // Thresholds are f32 bit patterns compared as signed integers (distances are >= -0 and never NaN); 0x7fffffff
    // lets everything pass.
    const uint32_t *threshold_bits = nullptr;  // one per row of A
    uint32_t *candidate_counts = nullptr;  // one per row of A; may run past `candidate_capacity` (overflow marker)
    uint2 *candidates = nullptr;           // rows x candidate_capacity
    uint32_t candidate_capacity = 0;
    uint32_t column_id_base = 0;
};
// Enqueues exactly one kernel.
cudaError_t launch_gemm_tc(const GemmArgs &args, cudaStream_t stream);
// SMs the persistent tensor-core kernels may occupy (0 = all of them), as set by nkb_set_sm_budget.
int sm_budget();
// Limits of the kernels' bounded waits, one per wait site (microseconds; see nkb_ptx.cuh), as set by nkb_set_wait_limit_ns.
void wait_limits_us(uint32_t (&out)[kWaitSites]);
// Accumulation span (pipeline stages of 128 bytes of depth per tensor-core accumulation chain) the GEMM uses for a
// floating-point element type at this depth when the caller has not forced one.
uint32_t default_accumulation_span(uint32_t dtype, uint64_t depth);

// f32 x f32 -> f64 on CUDA cores. `b` is the padded row-major f32 payload.
cudaError_t launch_gemm_f32(int epilogue, const float *a, uint64_t a_stride, const float *b, uint64_t b_stride,
                            const double *b_norms, const double *a_norms, double *c, uint64_t c_stride,
                            uint64_t m, uint64_t n, uint64_t k, cudaStream_t stream, int32_t tri_diag = -1);
// f64 x f64 -> f64 with the reference's two-lane Dot2 accumulation (bit-identical dots). Same layout rules.
cudaError_t launch_gemm_f64(int epilogue, const double *a, uint64_t a_stride, const double *b, uint64_t b_stride,
                            const double *b_norms, const double *a_norms, double *c, uint64_t c_stride,
                            uint64_t m, uint64_t n, uint64_t k, cudaStream_t stream, int32_t tri_diag = -1);

// Resolves cuTensorMapEncodeTiled through the runtime (no link-time dependency on libcuda).
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn get_encode_tiled();

} // namespace nkb
