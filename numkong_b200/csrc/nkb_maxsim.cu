// MaxSim late interaction, fused: the query-token x document-token similarity tile lives only in
// TMEM; the epilogue keeps a running (max, argmax) per query token and document, normalises the
// winner, and adds the per-query sums. The full similarity matrix is never written to memory.
//
// Replaces NumKong's nk_maxsim_packed_<t> (include/numkong/maxsim.h:106-114). Semantics follow the
// reference's tensor-engine back end (include/numkong/maxsim/sapphireamx.h:716-861): the argmax is
// taken over the RAW dot with a strict comparison (first document token wins ties), only the winner
// is normalised with the inverse norms stored at pack time, the angular is clamped at 0, and the sum
// over query tokens is carried in f64.
//
// One kernel serves both the single (query, document) call of the reference API and the all-pairs
// batch (many queries x many ragged documents packed back to back). A CTA owns one tile of 128 query
// tokens and one contiguous run of whole documents. The run is cut into FOUR STREAMS of whole
// documents (equal shares of its tokens) and sixteen epilogue warps - one per TMEM lane quarter and
// stream - follow them. A warp therefore sees every document of its stream from its first token to
// its last: the running maximum of a document never leaves the warp's registers, no two warps ever
// have to merge partial maxima, and the per-(query, document) sum is finished by the one warp that
// holds the query's 32 rows (a plain store; only queries that straddle warps or tiles add their parts
// atomically - two parts commute).
//
// With the query tile resident in shared memory (depth <= 256 for 16-bit types) the four streams
// advance in lock-step, 64 tokens each per step: their four half chunks sit back to back in one
// stage, ONE N = 256 instruction per 32 bytes of depth multiplies all four, and TMEM holds two such
// 256-column buffers. A warp pulls its stream's 64 columns into registers, hands the buffer back at
// once and scans from registers while the tensor cores fill the other buffer, so no MMA waits for a
// scan. Deeper queries stream through the ring with the documents; the streams then own one
// 128-column accumulator each and take turns.
//
// The batch form first re-lays the documents on 32-token boundaries (maxsim_pad_rows_kernel), so
// that no 32-column chunk of the scan holds a document boundary.
#include <cstdio>
#include <cstring>
#include "nkb_internal.h"
#include "nkb_host.h"
#include "nkb_ptx.cuh"
#include "../../include/numkong_b200.h"

namespace nkb {

namespace {

constexpr int kMsBM = 128;                 // query tokens per CTA = TMEM lanes
constexpr int kMsBN = 128;                 // document tokens per tile = one 128-row block of the packed payload
constexpr int kMsStreams = 4;              // document streams per CTA (TMEM: 2 buffers x 4 x 64 columns, or 4 x 128 for deep queries)
constexpr int kMsEpilogueWarps = 4 * kMsStreams;
constexpr int kMsThreads = 64 + 32 * kMsEpilogueWarps;
// Shared memory: the query tile stays resident when it is at most four depth blocks long (depth <= 256 for 16-bit types:
// every late-interaction model in use), and only document chunks stream through the ring; deeper queries stream through the
// ring with the documents (half as many, twice as large stages).
constexpr int kMsResidentBlocks = 4;
constexpr int kMsResidentBytes = kMsResidentBlocks * (int)kChunkBytes;   // 64 KiB
constexpr int kMsRingBytes = 6 * (int)kChunkBytes;                       // 96 KiB: three stages of 32 KiB
constexpr int kMsRingOffset = kMsResidentBytes;
constexpr int kMsBarrierOffset = kMsRingOffset + kMsRingBytes;
constexpr int kMsMaxStages = 6;
// The epilogue warps run alone on their SM sub-partitions, so every global load they wait for is dead time. The
// inverse norms of the document tokens a CTA walks and the ends of its documents are therefore copied into shared
// memory once per CTA (lookups beyond these windows fall back to global memory).
constexpr int kMsRunTiles = 112;          // 128-token tiles per CTA: the set-up of a CTA (TMEM, barriers, query tile, these caches)
                                          // overlaps with nothing, so runs are as long as the caches below allow (measured:
                                          // 64 -> 128 tiles per run +5 %)
constexpr int kMsInvCache = (kMsRunTiles + 8) * kMsBN;   // tokens (a run plus one long document)
constexpr int kMsEndCache = 256;          // documents
constexpr int kMsCacheOffset = kMsBarrierOffset + 256;
constexpr int kMsSmemTotal = kMsCacheOffset + kMsInvCache * 4 + kMsEndCache * 4 + 1024;

struct MaxsimDev {
    const uint8_t *q_payload, *d_payload;
    const float *q_inv, *d_inv;          // inverse norms per token
    const uint64_t *q_offsets, *d_offsets;  // token offsets per query / document (device), length count+1
    const uint32_t *q_token_query;       // query index of every query token (filled by maxsim_prepare_kernel)
    const uint64_t *stream_bounds;       // first document of every stream, 4 per segment plus one closing entry (same kernel)
    uint64_t n_queries, n_docs;
    uint64_t q_tokens, d_tokens;
    uint32_t kblocks;
    uint32_t q_tiles, segments;
    uint32_t q_group;                    // query tiles that walk the same document segment side by side
    uint32_t idesc;        // M = 128, N = 128: one stream's tile
    uint32_t idesc_pair;   // M = 128, N = 256: the tiles of two neighbouring streams in one instruction
    float *scores_f32;                   // batch: n_queries x n_docs
    uint64_t score_stride;               // in floats
    double *total_f64;                   // single pair: one accumulator
    unsigned int *error_word;
};

// First index i in [0, n] with offsets[i] >= x (offsets ascending, offsets[n] = total).
__device__ __forceinline__ uint64_t lower_bound_offsets(const uint64_t *offsets, uint64_t n, uint64_t x) {
    uint64_t lo = 0, hi = n;
    while (lo < hi) {
        uint64_t mid = (lo + hi) >> 1;
        if (offsets[mid] < x) lo = mid + 1; else hi = mid;
    }
    return lo;
}

// Runs once before maxsim_kernel: the query each query token belongs to, and the first document of every stream. A segment
// is the run of documents whose first token falls into its equal share of all document tokens; its four streams are the
// documents whose first token falls into each quarter of the segment's own tokens.
__global__ void maxsim_prepare_kernel(const uint64_t *q_offsets, uint64_t n_queries, uint64_t q_tokens, uint32_t *q_token_query,
                                      const uint64_t *d_offsets, uint64_t n_docs, uint64_t d_tokens, uint32_t segments,
                                      uint64_t *stream_bounds) {
    const uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < q_tokens) q_token_query[i] = (uint32_t)(lower_bound_offsets(q_offsets, n_queries, i + 1) - 1);
    if (i <= (uint64_t)segments * kMsStreams) {
        const uint64_t per_seg = (d_tokens + segments - 1) / segments;
        const uint64_t seg = i / kMsStreams, part = i % kMsStreams;
        uint64_t bound = n_docs;
        if (seg < segments) {
            const uint64_t first = lower_bound_offsets(d_offsets, n_docs, seg * per_seg);
            bound = first;
            if (part != 0) {
                const uint64_t last = seg + 1 == segments ? n_docs : lower_bound_offsets(d_offsets, n_docs, (seg + 1) * per_seg);
                const uint64_t t0 = d_offsets[first], t1 = d_offsets[last];
                bound = lower_bound_offsets(d_offsets, n_docs, t0 + (t1 - t0) * part / kMsStreams);
                if (bound < first) bound = first;
                if (bound > last) bound = last;
            }
        }
        stream_bounds[i] = bound;
    }
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

constexpr float kLowest = -3.402823466e+38f;

// Largest value of a 32-column chunk held in registers and, on request, its FIRST position.
//   chunk_maximum()         four group maxima (8 columns each, three-input max) and their maximum: 18 instructions
//   chunk_maximum_masked()  the same when only the columns whose bit is set in `inside` count. The mask is the same for every
//                           thread of the warp (document boundaries), so whole groups inside or outside it cost no selects.
//   chunk_position()        first column equal to the maximum: the first group whose maximum matches is selected into eight
//                           values and scanned from the back. Only needed when the chunk beats the running maximum of some row.
// Equal dots resolve to the lower column, like a left-to-right scan with `>` does. A column outside the mask reads as the
// lowest float and can only "win" when every column inside holds that very value, which finite dots never do.
__device__ __forceinline__ float group_maximum(const uint32_t (&v)[32], int g) {
    return max3(max3(__uint_as_float(v[8 * g]), __uint_as_float(v[8 * g + 1]), __uint_as_float(v[8 * g + 2])),
                max3(__uint_as_float(v[8 * g + 3]), __uint_as_float(v[8 * g + 4]), __uint_as_float(v[8 * g + 5])),
                fmaxf(__uint_as_float(v[8 * g + 6]), __uint_as_float(v[8 * g + 7])));
}
__device__ __forceinline__ float chunk_maximum(const uint32_t (&v)[32], float (&group)[4]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) group[g] = group_maximum(v, g);
    return fmaxf(max3(group[0], group[1], group[2]), group[3]);
}
__device__ __forceinline__ float chunk_maximum_masked(const uint32_t (&v)[32], uint32_t inside, float (&group)[4]) {
#pragma unroll
    for (int g = 0; g < 4; ++g) {
        const uint32_t bits = (inside >> (8 * g)) & 0xffu;
        if (bits == 0xffu) group[g] = group_maximum(v, g);
        else if (bits == 0u) group[g] = kLowest;
        else {
            float x[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) x[i] = ((bits >> i) & 1u) ? __uint_as_float(v[8 * g + i]) : kLowest;
            group[g] = max3(max3(x[0], x[1], x[2]), max3(x[3], x[4], x[5]), fmaxf(x[6], x[7]));
        }
    }
    return fmaxf(max3(group[0], group[1], group[2]), group[3]);
}
__device__ __forceinline__ uint32_t chunk_position(const uint32_t (&v)[32], uint32_t inside, const float (&group)[4], float top) {
    const bool in0 = group[0] == top, in1 = group[1] == top, in2 = group[2] == top;
    const uint32_t first = in0 ? 0u : in1 ? 8u : in2 ? 16u : 24u;
    const uint32_t group_inside = inside >> first;
    uint32_t at = 7;
#pragma unroll
    for (int i = 6; i >= 0; --i) {
        const uint32_t raw = in0 ? v[i] : in1 ? v[8 + i] : in2 ? v[16 + i] : v[24 + i];
        const float w = ((group_inside >> i) & 1u) ? __uint_as_float(raw) : kLowest;
        at = w == top ? (uint32_t)i : at;
    }
    return first + at;
}

template <int kKind>
__global__ void __launch_bounds__(kMsThreads, 1) maxsim_kernel(const MaxsimDev p) {
    constexpr int kTmemCols = kMsStreams * kMsBN;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t *smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
    const uint32_t bar_base = smem_base + kMsBarrierOffset;
    auto full_bar = [&](int s) { return bar_base + 8u * s; };
    auto empty_bar = [&](int s) { return bar_base + 8u * (kMsMaxStages + s); };
    auto tmem_full_bar = [&](int a) { return bar_base + 8u * (2 * kMsMaxStages + a); };
    auto tmem_empty_bar = [&](int a) { return bar_base + 8u * (2 * kMsMaxStages + kMsStreams + a); };
    const uint32_t query_bar = bar_base + 8u * (2 * kMsMaxStages + 2 * kMsStreams);      // resident query tile has landed
    const uint32_t drain_bar = query_bar + 8u;                                            // all MMAs have retired
    volatile uint32_t *tmem_slot = reinterpret_cast<volatile uint32_t *>(smem_gen + kMsBarrierOffset + 8 * (2 * kMsMaxStages + 2 * kMsStreams + 2));

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    // Block order: `q_group` query tiles share a document segment (so a segment is fetched from HBM once per group and
    // from L2 by the others), then the next segment, and so on; then the next group of query tiles. Keeping the group
    // small keeps the number of SMs that ask L2 for the same lines at the same moment small.
    const uint32_t per_group = p.q_group * p.segments;
    const uint32_t q_tile = (blockIdx.x / per_group) * p.q_group + (blockIdx.x % per_group) % p.q_group;
    const uint32_t segment = (blockIdx.x % per_group) / p.q_group;
    if (q_tile >= p.q_tiles) return;  // padding blocks of the last group (nothing allocated yet)

    const bool resident = p.kblocks <= (uint32_t)kMsResidentBlocks;
    // A stage is 32 KiB. Query tile streamed (deep queries): a document chunk and the query chunk of the same depth block; every
    // stream then has one 128-column accumulator and the streams take turns (N = 128 instructions).
    // Query tile resident (the regular case): the four streams advance in LOCK-STEP, 64 tokens each per step. A stage holds
    // the four 64-token half chunks (8 KiB each) of one depth block back to back = 256 rows, and ONE N = 256 instruction
    // multiplies all four - a quarter of the instructions for the issuing thread, and the query chunk is read from shared
    // memory once per 256 columns (at N = 128 an instruction reads 8 KiB per 64 cycles: all the 128 bytes per cycle shared
    // memory delivers, while the copies of the next stages write into it). TMEM holds two such 256-column buffers; stream s owns
    // columns 64 s .. 64 s + 63 of either. An epilogue warp pulls its 64 columns into registers, hands the buffer back at once
    // and scans from registers while the tensor cores fill the other buffer: no MMA ever waits for a scan.
    const int stages = 3;
    const uint32_t stage_bytes = 2u * kChunkBytes;
    constexpr uint32_t kHalf = kMsBN / 2;                          // tokens per stream and step in lock-step mode
    constexpr uint32_t kHalfBytes = kHalf * kChunkRowBytes;        // 8 KiB: 64 rows of one depth block

    if (threadIdx.x == 0) {
        for (int s = 0; s < kMsMaxStages; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        // lock-step mode uses barriers 0 and 1 (one per buffer; every epilogue warp reports once per step)
        for (int a = 0; a < kMsStreams; ++a) { mbar_init(tmem_full_bar(a), 1); mbar_init(tmem_empty_bar(a), resident ? 4 * kMsStreams : 4 * 32); }
        mbar_init(query_bar, 1);
        mbar_init(drain_bar, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<1>(smem_u32(const_cast<uint32_t *>(tmem_slot)), kTmemCols);
        tmem_relinquish<1>();
    }
    // This CTA's run of whole documents and its four streams (bounds computed by maxsim_prepare_kernel).
    const uint64_t *bounds = p.stream_bounds + (uint64_t)segment * kMsStreams;
    const uint64_t doc_begin = bounds[0], doc_end = bounds[kMsStreams];
    const bool has_work = doc_begin < doc_end;
    const uint64_t tok_begin = has_work ? p.d_offsets[doc_begin] : 0;
    const uint64_t tok_end = has_work ? p.d_offsets[doc_end] : 0;
    // Shared-memory copies of what the epilogue looks up per document. Everything the epilogue indexes with is kept
    // relative to the first 128-token block the CTA touches / to its first document, in 32 bits (a run of 2^32 tokens or
    // documents would take hours): 64-bit compares cost the epilogue's busiest pipe twice as much.
    float *inv_cache = reinterpret_cast<float *>(smem_gen + kMsCacheOffset);
    uint32_t *end_cache = reinterpret_cast<uint32_t *>(smem_gen + kMsCacheOffset + kMsInvCache * 4);
    const uint64_t cache_base = tok_begin / kMsBN * kMsBN;  // first token held in inv_cache = origin of relative token positions
    const uint32_t run_hi = (uint32_t)(tok_end - cache_base);
    const uint32_t run_docs = (uint32_t)(doc_end - doc_begin);
    if (has_work) {
        for (uint32_t i = threadIdx.x; i < (uint32_t)kMsInvCache; i += blockDim.x)
            inv_cache[i] = cache_base + i < p.d_tokens ? __ldg(p.d_inv + cache_base + i) : 0.0f;
        for (uint32_t i = threadIdx.x; i < (uint32_t)kMsEndCache; i += blockDim.x)
            end_cache[i] = i < run_docs ? (uint32_t)(p.d_offsets[doc_begin + i + 1] - cache_base) : run_hi;
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // Inverse norm of the document token at relative position `rel`; end (relative) of the run's document number `doc`.
    auto inverse_norm_of = [&](uint32_t rel) {
        return rel < (uint32_t)kMsInvCache ? inv_cache[rel] : __ldg(p.d_inv + cache_base + rel);
    };
    auto end_of_doc = [&](uint32_t doc) {
        return doc < (uint32_t)kMsEndCache ? end_cache[doc] : (uint32_t)(p.d_offsets[doc_begin + doc + 1] - cache_base);
    };
    // Stream `s`: documents [first, last) of the run, tokens [lo, hi) relative to cache_base, and the 128-token blocks that
    // hold them (a block at the border between two streams is multiplied for both; each keeps its own documents' columns).
    struct Stream { uint32_t first_doc, last_doc, lo, hi, first_block, blocks, first_half, halves; };
    auto stream_of = [&](int s) {
        Stream st;
        st.first_doc = (uint32_t)(bounds[s] - doc_begin);
        st.last_doc = (uint32_t)(bounds[s + 1] - doc_begin);
        st.lo = st.first_doc == 0 ? (uint32_t)(tok_begin - cache_base) : end_of_doc(st.first_doc - 1);
        st.hi = st.last_doc == 0 ? st.lo : end_of_doc(st.last_doc - 1);
        st.first_block = st.lo / kMsBN;
        st.blocks = st.hi > st.lo ? (st.hi + kMsBN - 1) / kMsBN - st.first_block : 0u;
        st.first_half = st.lo / kHalf;                                                   // 64-token half blocks (lock-step mode)
        st.halves = st.hi > st.lo ? (st.hi + kHalf - 1) / kHalf - st.first_half : 0u;
        return st;
    };

    if (warp == 0) {
        if (lane == 0 && has_work) {
            Stream st[kMsStreams];
            uint32_t rounds = 0;
            for (int s = 0; s < kMsStreams; ++s) { st[s] = stream_of(s); rounds = st[s].blocks > rounds ? st[s].blocks : rounds; }
            const uint8_t *a_tile = p.q_payload + (uint64_t)q_tile * p.kblocks * kChunkBytes;
            if (resident) {
                mbar_expect_tx(query_bar, p.kblocks * kChunkBytes);
                for (uint32_t kb = 0; kb < p.kblocks; ++kb)
                    bulk_load(smem_base + kb * kChunkBytes, a_tile + (uint64_t)kb * kChunkBytes, kChunkBytes, query_bar);
            }
            int stage = 0;
            uint32_t phase = 0, issued = 0;
            bool ok = true;
            auto tile_of = [&](int s, uint32_t r) {
                return p.d_payload + (cache_base / kMsBN + st[s].first_block + r) * (uint64_t)p.kblocks * kChunkBytes;
            };
            if (resident) {
                uint32_t steps = 0;
                for (int s = 0; s < kMsStreams; ++s) steps = st[s].halves > steps ? st[s].halves : steps;
                for (uint32_t t = 0; t < steps && ok; ++t) {
                    uint32_t active = 0;
                    for (int s = 0; s < kMsStreams; ++s) active += t < st[s].halves ? 1u : 0u;
                    for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, 1, p.error_word)) { ok = false; break; }
                        const uint32_t dst = smem_base + kMsRingOffset + stage * stage_bytes;
                        mbar_expect_tx(full_bar(stage), active * kHalfBytes);
                        for (int s = 0; s < kMsStreams; ++s) {
                            if (t >= st[s].halves) continue;  // this stream is done: its rows of the stage keep what they held
                            const uint64_t token = cache_base + (uint64_t)(st[s].first_half + t) * kHalf;
                            const uint8_t *src = p.d_payload + ((token >> 7) * p.kblocks + kb) * (uint64_t)kChunkBytes + (token & 64u) * kChunkRowBytes;
                            bulk_load(dst + s * kHalfBytes, src, kHalfBytes, full_bar(stage));
                        }
                        ++issued;
                        if (++stage == stages) { stage = 0; phase ^= 1u; }
                    }
                }
                rounds = 0;  // nothing left for the stream-by-stream loop below
            }
            for (uint32_t r = 0; r < rounds && ok; ++r) {
                for (int s = 0; s < kMsStreams && ok; ++s) {
                    if (r >= st[s].blocks) continue;
                    const uint8_t *b_tile = tile_of(s, r);
                    for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                        if (!mbar_wait(empty_bar(stage), phase ^ 1u, 1, p.error_word)) { ok = false; break; }
                        const uint32_t dst = smem_base + kMsRingOffset + stage * stage_bytes;
                        mbar_expect_tx(full_bar(stage), stage_bytes);
                        bulk_load(dst + kChunkBytes, a_tile + (uint64_t)kb * kChunkBytes, kChunkBytes, full_bar(stage));
                        bulk_load(dst, b_tile + (uint64_t)kb * kChunkBytes, kChunkBytes, full_bar(stage));
                        ++issued;
                        if (++stage == stages) { stage = 0; phase ^= 1u; }
                    }
                }
            }
            if (!ok) {
                // Copies issued last may still be in flight: wait (bounded) until their stages' barriers have counted them.
                int s = stage;
                uint32_t ph = phase;
                for (uint32_t i = 0; i < issued && i < (uint32_t)stages; ++i) {
                    if (s == 0) { s = stages; ph ^= 1u; }
                    --s;
                    if (!mbar_wait(full_bar(s), ph, 6, p.error_word)) break;
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && has_work) {
            Stream st[kMsStreams];
            uint32_t rounds = 0;
            for (int s = 0; s < kMsStreams; ++s) { st[s] = stream_of(s); rounds = st[s].blocks > rounds ? st[s].blocks : rounds; }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            if (resident && !mbar_wait(query_bar, 0u, 3, p.error_word)) ok = false;
            if (resident) {
                uint32_t steps = 0;
                for (int s = 0; s < kMsStreams; ++s) steps = st[s].halves > steps ? st[s].halves : steps;
                for (uint32_t t = 0; t < steps && ok; ++t) {
                    // Buffer t & 1 was handed out t / 2 times before: wait until all sixteen warps have pulled step t - 2 out of it.
                    const uint32_t buf = t & 1u;
                    if (!mbar_wait(tmem_empty_bar(buf), ((t >> 1) & 1u) ^ 1u, 2, p.error_word)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * (2u * kMsBN);
                    for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                        if (!mbar_wait(full_bar(stage), phase, 3, p.error_word)) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint64_t a_desc = make_smem_desc_sw128(smem_base + kb * kChunkBytes);
                        const uint64_t b_desc = make_smem_desc_sw128(smem_base + kMsRingOffset + stage * stage_bytes);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<kKind, 1>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc_pair, (kb | (uint32_t)k) != 0u);
                        umma_commit(empty_bar(stage));
                        if (++stage == stages) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) umma_commit(tmem_full_bar(buf));
                }
                rounds = 0;
            }
            for (uint32_t r = 0; r < rounds && ok; ++r) {
                for (int s = 0; s < kMsStreams && ok; ++s) {
                    if (r >= st[s].blocks) continue;
                    // Stream s's accumulator was handed out r times before: wait until its four warps have read round r - 1.
                    if (!mbar_wait(tmem_empty_bar(s), (r & 1u) ^ 1u, 2, p.error_word)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + s * kMsBN;
                    for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                        if (!mbar_wait(full_bar(stage), phase, 3, p.error_word)) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t b_src = smem_base + kMsRingOffset + stage * stage_bytes;
                        const uint32_t a_src = b_src + kChunkBytes;
                        const uint64_t a_desc = make_smem_desc_sw128(a_src);
                        const uint64_t b_desc = make_smem_desc_sw128(b_src);
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            umma<kKind, 1>(d_tmem, a_desc + 2u * k, b_desc + 2u * k, p.idesc, (kb | (uint32_t)k) != 0u);
                        umma_commit(empty_bar(stage));
                        if (++stage == stages) { stage = 0; phase ^= 1u; }
                    }
                    if (ok) umma_commit(tmem_full_bar(s));
                }
            }
            // No MMA may still be running when TMEM and shared memory are released below.
            umma_commit(drain_bar);
            mbar_wait(drain_bar, 0u, 5, p.error_word);
        }
    } else if (has_work) {
        // ------------------------------------------------------------ epilogue (warps 2..17)
        const uint32_t quarter = warp & 3u;                 // TMEM lanes 32 * quarter .. + 31 = 32 query tokens
        const int s = (warp - 2) >> 2;                      // the stream this warp follows
        const Stream st = stream_of(s);
        const uint64_t row = (uint64_t)q_tile * kMsBM + quarter * 32u + lane;
        const bool row_ok = row < p.q_tokens;
        const float q_inv = row_ok ? p.q_inv[row] : 0.0f;
        constexpr uint32_t kNoQuery = 0xffffffffu;  // padding rows
        const uint32_t qid = row_ok ? p.q_token_query[row] : kNoQuery;
        const uint32_t qid_above = __shfl_up_sync(0xffffffffu, qid, 1);
        const bool segment_head = qid != kNoQuery && (lane == 0 || qid_above != qid);
        // Bit b: the lane 2^b further down belongs to the same query (the per-document sums are segmented by query).
        uint32_t joins = 0;
#pragma unroll
        for (int b = 0; b < 5; ++b) {
            const uint32_t other_q = __shfl_down_sync(0xffffffffu, qid, 1u << b);
            if (lane + (1 << b) < 32 && other_q == qid) joins |= 1u << b;
        }
        // Where this query's scores of the run's documents go (segment heads of the all-pairs call only), and whether this
        // warp holds ALL of the query's tokens (then the sum is final and stored; otherwise the parts are added atomically).
        float *score_row = segment_head && p.scores_f32 ? p.scores_f32 + (uint64_t)qid * p.score_stride + doc_begin : nullptr;
        bool whole_query = false;
        if (segment_head) {
            const uint64_t warp_row0 = (uint64_t)q_tile * kMsBM + quarter * 32u;
            whole_query = p.q_offsets[qid] >= warp_row0 && p.q_offsets[qid + 1] <= warp_row0 + 32u;
        }

        uint32_t cur_doc = st.first_doc;                          // number of the current document within the run
        uint32_t cur_end = st.blocks ? end_of_doc(cur_doc) : 0u;  // its end, relative
        float run = kLowest;
        uint32_t arg = 0;                                         // relative position of the running winner

        // Closes the current document: normalise the winner, add the query's tokens up (f64, segmented by query), write.
        auto finish_doc = [&]() {
            float angular = 0.0f;
            if (row_ok) {
                const float cosine = run * q_inv * inverse_norm_of(arg);
                angular = 1.0f - cosine;
                if (!(angular > 0.0f)) angular = angular < 0.0f ? 0.0f : angular;  // clamp, keep NaN
            }
            double sum = (double)angular;
#pragma unroll
            for (int b = 0; b < 5; ++b) {
                const double other = __shfl_down_sync(0xffffffffu, sum, 1u << b);
                if ((joins >> b) & 1u) sum += other;
            }
            if (segment_head) {
                if (p.total_f64) atomicAdd(p.total_f64, sum);
                else if (whole_query) score_row[cur_doc] = (float)sum;
                else atomicAdd(score_row + cur_doc, (float)sum);
            }
            run = kLowest;
            arg = 0;
        };
        // One 32-column chunk whose column 0 sits at relative position c0.
        auto scan_chunk = [&](const uint32_t (&v)[32], uint32_t c0) {
            float group[4];
            if (c0 >= st.lo && c0 + 32u <= cur_end) {
                // The whole chunk lies inside the current document.
                const float best = chunk_maximum(v, group);
                if (best > run) { run = best; arg = c0 + chunk_position(v, 0xffffffffu, group, best); }
                return;
            }
            // Document boundaries (or an end of the stream) fall inside or before the chunk: walk it piece by piece, masking
            // the columns outside the piece. Boundaries are the same for every thread.
            const uint32_t hi = c0 + 32u < st.hi ? c0 + 32u : st.hi;
            uint32_t pos = c0 > st.lo ? c0 : st.lo;
            while (pos < hi) {
                while (pos >= cur_end) {
                    finish_doc();
                    ++cur_doc;
                    cur_end = end_of_doc(cur_doc);
                }
                const uint32_t piece_end = cur_end < hi ? cur_end : hi;
                const uint32_t j0 = pos - c0, j1 = piece_end - c0;  // 0 <= j0 < j1 <= 32
                if (j0 == 0u && j1 == 32u) {
                    // The chunk begins a document and lies inside it (every document's first chunk once documents sit on
                    // 32-token boundaries): no column is masked.
                    const float best = chunk_maximum(v, group);
                    if (best > run) { run = best; arg = c0 + chunk_position(v, 0xffffffffu, group, best); }
                    return;
                }
                const uint32_t inside = (0xffffffffu >> (32u - j1)) & (0xffffffffu << j0);
                const float best = chunk_maximum_masked(v, inside, group);
                if (best > run) { run = best; arg = c0 + chunk_position(v, inside, group, best); }
                pos = piece_end;
            }
        };

        if (resident) {
            // Lock-step mode: every warp walks all steps (the buffer goes back when all sixteen have reported), a warp whose
            // stream is done just reports.
            uint32_t steps = 0;
            for (int i = 0; i < kMsStreams; ++i) { const uint32_t h = stream_of(i).halves; steps = h > steps ? h : steps; }
            for (uint32_t t = 0; t < steps; ++t) {
                const uint32_t buf = t & 1u;
                if (!mbar_wait(tmem_full_bar(buf), (t >> 1) & 1u, 4, p.error_word)) break;  // the issuer's own bounded wait ends the others
                tc_fence_after_sync();
                const bool mine = t < st.halves;
                uint32_t v0[32], v1[32];
                if (mine) {
                    const uint32_t t_addr = tmem_base + ((quarter * 32u) << 16) + buf * (2u * kMsBN) + (uint32_t)s * kHalf;
                    tmem_ld_32x32(t_addr, v0);
                    tmem_ld_32x32(t_addr + 32, v1);
                    tmem_ld_wait_for(v0);
                    tmem_ld_wait_for(v1);
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(tmem_empty_bar(buf));   // both chunks are in registers: the buffer can be refilled
                if (!mine) continue;
                const uint32_t c0 = (st.first_half + t) * kHalf;   // relative position of the step's column 0
                scan_chunk(v0, c0);
                scan_chunk(v1, c0 + 32u);
                // Documents that end inside this step are complete.
                const uint32_t step_hi = c0 + kHalf < st.hi ? c0 + kHalf : st.hi;
                while (cur_doc < st.last_doc && cur_end <= step_hi) {
                    finish_doc();
                    ++cur_doc;
                    cur_end = cur_doc < st.last_doc ? end_of_doc(cur_doc) : 0u;  // 0: no chunk is "inside" once the stream is done
                }
            }
        }
        for (uint32_t r = 0; r < (resident ? 0u : st.blocks); ++r) {
            if (!mbar_wait(tmem_full_bar(s), r & 1u, 4, p.error_word)) break;  // nothing else waits for this warp
            tc_fence_after_sync();
            const uint32_t t_addr = tmem_base + ((quarter * 32u) << 16) + s * kMsBN;
            const uint32_t tile_c0 = (st.first_block + r) * kMsBN;  // relative position of the tile's column 0
            // Two chunks in flight: the next one is on its way from TMEM while the current one is scanned.
            uint32_t v0[32], v1[32];
            tmem_ld_32x32(t_addr, v0);
            tmem_ld_wait_for(v0);
            tmem_ld_32x32(t_addr + 32, v1);
            scan_chunk(v0, tile_c0);
            tmem_ld_wait_for(v1);
            tmem_ld_32x32(t_addr + 64, v0);
            scan_chunk(v1, tile_c0 + 32u);
            tmem_ld_wait_for(v0);
            tmem_ld_32x32(t_addr + 96, v1);
            scan_chunk(v0, tile_c0 + 64u);
            tmem_ld_wait_for(v1);
            tc_fence_before_sync();
            mbar_arrive(tmem_empty_bar(s));   // everything this warp needs of the tile is in registers
            scan_chunk(v1, tile_c0 + 96u);
            // Documents that end inside this tile are complete.
            const uint32_t tile_hi = tile_c0 + kMsBN < st.hi ? tile_c0 + kMsBN : st.hi;
            while (cur_doc < st.last_doc && cur_end <= tile_hi) {
                finish_doc();
                ++cur_doc;
                cur_end = cur_doc < st.last_doc ? end_of_doc(cur_doc) : 0u;  // 0: no chunk is "inside" once the stream is done
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<1>(tmem_base, kTmemCols);
    }
}

// f32 inputs: CUDA cores, f64 dots (include/numkong/maxsim/serial.h:426-459 keeps dot, cosine and
// angular in f64). One warp per query token; lanes split the depth.
__global__ void maxsim_f32_kernel(const float *__restrict__ q, const float *__restrict__ d, uint64_t q_stride_elems,
                                  uint64_t d_stride_elems, const float *__restrict__ q_inv, const float *__restrict__ d_inv,
                                  uint64_t nq, uint64_t nd, uint64_t depth, double *total) {
    const int lane = threadIdx.x & 31;
    const uint64_t warps = ((uint64_t)gridDim.x * blockDim.x) >> 5;
    for (uint64_t i = ((uint64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5; i < nq; i += warps) {
        const float *x = q + i * q_stride_elems;
        double run = -1.7976931348623157e308;
        uint64_t arg = 0;
        for (uint64_t j = 0; j < nd; ++j) {
            const float *y = d + j * d_stride_elems;
            double s = 0.0;
            for (uint64_t l = lane; l < depth; l += 32) s = fma((double)x[l], (double)y[l], s);
#pragma unroll
            for (int off = 16; off > 0; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
            if (s > run) { run = s; arg = j; }
        }
        if (lane == 0) {
            double angular = 1.0 - run * (double)q_inv[i] * (double)d_inv[arg];
            if (angular < 0.0) angular = 0.0;
            atomicAdd(total, angular);
        }
    }
}

__global__ void iota_offsets_kernel(uint64_t *out, uint64_t a, uint64_t b) { out[0] = a; out[1] = b; }

// ---- documents re-laid on 32-token boundaries (batch form) ------------------------------------------------------------
// The epilogue scans the similarity tile 32 columns at a time. A document boundary inside such a chunk costs it several times
// a plain chunk (two masked maxima, two position searches, the close of a document in mid-chunk), and with documents of
// 64 - 300 tokens every fifth or sixth chunk holds one: measured, treating every chunk as plain makes the kernel 38 % faster.
// So the batch call first copies the documents into a scratch blob in which every document starts on a multiple of 32 tokens:
// the tail of its last chunk repeats the document's LAST token. A repeated token can tie with the real one but never beat it,
// and ties go to the lower position, so maxima, winners and sums are the same bits as on the caller's layout; inverse norms
// are repeated alongside. Costs one pass over the packed documents (read + write at HBM rate, about 3 % of the call at depth
// 128), 9 % more columns on average for documents of late-interaction size, and the scratch.
constexpr int kPadScanBlock = 1024;
__device__ __forceinline__ uint64_t padded_length(const uint64_t *offsets, uint64_t doc) {
    return (offsets[doc + 1] - offsets[doc] + 31u) & ~(uint64_t)31u;
}
// (a) sum of the padded lengths of every block of 1024 documents
__global__ void __launch_bounds__(kPadScanBlock) pad_block_sums_kernel(const uint64_t *offsets, uint64_t n_docs, uint64_t *block_sums) {
    __shared__ uint64_t warp_sums[kPadScanBlock / 32];
    const uint64_t doc = (uint64_t)blockIdx.x * kPadScanBlock + threadIdx.x;
    uint64_t v = doc < n_docs ? padded_length(offsets, doc) : 0;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_down_sync(0xffffffffu, v, o);
    if ((threadIdx.x & 31) == 0) warp_sums[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint64_t w = warp_sums[threadIdx.x];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) w += __shfl_down_sync(0xffffffffu, w, o);
        if (threadIdx.x == 0) block_sums[blockIdx.x] = w;
    }
}
// (b) exclusive scan of the block sums, in place, by one thread block; the grand total goes behind the last entry
__global__ void __launch_bounds__(kPadScanBlock) pad_scan_blocks_kernel(uint64_t *block_sums, uint64_t blocks) {
    __shared__ uint64_t warp_sums[kPadScanBlock / 32];
    __shared__ uint64_t carry;
    if (threadIdx.x == 0) carry = 0;
    __syncthreads();
    for (uint64_t base = 0; base < blocks; base += kPadScanBlock) {
        const uint64_t i = base + threadIdx.x;
        const uint64_t own = i < blocks ? block_sums[i] : 0;
        uint64_t v = own;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint64_t up = __shfl_up_sync(0xffffffffu, v, o);
            if ((threadIdx.x & 31) >= o) v += up;
        }
        if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = v;
        __syncthreads();
        if (threadIdx.x < 32) {
            uint64_t w = warp_sums[threadIdx.x];
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const uint64_t up = __shfl_up_sync(0xffffffffu, w, o);
                if (threadIdx.x >= o) w += up;
            }
            warp_sums[threadIdx.x] = w;  // inclusive over warps
        }
        __syncthreads();
        const uint64_t before = carry + ((threadIdx.x >> 5) ? warp_sums[(threadIdx.x >> 5) - 1] : 0) + v - own;
        if (i < blocks) block_sums[i] = before;
        __syncthreads();
        if (threadIdx.x == kPadScanBlock - 1) carry = before + own;
        __syncthreads();
    }
    if (threadIdx.x == 0) block_sums[blocks] = carry;
}
// (c) the padded offsets: exclusive scan inside every block of 1024 documents plus the block's base
__global__ void __launch_bounds__(kPadScanBlock) pad_offsets_kernel(const uint64_t *offsets, uint64_t n_docs, const uint64_t *block_bases,
                                                                  uint64_t *padded_offsets) {
    __shared__ uint64_t warp_sums[kPadScanBlock / 32];
    const uint64_t doc = (uint64_t)blockIdx.x * kPadScanBlock + threadIdx.x;
    const uint64_t own = doc < n_docs ? padded_length(offsets, doc) : 0;
    uint64_t v = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint64_t up = __shfl_up_sync(0xffffffffu, v, o);
        if ((threadIdx.x & 31) >= o) v += up;
    }
    if ((threadIdx.x & 31) == 31) warp_sums[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        uint64_t w = warp_sums[threadIdx.x];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const uint64_t up = __shfl_up_sync(0xffffffffu, w, o);
            if (threadIdx.x >= o) w += up;
        }
        warp_sums[threadIdx.x] = w;
    }
    __syncthreads();
    const uint64_t before = block_bases[blockIdx.x] + ((threadIdx.x >> 5) ? warp_sums[(threadIdx.x >> 5) - 1] : 0) + v - own;
    if (doc < n_docs) padded_offsets[doc] = before;
    if (doc + 1 == n_docs) padded_offsets[n_docs] = before + own;
}
// One warp per document: its rows (128 bytes per depth block, eight 16-byte pieces stored at piece ^ (row & 7) inside the
// 128-row chunk of their depth block) move to their new row numbers, the last row is repeated up to the next multiple of 32.
__global__ void __launch_bounds__(256) maxsim_pad_rows_kernel(const uint4 *__restrict__ src, const float *__restrict__ src_inv,
                                                             const uint64_t *__restrict__ offsets, const uint64_t *__restrict__ padded_offsets,
                                                             uint64_t n_docs, uint32_t kblocks, uint4 *__restrict__ dst, float *__restrict__ dst_inv) {
    const uint64_t warps = (uint64_t)gridDim.x * (blockDim.x >> 5);
    const int lane = threadIdx.x & 31;
    const uint32_t pieces_per_row = kblocks * 8u;
    for (uint64_t doc = (uint64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5); doc < n_docs; doc += warps) {
        const uint64_t from = offsets[doc], length = offsets[doc + 1] - from, to = padded_offsets[doc];
        const uint64_t padded = padded_offsets[doc + 1] - to;
        if (length == 0) continue;
        for (uint64_t x = lane; x < padded * pieces_per_row; x += 32) {
            const uint64_t j = x / pieces_per_row;
            const uint32_t pc = (uint32_t)(x % pieces_per_row), kb = pc >> 3, piece = pc & 7u;
            const uint64_t s_row = from + (j < length ? j : length - 1), d_row = to + j;
            const uint64_t s_at = ((s_row >> 7) * kblocks + kb) * 1024u + (s_row & 127u) * 8u + (piece ^ (uint32_t)(s_row & 7u));
            const uint64_t d_at = ((d_row >> 7) * kblocks + kb) * 1024u + (d_row & 127u) * 8u + (piece ^ (uint32_t)(d_row & 7u));
            dst[d_at] = src[s_at];
        }
        for (uint64_t j = lane; j < padded; j += 32) dst_inv[to + j] = src_inv[from + (j < length ? j : length - 1)];
    }
}

cudaError_t launch_maxsim_tc(uint32_t dt, const MaxsimDev &dev_in, cudaStream_t stream) {
    MaxsimDev dev = dev_in;
    dev.idesc = make_idesc(1, dt == kBF16 ? 1 : 0, kMsBM, kMsBN);
    dev.idesc_pair = make_idesc(1, dt == kBF16 ? 1 : 0, kMsBM, 2 * kMsBN);
    static bool configured[64] = {false};
    int d = 0;
    cudaGetDevice(&d);
    if (d >= 0 && d < 64 && !configured[d]) {
        cudaError_t e = cudaFuncSetAttribute(maxsim_kernel<kKindF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, kMsSmemTotal);
        if (e != cudaSuccess) return e;
        configured[d] = true;
    }
    // Group size: 8 query tiles per segment unless overridden for tuning (bits 16..23 of the variant word).
    uint32_t group = ((uint32_t)current_variant() >> 16) & 0xffu;
    if (group == 0) group = 8;
    if (group > dev.q_tiles) group = dev.q_tiles;
    dev.q_group = group;
    uint64_t grid = (uint64_t)((dev.q_tiles + group - 1) / group) * group * dev.segments;
    if (grid == 0 || grid > 0x7fffffffull || dev.q_tokens > 0xffffffffull) return cudaErrorInvalidValue;
    // Look-up tables for the main kernel: token -> query, stream -> first document (four streams per segment).
    const uint64_t map_bytes = round_up(dev.q_tokens * 4, 16);
    const uint64_t bound_count = (uint64_t)dev.segments * kMsStreams + 1;
    uint8_t *tables = static_cast<uint8_t *>(scratch(kSlotNorms, map_bytes + bound_count * 8));
    if (!tables) return cudaErrorMemoryAllocation;
    uint32_t *token_query = reinterpret_cast<uint32_t *>(tables);
    uint64_t *bounds = reinterpret_cast<uint64_t *>(tables + map_bytes);
    const uint64_t items = dev.q_tokens > bound_count ? dev.q_tokens : bound_count;
    maxsim_prepare_kernel<<<(unsigned)((items + 255) / 256), 256, 0, stream>>>(dev.q_offsets, dev.n_queries, dev.q_tokens, token_query,
                                                                             dev.d_offsets, dev.n_docs, dev.d_tokens, dev.segments, bounds);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return e;
    g_launches++;
    dev.q_token_query = token_query;
    dev.stream_bounds = bounds;
    maxsim_kernel<kKindF16><<<(unsigned)grid, kMsThreads, kMsSmemTotal, stream>>>(dev);
    return cudaGetLastError();
}

uint32_t pick_segments(uint64_t d_tokens, uint32_t q_tiles) {
    // Runs of about kMsRunTiles document tiles (14,336 tokens, some 80 documents of late-interaction size: twenty per stream)
    // per CTA, but at least two CTAs per SM when the work allows it.
    uint64_t tiles = (d_tokens + kMsBN - 1) / kMsBN;
    uint64_t seg = (tiles + kMsRunTiles - 1) / kMsRunTiles;
    const uint64_t min_ctas = 2 * 148;
    if ((uint64_t)q_tiles * seg < min_ctas) {
        uint64_t want = (min_ctas + q_tiles - 1) / q_tiles;
        seg = want < tiles ? want : tiles;
    }
    if (seg < 1) seg = 1;
    if (seg > 0x7fffffull) seg = 0x7fffffull;
    return (uint32_t)seg;
}

uint64_t maxsim_size_impl(uint32_t dt, uint64_t count, uint64_t depth) {
    if (dt != kBF16 && dt != kF16 && dt != kF32) return 0;
    return packed_geometry(dt, count, depth).total_bytes;
}

} // namespace

// Shared with the dots blobs: same header, chunk grid and kernels; the norm slot holds 1/|v| as f32.
void maxsim_pack_impl(uint32_t dt, const void *vectors, uint64_t count, uint64_t depth, uint64_t stride, void *packed);

namespace {

void maxsim_single_impl(uint32_t dt, const void *q_packed, const void *d_packed, uint64_t nq, uint64_t nd, uint64_t depth,
                        void *result) {
    clear_error();
    const bool wide = dt == kF32;
    auto fail = [&]() { if (result) std::memset(result, 0xFF, wide ? 8 : 4); };
    if (!result) { set_error("maxsim_packed: null result%s", ""); return; }
    const MemKind r_kind = classify(result);
    auto write_result = [&](double v) {
        float f = (float)v;
        if (r_kind == kMemHost) { if (wide) std::memcpy(result, &v, 8); else std::memcpy(result, &f, 4); }
        else cudaMemcpyAsync(result, wide ? (void *)&v : (void *)&f, wide ? 8 : 4, cudaMemcpyHostToDevice, current_stream());
    };
    if (dt != kBF16 && dt != kF16 && dt != kF32) { set_error("maxsim_packed: unsupported element type%s", ""); fail(); return; }
    if (!q_packed || !d_packed) { set_error("maxsim_packed: null packed operand%s", ""); fail(); return; }
    if (nq == 0) { write_result(0.0); return; }
    if (nd == 0) { set_error("maxsim_packed: a document needs at least one vector%s", ""); fail(); return; }
    cudaStream_t stream = current_stream();
    PackedHeader qh, dh;
    const uint8_t *qb = resident_blob(q_packed, classify(q_packed), kMagicMaxsim, dt, nq, depth, &qh);
    if (!qb) { fail(); return; }
    const uint8_t *db = resident_blob(d_packed, classify(d_packed), kMagicMaxsim, dt, nd, depth, &dh);
    if (!db) { fail(); return; }
    unsigned int *err = device_error_word();
    double *total = static_cast<double *>(scratch(kSlotAux, 64));
    if (!err || !total) { set_error("maxsim_packed: could not allocate device scratch%s", ""); fail(); return; }
    bool ok = cuda_ok(cudaMemsetAsync(total, 0, 8, stream), "clear accumulator");
    if (ok && dt == kF32) {
        int blocks = (int)((nq * 32 + 255) / 256);
        if (blocks > 148 * 8) blocks = 148 * 8;
        maxsim_f32_kernel<<<blocks, 256, 0, stream>>>(reinterpret_cast<const float *>(qb + qh.payload_offset),
                                                      reinterpret_cast<const float *>(db + dh.payload_offset),
                                                      qh.depth_padded_bytes / 4, dh.depth_padded_bytes / 4,
                                                      reinterpret_cast<const float *>(qb + qh.norms_offset),
                                                      reinterpret_cast<const float *>(db + dh.norms_offset), nq, nd, depth, total);
        ok = cuda_ok(cudaGetLastError(), "f32 MaxSim kernel");
        g_launches++;
    } else if (ok) {
        uint64_t *offsets = reinterpret_cast<uint64_t *>(total + 1);  // [0,nq] and [0,nd], same scratch slot
        iota_offsets_kernel<<<1, 1, 0, stream>>>(offsets, 0, nq);
        iota_offsets_kernel<<<1, 1, 0, stream>>>(offsets + 2, 0, nd);
        g_launches += 2;
        MaxsimDev dev{};
        dev.q_payload = qb + qh.payload_offset; dev.d_payload = db + dh.payload_offset;
        dev.q_inv = reinterpret_cast<const float *>(qb + qh.norms_offset);
        dev.d_inv = reinterpret_cast<const float *>(db + dh.norms_offset);
        dev.q_offsets = offsets; dev.d_offsets = offsets + 2;
        dev.n_queries = 1; dev.n_docs = 1; dev.q_tokens = nq; dev.d_tokens = nd;
        dev.kblocks = (uint32_t)(qh.depth_padded_bytes / kChunkRowBytes);
        dev.q_tiles = (uint32_t)((nq + kMsBM - 1) / kMsBM);
        dev.segments = 1;  // one document: its tokens cannot be split across CTAs
        dev.scores_f32 = nullptr; dev.score_stride = 0; dev.total_f64 = total; dev.error_word = err;
        ok = cuda_ok(launch_maxsim_tc(dt, dev, stream), "MaxSim kernel");
        g_launches++;
    }
    double host_total = 0.0;
    if (ok) ok = cuda_ok(cudaMemcpyAsync(&host_total, total, 8, cudaMemcpyDeviceToHost, stream), "read accumulator");
    if (ok) ok = cuda_ok(cudaStreamSynchronize(stream), "maxsim_packed");
    if (ok) {
        uint32_t w = read_device_error();
        if (w) { char buf[64]; std::snprintf(buf, sizeof buf, "0x%08x", w); set_error("a pipeline wait inside the MaxSim kernel gave up (error word %s)", buf); ok = false; }
    }
    if (!ok) { fail(); return; }
    write_result(host_total);
}

void maxsims_batch_impl(uint32_t dt, const void *q_packed, const void *q_offsets, uint64_t n_queries, const void *d_packed,
                        const void *d_offsets, uint64_t n_docs, uint64_t depth, void *scores, uint64_t score_stride) {
    clear_error();
    if (n_queries == 0 || n_docs == 0) return;
    const MemKind s_kind = classify(scores);
    const uint64_t row_bytes = n_docs * 4;
    auto fail = [&]() { fill_error_output(scores, s_kind, n_queries, row_bytes, score_stride < row_bytes ? row_bytes : score_stride); };
    if ((dt != kBF16 && dt != kF16) || !q_packed || !d_packed || !q_offsets || !d_offsets || !scores) {
        set_error("maxsims_packed: unsupported element type or null pointer%s", ""); fail(); return;
    }
    if (score_stride % 4 || (n_queries > 1 && score_stride < row_bytes)) { set_error("maxsims_packed: bad score stride%s", ""); fail(); return; }
    cudaStream_t stream = current_stream();
    // Offsets: bring to the device when they are host arrays; the totals are needed on the host.
    uint64_t totals[2] = {0, 0};
    const uint64_t *q_off_dev = nullptr, *d_off_dev = nullptr;
    const void *srcs[2] = {q_offsets, d_offsets};
    const uint64_t counts[2] = {n_queries, n_docs};
    const int slots[2] = {kSlotAux, kSlotAux2};
    bool ok = true;
    for (int s = 0; s < 2 && ok; ++s) {
        MemKind kind = classify(srcs[s]);
        const uint64_t *dev_ptr;
        if (kind == kMemHost) {
            totals[s] = static_cast<const uint64_t *>(srcs[s])[counts[s]];
            void *buf = scratch(slots[s], (counts[s] + 1) * 8);
            ok = buf && cuda_ok(cudaMemcpyAsync(buf, srcs[s], (counts[s] + 1) * 8, cudaMemcpyHostToDevice, stream), "upload offsets");
            dev_ptr = static_cast<const uint64_t *>(buf);
        } else {
            ok = cuda_ok(cudaMemcpyAsync(&totals[s], static_cast<const uint64_t *>(srcs[s]) + counts[s], 8, cudaMemcpyDeviceToHost, stream), "read offsets") &&
                 cuda_ok(cudaStreamSynchronize(stream), "read offsets");
            dev_ptr = static_cast<const uint64_t *>(srcs[s]);
        }
        if (s == 0) q_off_dev = dev_ptr; else d_off_dev = dev_ptr;
    }
    if (!ok) { fail(); return; }
    const uint64_t q_tokens = totals[0], d_tokens = totals[1];
    PackedHeader qh, dh;
    const uint8_t *qb = resident_blob(q_packed, classify(q_packed), kMagicMaxsim, dt, q_tokens, depth, &qh);
    if (!qb) { fail(); return; }
    const uint8_t *db = resident_blob(d_packed, classify(d_packed), kMagicMaxsim, dt, d_tokens, depth, &dh);
    if (!db) { fail(); return; }
    unsigned int *err = device_error_word();
    if (!err) { set_error("maxsims_packed: could not allocate the device error word%s", ""); fail(); return; }

    float *s_dev = static_cast<float *>(scores);
    uint64_t s_pitch = score_stride;
    if (s_kind == kMemHost) {
        s_pitch = row_bytes;
        s_dev = static_cast<float *>(scratch(kSlotC, n_queries * row_bytes));
        if (!s_dev) { fail(); return; }
    }
    ok = cuda_ok(cudaMemset2DAsync(s_dev, s_pitch, 0, row_bytes, n_queries, stream), "clear scores");
    if (ok && q_tokens && d_tokens) {
        MaxsimDev dev{};
        dev.q_payload = qb + qh.payload_offset; dev.d_payload = db + dh.payload_offset;
        dev.q_inv = reinterpret_cast<const float *>(qb + qh.norms_offset);
        dev.d_inv = reinterpret_cast<const float *>(db + dh.norms_offset);
        dev.q_offsets = q_off_dev; dev.d_offsets = d_off_dev;
        dev.n_queries = n_queries; dev.n_docs = n_docs; dev.q_tokens = q_tokens; dev.d_tokens = d_tokens;
        dev.kblocks = (uint32_t)(qh.depth_padded_bytes / kChunkRowBytes);
        dev.q_tiles = (uint32_t)((q_tokens + kMsBM - 1) / kMsBM);
        // Documents on 32-token boundaries (see maxsim_pad_rows_kernel), unless switched off for comparisons (bit 24 of the
        // variant word), the scratch would take more than half of the free device memory, or they sit on such boundaries already.
        if ((((uint32_t)current_variant() >> 24) & 1u) == 0u) {
            const uint64_t blocks = (n_docs + kPadScanBlock - 1) / kPadScanBlock;
            const uint64_t bound_rows = round_up(d_tokens + 31 * n_docs, kRowPad);
            const uint64_t offsets_bytes = round_up((n_docs + 1) * 8, 256), sums_bytes = round_up((blocks + 1) * 8, 256);
            const uint64_t inv_bytes = round_up(bound_rows * 4, 256), payload_bytes = bound_rows * dh.depth_padded_bytes;
            const uint64_t need = offsets_bytes + sums_bytes + inv_bytes + payload_bytes;
            size_t free_bytes = 0, total_bytes = 0;
            if (cudaMemGetInfo(&free_bytes, &total_bytes) != cudaSuccess) { cudaGetLastError(); free_bytes = 0; }
            uint8_t *pad = need <= free_bytes / 2 || scratch_capacity(kSlotA) >= need ? static_cast<uint8_t *>(scratch(kSlotA, need)) : nullptr;
            if (pad) {
                uint64_t *padded_offsets = reinterpret_cast<uint64_t *>(pad), *sums = reinterpret_cast<uint64_t *>(pad + offsets_bytes);
                float *padded_inv = reinterpret_cast<float *>(pad + offsets_bytes + sums_bytes);
                uint4 *padded_payload = reinterpret_cast<uint4 *>(pad + offsets_bytes + sums_bytes + inv_bytes);
                pad_block_sums_kernel<<<(unsigned)blocks, kPadScanBlock, 0, stream>>>(d_off_dev, n_docs, sums);
                pad_scan_blocks_kernel<<<1, kPadScanBlock, 0, stream>>>(sums, blocks);
                pad_offsets_kernel<<<(unsigned)blocks, kPadScanBlock, 0, stream>>>(d_off_dev, n_docs, sums, padded_offsets);
                uint64_t padded_tokens = 0;
                ok = cuda_ok(cudaGetLastError(), "padded offsets") &&
                     cuda_ok(cudaMemcpyAsync(&padded_tokens, padded_offsets + n_docs, 8, cudaMemcpyDeviceToHost, stream), "read padded size") &&
                     cuda_ok(cudaStreamSynchronize(stream), "read padded size");
                g_launches += 3;
                if (ok && padded_tokens != d_tokens && padded_tokens <= bound_rows) {
                    const uint64_t warps_wanted = n_docs < 148 * 64 ? n_docs : 148 * 64;
                    maxsim_pad_rows_kernel<<<(unsigned)((warps_wanted + 7) / 8), 256, 0, stream>>>(
                        reinterpret_cast<const uint4 *>(dev.d_payload), dev.d_inv, d_off_dev, padded_offsets, n_docs, dev.kblocks, padded_payload, padded_inv);
                    ok = cuda_ok(cudaGetLastError(), "document re-layout kernel");
                    g_launches++;
                    dev.d_payload = reinterpret_cast<const uint8_t *>(padded_payload);
                    dev.d_inv = padded_inv;
                    dev.d_offsets = padded_offsets;
                    dev.d_tokens = padded_tokens;
                }
            }
        }
        dev.segments = pick_segments(dev.d_tokens, dev.q_tiles);
        dev.scores_f32 = s_dev; dev.score_stride = s_pitch / 4; dev.total_f64 = nullptr; dev.error_word = err;
        ok = cuda_ok(launch_maxsim_tc(dt, dev, stream), "MaxSim kernel");
        g_launches++;
    }
    if (ok && s_kind == kMemHost)
        ok = cuda_ok(cudaMemcpy2DAsync(scores, score_stride < row_bytes ? row_bytes : score_stride, s_dev, s_pitch, row_bytes, n_queries,
                                       cudaMemcpyDeviceToHost, stream), "download scores");
    const bool must_sync = s_kind == kMemHost || classify(q_packed) == kMemHost || classify(d_packed) == kMemHost ||
                           classify(q_offsets) == kMemHost || classify(d_offsets) == kMemHost;
    if (ok && must_sync) {
        ok = cuda_ok(cudaStreamSynchronize(stream), "maxsims_packed");
        if (ok) {
            uint32_t w = read_device_error();
            if (w) { char buf[64]; std::snprintf(buf, sizeof buf, "0x%08x", w); set_error("a pipeline wait inside the MaxSim kernel gave up (error word %s)", buf); ok = false; }
        }
    }
    if (!ok) fail();
}

} // namespace
} // namespace nkb

using namespace nkb;

extern "C" {

#define NKB_DEFINE_MAXSIM_FAMILY(T, DT)                                                                                \
    NKB_API nk_size_t nk_maxsim_packed_size_##T(nk_size_t count, nk_size_t depth) { return maxsim_size_impl(DT, count, depth); } \
    NKB_API void nk_maxsim_pack_##T(void const *vectors, nk_size_t count, nk_size_t depth, nk_size_t stride, void *packed) { \
        maxsim_pack_impl(DT, vectors, count, depth, stride, packed);                                                   \
    }                                                                                                                  \
    NKB_API void nk_maxsim_packed_##T(void const *q, void const *d, nk_size_t nq, nk_size_t nd, nk_size_t depth, void *result) { \
        maxsim_single_impl(DT, q, d, nq, nd, depth, result);                                                           \
    }

NKB_DEFINE_MAXSIM_FAMILY(bf16, kBF16)
NKB_DEFINE_MAXSIM_FAMILY(f16, kF16)
NKB_DEFINE_MAXSIM_FAMILY(f32, kF32)

NKB_API void nkb_maxsims_packed_bf16(void const *q_packed, void const *q_offsets, nk_size_t n_queries, void const *d_packed,
                                     void const *d_offsets, nk_size_t n_docs, nk_size_t depth, void *scores, nk_size_t score_stride) {
    maxsims_batch_impl(kBF16, q_packed, q_offsets, n_queries, d_packed, d_offsets, n_docs, depth, scores, score_stride);
}
NKB_API void nkb_maxsims_packed_f16(void const *q_packed, void const *q_offsets, nk_size_t n_queries, void const *d_packed,
                                    void const *d_offsets, nk_size_t n_docs, nk_size_t depth, void *scores, nk_size_t score_stride) {
    maxsims_batch_impl(kF16, q_packed, q_offsets, n_queries, d_packed, d_offsets, n_docs, depth, scores, score_stride);
}

} // extern "C"
