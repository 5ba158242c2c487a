// Top-k selection for results that are too large to hand back whole.
//
// NumKong's batched distances and MaxSim return full matrices / one scalar per call
// (include/numkong/spatials.h:72-, include/numkong/maxsim.h:106-114); at 65,536 queries x 10,000,000
// corpus rows the full matrix is 2.6 TB, so the nearest-k per query have to be selected on the device.
// These entry points are additions: each equals "call the reference function, then keep the k smallest
// of every row (ties broken by the lower id)", which is how the tests check them.
//
//   topk_smallest_kernel   one CTA per row: exact radix select (4 x 8-bit passes over order-preserving
//                          integer keys), ordered tie handling, bitonic sort of the survivors
//   merge_topk_kernel      merges a panel's k best into the running k best
//   filter_init_kernel / filter_refine_kernel   thresholds and running lists of the filtered path
// The batched-distance top-k walks the packed B matrix in column panels. Materialising path: tensor-core GEMM
// with the distance epilogue into a scratch panel, select, merge. Filtered path (k <= 128, large packed
// matrices): only a first narrow panel is materialised; it gives every row a threshold (its k-th smallest so
// far), and the remaining, ever wider panels run the GEMM with a filter epilogue that writes nothing but the few
// values below the threshold, which a refine kernel folds into the running lists. Both paths return the same
// bits; a candidate list that overflows sends the call back to the materialising path.
#include <atomic>
#include <cstdio>
#include <cstring>
#include "nkb_internal.h"
#include "nkb_host.h"
#include "../../include/numkong_b200.h"

namespace nkb {

namespace {

std::atomic<uint64_t> g_panel_rows{0};  // 0 = choose by scratch size
std::atomic<int> g_filter_mode{1};      // 0 = always materialise; 1 = filter when the shape allows; >= 256 = bootstrap width
std::atomic<uint64_t> g_filter_fallbacks{0};  // calls redone without the filter after a candidate list overflowed

constexpr int kTopThreads = 256;
constexpr int kTopMax = 1024;  // largest k supported

__device__ __forceinline__ uint32_t order_key(float f) { return selection_key(f); }
__device__ __forceinline__ float key_value(uint32_t k) { return selection_value(k); }

// Sorts `n` (a power of two) 64-bit words ascending in shared memory.
__device__ void bitonic_sort_u64(unsigned long long *data, int n) {
    for (int size = 2; size <= n; size <<= 1) {
        for (int stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (int i = threadIdx.x; i < n / 2; i += blockDim.x) {
                int lo = 2 * i - (i & (stride - 1));
                int hi = lo + stride;
                bool ascending = (lo & size) == 0;
                unsigned long long a = data[lo], b = data[hi];
                if ((a > b) == ascending) { data[lo] = b; data[hi] = a; }
            }
        }
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kTopThreads)
topk_smallest_kernel(const float *__restrict__ scores, uint64_t cols, uint64_t stride_elems, uint32_t top,
                     uint64_t id_base, float *__restrict__ out_vals, long long *__restrict__ out_ids) {
    __shared__ uint32_t hist[256];
    __shared__ uint32_t s_prefix, s_remaining, s_equal, s_count, s_eq_seen;
    __shared__ uint32_t warp_tot[kTopThreads / 32];
    __shared__ unsigned long long cand[kTopMax];
    const float *row = scores + (uint64_t)blockIdx.x * stride_elems;
    const uint32_t want = cols < top ? (uint32_t)cols : top;
    uint32_t padded = 1;
    while (padded < top) padded <<= 1;

    uint32_t prefix = 0, mask = 0, remaining = want;
    if (want > 0) {
        for (int pass = 0; pass < 4; ++pass) {
            const int shift = 24 - 8 * pass;
            for (int i = threadIdx.x; i < 256; i += blockDim.x) hist[i] = 0;
            __syncthreads();
            for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) {
                uint32_t key = order_key(row[c]);
                if ((key & mask) == prefix) atomicAdd(&hist[(key >> shift) & 0xffu], 1u);
            }
            __syncthreads();
            {
                // One bin per thread (the block has exactly 256): inclusive prefix sum over the bins, then the one
                // thread whose bin holds the remaining-th smallest key publishes it.
                const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
                const uint32_t mine = hist[threadIdx.x];
                uint32_t incl = mine;
#pragma unroll
                for (int off = 1; off < 32; off <<= 1) {
                    const uint32_t o = __shfl_up_sync(0xffffffffu, incl, off);
                    if (lane >= off) incl += o;
                }
                if (lane == 31) warp_tot[w] = incl;
                __syncthreads();
                for (int i = 0; i < w; ++i) incl += warp_tot[i];
                const uint32_t excl = incl - mine;
                if (excl < remaining && incl >= remaining) {
                    s_prefix = prefix | ((uint32_t)threadIdx.x << shift);
                    s_remaining = remaining - excl;
                    s_equal = mine;
                }
            }
            __syncthreads();
            prefix = s_prefix;
            remaining = s_remaining;
            mask |= 0xffu << shift;
            __syncthreads();
        }
    }
    // `prefix` is now the key of the want-th smallest element; `remaining` of the elements equal to it
    // are taken, lowest columns first.
    if (threadIdx.x == 0) { s_count = 0; s_eq_seen = 0; }
    for (int i = threadIdx.x; i < (int)padded; i += blockDim.x) cand[i] = ~0ull;
    __syncthreads();
    if (want > 0 && s_equal == remaining) {
        // Every element equal to the k-th smallest is kept: no order to respect while collecting (the sort restores it).
        for (uint64_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const uint32_t key = order_key(row[c]);
            if (key <= prefix) {
                const uint32_t slot = atomicAdd(&s_count, 1u);
                if (slot < kTopMax) cand[slot] = ((unsigned long long)key << 32) | (unsigned long long)(uint32_t)c;
            }
        }
    } else if (want > 0) {
        const uint64_t rounds = (cols + blockDim.x - 1) / blockDim.x;
        for (uint64_t r = 0; r < rounds; ++r) {
            const uint64_t c = r * blockDim.x + threadIdx.x;
            uint32_t key = 0xffffffffu;
            bool less = false, equal = false;
            if (c < cols) { key = order_key(row[c]); less = key < prefix; equal = key == prefix; }
            // Rank of this thread among the "equal" elements of the round (block-wide exclusive count).
            const uint32_t ballot = __ballot_sync(0xffffffffu, equal);
            const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
            if (lane == 0) warp_tot[w] = __popc(ballot);
            __syncthreads();
            uint32_t before = __popc(ballot & ((1u << lane) - 1u));
            for (int i = 0; i < w; ++i) before += warp_tot[i];
            uint32_t round_total = 0;
            for (int i = 0; i < kTopThreads / 32; ++i) round_total += warp_tot[i];
            const uint32_t eq_seen = s_eq_seen;
            if (less || (equal && eq_seen + before < remaining)) {
                uint32_t slot = atomicAdd(&s_count, 1u);
                if (slot < kTopMax) cand[slot] = ((unsigned long long)key << 32) | (unsigned long long)(uint32_t)c;
            }
            __syncthreads();
            if (threadIdx.x == 0) s_eq_seen = eq_seen + round_total;
            __syncthreads();
        }
    }
    bitonic_sort_u64(cand, (int)padded);
    for (uint32_t i = threadIdx.x; i < top; i += blockDim.x) {
        unsigned long long e = cand[i];
        const uint64_t o = (uint64_t)blockIdx.x * top + i;
        if (i < want && e != ~0ull) {
            out_vals[o] = key_value((uint32_t)(e >> 32));
            out_ids[o] = (long long)(id_base + (uint32_t)e);
        } else {
            out_vals[o] = __uint_as_float(0x7f800000u);
            out_ids[o] = -1;
        }
    }
}

// run <- k smallest of (run ++ fresh), ordered by (value, id). One CTA per row.
__global__ void __launch_bounds__(kTopThreads)
merge_topk_kernel(float *__restrict__ run_vals, long long *__restrict__ run_ids, const float *__restrict__ new_vals,
                  const long long *__restrict__ new_ids, uint32_t top) {
    __shared__ unsigned long long keys[2 * kTopMax];   // (order key << 32) | position in the combined list
    __shared__ long long ids[2 * kTopMax];
    uint32_t padded = 1;
    while (padded < 2 * top) padded <<= 1;
    const uint64_t base = (uint64_t)blockIdx.x * top;
    // Both lists are already sorted by (value, id) and the running list holds the lower ids, so the
    // position in the combined list breaks value ties exactly like the id does.
    for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) {
        if (i < 2 * top) {
            const bool from_run = i < top;
            const float v = from_run ? run_vals[base + i] : new_vals[base + i - top];
            const long long id = from_run ? run_ids[base + i] : new_ids[base + i - top];
            ids[i] = id;
            keys[i] = id < 0 ? ~0ull : (((unsigned long long)order_key(v) << 32) | i);
        } else keys[i] = ~0ull;
    }
    __syncthreads();
    bitonic_sort_u64(keys, (int)padded);
    for (uint32_t i = threadIdx.x; i < top; i += blockDim.x) {
        const unsigned long long e = keys[i];
        if (e != ~0ull) {
            run_vals[base + i] = key_value((uint32_t)(e >> 32));
            run_ids[base + i] = ids[(uint32_t)e];
        } else {
            run_vals[base + i] = __uint_as_float(0x7f800000u);
            run_ids[base + i] = -1;
        }
    }
}

// Merges `parts` lists per row (each `top` long, any order, empty slots marked by id < 0) into the `top` smallest by
// (value, id). Lists are laid out [part][row][top]: what a gather of per-shard results delivers. One CTA per row;
// dynamic shared memory holds `padded` (a power of two >= parts * top) ids followed by as many 32-bit value keys.
// Unlike merge_topk_kernel this makes no assumption about which list holds the lower ids.
__global__ void __launch_bounds__(kTopThreads)
merge_parts_kernel(const float *__restrict__ vals, const long long *__restrict__ ids, uint32_t parts, uint64_t rows, uint32_t top,
                   uint32_t padded, float *__restrict__ out_vals, long long *__restrict__ out_ids) {
    extern __shared__ unsigned long long merge_smem[];
    long long *s_id = reinterpret_cast<long long *>(merge_smem);
    uint32_t *s_key = reinterpret_cast<uint32_t *>(s_id + padded);
    const uint64_t row = blockIdx.x;
    const uint32_t total = parts * top;
    constexpr long long kNoId = 0x7fffffffffffffffll;
    for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) {
        uint32_t key = 0xffffffffu;
        long long id = kNoId;
        if (i < total) {
            const uint64_t at = ((uint64_t)(i / top) * rows + row) * top + i % top;
            const long long got = ids[at];
            if (got >= 0) { id = got; key = order_key(vals[at]); }
        }
        s_key[i] = key;
        s_id[i] = id;
    }
    for (uint32_t size = 2; size <= padded; size <<= 1) {
        for (uint32_t stride = size >> 1; stride > 0; stride >>= 1) {
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < padded / 2; i += blockDim.x) {
                const uint32_t lo = 2 * i - (i & (stride - 1)), hi = lo + stride;
                const bool ascending = (lo & size) == 0;
                const uint32_t ka = s_key[lo], kb = s_key[hi];
                const long long ia = s_id[lo], ib = s_id[hi];
                const bool a_after_b = ka > kb || (ka == kb && ia > ib);
                if (a_after_b == ascending) { s_key[lo] = kb; s_key[hi] = ka; s_id[lo] = ib; s_id[hi] = ia; }
            }
        }
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < top; i += blockDim.x) {
        const bool empty = s_id[i] == kNoId;
        out_vals[row * top + i] = empty ? __uint_as_float(0x7f800000u) : key_value(s_key[i]);
        out_ids[row * top + i] = empty ? -1 : s_id[i];
    }
}

constexpr uint32_t kMergeMaxEntries = 16384;  // parts * top, rounded up to a power of two: 192 KiB of shared memory

void merge_topk_impl(const void *values, const void *ids, uint64_t parts, uint64_t rows, uint64_t top, void *out_vals, void *out_ids) {
    clear_error();
    if (rows == 0 || top == 0) return;
    const MemKind v_kind = classify(out_vals), i_kind = classify(out_ids);
    auto fail = [&]() {
        fill_error_output(out_vals, v_kind, rows, top * 4, top * 4);
        fill_error_output(out_ids, i_kind, rows, top * 8, top * 8);
    };
    if (!values || !ids || !out_vals || !out_ids) { set_error("merge_topk: null pointer%s", ""); return; }
    uint32_t padded = 2;
    while (padded < parts * top && padded < 2 * kMergeMaxEntries) padded <<= 1;
    if (parts == 0 || top > kTopMax || padded > kMergeMaxEntries || rows > 0x7fffffffull) {
        set_error("merge_topk: at most 1024 per list and 16384 entries per row (parts x top)%s", "");
        fail();
        return;
    }
    cudaStream_t stream = current_stream();
    const uint64_t n = parts * rows * top;
    const MemKind sv_kind = classify(values), si_kind = classify(ids);
    const float *v_in = static_cast<const float *>(values);
    const long long *i_in = static_cast<const long long *>(ids);
    bool ok = true;
    if (sv_kind == kMemHost) {
        void *buf = scratch(kSlotA, n * 4);
        ok = buf && cuda_ok(cudaMemcpyAsync(buf, values, n * 4, cudaMemcpyHostToDevice, stream), "upload of top-k values");
        v_in = static_cast<const float *>(buf);
    }
    if (ok && si_kind == kMemHost) {
        void *buf = scratch(kSlotC, n * 8);
        ok = buf && cuda_ok(cudaMemcpyAsync(buf, ids, n * 8, cudaMemcpyHostToDevice, stream), "upload of top-k ids");
        i_in = static_cast<const long long *>(buf);
    }
    float *v_dev = static_cast<float *>(out_vals);
    long long *i_dev = static_cast<long long *>(out_ids);
    if (ok && v_kind == kMemHost) { v_dev = static_cast<float *>(scratch(kSlotAux, rows * top * 4)); ok = v_dev != nullptr; }
    if (ok && i_kind == kMemHost) { i_dev = static_cast<long long *>(scratch(kSlotAux2, rows * top * 8)); ok = i_dev != nullptr; }
    if (ok) {
        const size_t smem = (size_t)padded * 12;
        static bool configured[64] = {false};
        int d = 0;
        cudaGetDevice(&d);
        if (d >= 0 && d < 64 && !configured[d]) {
            ok = cuda_ok(cudaFuncSetAttribute(merge_parts_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kMergeMaxEntries * 12), "merge kernel set-up");
            configured[d] = ok;
        }
        if (ok) {
            merge_parts_kernel<<<(unsigned)rows, kTopThreads, smem, stream>>>(v_in, i_in, (uint32_t)parts, rows, (uint32_t)top, padded, v_dev, i_dev);
            g_launches++;
            ok = cuda_ok(cudaGetLastError(), "merge kernel");
        }
    }
    if (ok && v_kind == kMemHost) ok = cuda_ok(cudaMemcpyAsync(out_vals, v_dev, rows * top * 4, cudaMemcpyDeviceToHost, stream), "download of merged values");
    if (ok && i_kind == kMemHost) ok = cuda_ok(cudaMemcpyAsync(out_ids, i_dev, rows * top * 8, cudaMemcpyDeviceToHost, stream), "download of merged ids");
    if (ok && (v_kind == kMemHost || i_kind == kMemHost || sv_kind == kMemHost || si_kind == kMemHost)) ok = cuda_ok(cudaStreamSynchronize(stream), "merge_topk");
    if (!ok) fail();
}

// ---- fused selection: the GEMM epilogue filters, these kernels keep the running lists -------------------
constexpr uint32_t kFilterTopMax = 128;       // largest k the filtered path serves
constexpr uint32_t kFilterCapacity = 512;     // candidates kept per row and panel
constexpr uint32_t kFilterBootstrap = 2048;   // packed rows selected from a materialised panel to get first thresholds
// Thresholds travel as f32 bit patterns that the epilogue compares as signed integers (distances are >= -0, never NaN);
// the largest positive pattern lets every value pass.
constexpr uint32_t kPassAll = 0x7fffffffu;

// Sets every row's threshold from its running list (k-th entry, or "everything passes" while the list is short)
// and clears the candidate counts and the overflow word.
__global__ void filter_init_kernel(const float *__restrict__ run_vals, const long long *__restrict__ run_ids, uint32_t top,
                                   uint64_t rows, uint32_t *__restrict__ threshold_bits, uint32_t *__restrict__ counts,
                                   uint32_t *__restrict__ overflow) {
    const uint64_t row = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (row == 0) *overflow = 0;
    if (row >= rows) return;
    const uint64_t last = row * top + top - 1;
    threshold_bits[row] = run_ids[last] < 0 ? kPassAll : __float_as_uint(run_vals[last]);
    counts[row] = 0;
}

// run <- k smallest of (run ++ this row's candidates), ordered by (value, id); then the row's threshold key is renewed
// and its candidate count cleared. Candidates come from packed rows after everything the running list has seen, so
// their ids are larger: positions in the combined list break value ties exactly like ids do. One CTA per row.
__global__ void __launch_bounds__(kTopThreads)
filter_refine_kernel(float *__restrict__ run_vals, long long *__restrict__ run_ids, const uint2 *__restrict__ candidates,
                     uint32_t *__restrict__ counts, uint32_t *__restrict__ threshold_bits, uint32_t capacity, uint32_t top,
                     uint64_t id_origin, uint32_t *__restrict__ overflow) {
    __shared__ unsigned long long keys[1024];
    __shared__ long long old_ids[kFilterTopMax];
    const uint64_t row = blockIdx.x;
    uint32_t count = counts[row];
    if (count == 0) return;  // uniform for the CTA: nothing beat the threshold
    if (count > capacity) {
        if (threadIdx.x == 0) atomicOr(overflow, 1u);
        count = capacity;
    }
    uint32_t padded = 2;
    while (padded < top + count) padded <<= 1;
    const uint64_t base = row * top;
    for (uint32_t i = threadIdx.x; i < padded; i += blockDim.x) {
        unsigned long long key = ~0ull;
        if (i < top) {
            const long long id = run_ids[base + i];
            old_ids[i] = id;
            if (id >= 0) key = ((unsigned long long)order_key(run_vals[base + i]) << 32) | i;
        } else if (i < top + count) {
            const uint2 c = candidates[row * capacity + (i - top)];
            key = ((unsigned long long)order_key(__uint_as_float(c.x)) << 32) | (unsigned long long)(top + c.y);
        }
        keys[i] = key;
    }
    bitonic_sort_u64(keys, (int)padded);  // starts and ends with a block-wide barrier
    for (uint32_t i = threadIdx.x; i < top; i += blockDim.x) {
        const unsigned long long e = keys[i];
        const uint32_t low = (uint32_t)e;
        if (e != ~0ull) {
            run_vals[base + i] = key_value((uint32_t)(e >> 32));
            run_ids[base + i] = low < top ? old_ids[low] : (long long)(id_origin + (low - top));
        } else {
            run_vals[base + i] = __uint_as_float(0x7f800000u);
            run_ids[base + i] = -1;
        }
        if (i == top - 1) threshold_bits[row] = e != ~0ull ? __float_as_uint(key_value((uint32_t)(e >> 32))) : kPassAll;
    }
    if (threadIdx.x == 0) counts[row] = 0;
}

// Widest panel the filter may scan after `seen` packed rows: the number of later values below the k-th smallest of
// `seen` grows like (panel / seen) * Gamma(k), so the ratio is chosen to keep k + 8 sqrt(k) + 8 "expected" candidates,
// scaled by the ratio, inside the capacity (an overflow is still detected and the call redone without the filter).
uint64_t filter_growth(uint32_t top) {
    uint32_t root = 1;
    while (root * root < top) ++root;
    const uint32_t budget = top + 8 * root + 8;
    uint32_t ratio = kFilterCapacity / budget;
    return ratio > 8 ? 8 : ratio;
}

bool topk_on_device(const float *scores, uint64_t rows, uint64_t cols, uint64_t stride_bytes, uint32_t top,
                    uint64_t id_base, float *vals, long long *ids, cudaStream_t stream) {
    if (rows == 0) return true;
    topk_smallest_kernel<<<(unsigned)rows, kTopThreads, 0, stream>>>(scores, cols, stride_bytes / 4, top, id_base, vals, ids);
    g_launches++;
    return cuda_ok(cudaGetLastError(), "top-k kernel");
}

void topk_smallest_impl(const void *scores, uint64_t rows, uint64_t cols, uint64_t stride, uint64_t top, uint64_t id_base,
                        void *out_vals, void *out_ids) {
    clear_error();
    if (rows == 0 || top == 0) return;
    const MemKind v_kind = classify(out_vals), i_kind = classify(out_ids), s_kind = classify(scores);
    auto fail = [&]() {
        fill_error_output(out_vals, v_kind, rows, top * 4, top * 4);
        fill_error_output(out_ids, i_kind, rows, top * 8, top * 8);
    };
    if (!scores || !out_vals || !out_ids) { set_error("topk: null pointer%s", ""); return; }
    if (top > kTopMax) { set_error("topk: k is limited to 1024%s", ""); fail(); return; }
    if (rows > 0x7fffffffull || cols > 0xffffffffull || stride % 4) { set_error("topk: unsupported shape or stride%s", ""); fail(); return; }
    cudaStream_t stream = current_stream();
    const float *s_dev = static_cast<const float *>(scores);
    uint64_t s_pitch = stride;
    bool ok = true;
    if (s_kind == kMemHost) {
        s_pitch = cols * 4;
        void *buf = scratch(kSlotC, rows * s_pitch + 16);
        ok = buf && cuda_ok(cudaMemcpy2DAsync(buf, s_pitch, scores, stride < s_pitch ? s_pitch : stride, s_pitch, rows, cudaMemcpyHostToDevice, stream), "upload scores");
        s_dev = static_cast<const float *>(buf);
    }
    float *v_dev = static_cast<float *>(out_vals);
    long long *i_dev = static_cast<long long *>(out_ids);
    if (ok && v_kind == kMemHost) { v_dev = static_cast<float *>(scratch(kSlotAux, rows * top * 4)); ok = v_dev != nullptr; }
    if (ok && i_kind == kMemHost) { i_dev = static_cast<long long *>(scratch(kSlotAux2, rows * top * 8)); ok = i_dev != nullptr; }
    if (ok) ok = topk_on_device(s_dev, rows, cols, s_pitch, (uint32_t)top, id_base, v_dev, i_dev, stream);
    if (ok && v_kind == kMemHost) ok = cuda_ok(cudaMemcpyAsync(out_vals, v_dev, rows * top * 4, cudaMemcpyDeviceToHost, stream), "download top-k values");
    if (ok && i_kind == kMemHost) ok = cuda_ok(cudaMemcpyAsync(out_ids, i_dev, rows * top * 8, cudaMemcpyDeviceToHost, stream), "download top-k ids");
    if (ok && (v_kind == kMemHost || i_kind == kMemHost || s_kind == kMemHost)) ok = cuda_ok(cudaStreamSynchronize(stream), "topk");
    if (!ok) fail();
}

// Nearest-k rows of the packed matrix for every row of A, without materialising the distance matrix.
void spatial_topk_impl(uint32_t dt, int epilogue, const void *a, const void *b_packed, uint64_t m, uint64_t n, uint64_t k,
                       uint64_t a_stride, uint64_t top, void *out_vals, void *out_ids, uint64_t id_base,
                       bool allow_filter = true) {
    clear_error();
    if (m == 0 || top == 0) return;
    const MemKind v_kind = classify(out_vals), i_kind = classify(out_ids);
    auto fail = [&]() {
        fill_error_output(out_vals, v_kind, m, top * 4, top * 4);
        fill_error_output(out_ids, i_kind, m, top * 8, top * 8);
    };
    if (!a || !b_packed || !out_vals || !out_ids) { set_error("packed_topk: null pointer%s", ""); return; }
    if (top > kTopMax) { set_error("packed_topk: k is limited to 1024%s", ""); fail(); return; }
    if (n == 0 || k == 0) { set_error("packed_topk: empty packed matrix%s", ""); fail(); return; }
    cudaStream_t stream = current_stream();
    const MemKind a_kind = classify(a), b_kind = classify(b_packed);
    PackedHeader h;
    const uint8_t *blob = resident_blob(b_packed, b_kind, kMagicDots, dt, n, k, &h);
    if (!blob) { fail(); return; }
    unsigned int *err = device_error_word();
    uint64_t a_pitch = 0;
    const void *a_dev = resident_matrix(a, a_kind, m, k * dtype_bytes(dt), a_stride, kSlotA, kPieceNone, &a_pitch);
    if (!err || !a_dev) { fail(); return; }

    // Filtered path: only a first narrow panel is materialised and selected from; it gives every row a threshold
    // (its k-th smallest so far). Wider and wider panels then go through the GEMM with the filter epilogue, which
    // stores nothing but the few values below the threshold, and a refine kernel folds those into the running lists.
    const int filter_mode = g_filter_mode.load();
    const uint64_t bootstrap = filter_mode >= 256 ? round_up((uint64_t)filter_mode, 256) : kFilterBootstrap;
    const uint64_t growth = filter_growth((uint32_t)top);
    const bool filtered = allow_filter && filter_mode != 0 && top <= kFilterTopMax && growth >= 2 && bootstrap >= 2 * top &&
                          (filter_mode >= 256 ? n > bootstrap : n >= 4 * bootstrap) && m <= 131072;

    // Panel width: a multiple of 256 packed rows whose m x width f32 scratch stays near 1 GiB.
    uint64_t width = ((1ull << 30) / (m * 4)) / 256 * 256;
    if (g_panel_rows.load()) width = round_up(g_panel_rows.load(), 256);
    if (filtered) width = bootstrap;
    if (width < 256) width = 256;
    if (width > h.rows_padded) width = h.rows_padded;
    const uint64_t panels = filtered ? 1 : (n + width - 1) / width;

    float *a_norms = static_cast<float *>(scratch(kSlotNorms, m * 4));
    float *panel = static_cast<float *>(scratch(kSlotC, m * width * 4));
    // Running and per-panel results share one allocation: [run vals | new vals | run ids | new ids].
    uint8_t *lists = static_cast<uint8_t *>(scratch(kSlotAux, m * top * 24 + 64));
    if (!a_norms || !panel || !lists) { fail(); return; }
    float *run_vals = reinterpret_cast<float *>(lists);
    float *new_vals = run_vals + m * top;
    long long *run_ids = reinterpret_cast<long long *>(lists + round_up(m * top * 8, 8));
    long long *new_ids = run_ids + m * top;
    if (v_kind == kMemDevice) run_vals = static_cast<float *>(out_vals);
    if (i_kind == kMemDevice) run_ids = static_cast<long long *>(out_ids);

    bool ok = cuda_ok(launch_row_sumsq(dt, a_dev, m, k, a_pitch, a_norms, true, false, stream), "row norm kernel");
    g_launches++;
    const uint32_t kblocks = (uint32_t)(h.depth_padded_bytes / kChunkRowBytes);
    for (uint64_t p = 0; p < panels && ok; ++p) {
        const uint64_t col0 = p * width;
        const uint64_t cols = n - col0 < width ? n - col0 : width;
        GemmArgs g;
        g.dtype = dt; g.epilogue = epilogue; g.a = a_dev; g.a_stride = a_pitch;
        g.b_payload = blob + h.payload_offset + (col0 / kChunkRows) * (uint64_t)kblocks * kChunkBytes;
        g.b_norms = blob + h.norms_offset + col0 * 4;
        g.a_norms = a_norms;
        g.c = panel; g.c_stride = width * 4; g.m = m; g.n = cols; g.k = k;
        g.depth_padded_bytes = h.depth_padded_bytes; g.error_word = err; g.variant = current_variant();
        ok = cuda_ok(launch_gemm_tc(g, stream), "tensor-core GEMM kernel");
        g_launches++;
        if (!ok) break;
        float *pv = p == 0 ? run_vals : new_vals;
        long long *pi = p == 0 ? run_ids : new_ids;
        ok = topk_on_device(panel, m, cols, width * 4, (uint32_t)top, id_base + col0, pv, pi, stream);
        if (ok && p > 0) {
            merge_topk_kernel<<<(unsigned)m, kTopThreads, 0, stream>>>(run_vals, run_ids, new_vals, new_ids, (uint32_t)top);
            g_launches++;
            ok = cuda_ok(cudaGetLastError(), "merge kernel");
        }
    }
    if (ok && filtered) {
        // [candidates: m x capacity x 8 B | threshold keys: m x 4 B | counts: m x 4 B | overflow word]
        const uint64_t cand_bytes = m * kFilterCapacity * 8;
        uint8_t *filter_mem = static_cast<uint8_t *>(scratch(kSlotAux2, cand_bytes + m * 8 + 64));
        if (!filter_mem) { fail(); return; }
        uint2 *candidates = reinterpret_cast<uint2 *>(filter_mem);
        uint32_t *threshold_bits = reinterpret_cast<uint32_t *>(filter_mem + cand_bytes);
        uint32_t *counts = threshold_bits + m;
        uint32_t *overflow = counts + m;
        filter_init_kernel<<<(unsigned)((m + 255) / 256), 256, 0, stream>>>(run_vals, run_ids, (uint32_t)top, m, threshold_bits,
                                                                           counts, overflow);
        g_launches++;
        ok = cuda_ok(cudaGetLastError(), "filter init kernel");
        uint64_t seen = width;
        while (ok && seen < n) {
            uint64_t cols = growth * seen / 256 * 256;
            if (cols > n - seen) cols = n - seen;
            GemmArgs g;
            g.dtype = dt; g.epilogue = epilogue; g.a = a_dev; g.a_stride = a_pitch;
            g.b_payload = blob + h.payload_offset + (seen / kChunkRows) * (uint64_t)kblocks * kChunkBytes;
            g.b_norms = blob + h.norms_offset + seen * 4;
            g.a_norms = a_norms;
            g.c = nullptr; g.c_stride = 0; g.m = m; g.n = cols; g.k = k;
            g.depth_padded_bytes = h.depth_padded_bytes; g.error_word = err; g.variant = current_variant();
            g.threshold_bits = threshold_bits; g.candidate_counts = counts; g.candidates = candidates;
            g.candidate_capacity = kFilterCapacity; g.column_id_base = 0;
            ok = cuda_ok(launch_gemm_tc(g, stream), "tensor-core GEMM kernel (filter)");
            g_launches++;
            if (!ok) break;
            filter_refine_kernel<<<(unsigned)m, kTopThreads, 0, stream>>>(run_vals, run_ids, candidates, counts, threshold_bits,
                                                                         kFilterCapacity, (uint32_t)top, id_base + seen, overflow);
            g_launches++;
            ok = cuda_ok(cudaGetLastError(), "filter refine kernel");
            seen += cols;
        }
        // A row whose candidates did not fit lost values: redo the whole call on the materialising path. Reading the
        // word back makes the filtered path synchronise with its stream before it returns.
        uint32_t overflowed = 0;
        if (ok) ok = cuda_ok(cudaMemcpyAsync(&overflowed, overflow, 4, cudaMemcpyDeviceToHost, stream), "read overflow word") &&
                     cuda_ok(cudaStreamSynchronize(stream), "packed_topk");
        if (ok && read_device_error()) { set_error("a pipeline wait inside the GEMM kernel gave up%s", ""); ok = false; }
        if (ok && overflowed) {
            g_filter_fallbacks++;
            spatial_topk_impl(dt, epilogue, a, b_packed, m, n, k, a_stride, top, out_vals, out_ids, id_base, false);
            return;
        }
    }
    if (ok && v_kind == kMemHost) ok = cuda_ok(cudaMemcpyAsync(out_vals, run_vals, m * top * 4, cudaMemcpyDeviceToHost, stream), "download top-k values");
    if (ok && i_kind == kMemHost) ok = cuda_ok(cudaMemcpyAsync(out_ids, run_ids, m * top * 8, cudaMemcpyDeviceToHost, stream), "download top-k ids");
    if (ok && (v_kind == kMemHost || i_kind == kMemHost || a_kind == kMemHost || b_kind == kMemHost)) {
        ok = cuda_ok(cudaStreamSynchronize(stream), "packed_topk");
        if (ok && read_device_error()) { set_error("a pipeline wait inside the GEMM kernel gave up%s", ""); ok = false; }
    }
    if (!ok) fail();
}

} // namespace
} // namespace nkb

using namespace nkb;

extern "C" {

NKB_API void nkb_set_topk_panel_rows(nk_size_t rows) { g_panel_rows.store(rows); }
NKB_API void nkb_set_topk_filter(int mode) { g_filter_mode.store(mode < 0 ? 0 : mode); }
NKB_API nk_size_t nkb_topk_filter_fallbacks(void) { return g_filter_fallbacks.load(); }

NKB_API void nkb_topk_smallest_f32(void const *scores, nk_size_t rows, nk_size_t cols, nk_size_t stride, nk_size_t top,
                                   nk_size_t id_base, void *out_values, void *out_ids) {
    topk_smallest_impl(scores, rows, cols, stride, top, id_base, out_values, out_ids);
}

NKB_API void nkb_merge_topk(void const *values, void const *ids, nk_size_t parts, nk_size_t rows, nk_size_t top,
                            void *out_values, void *out_ids) {
    merge_topk_impl(values, ids, parts, rows, top, out_values, out_ids);
}

#define NKB_DEFINE_TOPK(T, DT)                                                                                         \
    NKB_API void nkb_angulars_packed_topk_##T(void const *a, void const *b_packed, nk_size_t height, nk_size_t width,  \
                                              nk_size_t depth, nk_size_t a_stride, nk_size_t top, void *distances,     \
                                              void *ids, nk_size_t id_base) {                                          \
        spatial_topk_impl(DT, kEpiAngular, a, b_packed, height, width, depth, a_stride, top, distances, ids, id_base); \
    }                                                                                                                  \
    NKB_API void nkb_euclideans_packed_topk_##T(void const *a, void const *b_packed, nk_size_t height, nk_size_t width, \
                                                nk_size_t depth, nk_size_t a_stride, nk_size_t top, void *distances,   \
                                                void *ids, nk_size_t id_base) {                                        \
        spatial_topk_impl(DT, kEpiEuclidean, a, b_packed, height, width, depth, a_stride, top, distances, ids, id_base); \
    }

NKB_DEFINE_TOPK(f16, kF16)
NKB_DEFINE_TOPK(bf16, kBF16)

} // extern "C"
