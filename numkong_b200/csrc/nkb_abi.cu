// Host side of the C ABI declared in include/numkong_b200.h: argument checks, pointer
// classification, staging of host-resident operands, the device cache of host-resident packed
// blobs, and the NumKong failure convention (fill the output with 0xFF, c/numkong.c:78-81).
// It plays the role of NumKong's dispatch layer (c/numkong.c:347-380, 628-765): one indirection
// between the exported nk_* symbol and the kernel that does the work.
#include <atomic>
#include <chrono>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "../../include/numkong_b200.h"
#include "nkb_host.h"

namespace nkb {

std::atomic<uint64_t> g_launches{0};

namespace {

std::atomic<int> g_variant{0};
std::atomic<int> g_fp6_native{1};
std::atomic<uint64_t> g_nonce_counter{0};
std::atomic<int> g_sm_budget{0};
// Limit of every bounded wait of the tensor-core kernels, by wait site (microseconds); see nkb_set_wait_limit_ns.
std::atomic<uint32_t> g_wait_us[kWaitSites] = {{kDefaultWaitLimitUs}, {kDefaultWaitLimitUs}, {kDefaultWaitLimitUs}, {kDefaultWaitLimitUs},
                                               {kDefaultWaitLimitUs}, {kDefaultWaitLimitUs}, {kDefaultWaitLimitUs}, {kDefaultWaitLimitUs},
                                               {kDefaultWaitLimitUs}};

// ---------------------------------------------------------------- per-thread context
struct Scratch {
    void *ptr = nullptr;
    size_t bytes = 0;
    int device = -1;
};

struct ThreadCtx {
    cudaStream_t stream = nullptr;
    std::string error;
    Scratch slots[kScratchSlots];
    // Row-pipelined host calls alternate between two private streams, each with its own set of staging buffers.
    cudaStream_t pipe[2] = {nullptr, nullptr};
    cudaEvent_t pipe_done[2] = {nullptr, nullptr};
    cudaEvent_t fork = nullptr;
    int pipe_device = -1;
    int slot_set = 0;
    cudaStream_t override_stream = nullptr;
    bool use_override = false;
    cudaEvent_t stream_switch = nullptr;  // orders a newly selected stream behind the work already enqueued on the old one
    // Cached device copies of host-resident blobs the current call works on: (nonce, device) pairs, pinned against eviction
    // until this thread's next call begins.
    std::vector<std::pair<uint64_t, int>> pins;
    ~ThreadCtx();  // device memory is reclaimed with the context at process exit
};
thread_local ThreadCtx t_ctx;

// ---------------------------------------------------------------- per-device state
struct DeviceState {
    unsigned int *error_word = nullptr;
};
std::mutex g_state_mutex;
DeviceState g_devices[64];

// ---------------------------------------------------------------- cache of host-resident blobs
struct CachedBlob {
    uint64_t nonce = 0, bytes = 0;
    int device = -1;
    void *dev_ptr = nullptr;
    uint64_t last_use = 0;
    int pins = 0;  // calls (of any thread) that looked this entry up and may not have enqueued their kernels yet
};
std::mutex g_cache_mutex;
std::vector<CachedBlob> g_cache;
uint64_t g_cache_clock = 0;
constexpr size_t kCacheMaxEntries = 8;

// Makes room for one more entry: frees the least recently used entry that no call has pinned. A pinned entry may belong
// to a thread that has the pointer but has not launched yet, which the device-wide synchronisation before the free
// would not cover; when every entry is pinned the cache grows past its nominal size instead. Caller holds g_cache_mutex.
void evict_for_insert() {
    if (g_cache.size() < kCacheMaxEntries) return;
    size_t victim = g_cache.size();
    for (size_t i = 0; i < g_cache.size(); ++i)
        if (g_cache[i].pins == 0 && (victim == g_cache.size() || g_cache[i].last_use < g_cache[victim].last_use)) victim = i;
    if (victim == g_cache.size()) return;
    cudaDeviceSynchronize();  // kernels already enqueued on any stream may still read the victim
    cudaFree(g_cache[victim].dev_ptr);
    g_cache.erase(g_cache.begin() + victim);
}

// Drops the pins the calling thread took during its previous call.
void release_pins() {
    if (t_ctx.pins.empty()) return;
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    for (const auto &pin : t_ctx.pins)
        for (auto &e : g_cache)
            if (e.nonce == pin.first && e.device == pin.second && e.pins > 0) { --e.pins; break; }
    t_ctx.pins.clear();
}

uint64_t fresh_nonce() {
    uint64_t t = (uint64_t)std::chrono::steady_clock::now().time_since_epoch().count();
    uint64_t c = g_nonce_counter.fetch_add(1) + 1;
    uint64_t x = t ^ (c * 0x9E3779B97F4A7C15ull) ^ (uint64_t)(uintptr_t)&t_ctx;
    x ^= x >> 31; x *= 0xBF58476D1CE4E5B9ull; x ^= x >> 29;
    return x ? x : 1;
}

ThreadCtx::~ThreadCtx() { release_pins(); }

} // namespace

// ---------------------------------------------------------------- helpers shared with other host files
void set_error(const char *fmt, const char *detail) {
    char buf[512];
    std::snprintf(buf, sizeof buf, fmt, detail ? detail : "");
    t_ctx.error = buf;
}
// Every entry point starts here: the thread's previous call has enqueued all its kernels by now, so its pins go.
void clear_error() {
    t_ctx.error.clear();
    release_pins();
}
void wait_limits_us(uint32_t (&out)[kWaitSites]) {
    for (int i = 0; i < kWaitSites; ++i) out[i] = g_wait_us[i].load();
}
cudaStream_t current_stream() { return t_ctx.use_override ? t_ctx.override_stream : t_ctx.stream; }
int current_variant() { return g_variant.load(); }
int fp6_native() { return g_fp6_native.load(); }
int sm_budget() { return g_sm_budget.load(); }

bool cuda_ok(cudaError_t e, const char *what) {
    if (e == cudaSuccess) return true;
    char buf[512];
    std::snprintf(buf, sizeof buf, "%s: %s", what, cudaGetErrorString(e));
    t_ctx.error = buf;
    cudaGetLastError();  // clear the sticky-less error state
    return false;
}

MemKind classify(const void *p) {
    if (!p) return kMemHost;
    cudaPointerAttributes attr;
    cudaError_t e = cudaPointerGetAttributes(&attr, p);
    if (e != cudaSuccess) { cudaGetLastError(); return kMemHost; }
    if (attr.type == cudaMemoryTypeDevice || attr.type == cudaMemoryTypeManaged) return kMemDevice;
    return kMemHost;
}

void *scratch(int slot, size_t bytes) {
    Scratch &s = t_ctx.slots[slot + t_ctx.slot_set * kSlotsPerSet];
    int dev = 0;
    cudaGetDevice(&dev);
    if (s.ptr && s.device == dev && s.bytes >= bytes) return s.ptr;
    if (s.ptr) {
        cudaDeviceSynchronize();  // earlier calls on any stream may still be using the old buffer
        cudaFree(s.ptr);
        s.ptr = nullptr; s.bytes = 0;
    }
    size_t want = bytes < 256 ? 256 : bytes;
    void *p = nullptr;
    if (!cuda_ok(cudaMalloc(&p, want), "cudaMalloc(staging)")) return nullptr;
    s.ptr = p; s.bytes = want; s.device = dev;
    return p;
}

size_t scratch_capacity(int slot) {
    const Scratch &s = t_ctx.slots[slot + t_ctx.slot_set * kSlotsPerSet];
    int dev = 0;
    cudaGetDevice(&dev);
    return s.ptr && s.device == dev ? s.bytes : 0;
}

unsigned int *device_error_word() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lock(g_state_mutex);
    DeviceState &st = g_devices[dev];
    if (!st.error_word) {
        unsigned int *p = nullptr;
        if (cudaMalloc(&p, 256) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        cudaMemset(p, 0, 256);
        st.error_word = p;
    }
    return st.error_word;
}

// The current device's error word if some call created it already; never allocates.
static unsigned int *existing_error_word() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    std::lock_guard<std::mutex> lock(g_state_mutex);
    return g_devices[dev].error_word;
}

// Reads one error word and, when it reports a failed wait, clears it again: the failure is reported once, to the caller
// that synchronised first, and later calls start clean (the kernels of the failed call have all retired by then).
uint32_t take_error_word(unsigned int *word) {
    if (!word) return 0;
    unsigned int v = 0;
    if (cudaMemcpy(&v, word, 4, cudaMemcpyDeviceToHost) != cudaSuccess) { cudaGetLastError(); return 0xffffffffu; }
    if (v != 0) { cudaMemset(word, 0, 4); cudaGetLastError(); }
    return v;
}

// Error status of the current device: the word of the regular entry points (when one of them has run) or else the fixed
// word of the allocation-free entry point (when that has run). Allocates nothing.
uint32_t read_device_error() {
    const uint32_t regular = take_error_word(existing_error_word());
    const uint32_t fixed = take_error_word(noalloc_error_word());
    return regular ? regular : fixed;
}

void fill_error_output(void *out, MemKind kind, uint64_t rows, uint64_t row_bytes, uint64_t stride) {
    if (!out || rows == 0 || row_bytes == 0) return;
    if (kind == kMemHost) {
        for (uint64_t r = 0; r < rows; ++r) std::memset(static_cast<uint8_t *>(out) + r * stride, 0xFF, row_bytes);
    } else {
        cudaMemset2DAsync(out, stride, 0xFF, row_bytes, rows, t_ctx.stream);
        cudaGetLastError();
    }
}

// Device pointer of a packed blob. Host-resident blobs are uploaded once and found again by nonce.
const uint8_t *resident_blob(const void *blob, MemKind kind, uint32_t magic, uint32_t dtype, uint64_t rows,
                             uint64_t depth, PackedHeader *header_out) {
    if (kind == kMemDevice) {
        // Geometry is a pure function of (dtype, rows, depth); the header is not read back, which
        // keeps device-resident calls free of synchronisation.
        PackedGeometry g = packed_geometry(dtype, rows, depth);
        if (header_out) {
            std::memset(header_out, 0, sizeof *header_out);
            header_out->magic = magic; header_out->dtype = dtype; header_out->rows = rows; header_out->depth = depth;
            header_out->rows_padded = g.rows_padded; header_out->depth_padded_bytes = g.depth_padded_bytes;
            header_out->payload_offset = g.payload_offset; header_out->norms_offset = g.norms_offset;
            header_out->total_bytes = g.total_bytes;
        }
        if (reinterpret_cast<uintptr_t>(blob) & 15u) { set_error("packed blob in device memory must be 16-byte aligned%s", ""); return nullptr; }
        return static_cast<const uint8_t *>(blob);
    }
    PackedHeader h;
    std::memcpy(&h, blob, sizeof h);
    if (h.magic != magic) { set_error("packed blob was not produced by the matching pack function of this library%s", ""); return nullptr; }
    if (h.dtype != dtype) { set_error("packed blob holds a different element type%s", ""); return nullptr; }
    if (h.rows != rows || h.depth != depth) { set_error("packed blob was packed for a different width/depth%s", ""); return nullptr; }
    PackedGeometry g = packed_geometry(dtype, rows, depth);
    if (h.total_bytes != g.total_bytes) { set_error("packed blob header is inconsistent%s", ""); return nullptr; }
    if (header_out) *header_out = h;
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    for (auto &e : g_cache)
        if (e.nonce == h.nonce && e.bytes == h.total_bytes && e.device == dev) {
            e.last_use = ++g_cache_clock;
            ++e.pins;
            t_ctx.pins.emplace_back(e.nonce, dev);
            return static_cast<const uint8_t *>(e.dev_ptr);
        }
    evict_for_insert();
    void *d = nullptr;
    if (!cuda_ok(cudaMalloc(&d, h.total_bytes), "cudaMalloc(packed blob copy)")) return nullptr;
    if (!cuda_ok(cudaMemcpyAsync(d, blob, h.total_bytes, cudaMemcpyHostToDevice, t_ctx.stream), "upload of packed blob")) { cudaFree(d); return nullptr; }
    CachedBlob e; e.nonce = h.nonce; e.bytes = h.total_bytes; e.device = dev; e.dev_ptr = d; e.last_use = ++g_cache_clock;
    e.pins = 1;
    t_ctx.pins.emplace_back(e.nonce, dev);
    g_cache.push_back(e);
    return static_cast<const uint8_t *>(d);
}

void remember_blob(uint64_t nonce, uint64_t bytes, void *dev_ptr) {
    int dev = 0;
    cudaGetDevice(&dev);
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    evict_for_insert();
    CachedBlob e; e.nonce = nonce; e.bytes = bytes; e.device = dev; e.dev_ptr = dev_ptr; e.last_use = ++g_cache_clock;
    g_cache.push_back(e);
}

__global__ void write_header_kernel(PackedHeader *dst, PackedHeader h) { *dst = h; }

// Brings a strided matrix into device memory that TMA can address (16-byte aligned base and pitch).
// Returns the device pointer and pitch; uses `slot` when a copy is needed.
const void *resident_matrix(const void *src, MemKind kind, uint64_t rows, uint64_t row_bytes, uint64_t stride,
                            int slot, int piece_mode, uint64_t *pitch_out) {
    if (rows <= 1 && stride < row_bytes) stride = row_bytes;
    const bool aligned = ((reinterpret_cast<uintptr_t>(src) & 15u) == 0) && ((stride & 15u) == 0);
    if (kind == kMemDevice && aligned && piece_mode == kPieceNone) { *pitch_out = stride; return src; }
    const int shift = piece_mode_shift(piece_mode);  // sub-byte rows come out 2 or 8 times as long
    const bool expands = shift != 0;
    uint64_t pitch = round_up(row_bytes << shift, 16);
    void *dst = scratch(slot, rows * pitch + 16 + (expands && kind == kMemHost ? rows * row_bytes + 16 : 0));
    if (!dst) return nullptr;
    if (kind == kMemHost && expands) {
        // Raw rows are uploaded behind the destination, then expanded into it.
        uint8_t *raw = static_cast<uint8_t *>(dst) + round_up(rows * pitch, 16);
        if (!cuda_ok(cudaMemcpy2DAsync(raw, row_bytes, src, stride, row_bytes, rows, cudaMemcpyHostToDevice, current_stream()), "upload of input matrix")) return nullptr;
        if (!cuda_ok(launch_restride(raw, rows, row_bytes, row_bytes, dst, pitch, piece_mode, current_stream()), "operand expansion kernel")) return nullptr;
        g_launches++;
    } else if (kind == kMemHost) {
        if (pitch != row_bytes) {
            if (!cuda_ok(cudaMemsetAsync(dst, 0, rows * pitch, current_stream()), "clear staging")) return nullptr;
        }
        if (!cuda_ok(cudaMemcpy2DAsync(dst, pitch, src, stride, row_bytes, rows, cudaMemcpyHostToDevice, current_stream()), "upload of input matrix")) return nullptr;
        if (piece_mode != kPieceNone) {  // in place: every piece is read and written by the same thread
            if (!cuda_ok(launch_restride(dst, rows, pitch, pitch, dst, pitch, piece_mode, current_stream()), "operand rewrite kernel")) return nullptr;
            g_launches++;
        }
    } else {
        if (!cuda_ok(launch_restride(src, rows, row_bytes, stride, dst, pitch, piece_mode, current_stream()), "restride kernel")) return nullptr;
        g_launches++;
    }
    *pitch_out = pitch;
    return dst;
}

namespace {

// ---------------------------------------------------------------- the three entry-point bodies
uint64_t packed_size_impl(uint32_t dt, uint64_t rows, uint64_t depth) {
    if (!dtype_supported(dt)) return 0;
    return packed_geometry(dt, rows, depth).total_bytes;
}

void pack_impl(uint32_t magic, uint32_t dt, const void *b, uint64_t rows, uint64_t depth, uint64_t stride, void *packed,
               bool inverse_norms) {
    clear_error();
    if (!dtype_supported(dt) || !packed) { set_error("pack: unsupported element type or null output%s", ""); return; }
    if (rows && depth && !b) { set_error("pack: null input%s", ""); return; }
    const PackedGeometry g = packed_geometry(dt, rows, depth);
    const MemKind out_kind = classify(packed), in_kind = classify(b);
    cudaStream_t stream = t_ctx.stream;

    PackedHeader h;
    std::memset(&h, 0, sizeof h);
    h.magic = magic; h.dtype = dt; h.element_bytes = dtype_bytes(dt); h.norm_bytes = norm_bytes(dt);
    h.rows = rows; h.depth = depth; h.rows_padded = g.rows_padded; h.depth_padded_bytes = g.depth_padded_bytes;
    h.payload_offset = g.payload_offset; h.norms_offset = g.norms_offset; h.total_bytes = g.total_bytes;
    h.nonce = fresh_nonce();

    uint8_t *dev_blob = nullptr;
    bool owned = false;
    if (out_kind == kMemDevice) {
        if (reinterpret_cast<uintptr_t>(packed) & 15u) { set_error("pack: device output must be 16-byte aligned%s", ""); return; }
        dev_blob = static_cast<uint8_t *>(packed);
    } else {
        void *d = nullptr;
        if (!cuda_ok(cudaMalloc(&d, g.total_bytes), "cudaMalloc(packed blob)")) { std::memset(packed, 0xFF, g.total_bytes); return; }
        dev_blob = static_cast<uint8_t *>(d);
        owned = true;
    }
    bool ok = true;
    const void *b_dev = b;
    uint64_t b_pitch = stride;
    if (rows && depth) {
        if (in_kind == kMemHost) {
            // Dense upload; the pack kernel reads any alignment, so no re-pitching is needed.
            uint64_t row_bytes = source_row_bytes(dt, depth);
            void *stage = scratch(kSlotA, rows * row_bytes + 16);
            ok = stage && cuda_ok(cudaMemcpy2DAsync(stage, row_bytes, b, stride < row_bytes ? row_bytes : stride, row_bytes, rows,
                                                    cudaMemcpyHostToDevice, stream), "upload of matrix to pack");
            b_dev = stage; b_pitch = row_bytes;
        }
        if (ok) {
            ok = cuda_ok(launch_pack_payload(dt, b_dev, rows, depth, b_pitch, dev_blob + g.payload_offset, g.rows_padded,
                                             g.depth_padded_bytes, piece_mode_for(dt), stream), "pack kernel");
            g_launches++;
        }
        if (ok) {
            ok = cuda_ok(launch_row_sumsq(dt, b_dev, rows, depth, b_pitch, dev_blob + g.norms_offset, false, inverse_norms, stream), "norm kernel");
            g_launches++;
        }
    } else if (ok) {
        ok = cuda_ok(cudaMemsetAsync(dev_blob + g.payload_offset, 0, g.total_bytes - g.payload_offset, stream), "clear blob");
    }
    if (ok) {
        write_header_kernel<<<1, 1, 0, stream>>>(reinterpret_cast<PackedHeader *>(dev_blob), h);
        ok = cuda_ok(cudaGetLastError(), "header kernel");
        g_launches++;
    }
    if (out_kind == kMemHost) {
        if (ok) ok = cuda_ok(cudaMemcpyAsync(packed, dev_blob, g.total_bytes, cudaMemcpyDeviceToHost, stream), "download of packed blob");
        if (ok) ok = cuda_ok(cudaStreamSynchronize(stream), "pack");
        if (ok) remember_blob(h.nonce, g.total_bytes, dev_blob);  // later calls with this host blob skip the upload
        else { if (owned) cudaFree(dev_blob); std::memset(packed, 0xFF, g.total_bytes); }
    } else if (!ok) {
        cudaMemsetAsync(dev_blob, 0xFF, g.total_bytes, stream);
        cudaGetLastError();
    } else if (in_kind == kMemHost) {
        cuda_ok(cudaStreamSynchronize(stream), "pack");
    }
}

bool ensure_pipe_streams() {
    int dev = 0;
    cudaGetDevice(&dev);
    if (t_ctx.pipe[0] && t_ctx.pipe_device == dev) return true;
    for (int s = 0; s < 2; ++s) {
        if (cudaStreamCreateWithFlags(&t_ctx.pipe[s], cudaStreamNonBlocking) != cudaSuccess) { cudaGetLastError(); t_ctx.pipe[0] = nullptr; return false; }
        if (cudaEventCreateWithFlags(&t_ctx.pipe_done[s], cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); t_ctx.pipe[0] = nullptr; return false; }
    }
    if (cudaEventCreateWithFlags(&t_ctx.fork, cudaEventDisableTiming) != cudaSuccess) { cudaGetLastError(); t_ctx.pipe[0] = nullptr; return false; }
    t_ctx.pipe_device = dev;
    return true;
}

// One packed call on `stream` without the final synchronisation: stages A and C as needed, launches the
// kernels, copies C back. Returns false (error text set) on failure.
// `first_column` (a multiple of 256) selects the packed rows [first_column, first_column + n) of the blob; `c` then points at
// the cell of the first of those columns.
bool packed_core(uint32_t dt, int epilogue, const void *a, MemKind a_kind, const uint8_t *blob, const PackedHeader &h,
                 unsigned int *err, void *c, MemKind c_kind, uint64_t m, uint64_t n, uint64_t k, uint64_t a_stride,
                 uint64_t c_stride, cudaStream_t stream, uint64_t first_column = 0) {
    // Packed rows are stored in blocks of 128 (tensor-core types: one chunk column of depth_padded_bytes / 128 chunks per
    // block) or one after the other (f32 / f64), so a column range is a byte offset into the payload and the norms.
    const uint8_t *payload = blob + h.payload_offset + first_column * h.depth_padded_bytes;
    const uint8_t *norms = blob + h.norms_offset + first_column * norm_bytes(dt);
    const uint32_t out_bytes = dot_out_bytes(dt);
    const uint64_t c_row_bytes = n * out_bytes;
    // Output: in place when it is device memory with 4-byte aligned rows, else a dense device copy.
    uint8_t *c_dev = static_cast<uint8_t *>(c);
    uint64_t c_pitch = c_stride;
    const bool c_direct = c_kind == kMemDevice && (reinterpret_cast<uintptr_t>(c) % out_bytes) == 0;
    if (!c_direct) {
        c_pitch = round_up(c_row_bytes, 16);
        c_dev = static_cast<uint8_t *>(scratch(kSlotC, m * c_pitch));
        if (!c_dev) return false;
    }
    bool ok = true;
    if (k == 0) {
        ok = cuda_ok(cudaMemset2DAsync(c_dev, c_pitch, 0, c_row_bytes, m, stream), "clear result");
    } else if (is_cuda_core_dtype(dt)) {
        const uint32_t eb = dtype_bytes(dt);
        const void *a_dev = a;
        uint64_t a_pitch = a_stride;
        if (a_kind == kMemHost || (reinterpret_cast<uintptr_t>(a) & (eb - 1)) || (a_stride & (eb - 1))) {
            a_dev = resident_matrix(a, a_kind, m, k * eb, a_stride, kSlotA, kPieceNone, &a_pitch);
            if (!a_dev) return false;
        }
        double *a_norms = nullptr;
        if (epilogue != kEpiDot) {
            a_norms = static_cast<double *>(scratch(kSlotNorms, m * 8));
            ok = a_norms && cuda_ok(launch_row_sumsq(dt, a_dev, m, k, a_pitch, a_norms, false, false, stream), "row norm kernel");
            g_launches++;
        }
        if (ok && dt == kF32) {
            ok = cuda_ok(launch_gemm_f32(epilogue, static_cast<const float *>(a_dev), a_pitch,
                                         reinterpret_cast<const float *>(payload), h.depth_padded_bytes,
                                         reinterpret_cast<const double *>(norms), a_norms,
                                         reinterpret_cast<double *>(c_dev), c_pitch, m, n, k, stream), "f32 GEMM kernel");
            g_launches++;
        } else if (ok) {
            ok = cuda_ok(launch_gemm_f64(epilogue, static_cast<const double *>(a_dev), a_pitch,
                                         reinterpret_cast<const double *>(payload), h.depth_padded_bytes,
                                         reinterpret_cast<const double *>(norms), a_norms,
                                         reinterpret_cast<double *>(c_dev), c_pitch, m, n, k, stream), "f64 GEMM kernel");
            g_launches++;
        }
    } else {
        // FP6 operands are rewritten for the tensor cores (see transform_piece); their norms are taken
        // from the caller's bytes first.
        const int piece_mode = piece_mode_for(dt);
        uint64_t a_pitch = 0;
        const void *a_dev = nullptr;
        float *a_norms = nullptr;
        if (epilogue != kEpiDot) {
            a_norms = static_cast<float *>(scratch(kSlotNorms, m * 4));
            if (!a_norms) return false;
        }
        if (is_subbyte(dt)) {
            // Sub-byte rows are expanded to one byte per value on their way into the staging buffer; norms come from that copy.
            a_dev = resident_matrix(a, a_kind, m, source_row_bytes(dt, k), a_stride, kSlotA, piece_mode, &a_pitch);
            if (!a_dev) return false;
            if (a_norms) {
                ok = cuda_ok(launch_row_sumsq(operand_dtype(dt), a_dev, m, operand_depth(dt, k), a_pitch, a_norms, true, false, stream), "row norm kernel");
                g_launches++;
            }
        } else if (piece_mode == kPieceNone) {
            a_dev = resident_matrix(a, a_kind, m, k * dtype_bytes(dt), a_stride, kSlotA, kPieceNone, &a_pitch);
            if (!a_dev) return false;
            if (a_norms) {
                ok = cuda_ok(launch_row_sumsq(dt, a_dev, m, k, a_pitch, a_norms, true, false, stream), "row norm kernel");
                g_launches++;
            }
        } else if (a_kind == kMemDevice) {
            if (a_norms) {
                ok = cuda_ok(launch_row_sumsq(dt, a, m, k, a_stride, a_norms, true, false, stream), "row norm kernel");
                g_launches++;
            }
            a_dev = resident_matrix(a, a_kind, m, k, a_stride, kSlotA, piece_mode, &a_pitch);
            if (!a_dev) return false;
        } else {
            a_dev = resident_matrix(a, a_kind, m, k, a_stride, kSlotA, kPieceNone, &a_pitch);
            if (!a_dev) return false;
            if (a_norms) {
                ok = cuda_ok(launch_row_sumsq(dt, a_dev, m, k, a_pitch, a_norms, true, false, stream), "row norm kernel");
                g_launches++;
            }
            // In place: each 16-byte piece is read and written by the same thread.
            ok = ok && cuda_ok(launch_restride(a_dev, m, a_pitch, a_pitch, const_cast<void *>(a_dev), a_pitch, piece_mode, stream), "operand rewrite kernel");
            g_launches++;
        }
        if (ok) {
            GemmArgs g;
            g.dtype = operand_dtype(dt); g.epilogue = epilogue; g.a = a_dev; g.a_stride = a_pitch;
            g.b_payload = payload; g.b_norms = norms; g.a_norms = a_norms;
            g.c = c_dev; g.c_stride = c_pitch; g.m = m; g.n = n; g.k = operand_depth(dt, k);
            g.depth_padded_bytes = h.depth_padded_bytes; g.error_word = err; g.variant = g_variant.load();
            ok = cuda_ok(launch_gemm_tc(g, stream), "tensor-core GEMM kernel");
            g_launches++;
        }
    }
    if (ok && !c_direct) {
        cudaMemcpyKind kind = c_kind == kMemHost ? cudaMemcpyDeviceToHost : cudaMemcpyDeviceToDevice;
        ok = cuda_ok(cudaMemcpy2DAsync(c, c_stride < c_row_bytes ? c_row_bytes : c_stride, c_dev, c_pitch, c_row_bytes, m, kind, stream), "download of result");
    }
    return ok;
}

// `first_column` / `column_count` restrict the call to a range of packed rows (columns of the result); `c` always points at
// cell (0, 0) of the full result. column_count == ~0 means "all of them".
void packed_impl(uint32_t dt, int epilogue, const void *a, const void *b_packed, void *c, uint64_t m, uint64_t n,
                 uint64_t k, uint64_t a_stride, uint64_t c_stride, uint64_t first_column = 0, uint64_t column_count = ~0ull) {
    clear_error();
    const uint32_t out_bytes = dot_out_bytes(dt);  // distances share the cell width of the dots
    const uint64_t width = n;  // packed rows in the blob
    if (column_count != ~0ull) {
        if (first_column % kRowPad || first_column > n || column_count > n - first_column) {
            set_error("packed columns: the first column must be a multiple of 256 and the range must lie inside the packed matrix%s", "");
            return;
        }
        n = column_count;
        c = c ? static_cast<uint8_t *>(c) + first_column * out_bytes : c;
    }
    const uint64_t c_row_bytes = n * out_bytes;
    if (m == 0 || n == 0) return;
    const MemKind c_kind = classify(c);
    auto fail = [&]() { fill_error_output(c, c_kind, m, c_row_bytes, c_stride < c_row_bytes ? c_row_bytes : c_stride); };
    if (!dtype_supported(dt) || !a || !b_packed || !c) { set_error("packed: unsupported element type or null pointer%s", ""); fail(); return; }
    if (m > 1 && c_stride < c_row_bytes) { set_error("packed: c_stride is smaller than a row of the result%s", ""); fail(); return; }
    if (c_stride % out_bytes) { set_error("packed: c_stride must be a multiple of the output cell size%s", ""); fail(); return; }
    cudaStream_t stream = t_ctx.stream;
    const MemKind a_kind = classify(a), b_kind = classify(b_packed);

    PackedHeader h;
    const uint8_t *blob = resident_blob(b_packed, b_kind, kMagicDots, dt, width, k, &h);
    if (!blob) { fail(); return; }
    unsigned int *err = device_error_word();
    if (!err) { set_error("could not allocate the device error word%s", ""); fail(); return; }

    bool ok = true;
    // Large host-to-host calls are cut into row blocks that alternate between two private streams, so the
    // upload of one block, the kernels of another and the download of a third overlap.
    constexpr uint64_t kPipeRows = 1024;
    const bool pipelined = a_kind == kMemHost && c_kind == kMemHost && k > 0 && m >= 2 * kPipeRows && ensure_pipe_streams();
    if (pipelined) {
        ok = cuda_ok(cudaEventRecord(t_ctx.fork, stream), "pipeline fork");
        for (int s = 0; s < 2 && ok; ++s) ok = cuda_ok(cudaStreamWaitEvent(t_ctx.pipe[s], t_ctx.fork, 0), "pipeline fork");
        // The first blocks are short so that the download of results (the longest leg of a host-to-host call) starts
        // almost at once; after that, blocks of kPipeRows rows keep the copies long enough to run at full PCIe speed.
        int block = 0;
        uint64_t rows = 0;
        for (uint64_t r0 = 0; r0 < m && ok; r0 += rows, ++block) {
            const uint64_t ramp = block < 2 ? kPipeRows / 4 : block == 2 ? kPipeRows / 2 : kPipeRows;
            rows = m - r0 < ramp ? m - r0 : ramp;
            t_ctx.slot_set = block & 1;
            t_ctx.use_override = true;
            t_ctx.override_stream = t_ctx.pipe[block & 1];
            ok = packed_core(dt, epilogue, static_cast<const uint8_t *>(a) + r0 * a_stride, a_kind, blob, h, err,
                             static_cast<uint8_t *>(c) + r0 * c_stride, c_kind, rows, n, k, a_stride, c_stride, t_ctx.pipe[block & 1], first_column);
        }
        t_ctx.slot_set = 0;
        t_ctx.use_override = false;
        for (int s = 0; s < 2; ++s) {
            bool joined = cuda_ok(cudaEventRecord(t_ctx.pipe_done[s], t_ctx.pipe[s]), "pipeline join") &&
                          cuda_ok(cudaStreamWaitEvent(stream, t_ctx.pipe_done[s], 0), "pipeline join");
            ok = ok && joined;
        }
    } else {
        ok = packed_core(dt, epilogue, a, a_kind, blob, h, err, c, c_kind, m, n, k, a_stride, c_stride, stream, first_column);
    }
    const bool must_sync = a_kind == kMemHost || b_kind == kMemHost || c_kind == kMemHost;
    if (ok && must_sync) {
        ok = cuda_ok(cudaStreamSynchronize(stream), "packed call");
        if (ok) {
            uint32_t w = read_device_error();
            if (w) { char buf[64]; std::snprintf(buf, sizeof buf, "0x%08x", w); set_error("a pipeline wait inside the GEMM kernel gave up (error word %s)", buf); ok = false; }
        }
    }
    if (!ok) fail();
}

} // namespace

void maxsim_pack_impl(uint32_t dt, const void *vectors, uint64_t count, uint64_t depth, uint64_t stride, void *packed) {
    if (dt != kBF16 && dt != kF16 && dt != kF32) { clear_error(); set_error("maxsim_pack: unsupported element type%s", ""); return; }
    pack_impl(kMagicMaxsim, dt, vectors, count, depth, stride, packed, true);
}

} // namespace nkb

using namespace nkb;

extern "C" {

#define NKB_DEFINE_PACKED_FAMILY(T, DT)                                                                                \
    NKB_API nk_size_t nk_dots_packed_size_##T(nk_size_t width, nk_size_t depth) { return packed_size_impl(DT, width, depth); } \
    NKB_API void nk_dots_pack_##T(void const *b, nk_size_t width, nk_size_t depth, nk_size_t b_stride, void *b_packed) { \
        pack_impl(kMagicDots, DT, b, width, depth, b_stride, b_packed, false);                                        \
    }                                                                                                                  \
    NKB_API void nk_dots_packed_##T(void const *a, void const *b_packed, void *c, nk_size_t height, nk_size_t width,   \
                                    nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride) {                         \
        packed_impl(DT, kEpiDot, a, b_packed, c, height, width, depth, a_stride, c_stride);                            \
    }                                                                                                                  \
    NKB_API void nk_angulars_packed_##T(void const *a, void const *b_packed, void *c, nk_size_t height,                \
                                        nk_size_t width, nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride) {    \
        packed_impl(DT, kEpiAngular, a, b_packed, c, height, width, depth, a_stride, c_stride);                        \
    }                                                                                                                  \
    NKB_API void nk_euclideans_packed_##T(void const *a, void const *b_packed, void *c, nk_size_t height,              \
                                          nk_size_t width, nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride) {  \
        packed_impl(DT, kEpiEuclidean, a, b_packed, c, height, width, depth, a_stride, c_stride);                      \
    }

NKB_DEFINE_PACKED_FAMILY(i8, kI8)
NKB_DEFINE_PACKED_FAMILY(u8, kU8)
NKB_DEFINE_PACKED_FAMILY(bf16, kBF16)
NKB_DEFINE_PACKED_FAMILY(f16, kF16)
NKB_DEFINE_PACKED_FAMILY(e4m3, kE4M3)
NKB_DEFINE_PACKED_FAMILY(e5m2, kE5M2)
NKB_DEFINE_PACKED_FAMILY(e2m3, kE2M3)
NKB_DEFINE_PACKED_FAMILY(e3m2, kE3M2)
NKB_DEFINE_PACKED_FAMILY(f32, kF32)
NKB_DEFINE_PACKED_FAMILY(i4, kI4)
NKB_DEFINE_PACKED_FAMILY(u4, kU4)
NKB_DEFINE_PACKED_FAMILY(f64, kF64)

// One-bit vectors: the "dot" is the AND-popcount, the packed norms are population counts, and the two set distances are
// epilogues of the same product (include/numkong/sets.h:69-117, generators include/numkong/sets/serial.h:19-39).
NKB_API nk_size_t nk_dots_packed_size_u1(nk_size_t width, nk_size_t depth) { return packed_size_impl(kU1, width, depth); }
NKB_API void nk_dots_pack_u1(void const *b, nk_size_t width, nk_size_t depth, nk_size_t b_stride, void *b_packed) {
    pack_impl(kMagicDots, kU1, b, width, depth, b_stride, b_packed, false);
}
NKB_API void nk_dots_packed_u1(void const *a, void const *b_packed, void *c, nk_size_t height, nk_size_t width, nk_size_t depth,
                               nk_size_t a_stride, nk_size_t c_stride) {
    packed_impl(kU1, kEpiDot, a, b_packed, c, height, width, depth, a_stride, c_stride);
}
NKB_API void nk_hammings_packed_u1(void const *v, void const *q_packed, void *result, nk_size_t rows, nk_size_t cols, nk_size_t d,
                                   nk_size_t v_stride, nk_size_t r_stride) {
    packed_impl(kU1, kEpiHamming, v, q_packed, result, rows, cols, d, v_stride, r_stride);
}
NKB_API void nk_jaccards_packed_u1(void const *v, void const *q_packed, void *result, nk_size_t rows, nk_size_t cols, nk_size_t d,
                                   nk_size_t v_stride, nk_size_t r_stride) {
    packed_impl(kU1, kEpiJaccard, v, q_packed, result, rows, cols, d, v_stride, r_stride);
}

NKB_API void nkb_dots_packed_columns(uint32_t dtype, void const *a, void const *b_packed, void *c, nk_size_t height, nk_size_t width,
                                     nk_size_t depth, nk_size_t a_stride, nk_size_t c_stride, nk_size_t first_column,
                                     nk_size_t column_count) {
    if (!dtype_supported(dtype)) { clear_error(); set_error("packed columns: unsupported element type%s", ""); return; }
    packed_impl(dtype, kEpiDot, a, b_packed, c, height, width, depth, a_stride, c_stride, first_column, column_count);
}

NKB_API char const *nkb_last_error(void) { return t_ctx.error.c_str(); }
NKB_API void nkb_set_stream(void *cuda_stream) {
    cudaStream_t next = static_cast<cudaStream_t>(cuda_stream);
    if (next == t_ctx.stream) return;
    // The thread's staging buffers (row norms, re-strided operands, candidate lists) pass from call to call without
    // ordering of their own, so the new stream is put behind everything this thread has enqueued on the old one.
    cudaStreamCaptureStatus old_capture = cudaStreamCaptureStatusNone, new_capture = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(t_ctx.stream, &old_capture);
    cudaStreamIsCapturing(next, &new_capture);
    cudaGetLastError();
    if (old_capture == cudaStreamCaptureStatusNone && new_capture == cudaStreamCaptureStatusNone) {
        if (!t_ctx.stream_switch && cudaEventCreateWithFlags(&t_ctx.stream_switch, cudaEventDisableTiming) != cudaSuccess) t_ctx.stream_switch = nullptr;
        if (t_ctx.stream_switch && cudaEventRecord(t_ctx.stream_switch, t_ctx.stream) == cudaSuccess)
            cudaStreamWaitEvent(next, t_ctx.stream_switch, 0);
        cudaGetLastError();
    }
    t_ctx.stream = next;
}
NKB_API uint32_t nkb_synchronize(void) {
    clear_error();
    if (!cuda_ok(cudaStreamSynchronize(t_ctx.stream), "nkb_synchronize")) return 0xffffffffu;
    return read_device_error();
}
NKB_API void nkb_set_wait_limit_ns(int site, uint64_t nanoseconds) {
    uint64_t us = nanoseconds == 0 ? kDefaultWaitLimitUs : (nanoseconds + 999) / 1000;
    if (us > kDefaultWaitLimitUs) us = kDefaultWaitLimitUs;
    for (int i = 1; i < kWaitSites; ++i)
        if (site == 0 || site == i) g_wait_us[i].store((uint32_t)us);
}
NKB_API int nkb_test_set_error_word(int which, uint32_t value) {
    unsigned int *word = which == 0 ? device_error_word() : noalloc_error_word();
    if (!word) return 1;
    return cudaMemcpy(word, &value, 4, cudaMemcpyHostToDevice) == cudaSuccess ? 0 : 2;
}
NKB_API uint64_t nkb_cached_blob_count(void) {
    std::lock_guard<std::mutex> lock(g_cache_mutex);
    return g_cache.size();
}
NKB_API uint64_t nkb_launch_count(void) { return g_launches.load(); }
NKB_API void nkb_set_gemm_variant(int variant) { g_variant.store(variant); }
NKB_API void nkb_set_accumulation_span(int stages) {
    const int span = stages < 0 ? 0 : (stages > 255 ? 255 : stages);
    g_variant.store((g_variant.load() & ~0xff00) | (span << 8));
}
NKB_API void nkb_set_fp6_native(int native) { g_fp6_native.store(native ? 1 : 0); }
NKB_API void nkb_set_sm_budget(int sms) { g_sm_budget.store(sms < 0 ? 0 : sms); }
NKB_API void nkb_release_caches(void) {
    cudaDeviceSynchronize();
    {
        std::lock_guard<std::mutex> lock(g_cache_mutex);
        for (auto &e : g_cache) cudaFree(e.dev_ptr);
        g_cache.clear();
    }
    for (auto &s : t_ctx.slots) {
        if (s.ptr) cudaFree(s.ptr);
        s = Scratch();
    }
    cudaGetLastError();
}

NKB_API uint64_t nk_capabilities(void) {
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) { cudaGetLastError(); return 0; }
    int dev = 0, major = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
    return major == 10 ? NKB_CAPABILITY_B200 : 0;
}
NKB_API int nk_configure_thread(uint64_t) { return 1; }

} // extern "C"
