// Batched angular distances for callers that are not allowed to allocate device memory.
//
// The regular entry points (nk_angulars_packed_<t>) keep a per-thread scratch vector for the squared
// norms of the rows of A, obtained with cudaMalloc on first use and grown on demand. Some callers
// cannot tolerate that: code running between cudaStreamBeginCapture and cudaStreamEndCapture (an
// allocation is illegal there), real-time loops and services with a fixed memory budget where a
// cudaMalloc in the middle of serving is a latency spike or an out-of-memory risk, and plug-ins living
// inside a host application that owns the whole device heap through its own pool allocator.
//
// nkb_angulars_packed_noalloc does the same computation with the row-norm scratch (and the error word of
// the pipeline waits) in fixed device arrays that are part of this library's image. The price is a
// hard limit on the number of rows per call and one shared scratch per GPU.
//
// How such a caller learns that a pipeline wait gave up: nkb_synchronize() reads this fixed error word as well
// (a 4-byte copy from an address cached at set-up; it creates nothing), returns it when it is non-zero and
// clears it. A process that only ever uses this entry point therefore never allocates device memory here.
#include <cstdio>
#include <mutex>

#include "../../include/numkong_b200.h"
#include "nkb_host.h"

namespace nkb {
namespace {

// Every GPU that loads the library holds these 256 KiB + 256 B until the process exits.
constexpr uint64_t kNoAllocMaxRows = NKB_NOALLOC_MAX_ROWS;
static __device__ __align__(256) float g_noalloc_row_norms[kNoAllocMaxRows];
static __device__ __align__(256) unsigned int g_noalloc_error_word[64];

struct DeviceAddresses {
    float *row_norms = nullptr;
    unsigned int *error_word = nullptr;
};
std::mutex g_noalloc_mutex;
DeviceAddresses g_noalloc_addresses[64];

// In host code the names of the arrays above are only handles; a kernel needs the device addresses, which
// the runtime hands out per device. Looked up once per device, with that device current.
bool noalloc_setup(DeviceAddresses &out) {
    int dev = 0;
    if (!cuda_ok(cudaGetDevice(&dev), "cudaGetDevice")) return false;
    if (dev < 0 || dev >= 64) { set_error("noalloc: device ordinal out of range%s", ""); return false; }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    DeviceAddresses &slot = g_noalloc_addresses[dev];
    if (!slot.row_norms) {
        void *norms = nullptr, *word = nullptr;
        if (!cuda_ok(cudaGetSymbolAddress(&norms, g_noalloc_row_norms), "cudaGetSymbolAddress(row norms)")) return false;
        if (!cuda_ok(cudaGetSymbolAddress(&word, g_noalloc_error_word), "cudaGetSymbolAddress(error word)")) return false;
        // The error word must start at zero; the norms are fully rewritten by every call before they are read.
        if (!cuda_ok(cudaMemset(word, 0, sizeof(unsigned int) * 64), "clear error word")) return false;
        slot.row_norms = static_cast<float *>(norms);
        slot.error_word = static_cast<unsigned int *>(word);
    }
    out = slot;
    return true;
}

} // namespace

// For nkb_synchronize(): where this device's fixed error word lives, once the entry point below has set it up; nullptr
// before that. A lookup in a table the set-up filled in - no runtime call, no allocation.
unsigned int *noalloc_error_word() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { cudaGetLastError(); return nullptr; }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    return g_noalloc_addresses[dev].error_word;
}

} // namespace nkb

using namespace nkb;

extern "C" NKB_API int nkb_angulars_packed_noalloc(uint32_t dtype, void const *a, void const *b_packed, void *c,
                                                   nk_size_t height, nk_size_t width, nk_size_t depth,
                                                   nk_size_t a_stride, nk_size_t c_stride) {
    clear_error();
    if (dtype != kBF16 && dtype != kF16 && dtype != kE4M3 && dtype != kE5M2 && dtype != kI8 && dtype != kU8) {
        set_error("noalloc: supported element types are bf16, f16, e4m3, e5m2, i8, u8%s", "");
        return 1;
    }
    if (height > kNoAllocMaxRows) {
        char buf[64];
        std::snprintf(buf, sizeof buf, "%llu", (unsigned long long)kNoAllocMaxRows);
        set_error("noalloc: at most %s rows of A per call (fixed scratch); split the call by rows", buf);
        return 2;
    }
    if (height == 0 || width == 0) return 0;
    if (!a || !b_packed || !c || depth == 0) { set_error("noalloc: null pointer or zero depth%s", ""); return 3; }
    if (classify(a) != kMemDevice || classify(b_packed) != kMemDevice || classify(c) != kMemDevice) {
        set_error("noalloc: A, the packed blob and C must all be device (or managed) memory - staging host memory would allocate%s", "");
        return 4;
    }
    if ((reinterpret_cast<uintptr_t>(a) & 15u) || (a_stride & 15u) || (reinterpret_cast<uintptr_t>(b_packed) & 15u) ||
        (reinterpret_cast<uintptr_t>(c) & 3u) || (c_stride & 3u) || (height > 1 && c_stride < width * 4)) {
        set_error("noalloc: A and the blob must be 16-byte aligned (A's stride too), C 4-byte aligned with c_stride >= width*4%s", "");
        return 5;
    }
    DeviceAddresses addr;
    if (!noalloc_setup(addr)) return 6;
    cudaStream_t stream = current_stream();
    const PackedGeometry g = packed_geometry(dtype, width, depth);
    const uint8_t *blob = static_cast<const uint8_t *>(b_packed);
    if (!cuda_ok(launch_row_sumsq(dtype, a, height, depth, a_stride, addr.row_norms, true, false, stream), "row norm kernel")) return 7;
    g_launches++;
    GemmArgs args;
    args.dtype = dtype; args.epilogue = kEpiAngular; args.a = a; args.a_stride = a_stride;
    args.b_payload = blob + g.payload_offset; args.b_norms = blob + g.norms_offset; args.a_norms = addr.row_norms;
    args.c = c; args.c_stride = c_stride; args.m = height; args.n = width; args.k = depth;
    args.depth_padded_bytes = g.depth_padded_bytes; args.error_word = addr.error_word; args.variant = current_variant();
    if (!cuda_ok(launch_gemm_tc(args, stream), "tensor-core GEMM kernel")) return 8;
    g_launches++;
    return 0;
}
