// One-to-all delivery of a packed matrix through the NVSwitch: nkb_multicast_store(multicast_dst, src, bytes).
//
// The multi-GPU form of the packed product splits the rows of A between the GPUs and gives every GPU the whole packed B
// (NumKong's own threading model: "pass a slice of A's rows and the full packed B", README.md:199-212 of the reference). The
// blob is position independent, so delivering it is a byte copy. A ring or tree broadcast sends the bytes hop by hop; with
// an NVLink multicast mapping (cuMulticast*: one virtual address bound to the same buffer on every GPU) the sender issues
// each 16 bytes ONCE with `multimem.st` and the switch writes them into every GPU's copy, so the sender's link carries the
// blob once, whatever the number of receivers.
//
// The caller owns the mapping (torch.distributed._symmetric_memory or its own cuMulticast calls), passes the multicast
// address of the destination, and orders the receivers behind the copy with nkb_peer_barrier on their streams. Nothing
// waits in the copy kernel and nothing is allocated.
//
// nkb_peer_barrier(peer_flags, world, rank, epoch): one small kernel per GPU. Thread p stores `epoch` into slot `rank` of
// GPU p's flag buffer (a peer store, released at system scope behind everything this GPU's stream has finished) and then
// polls slot p of the GPU's own buffer until it holds `epoch` or more. Epochs only grow, so the flags are never reset and
// a GPU that is one barrier ahead cannot confuse one that is still polling. The poll is bounded (wait site 8).
#include <cstdint>
#include <cuda_runtime.h>
#include "nkb_host.h"
#include "nkb_ptx.cuh"
#include "../../include/numkong_b200.h"

namespace nkb {
namespace {

constexpr int kMulticastThreads = 256;
constexpr int kMulticastUnroll = 4;  // 16-byte loads a thread keeps in flight

__device__ __forceinline__ void multimem_store(uint4 *multicast_dst, uint4 v) {
    asm volatile("multimem.st.weak.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(multicast_dst), "f"(__uint_as_float(v.x)),
                 "f"(__uint_as_float(v.y)), "f"(__uint_as_float(v.z)), "f"(__uint_as_float(v.w))
                 : "memory");
}

__global__ void __launch_bounds__(kMulticastThreads) multicast_store_kernel(const uint4 *__restrict__ src, uint4 *multicast_dst, uint64_t pieces) {
    const uint64_t stride = (uint64_t)gridDim.x * kMulticastThreads;
    uint64_t i = (uint64_t)blockIdx.x * kMulticastThreads + threadIdx.x;
    for (; i + (kMulticastUnroll - 1) * stride < pieces; i += kMulticastUnroll * stride) {
        uint4 v[kMulticastUnroll];
#pragma unroll
        for (int u = 0; u < kMulticastUnroll; ++u) v[u] = __ldg(src + i + u * stride);
#pragma unroll
        for (int u = 0; u < kMulticastUnroll; ++u) multimem_store(multicast_dst + i + u * stride, v[u]);
    }
    for (; i < pieces; i += stride) multimem_store(multicast_dst + i, __ldg(src + i));
}

constexpr int kMaxPeers = 16;
struct PeerFlags { uint32_t *flags[kMaxPeers]; };

__global__ void peer_barrier_kernel(PeerFlags peers, int world, int rank, uint32_t epoch, unsigned int *error_word, uint32_t limit_us) {
    const int p = threadIdx.x;
    if (p >= world) return;
    __threadfence_system();
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(peers.flags[p] + rank), "r"(epoch) : "memory");
    const uint32_t *mine = peers.flags[rank] + p;
    const uint64_t start = global_timer_ns();
    while (true) {
        uint32_t seen;
        asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if ((int32_t)(seen - epoch) >= 0) break;
        if (global_timer_ns() - start > (uint64_t)limit_us * 1000ull) {
            atomicCAS(error_word, 0u, 0x80000000u | (8u << 16) | (uint32_t)p);
            break;
        }
        __nanosleep(100);
    }
}

} // namespace
} // namespace nkb

using namespace nkb;

NKB_API int nkb_multicast_store(void *multicast_dst, void const *src, nk_size_t bytes, int blocks) {
    clear_error();
    if (bytes == 0) return 0;
    if (!multicast_dst || !src || (reinterpret_cast<uintptr_t>(multicast_dst) & 15u) || (reinterpret_cast<uintptr_t>(src) & 15u) || (bytes & 15u)) {
        set_error("multicast store: addresses and size must be multiples of 16 bytes%s", "");
        return 1;
    }
    if (classify(src) != kMemDevice) {
        set_error("multicast store: the source must be device memory%s", "");
        return 2;
    }
    if (blocks <= 0) blocks = 64;
    if (blocks > 1024) blocks = 1024;
    multicast_store_kernel<<<blocks, kMulticastThreads, 0, current_stream()>>>(static_cast<const uint4 *>(src), static_cast<uint4 *>(multicast_dst), bytes / 16);
    g_launches++;
    return cuda_ok(cudaGetLastError(), "multicast store kernel") ? 0 : 3;
}

NKB_API int nkb_peer_barrier(void *const *peer_flags, int world, int rank, uint32_t epoch) {
    clear_error();
    if (!peer_flags || world < 1 || world > kMaxPeers || rank < 0 || rank >= world) {
        set_error("peer barrier: 1 <= world <= 16 and 0 <= rank < world%s", "");
        return 1;
    }
    PeerFlags peers = {};
    for (int p = 0; p < world; ++p) {
        if (!peer_flags[p] || (reinterpret_cast<uintptr_t>(peer_flags[p]) & 3u)) {
            set_error("peer barrier: a flag buffer address is null or misaligned%s", "");
            return 1;
        }
        peers.flags[p] = static_cast<uint32_t *>(peer_flags[p]);
    }
    unsigned int *error_word = device_error_word();
    if (!error_word) return 2;
    uint32_t limits[kWaitSites];
    wait_limits_us(limits);
    peer_barrier_kernel<<<1, 32, 0, current_stream()>>>(peers, world, rank, epoch, error_word, limits[8]);
    g_launches++;
    return cuda_ok(cudaGetLastError(), "peer barrier kernel") ? 0 : 3;
}
