// Host-side helpers shared by the files that implement the exported entry points.
#pragma once
#include <atomic>
#include "nkb_internal.h"

namespace nkb {

enum MemKind : int { kMemHost = 0, kMemDevice = 1 };

// Per-thread staging buffers (grow-only device allocations).
enum ScratchSlot : int { kSlotA = 0, kSlotC = 1, kSlotNorms = 2, kSlotAux = 3, kSlotAux2 = 4, kSlotsPerSet = 5, kScratchSlots = 10 };

extern std::atomic<uint64_t> g_launches;

void set_error(const char *fmt, const char *detail);
void clear_error();
bool cuda_ok(cudaError_t e, const char *what);
cudaStream_t current_stream();
int current_variant();

// Device/managed memory is used in place; everything else is treated as host memory.
MemKind classify(const void *p);
void *scratch(int slot, size_t bytes);
// Bytes the calling thread's staging buffer `slot` already holds on the current device (0: none yet).
size_t scratch_capacity(int slot);
unsigned int *device_error_word();
// Error status of the current device (0 = no bounded wait gave up since the last report); a reported failure is cleared.
uint32_t read_device_error();
// Device address of the allocation-free entry point's fixed error word on the current device, or nullptr when that entry
// point has not run there yet (nkb_noalloc.cu).
unsigned int *noalloc_error_word();
void fill_error_output(void *out, MemKind kind, uint64_t rows, uint64_t row_bytes, uint64_t stride);

const uint8_t *resident_blob(const void *blob, MemKind kind, uint32_t magic, uint32_t dtype, uint64_t rows,
                             uint64_t depth, PackedHeader *header_out);
void remember_blob(uint64_t nonce, uint64_t bytes, void *dev_ptr);
const void *resident_matrix(const void *src, MemKind kind, uint64_t rows, uint64_t row_bytes, uint64_t stride,
                            int slot, int piece_mode, uint64_t *pitch_out);

} // namespace nkb
