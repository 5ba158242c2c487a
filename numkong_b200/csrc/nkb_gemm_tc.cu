// Packed GEMM C = A * B^T on the 5th-generation tensor cores (tcgen05), with the
// dot / angular / euclidean epilogues fused into the TMEM read-out.
//
// Replaces the depth loops of NumKong's nk_dots_packed_<t> (include/numkong/dots/serial.h:520-1085,
// AMX form include/numkong/dots/sapphireamx.h:981-) and the second pass of
// nk_angulars_packed_<t> / nk_euclideans_packed_<t> (include/numkong/dots/serial.h:2756-2800).
//
// One persistent CTA per SM, six warps:
//   warp 0      producer: TMA tiled loads of A (128-byte swizzle) and untiled bulk copies of the
//               pre-swizzled B chunks into a multi-stage shared-memory ring (mbarrier full/empty pairs)
//   warp 1      allocates TMEM and issues tcgen05.mma from one thread; accumulators live in TMEM,
//               two of them, so reading one out overlaps the MMAs that fill the other
//   warps 2..9  epilogue: tcgen05.ld of their 32-lane quarter and column half, f32/i32 summation of the
//               accumulation spans in registers, finalisation, global stores
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
};

template <int kBN, int kStages>
struct SmemPlan {
    static constexpr int kABytes = kBM * kBKBytes;
    static constexpr int kBBytes = kBN * kBKBytes;
    static constexpr int kStageBytes = kABytes + kBBytes;
    static constexpr int kBarrierOffset = kStages * kStageBytes;
    static constexpr int kBarrierBytes = 256;
    static constexpr int kTotal = kBarrierOffset + kBarrierBytes + 1024;  // + slack for manual 1024-byte alignment
};

__device__ __forceinline__ void tile_coords(uint32_t tile, uint32_t tiles_m, uint32_t tiles_n, uint32_t &mt, uint32_t &nt) {
    uint32_t per_group = kGroupM * tiles_n;
    uint32_t group = tile / per_group;
    uint32_t first_m = group * kGroupM;
    uint32_t group_rows = min(tiles_m - first_m, (uint32_t)kGroupM);
    uint32_t in_group = tile % per_group;
    mt = first_m + in_group % group_rows;
    nt = in_group / group_rows;
}

template <int kEpi>
__device__ __forceinline__ float finalize(float dot, float a_norm, float b_norm) {
    if constexpr (kEpi == kEpiAngular) {
        // NumKong batched rule (include/numkong/spatial/serial.h:257-269): zero norm product gives
        // 0 when the dot is 0 and 1 otherwise; the result is clamped at 0.
        float product = a_norm * b_norm;
        if (product > 0.0f) {
            float r = rsqrtf(product);
            r = r * (1.5f - 0.5f * product * r * r);
            float v = 1.0f - dot * r;
            return v > 0.0f ? v : 0.0f;
        }
        return dot == 0.0f ? 0.0f : 1.0f;
    } else {
        // include/numkong/spatial/serial.h:272-278
        float d2 = a_norm + b_norm - 2.0f * dot;
        return d2 > 0.0f ? sqrtf(d2) : 0.0f;
    }
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
            uint32_t phase = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                uint32_t mt, nt;
                tile_coords(tile, p.tiles_m, p.tiles_n, mt, nt);
                const uint8_t *b_tile = p.b_payload + (uint64_t)nt * (kBN / kChunkRows) * p.kblocks * kChunkBytes;
                for (uint32_t kb = 0; kb < p.kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, 1, p.error_word)) { ok = false; break; }
                    uint32_t a_dst = smem_base + stage * Plan::kStageBytes;
                    uint32_t b_dst = a_dst + Plan::kABytes;
                    mbar_expect_tx(full_bar(stage), Plan::kStageBytes);
                    tma_load_2d(a_dst, &a_map, (int)(kb * p.elems_per_kblock), (int)(mt * kBM), full_bar(stage));
#pragma unroll
                    for (int j = 0; j < kBN / (int)kChunkRows; ++j)
                        bulk_load(b_dst + j * kChunkBytes, b_tile + ((uint64_t)j * p.kblocks + kb) * kChunkBytes,
                                  kChunkBytes, full_bar(stage));
                    if (++stage == kStages) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Give copies that are still in flight time to land before the CTA retires.
                for (int i = 0; i < 1000; ++i) __nanosleep(1000);
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
                for (uint32_t kb0 = 0; kb0 < p.kblocks && ok; kb0 += p.flush_kblocks, ++seq) {
                    const uint32_t buf = seq & 1u;
                    const uint32_t buf_phase = (seq >> 1) & 1u;
                    if (!mbar_wait(tmem_empty_bar(buf), buf_phase ^ 1u, 2, p.error_word)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + buf * kBN;
                    const uint32_t kb1 = min(kb0 + p.flush_kblocks, p.kblocks);
                    for (uint32_t kb = kb0; kb < kb1; ++kb) {
                        if (!mbar_wait(full_bar(stage), phase, 3, p.error_word)) { ok = false; break; }
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
        }
    } else {
        // ------------------------------------------------------------ epilogue (warps 2..9)
        const uint32_t quarter = warp & 3u;               // TMEM lanes this warp may read: 32*quarter .. +31
        const uint32_t half = (uint32_t)(warp - 2) >> 2;  // which half of the tile's columns
        uint32_t seq = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
            uint32_t mt, nt;
            tile_coords(tile, p.tiles_m, p.tiles_n, mt, nt);
            uint32_t acc[kColsPerThread];
#pragma unroll
            for (int j = 0; j < kColsPerThread; ++j) acc[j] = 0u;
            for (uint32_t kb0 = 0; kb0 < p.kblocks && ok; kb0 += p.flush_kblocks, ++seq) {
                const uint32_t buf = seq & 1u;
                const uint32_t buf_phase = (seq >> 1) & 1u;
                if (!mbar_wait(tmem_full_bar(buf), buf_phase, 4, p.error_word)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < kColsPerThread / 16; ++c) {
                    uint32_t v[16];
                    tmem_ld_32x16(tmem_base + ((quarter * 32u) << 16) + buf * kBN + half * kColsPerThread + c * 16, v);
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        if constexpr (kKind == kKindI8) acc[c * 16 + j] += v[j];
                        else acc[c * 16 + j] = __float_as_uint(__uint_as_float(acc[c * 16 + j]) + __uint_as_float(v[j]));
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(tmem_empty_bar(buf));
            }
            if (!ok) break;
            const uint32_t row = mt * kBM + quarter * 32u + lane;
            if (row >= p.m) continue;
            uint8_t *c_row = p.c + (uint64_t)row * p.c_stride;
            float a_norm = 0.0f;
            if constexpr (kEpi != kEpiDot) a_norm = p.a_norms[row];
#pragma unroll
            for (int c = 0; c < kColsPerThread / 32; ++c) {
                const uint32_t col0 = nt * kBN + half * kColsPerThread + c * 32;
                if (col0 >= p.n) break;
                if constexpr (kEpi != kEpiDot) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t raw = acc[c * 32 + j];
                        float dot = p.int_mode == 0 ? __uint_as_float(raw) : p.int_mode == 1 ? (float)(int32_t)raw : (float)raw;
                        float b_norm = 0.0f;
                        if (col0 + j < p.n)
                            b_norm = p.int_mode == 0 ? __ldg(reinterpret_cast<const float *>(p.b_norms) + col0 + j)
                                                     : (float)__ldg(reinterpret_cast<const uint32_t *>(p.b_norms) + col0 + j);
                        acc[c * 32 + j] = __float_as_uint(finalize<kEpi>(dot, a_norm, b_norm));
                    }
                }
                uint32_t *dst = reinterpret_cast<uint32_t *>(c_row) + col0;
                if (col0 + 32 <= p.n && (reinterpret_cast<uintptr_t>(dst) & 15u) == 0) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4)
                        *reinterpret_cast<uint4 *>(dst + j) = make_uint4(acc[c * 32 + j], acc[c * 32 + j + 1], acc[c * 32 + j + 2], acc[c * 32 + j + 3]);
                } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j)
                        if (col0 + j < p.n) dst[j] = acc[c * 32 + j];
                }
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
    uint32_t grid = tiles < (uint32_t)device_sm_count() ? tiles : (uint32_t)device_sm_count();
    kernel<<<grid, kThreads, Plan::kTotal, stream>>>(map, dev);
    return cudaGetLastError();
}

template <int kKind, int kEpi>
cudaError_t launch_by_tile(int bn, const CUtensorMap &map, const GemmDev &dev, cudaStream_t stream) {
    if (bn == 256) return launch_one<kKind, 256, 4, kEpi>(map, dev, stream);
    return launch_one<kKind, 128, 6, kEpi>(map, dev, stream);
}

template <int kKind>
cudaError_t launch_by_epilogue(int epi, int bn, const CUtensorMap &map, const GemmDev &dev, cudaStream_t stream) {
    switch (epi) {
    case kEpiDot: return launch_by_tile<kKind, kEpiDot>(bn, map, dev, stream);
    case kEpiAngular: return launch_by_tile<kKind, kEpiAngular>(bn, map, dev, stream);
    case kEpiEuclidean: return launch_by_tile<kKind, kEpiEuclidean>(bn, map, dev, stream);
    default: return cudaErrorInvalidValue;
    }
}

} // namespace

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

int gemm_tc_launch_count(const GemmArgs &) { return 1; }

cudaError_t launch_gemm_tc(const GemmArgs &args, cudaStream_t stream) {
    KindInfo ki;
    if (!kind_info(args.dtype, ki)) return cudaErrorInvalidValue;
    if (args.m == 0 || args.n == 0) return cudaSuccess;
    if (args.m > 0x7fffffffull || args.n > 0x7fffffffull || args.k > 0x7fffffffull) return cudaErrorInvalidValue;
    if ((reinterpret_cast<uintptr_t>(args.a) & 15u) || (args.a_stride & 15u)) return cudaErrorMisalignedAddress;

    const uint32_t eb = dtype_bytes(args.dtype);
    int bn = 256;
    if ((args.variant & 0xff) == 1) bn = 256;
    else if ((args.variant & 0xff) == 2) bn = 128;
    else {
        uint64_t tiles256 = ((args.m + kBM - 1) / kBM) * ((args.n + 255) / 256);
        if (args.n <= 128 || tiles256 < (uint64_t)device_sm_count()) bn = 128;
    }

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
    // Float kinds: spans of 16 stages (1024 16-bit or 2048 8-bit values): measured on B200, the normalised error
    // at depth 8192 is 8.6e-8 (bf16) / 1.0e-8 (e4m3), against 3.7e-7 / 3.7e-8 for one long chain, for ~3 % of the
    // run time (reading a 128 KiB accumulator out of TMEM stalls the MMAs for ~256 cycles). Integers are exact: one span.
    const uint32_t forced_flush = (uint32_t)args.variant >> 8;
    dev.flush_kblocks = ki.kind == kKindI8 ? dev.kblocks : (forced_flush ? forced_flush : 16u);
    if (dev.flush_kblocks == 0) dev.flush_kblocks = 1;
    dev.error_word = args.error_word;

    switch (ki.kind) {
    case kKindF16: return launch_by_epilogue<kKindF16>(args.epilogue, bn, map, dev, stream);
    case kKindF8F6F4: return launch_by_epilogue<kKindF8F6F4>(args.epilogue, bn, map, dev, stream);
    default: return launch_by_epilogue<kKindI8>(args.epilogue, bn, map, dev, stream);
    }
}

} // namespace nkb
