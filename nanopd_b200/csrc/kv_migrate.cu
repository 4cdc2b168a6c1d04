// Kernel 4: prefill -> decode KV page migration as one gather/scatter copy kernel.
//
// The reference moves a request's pages with two strided copy_ calls per block
// (nanoPD/workers/kv_transfer.py:73-79), i.e. up to thousands of launches per request, each a
// [layers] x 32 KiB strided copy.  Here one launch walks every (block pair, layer, K|V) unit —
// block_elems*elem bytes, contiguous on both sides.  Either side may be peer memory mapped over
// NVLink, so the same kernel pushes (source local) or pulls (destination local).
//
// Two data paths:
//   * bulk (default): one warp per CTA; an elected lane streams units through a ring of
//     shared-memory stages with cp.async.bulk (global -> shared on an mbarrier, shared -> global in
//     bulk groups): copies in flight without occupying registers or issue slots, in a CTA small
//     enough (one warp, 64 KiB) to sit beside a decode-attention CTA on the same SM.  No multicast.
//   * ld/st: 256 threads per CTA, 16-byte loads and stores, eight loads in flight per thread —
//     taken when one side is pinned host memory (the relay buffer of extract_kv_to_pinned /
//     load_kv_from_pinned, nanoPD/workers/kv_transfer.py:44-66, reached over PCIe through the
//     unified address space), or on request.
// Link- or HBM-bound: blocks * layers * 2 * block_bytes, one direction.
#include <cstdlib>

#include "npd_common.cuh"
#include "../../include/nanopd_b200_testing.h"

namespace {

using namespace npd;

int env_int(const char *name, int fallback) {
    const char *v = std::getenv(name);
    if (!v || !*v) return fallback;
    const int x = std::atoi(v);
    return x > 0 ? x : fallback;
}

struct MigrateParams {
    const uint8_t *src_k, *src_v;
    uint8_t *dst_k, *dst_v;
    const int32_t *src_blocks, *dst_blocks;
    int32_t *status;
    long long num_pairs;
    int num_layers;
    long long block_bytes;
    long long src_layer_stride, src_block_stride, dst_layer_stride, dst_block_stride;   // bytes
    int src_num_blocks, dst_num_blocks;
    int pieces_per_unit;      // bulk path: a unit is moved in pieces of at most piece_bytes
    int piece_bytes;          // bulk path: bytes per ring stage (a multiple of 16)
    int stages;               // bulk path: ring depth (<= kMaxBulkStages)
    long long wait_limit;     // bulk path: clocks a wait for a load may take before the kernel gives up
    long long withhold_piece; // testing only: this piece's load is announced but never issued (-1 = none)
};

constexpr int kThreads = 256;
constexpr int kUnroll = 8;
constexpr int kMaxBulkStages = 8;

__device__ __forceinline__ bool locate_unit(const MigrateParams &p, long long u, const uint8_t *&src, uint8_t *&dst) {
    // Unit order: pair-major, then layer, then K|V — consecutive units work on one block.
    const int kv = static_cast<int>(u & 1);
    const long long pl = u >> 1;
    const long long pair = pl / p.num_layers;
    const int layer = static_cast<int>(pl - pair * p.num_layers);
    const int sb = __ldg(p.src_blocks + pair), db = __ldg(p.dst_blocks + pair);
    if (sb < 0 || sb >= p.src_num_blocks || db < 0 || db >= p.dst_num_blocks) return false;
    src = (kv ? p.src_v : p.src_k) + layer * p.src_layer_stride + sb * p.src_block_stride;
    dst = (kv ? p.dst_v : p.dst_k) + layer * p.dst_layer_stride + db * p.dst_block_stride;
    return true;
}

__global__ void __launch_bounds__(kThreads) kv_migrate_ldst_kernel(const MigrateParams p) {
    const long long units = p.num_pairs * p.num_layers * 2;
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        const uint8_t *src8;
        uint8_t *dst8;
        if (!locate_unit(p, u, src8, dst8)) {
            if (p.status && threadIdx.x == 0) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
            continue;
        }
        const uint4 *src = reinterpret_cast<const uint4 *>(src8);
        uint4 *dst = reinterpret_cast<uint4 *>(dst8);
        const int n = static_cast<int>(p.block_bytes / 16);
        for (int base = 0; base < n; base += kThreads * kUnroll) {
            uint4 buf[kUnroll];
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) {
                const int idx = base + i * kThreads + threadIdx.x;
                if (idx < n) buf[i] = src[idx];
            }
#pragma unroll
            for (int i = 0; i < kUnroll; ++i) {
                const int idx = base + i * kThreads + threadIdx.x;
                if (idx < n) dst[idx] = buf[i];
            }
        }
    }
}

// ---- bulk-copy helpers (untiled cp.async.bulk: 16-byte aligned addresses and sizes) ----
__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}
__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src_smem, uint32_t bytes) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(src_smem), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() {     // at most N store groups still READING shared memory
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// One warp per CTA; lane 0 drives a ring of p.stages pieces: load piece i+S-1 while piece i is stored.
__global__ void __launch_bounds__(32) kv_migrate_bulk_kernel(const MigrateParams p) {
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t bars[kMaxBulkStages];
    if (threadIdx.x != 0) return;
    const int kBulkStages = p.stages, kPieceBytes = p.piece_bytes;
    for (int i = 0; i < kBulkStages; ++i) mbar_init(smem_u32(&bars[i]), 1);
    mbar_fence_init();
    fence_proxy_async_smem();

    const long long units = p.num_pairs * p.num_layers * 2;
    const long long pieces = units * p.pieces_per_unit;
    // this CTA's pieces: blockIdx.x, blockIdx.x + gridDim.x, ...
    const long long my_count = pieces > blockIdx.x ? (pieces - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;

    auto piece_ptrs = [&](long long i, const uint8_t *&src, uint8_t *&dst, uint32_t &bytes) {
        const long long piece = blockIdx.x + i * gridDim.x;
        const long long u = piece / p.pieces_per_unit;
        const int part = static_cast<int>(piece - u * p.pieces_per_unit);
        const uint8_t *s;
        uint8_t *d;
        if (!locate_unit(p, u, s, d)) {
            if (p.status) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
            return false;
        }
        const long long off = (long long)part * kPieceBytes;
        const long long left = p.block_bytes - off;
        bytes = static_cast<uint32_t>(left < kPieceBytes ? left : kPieceBytes);
        src = s + off;
        dst = d + off;
        return true;
    };

    long long dead_at = -1;
    long long issued = 0;
    auto issue_load = [&](long long i) {
        const int st = static_cast<int>(i % kBulkStages);
        const uint8_t *src;
        uint8_t *dst;
        uint32_t bytes = 0;
        const uint32_t bar = smem_u32(&bars[st]);
        if (piece_ptrs(i, src, dst, bytes)) {
            mbar_expect_tx(bar, bytes);
            if (blockIdx.x + i * gridDim.x != p.withhold_piece)
                bulk_g2s(smem_u32(smem + (size_t)st * kPieceBytes), src, bytes, bar);
        } else {
            mbar_arrive(bar);          // skipped piece: keep the ring's phases in step
        }
    };
    for (; issued < my_count && issued < kBulkStages - 1; ++issued) issue_load(issued);

    for (long long i = 0; i < my_count; ++i) {
        const int st = static_cast<int>(i % kBulkStages);
        if (!mbar_wait_bounded(smem_u32(&bars[st]), static_cast<uint32_t>((i / kBulkStages) & 1), p.wait_limit)) {
            if (p.status) atomicOr(p.status, NPD_STATUS_WAIT_TIMEOUT);
            dead_at = i;
            break;
        }
        const uint8_t *src;
        uint8_t *dst;
        uint32_t bytes = 0;
        if (piece_ptrs(i, src, dst, bytes)) bulk_s2g(dst, smem_u32(smem + (size_t)st * kPieceBytes), bytes);
        bulk_commit();
        // The next load reuses the stage whose store was committed one iteration ago: wait until at most
        // one store group (the one just committed) is still reading shared memory.
        if (issued < my_count) {
            bulk_wait_read<1>();
            issue_load(issued);
            ++issued;
        }
    }
    if (dead_at >= 0) {
        // Loads issued behind the one that never arrived may still be writing this CTA's shared memory: give each a
        // bounded chance to land before the CTA ends and the SM hands the memory to another CTA.
        for (long long j = dead_at + 1; j < issued; ++j)
            (void)mbar_wait_bounded(smem_u32(&bars[j % kBulkStages]), static_cast<uint32_t>((j / kBulkStages) & 1),
                                    200000000LL);
    }
    bulk_wait_all();     // all stores have landed before the kernel (and its stream position) completes
}

}  // namespace

namespace {

int kv_migrate_impl(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                    const int32_t *src_blocks, const int32_t *dst_blocks, int64_t num_pairs,
                    int64_t num_layers, int64_t block_elems, int elem_bytes,
                    int64_t src_layer_stride, int64_t src_block_stride, int64_t src_num_blocks,
                    int64_t dst_layer_stride, int64_t dst_block_stride, int64_t dst_num_blocks,
                    int max_ctas, int32_t *status, void *stream, long long withhold_piece, long long wait_limit) {
    NPD_REQUIRE(num_pairs >= 0 && num_layers > 0 && block_elems > 0 && elem_bytes > 0, NPD_ERR_INVALID_ARG,
                "npd_kv_migrate: non-positive dimension");
    if (num_pairs == 0) return NPD_OK;
    NPD_REQUIRE(src_k && src_v && dst_k && dst_v && src_blocks && dst_blocks, NPD_ERR_INVALID_ARG,
                "npd_kv_migrate: NULL pointer");
    NPD_REQUIRE((block_elems * elem_bytes) % 16 == 0, NPD_ERR_INVALID_ARG,
                "npd_kv_migrate: block size in bytes must be a multiple of 16");
    NPD_REQUIRE(npd::aligned16(src_k) && npd::aligned16(src_v) && npd::aligned16(dst_k) && npd::aligned16(dst_v),
                NPD_ERR_INVALID_ARG, "npd_kv_migrate: pool pointers must be 16-byte aligned");
    const int64_t strides[4] = {src_layer_stride, src_block_stride, dst_layer_stride, dst_block_stride};
    for (int i = 0; i < 4; ++i)
        NPD_REQUIRE(strides[i] >= 0 && (strides[i] * elem_bytes) % 16 == 0, NPD_ERR_INVALID_ARG,
                    "npd_kv_migrate: strides must be non-negative multiples of 16 bytes");
    NPD_REQUIRE(src_block_stride >= block_elems && dst_block_stride >= block_elems, NPD_ERR_INVALID_ARG,
                "npd_kv_migrate: block stride smaller than a block");
    NPD_REQUIRE(src_num_blocks > 0 && dst_num_blocks > 0 && src_num_blocks < INT32_MAX && dst_num_blocks < INT32_MAX &&
                    num_layers < INT32_MAX && block_elems * elem_bytes / 16 < INT32_MAX,
                NPD_ERR_INVALID_ARG, "npd_kv_migrate: dimension out of range");

    MigrateParams p;
    p.src_k = static_cast<const uint8_t *>(src_k);
    p.src_v = static_cast<const uint8_t *>(src_v);
    p.dst_k = static_cast<uint8_t *>(dst_k);
    p.dst_v = static_cast<uint8_t *>(dst_v);
    p.src_blocks = src_blocks;
    p.dst_blocks = dst_blocks;
    p.status = status;
    p.num_pairs = num_pairs;
    p.num_layers = static_cast<int>(num_layers);
    p.block_bytes = block_elems * elem_bytes;
    p.src_layer_stride = src_layer_stride * elem_bytes;
    p.src_block_stride = src_block_stride * elem_bytes;
    p.dst_layer_stride = dst_layer_stride * elem_bytes;
    p.dst_block_stride = dst_block_stride * elem_bytes;
    p.src_num_blocks = static_cast<int>(src_num_blocks);
    p.dst_num_blocks = static_cast<int>(dst_num_blocks);
    p.withhold_piece = withhold_piece;
    p.wait_limit = wait_limit > 0 ? wait_limit : 4000000000LL;
    // Ring of the bulk path: 4 stages of 16 KiB.  64 KiB of shared memory and one warp fit beside a decode-attention
    // CTA on the same SM (132 KiB, 8 warps x 224 registers), so a migration on a side stream does not take SMs away
    // from the compute stream; 64 such CTAs keep ~3 MB in flight, enough for an NVLink on every box seen (with 48 the
    // same build reached 771 GB/s on one box and 708 GB/s on another; with 64, 762-772 GB/s).
    // A copy between two pools of ONE GPU has three times an NVLink's bandwidth to fill and nothing to gain from
    // being small: it takes the larger ring (6 x 32 KiB).
    cudaPointerAttributes src_attr{}, dst_attr{};
    const bool known = cudaPointerGetAttributes(&src_attr, src_k) == cudaSuccess &&
                       cudaPointerGetAttributes(&dst_attr, dst_k) == cudaSuccess;
    (void)cudaGetLastError();
    const bool same_gpu = known && src_attr.type == cudaMemoryTypeDevice && dst_attr.type == cudaMemoryTypeDevice &&
                          src_attr.device == dst_attr.device;
    // One side in pinned host memory (the relay buffer): plain loads and stores over PCIe, a small grid.
    const bool host_side = known && (src_attr.type == cudaMemoryTypeHost || dst_attr.type == cudaMemoryTypeHost);
    if (known)
        NPD_REQUIRE(src_attr.type != cudaMemoryTypeUnregistered && dst_attr.type != cudaMemoryTypeUnregistered,
                    NPD_ERR_INVALID_ARG, "npd_kv_migrate: a pool lies in pageable host memory (pin it first)");
    if (host_side && max_ctas >= 0) max_ctas = max_ctas > 0 ? -max_ctas : -32;
    if (host_side) {
        // the kernel needs the DEVICE alias of a pinned host pointer (the same number under unified addressing,
        // but asked for rather than assumed)
        const void *ptrs[4] = {p.src_k, p.src_v, p.dst_k, p.dst_v};
        for (int i = 0; i < 4; ++i) {
            cudaPointerAttributes a{};
            NPD_CUDA_TRY(cudaPointerGetAttributes(&a, ptrs[i]));
            if (a.type == cudaMemoryTypeHost) {
                NPD_REQUIRE(a.devicePointer != nullptr, NPD_ERR_INVALID_ARG,
                            "npd_kv_migrate: a pinned host pool is not mapped into the device's address space");
                ptrs[i] = a.devicePointer;
            }
        }
        p.src_k = static_cast<const uint8_t *>(ptrs[0]);
        p.src_v = static_cast<const uint8_t *>(ptrs[1]);
        p.dst_k = static_cast<uint8_t *>(const_cast<void *>(ptrs[2]));
        p.dst_v = static_cast<uint8_t *>(const_cast<void *>(ptrs[3]));
    }
    // tuning knobs from the environment, read once per process
    static const int knob_piece_kb = env_int("NPD_MIGRATE_PIECE_KB", 0), knob_stages = env_int("NPD_MIGRATE_STAGES", 0);
    p.piece_bytes = (knob_piece_kb > 0 ? knob_piece_kb : (same_gpu ? 32 : 16)) * 1024;
    p.stages = knob_stages > 0 ? knob_stages : (same_gpu ? 6 : 4);
    if (p.stages > kMaxBulkStages) p.stages = kMaxBulkStages;
    if (p.stages < 2) p.stages = 2;
    while ((long long)p.piece_bytes * p.stages > 200 * 1024 && p.piece_bytes > 4096) p.piece_bytes /= 2;
    p.pieces_per_unit = static_cast<int>((p.block_bytes + p.piece_bytes - 1) / p.piece_bytes);

    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    const long long units = num_pairs * num_layers * 2;
    cudaStream_t st = static_cast<cudaStream_t>(stream);

    // max_ctas < 0 selects the load/store path with -max_ctas CTAs (kept for comparison and as a fallback).
    if (max_ctas >= 0) {
        const long long pieces = units * p.pieces_per_unit;
        long long grid = max_ctas > 0 ? max_ctas : 64;
        if (grid > npd::sm_count(dev)) grid = npd::sm_count(dev);
        if (grid > pieces) grid = pieces;
        const size_t smem = (size_t)p.stages * p.piece_bytes;
        NPD_CUDA_TRY(cudaFuncSetAttribute(kv_migrate_bulk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        // Ask for the largest shared-memory carve-out: an SM configured for this small CTA alone could not take a
        // decode-attention CTA of the compute stream beside it, and a persistent kernel that is one CTA short
        // runs in two waves.
        NPD_CUDA_TRY(cudaFuncSetAttribute(kv_migrate_bulk_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
        kv_migrate_bulk_kernel<<<static_cast<unsigned>(grid), 32, smem, st>>>(p);
    } else {
        long long grid = -static_cast<long long>(max_ctas);
        if (grid > units) grid = units;
        NPD_CUDA_TRY(cudaFuncSetAttribute(kv_migrate_ldst_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                                          cudaSharedmemCarveoutMaxShared));
        kv_migrate_ldst_kernel<<<static_cast<unsigned>(grid), kThreads, 0, st>>>(p);
    }
    NPD_CUDA_TRY(cudaGetLastError());
    return NPD_OK;
}

}  // namespace

extern "C" int npd_kv_migrate(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                              const int32_t *src_blocks, const int32_t *dst_blocks, int64_t num_pairs,
                              int64_t num_layers, int64_t block_elems, int elem_bytes,
                              int64_t src_layer_stride, int64_t src_block_stride, int64_t src_num_blocks,
                              int64_t dst_layer_stride, int64_t dst_block_stride, int64_t dst_num_blocks,
                              int max_ctas, int32_t *status, void *stream) {
    return kv_migrate_impl(src_k, src_v, dst_k, dst_v, src_blocks, dst_blocks, num_pairs, num_layers, block_elems,
                           elem_bytes, src_layer_stride, src_block_stride, src_num_blocks, dst_layer_stride,
                           dst_block_stride, dst_num_blocks, max_ctas, status, stream, -1, 0);
}

extern "C" int npd_testing_kv_migrate_withheld(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                                               const int32_t *src_blocks, const int32_t *dst_blocks, int64_t num_pairs,
                                               int64_t num_layers, int64_t block_elems, int elem_bytes,
                                               int64_t src_layer_stride, int64_t src_block_stride,
                                               int64_t src_num_blocks, int64_t dst_layer_stride,
                                               int64_t dst_block_stride, int64_t dst_num_blocks, int max_ctas,
                                               int32_t *status, void *stream, int64_t withhold_piece,
                                               int64_t wait_limit_clocks) {
    NPD_REQUIRE(max_ctas > 0, NPD_ERR_INVALID_ARG, "npd_testing_kv_migrate_withheld: the bulk path only (max_ctas > 0)");
    NPD_REQUIRE(wait_limit_clocks > 0 && wait_limit_clocks <= 2000000000LL, NPD_ERR_INVALID_ARG,
                "npd_testing_kv_migrate_withheld: wait limit must be in (0, 2e9] clocks");
    return kv_migrate_impl(src_k, src_v, dst_k, dst_v, src_blocks, dst_blocks, num_pairs, num_layers, block_elems,
                           elem_bytes, src_layer_stride, src_block_stride, src_num_blocks, dst_layer_stride,
                           dst_block_stride, dst_num_blocks, max_ctas, status, stream, withhold_piece,
                           wait_limit_clocks);
}
