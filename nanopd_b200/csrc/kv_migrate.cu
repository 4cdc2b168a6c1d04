// Kernel 4: prefill -> decode KV page migration as one gather/scatter copy kernel.
//
// The reference moves a request's pages with two strided copy_ calls per block
// (nanoPD/workers/kv_transfer.py:73-79), i.e. up to thousands of launches per request, each a
// [layers] x 32 KiB strided copy.  Here one launch walks every (block pair, layer, K|V) unit —
// block_elems*elem bytes, contiguous on both sides — with 16-byte loads and stores, eight
// loads in flight per thread before the first store.  Either side may be peer memory mapped
// over NVLink, so the same kernel pushes (source local) or pulls (destination local).  It
// runs on a side stream with a capped CTA count so the compute stream keeps most SMs.
// Link- or HBM-bound: blocks * layers * 2 * block_bytes, one direction.
#include "npd_common.cuh"

namespace {

struct MigrateParams {
    const uint4 *src_k, *src_v;
    uint4 *dst_k, *dst_v;
    const int32_t *src_blocks, *dst_blocks;
    int32_t *status;
    long long num_pairs;
    int num_layers;
    int chunks_per_block;              // block bytes / 16
    long long src_layer_stride, src_block_stride, dst_layer_stride, dst_block_stride;   // 16-byte units
    int src_num_blocks, dst_num_blocks;
};

constexpr int kThreads = 256;
constexpr int kUnroll = 8;

__global__ void __launch_bounds__(kThreads) kv_migrate_kernel(const MigrateParams p) {
    const long long units = p.num_pairs * p.num_layers * 2;
    for (long long u = blockIdx.x; u < units; u += gridDim.x) {
        // Unit order: pair-major, then layer, then K|V — consecutive CTAs work on one block.
        const int kv = static_cast<int>(u & 1);
        const long long pl = u >> 1;
        const long long pair = pl / p.num_layers;
        const int layer = static_cast<int>(pl - pair * p.num_layers);
        const int sb = __ldg(p.src_blocks + pair), db = __ldg(p.dst_blocks + pair);
        if (sb < 0 || sb >= p.src_num_blocks || db < 0 || db >= p.dst_num_blocks) {
            if (p.status && threadIdx.x == 0) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
            continue;
        }
        const uint4 *src = (kv ? p.src_v : p.src_k) + layer * p.src_layer_stride + sb * p.src_block_stride;
        uint4 *dst = (kv ? p.dst_v : p.dst_k) + layer * p.dst_layer_stride + db * p.dst_block_stride;
        const int n = p.chunks_per_block;
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

}  // namespace

extern "C" int npd_kv_migrate(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                              const int32_t *src_blocks, const int32_t *dst_blocks, int64_t num_pairs,
                              int64_t num_layers, int64_t block_elems, int elem_bytes,
                              int64_t src_layer_stride, int64_t src_block_stride, int64_t src_num_blocks,
                              int64_t dst_layer_stride, int64_t dst_block_stride, int64_t dst_num_blocks,
                              int max_ctas, int32_t *status, void *stream) {
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
    p.src_k = static_cast<const uint4 *>(src_k);
    p.src_v = static_cast<const uint4 *>(src_v);
    p.dst_k = static_cast<uint4 *>(dst_k);
    p.dst_v = static_cast<uint4 *>(dst_v);
    p.src_blocks = src_blocks;
    p.dst_blocks = dst_blocks;
    p.status = status;
    p.num_pairs = num_pairs;
    p.num_layers = static_cast<int>(num_layers);
    p.chunks_per_block = static_cast<int>(block_elems * elem_bytes / 16);
    p.src_layer_stride = src_layer_stride * elem_bytes / 16;
    p.src_block_stride = src_block_stride * elem_bytes / 16;
    p.dst_layer_stride = dst_layer_stride * elem_bytes / 16;
    p.dst_block_stride = dst_block_stride * elem_bytes / 16;
    p.src_num_blocks = static_cast<int>(src_num_blocks);
    p.dst_num_blocks = static_cast<int>(dst_num_blocks);

    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    long long grid = max_ctas > 0 ? max_ctas : npd::sm_count(dev);
    const long long units = num_pairs * num_layers * 2;
    if (grid > units) grid = units;
    kv_migrate_kernel<<<static_cast<unsigned>(grid), kThreads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    NPD_CUDA_TRY(cudaGetLastError());
    return NPD_OK;
}
