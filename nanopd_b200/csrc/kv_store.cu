// Kernel 1: paged KV store — a vectorised, coalesced scatter of new K/V rows into block slots.
//
// One thread moves one 16-byte piece of a (token, kv-head) row of K and the same piece of V,
// so a 128-element 16-bit row is 16 consecutive lanes and a warp covers two rows with
// full 128-byte transactions on both sides.  Offsets are 64-bit (the reference's 32-bit
// index math, nanoPD/paged_attention/csrc/kvstore/paged_kv_store_kernel.cu:41-54,
// overflows past 2^31 elements).  HBM-bound: T*Hkv*D*e*2 bytes read + the same written.
#include "npd_common.cuh"

namespace {

struct StoreParams {
    uint4 *k_cache;
    uint4 *v_cache;
    const uint4 *k_src;
    const uint4 *v_src;
    const int32_t *block_tables;
    const int32_t *positions;
    int32_t *status;
    long long num_rows;          // T * Hkv
    int num_kv_heads;
    int chunks_per_row;          // D * e / 16
    int block_size;
    int num_blocks;
    int max_blocks_per_seq;
    long long cache_block_stride;   // in 16-byte units
    long long src_head_stride;      // in 16-byte units
    long long src_token_stride;     // in 16-byte units
    long long bt_row_stride;        // in int32
};

__global__ void __launch_bounds__(256) paged_kv_store_kernel(const StoreParams p) {
    const long long total = p.num_rows * p.chunks_per_row;
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / p.chunks_per_row;
        const int chunk = static_cast<int>(i - row * p.chunks_per_row);
        const long long t = row / p.num_kv_heads;
        const int h = static_cast<int>(row - t * p.num_kv_heads);

        const int pos = __ldg(p.positions + t);
        const int blk_idx = pos / p.block_size;
        const int off = pos - blk_idx * p.block_size;
        if (pos < 0 || blk_idx >= p.max_blocks_per_seq) {
            if (p.status && chunk == 0) atomicOr(p.status, NPD_STATUS_BAD_POSITION);
            continue;
        }
        const int phys = __ldg(p.block_tables + t * p.bt_row_stride + blk_idx);
        if (phys < 0 || phys >= p.num_blocks) {
            if (p.status && chunk == 0) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
            continue;
        }
        const long long src = h * p.src_head_stride + t * p.src_token_stride + chunk;
        const long long dst = phys * p.cache_block_stride +
                              ((long long)h * p.block_size + off) * p.chunks_per_row + chunk;
        const uint4 kv = __ldg(p.k_src + src);
        const uint4 vv = __ldg(p.v_src + src);
        p.k_cache[dst] = kv;
        p.v_cache[dst] = vv;
    }
}

}  // namespace

extern "C" int npd_kv_store(void *k_cache, void *v_cache, const void *k_src, const void *v_src,
                            const int32_t *block_tables, const int32_t *positions,
                            int64_t num_tokens, int64_t num_kv_heads, int64_t head_dim,
                            int64_t block_size, int64_t num_blocks, int64_t max_blocks_per_seq,
                            int64_t cache_block_stride, int64_t src_head_stride,
                            int64_t src_token_stride, int64_t bt_row_stride,
                            int dtype, int32_t *status, void *stream) {
    NPD_REQUIRE(dtype == NPD_DTYPE_F16 || dtype == NPD_DTYPE_BF16 || dtype == NPD_DTYPE_F32,
                NPD_ERR_UNSUPPORTED, "npd_kv_store: unsupported dtype code %d", dtype);
    const int elem = dtype == NPD_DTYPE_F32 ? 4 : 2;
    NPD_REQUIRE(num_tokens >= 0 && num_kv_heads > 0 && head_dim > 0 && block_size > 0 && num_blocks > 0 &&
                    max_blocks_per_seq > 0,
                NPD_ERR_INVALID_ARG, "npd_kv_store: non-positive dimension");
    if (num_tokens == 0) return NPD_OK;
    NPD_REQUIRE(k_cache && v_cache && k_src && v_src && block_tables && positions, NPD_ERR_INVALID_ARG,
                "npd_kv_store: NULL pointer");
    NPD_REQUIRE((head_dim * elem) % 16 == 0, NPD_ERR_UNSUPPORTED,
                "npd_kv_store: head_dim*elem_size (%lld bytes) must be a multiple of 16",
                (long long)(head_dim * elem));
    NPD_REQUIRE(npd::aligned16(k_cache) && npd::aligned16(v_cache) && npd::aligned16(k_src) &&
                    npd::aligned16(v_src),
                NPD_ERR_INVALID_ARG, "npd_kv_store: pointers must be 16-byte aligned");
    const int per16 = 16 / elem;
    NPD_REQUIRE(cache_block_stride % per16 == 0 && src_head_stride % per16 == 0 && src_token_stride % per16 == 0,
                NPD_ERR_INVALID_ARG, "npd_kv_store: strides must be multiples of 16 bytes");
    NPD_REQUIRE(cache_block_stride >= num_kv_heads * block_size * head_dim, NPD_ERR_INVALID_ARG,
                "npd_kv_store: cache block stride smaller than one block");
    NPD_REQUIRE(num_blocks <= INT32_MAX && max_blocks_per_seq <= INT32_MAX && block_size <= INT32_MAX,
                NPD_ERR_INVALID_ARG, "npd_kv_store: dimension exceeds int32");

    StoreParams p;
    p.k_cache = static_cast<uint4 *>(k_cache);
    p.v_cache = static_cast<uint4 *>(v_cache);
    p.k_src = static_cast<const uint4 *>(k_src);
    p.v_src = static_cast<const uint4 *>(v_src);
    p.block_tables = block_tables;
    p.positions = positions;
    p.status = status;
    p.num_rows = num_tokens * num_kv_heads;
    p.num_kv_heads = static_cast<int>(num_kv_heads);
    p.chunks_per_row = static_cast<int>(head_dim * elem / 16);
    p.block_size = static_cast<int>(block_size);
    p.num_blocks = static_cast<int>(num_blocks);
    p.max_blocks_per_seq = static_cast<int>(max_blocks_per_seq);
    p.cache_block_stride = cache_block_stride / per16;
    p.src_head_stride = src_head_stride / per16;
    p.src_token_stride = src_token_stride / per16;
    p.bt_row_stride = bt_row_stride;

    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    const long long total = p.num_rows * p.chunks_per_row;
    const int threads = 256;
    long long blocks = (total + threads - 1) / threads;
    const long long cap = (long long)npd::sm_count(dev) * 8;   // 8 resident CTAs of 256 threads per SM
    if (blocks > cap) blocks = cap;
    paged_kv_store_kernel<<<static_cast<unsigned>(blocks), threads, 0, static_cast<cudaStream_t>(stream)>>>(p);
    NPD_CUDA_TRY(cudaGetLastError());
    return NPD_OK;
}
