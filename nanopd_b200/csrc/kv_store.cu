// Kernel 1: paged KV store — a vectorised, coalesced scatter of new K/V rows into block slots.
//
// One thread moves one 16-byte piece of the K and V rows of one or four kv heads of a token; consecutive
// lanes take consecutive pieces, so a 128-element 16-bit row is 16 consecutive lanes and a warp
// covers two rows per head with full 128-byte transactions on both sides.  Offsets are 64-bit (the reference's 32-bit
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

// A thread moves one 16-byte piece (`chunk`) of the K and V rows of up to kHeadsPerThread consecutive kv heads of one
// token: the token's position and its page lookup (two dependent loads) and the split of the flat index are paid
// once per group of heads instead of once per piece, and the group's loads are all issued before its stores.
// Index math is 32-bit when the launch has fewer than 2^31 pieces (Index = unsigned), 64-bit otherwise.  Small
// launches (a decode batch) take one head per thread: they are bound by latency, and more threads hide more of it
// (256 tokens: 2.1 us against 2.4 with four heads per thread; 8192 tokens: 13.7 us against 12.7).
template <typename Index, int kHeadsPerThread>
__global__ void __launch_bounds__(256) paged_kv_store_kernel(const StoreParams p) {
    const int head_groups = (p.num_kv_heads + kHeadsPerThread - 1) / kHeadsPerThread;
    const Index per_token = static_cast<Index>(head_groups) * static_cast<Index>(p.chunks_per_row);
    const Index total = static_cast<Index>(p.num_rows / p.num_kv_heads) * per_token;
    for (Index i = blockIdx.x * static_cast<Index>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<Index>(gridDim.x) * blockDim.x) {
        const Index t_ = i / per_token;
        const int rest = static_cast<int>(i - t_ * per_token);
        const int hg = rest / p.chunks_per_row;
        const int chunk = rest - hg * p.chunks_per_row;
        const long long t = static_cast<long long>(t_);
        const int h0 = hg * kHeadsPerThread;

        const int pos = __ldg(p.positions + t);
        const int blk_idx = pos / p.block_size;
        const int off = pos - blk_idx * p.block_size;
        if (pos < 0 || blk_idx >= p.max_blocks_per_seq) {
            if (p.status && rest == 0) atomicOr(p.status, NPD_STATUS_BAD_POSITION);
            continue;
        }
        const int phys = __ldg(p.block_tables + t * p.bt_row_stride + blk_idx);
        if (phys < 0 || phys >= p.num_blocks) {
            if (p.status && rest == 0) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
            continue;
        }
        const long long src0 = t * p.src_token_stride + chunk;
        const long long dst0 = phys * p.cache_block_stride + (long long)off * p.chunks_per_row + chunk;
        uint4 kv[kHeadsPerThread], vv[kHeadsPerThread];
#pragma unroll
        for (int j = 0; j < kHeadsPerThread; ++j) {
            if (h0 + j < p.num_kv_heads) {
                kv[j] = __ldg(p.k_src + src0 + (h0 + j) * p.src_head_stride);
                vv[j] = __ldg(p.v_src + src0 + (h0 + j) * p.src_head_stride);
            }
        }
#pragma unroll
        for (int j = 0; j < kHeadsPerThread; ++j) {
            if (h0 + j < p.num_kv_heads) {
                const long long dst = dst0 + (long long)(h0 + j) * p.block_size * p.chunks_per_row;
                p.k_cache[dst] = kv[j];
                p.v_cache[dst] = vv[j];
            }
        }
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
    const int threads = 256;
    const long long cap = (long long)npd::sm_count(dev) * 8;   // 8 resident CTAs of 256 threads per SM
    const long long pieces = p.num_rows * p.chunks_per_row;
    const int heads_per_thread = pieces >= cap * threads ? 4 : 1;      // one head per thread until every slot has work
    const long long head_groups = (num_kv_heads + heads_per_thread - 1) / heads_per_thread;
    const long long total = num_tokens * head_groups * p.chunks_per_row;      // threads' worth of work
    long long blocks = (total + threads - 1) / threads;
    if (blocks > cap) blocks = cap;
    const bool small = total + cap * threads < (1LL << 31);
    const unsigned grid = static_cast<unsigned>(blocks);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (heads_per_thread == 1) {
        if (small) paged_kv_store_kernel<unsigned, 1><<<grid, threads, 0, st>>>(p);
        else paged_kv_store_kernel<long long, 1><<<grid, threads, 0, st>>>(p);
    } else {
        if (small) paged_kv_store_kernel<unsigned, 4><<<grid, threads, 0, st>>>(p);
        else paged_kv_store_kernel<long long, 4><<<grid, threads, 0, st>>>(p);
    }
    NPD_CUDA_TRY(cudaGetLastError());
    return NPD_OK;
}
