// Fused per-head RMSNorm (optional) + rotary embedding of Q and K, with K and V written straight
// into their paged block slots.
//
// The caller of the paged kernels produces the store's input with a chain of element-wise passes
// just before it (nanoPD/engine/model_runner.py:97-115: q_norm, k_norm, three transposes, rotary
// embedding on Q and K, then paged_kv_store at :142-149 / :188-194).  Here one launch reads the
// projection output once and writes the rotated Q (token-major, the layout the attention kernels
// take) and the K/V page slots: bytes moved = T*(Hq+2*Hkv)*D*e read + the same written, instead of
// a round trip through HBM per pass.
//
// Arithmetic follows the Hugging Face modules the reference calls, rounding where they round:
//   RMSNorm (Qwen3RMSNorm): x32 = float(x); y = T(x32 * rsqrt(mean(x32^2) + eps)); y = T(w * y)
//   rotary (apply_rotary_pos_emb): out = T(T(y * cos) + T(rotate_half(y) * sin)),
//   rotate_half(y) = concat(-y[D/2:], y[:D/2]),   T(.) = round to the tensor's 16-bit type.
// A (token, head) row is D/8 lanes of 16 bytes; the two elements a rotation pairs sit at the same place
// of two lanes half a row apart (one shuffle), the mean of squares is a reduction over the row's lanes,
// a warp works through eight passes of rows of one token with all their loads in flight, and the products and
// sums that the reference rounds to 16 bits are packed 16-bit instructions.  HBM-bound, launch-latency bound at
// decode sizes.
#include "npd_common.cuh"

namespace {

struct RopeStoreParams {
    void *q_out;
    const void *q, *k, *v;
    const void *q_w, *k_w;          // per-head-dim norm weights or nullptr
    const void *cos, *sin;          // [T, D]
    void *k_cache, *v_cache;
    const int32_t *block_tables;
    const int32_t *positions;
    int32_t *status;
    float eps;
    long long num_tokens;
    int num_q_heads, num_kv_heads;
    int block_size, num_blocks, max_blocks_per_seq;
    long long cache_block_stride;   // elements
    long long q_token_stride, k_token_stride, v_token_stride, q_out_token_stride, cs_row_stride;   // elements
    long long bt_row_stride;
};

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// 8 elements (16 bytes) of T <-> 8 floats
template <typename T>
__device__ __forceinline__ void unpack8(const uint4 &raw, float (&out)[8]) {
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = to_f<T>(e[i]);
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float (&in)[8]) {
    uint4 raw;
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f<T>(in[i]);
    return raw;
}

// Packed 16-bit arithmetic: one instruction per pair, one rounding per operation — what the 16-bit tensor
// arithmetic of the reference does (a product of two 16-bit values is exact in fp32, so "multiply in fp32 and
// round" and the native packed multiply give the same bits; likewise for the sum).
template <typename T> struct Pair;
template <> struct Pair<__half> { using type = __half2; };
template <> struct Pair<__nv_bfloat16> { using type = __nv_bfloat162; };
template <typename T>
__device__ __forceinline__ uint32_t mul2(uint32_t a, uint32_t b) {
    using P = typename Pair<T>::type;
    P r = __hmul2_rn(*reinterpret_cast<P *>(&a), *reinterpret_cast<P *>(&b));     // _rn: never fused with the add
    return *reinterpret_cast<uint32_t *>(&r);
}
template <typename T>
__device__ __forceinline__ uint32_t add2(uint32_t a, uint32_t b) {
    using P = typename Pair<T>::type;
    P r = __hadd2_rn(*reinterpret_cast<P *>(&a), *reinterpret_cast<P *>(&b));
    return *reinterpret_cast<uint32_t *>(&r);
}

// A row of D elements is D/8 pieces of 16 bytes, one per lane: LPR = D/8 lanes per row, 32/LPR rows per warp pass,
// the lower LPR/2 lanes of a row hold its first half and the upper ones the second half, so the element a rotation
// pairs with sits at the same place of lane ^ (LPR/2).
// A warp takes a UNIT at a time: kPasses consecutive passes over the rows of ONE token (8 rows at head_dim 128; a
// token of the Qwen3-8B shape, 32 q + 8 k + 8 v rows, is six units).  What the rows of a token share is then
// fetched once per unit instead of once per row: the lane's piece of the token's cos and sin rows (which were two
// of every three load instructions), the position and the page lookup.  All row loads of a unit are issued before
// the first is used.
// Four passes per unit and at least four CTAs of 256 threads per SM (64 registers): 42 us for 8192 tokens of the
// Qwen3-8B shape; eight passes per unit at the 80-95 registers the compiler then takes (two or three CTAs per SM)
// 47-55 us, eight passes squeezed into 64 registers 43 us, six CTAs per SM (40 registers, spills) 54 us.
#ifndef NPD_ROPE_PASSES
#define NPD_ROPE_PASSES 4
#endif
#ifndef NPD_ROPE_MIN_CTAS
#define NPD_ROPE_MIN_CTAS 4
#endif
template <typename T, int D>
__global__ void __launch_bounds__(256, NPD_ROPE_MIN_CTAS) qk_norm_rope_store_kernel(const RopeStoreParams p) {
    constexpr int LPR = D / 8;                 // lanes per row
    constexpr int RPW = 32 / LPR;              // rows per warp pass
    constexpr int kPasses = NPD_ROPE_PASSES;   // passes per unit
    constexpr int kChunk = RPW * kPasses;      // rows per unit
    const int lane = threadIdx.x & 31;
    const int sub = lane % LPR, row_in_pass = lane / LPR;
    const bool upper = sub >= LPR / 2;
    const int rows_per_token = p.num_q_heads + 2 * p.num_kv_heads;
    const unsigned units_per_token = static_cast<unsigned>((rows_per_token + kChunk - 1) / kChunk);
    const unsigned total = static_cast<unsigned>(p.num_tokens) * units_per_token;      // < 2^31, checked by the host
    const unsigned warps = gridDim.x * (blockDim.x >> 5);
    const unsigned w0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const uint32_t sign = upper ? 0u : 0x80008000u;            // rotate_half: (-second half, first half)
    const uint4 zero4 = make_uint4(0, 0, 0, 0);
    // the norm weights are the same for every row of a kind
    const uint4 q_wv = p.q_w ? __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(p.q_w) + sub * 8)) : zero4;
    const uint4 k_wv = p.k_w ? __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(p.k_w) + sub * 8)) : zero4;
    for (unsigned unit = w0; unit < total; unit += warps) {
        const unsigned t32 = unit / units_per_token;
        const int row0 = static_cast<int>(unit - t32 * units_per_token) * kChunk;
        const int row_end = min(row0 + kChunk, rows_per_token);
        const long long t = t32;
        // ---- what the unit's rows share ----
        uint4 c = zero4, sn = zero4;
        if (row0 < p.num_q_heads + p.num_kv_heads) {           // it has q or k rows
            c = __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(p.cos) + t * p.cs_row_stride + sub * 8));
            sn = __ldg(reinterpret_cast<const uint4 *>(static_cast<const T *>(p.sin) + t * p.cs_row_stride + sub * 8));
        }
        long long slot = -1;                                    // element offset of (head 0, this position) in the page
        if (row_end > p.num_q_heads) {                          // it has k or v rows: their page slot
            const int pos = __ldg(p.positions + t);
            const int blk_idx = pos / p.block_size;
            const int off = pos - blk_idx * p.block_size;
            if (pos < 0 || blk_idx >= p.max_blocks_per_seq) {
                if (p.status && lane == 0) atomicOr(p.status, NPD_STATUS_BAD_POSITION);
            } else {
                const int phys = __ldg(p.block_tables + t * p.bt_row_stride + blk_idx);
                if (phys < 0 || phys >= p.num_blocks) {
                    if (p.status && lane == 0) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
                } else {
                    slot = phys * p.cache_block_stride + (long long)off * D;
                }
            }
        }
        // ---- the rows: all loads first ----
        uint4 raw[kPasses];
#pragma unroll
        for (int u = 0; u < kPasses; ++u) {
            const int r = row0 + u * RPW + row_in_pass;
            raw[u] = zero4;
            if (r >= row_end) continue;
            const int kd = r < p.num_q_heads ? 0 : (r < p.num_q_heads + p.num_kv_heads ? 1 : 2);   // q, k, v
            const int h = kd == 0 ? r : (kd == 1 ? r - p.num_q_heads : r - p.num_q_heads - p.num_kv_heads);
            const T *src = kd == 0 ? static_cast<const T *>(p.q) + t * p.q_token_stride
                         : kd == 1 ? static_cast<const T *>(p.k) + t * p.k_token_stride
                                   : static_cast<const T *>(p.v) + t * p.v_token_stride;
            // a plain (coherent) load: q_out may alias q, and a non-coherent load of memory the same kernel writes
            // is undefined
            raw[u] = *reinterpret_cast<const uint4 *>(src + (long long)h * D + sub * 8);
        }
#pragma unroll
        for (int u = 0; u < kPasses; ++u) {
            // every lane takes part in the shuffles; rows without work carry zeros
            const int r = row0 + u * RPW + row_in_pass;
            const int kd = r >= row_end ? 3 : (r < p.num_q_heads ? 0 : (r < p.num_q_heads + p.num_kv_heads ? 1 : 2));
            const int h = kd == 0 ? r : (kd == 1 ? r - p.num_q_heads : r - p.num_q_heads - p.num_kv_heads);
            float x[8];
            unpack8<T>(raw[u], x);
            const bool normed = (kd == 0 && p.q_w != nullptr) || (kd == 1 && p.k_w != nullptr);
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; ++i) ss += x[i] * x[i];
#pragma unroll
            for (int s2 = LPR / 2; s2 > 0; s2 >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, s2);
            uint4 mine = raw[u];
            if (normed) {
                const float inv = rsqrtf(ss * (1.f / D) + p.eps);
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] *= inv;
                const uint4 y = pack8<T>(x);                       // rounded to T, as the norm module does
                const uint4 wv = kd == 0 ? q_wv : k_wv;
                mine = make_uint4(mul2<T>(wv.x, y.x), mul2<T>(wv.y, y.y), mul2<T>(wv.z, y.z), mul2<T>(wv.w, y.w));
            }
            // the partner half of the row, as the 16-bit values the rotation reads
            uint4 other;
            other.x = __shfl_xor_sync(0xffffffffu, mine.x, LPR / 2);
            other.y = __shfl_xor_sync(0xffffffffu, mine.y, LPR / 2);
            other.z = __shfl_xor_sync(0xffffffffu, mine.z, LPR / 2);
            other.w = __shfl_xor_sync(0xffffffffu, mine.w, LPR / 2);
            if (kd < 2) {
                mine.x = add2<T>(mul2<T>(mine.x, c.x), mul2<T>(other.x ^ sign, sn.x));
                mine.y = add2<T>(mul2<T>(mine.y, c.y), mul2<T>(other.y ^ sign, sn.y));
                mine.z = add2<T>(mul2<T>(mine.z, c.z), mul2<T>(other.z ^ sign, sn.z));
                mine.w = add2<T>(mul2<T>(mine.w, c.w), mul2<T>(other.w ^ sign, sn.w));
            }
            if (kd == 0) {
                *reinterpret_cast<uint4 *>(static_cast<T *>(p.q_out) + t * p.q_out_token_stride + (long long)h * D + sub * 8) = mine;
            } else if (kd < 3 && slot >= 0) {
                *reinterpret_cast<uint4 *>(static_cast<T *>(kd == 1 ? p.k_cache : p.v_cache) + slot +
                                           (long long)h * p.block_size * D + sub * 8) = mine;
            }
        }
    }
}

template <typename T>
int launch(const RopeStoreParams &p, int head_dim, int device, cudaStream_t stream) {
    const int rows_per_unit = (32 / (head_dim / 8)) * NPD_ROPE_PASSES;         // rows per warp pass x passes per unit
    const long long units = p.num_tokens * ((p.num_q_heads + 2 * p.num_kv_heads + rows_per_unit - 1) / rows_per_unit);
    const int threads = 256;
    long long blocks = (units + 7) / 8;                                        // one unit per warp
    const long long cap = (long long)npd::sm_count(device) * 8;
    if (blocks > cap) blocks = cap;
    switch (head_dim) {
        case 64: qk_norm_rope_store_kernel<T, 64><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p); break;
        case 128: qk_norm_rope_store_kernel<T, 128><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p); break;
        case 256: qk_norm_rope_store_kernel<T, 256><<<static_cast<unsigned>(blocks), threads, 0, stream>>>(p); break;
        default: return npd::fail(NPD_ERR_UNSUPPORTED, "npd_qk_norm_rope_store: head_dim %d not in {64,128,256}", head_dim);
    }
    NPD_CUDA_TRY(cudaGetLastError());
    return NPD_OK;
}

}  // namespace

extern "C" int npd_qk_norm_rope_store(void *q_out, const void *q, const void *k, const void *v,
                                      const void *q_norm_weight, const void *k_norm_weight,
                                      const void *cos, const void *sin, float eps,
                                      void *k_cache, void *v_cache, const int32_t *block_tables,
                                      const int32_t *positions, int64_t num_tokens, int64_t num_q_heads,
                                      int64_t num_kv_heads, int64_t head_dim, int64_t block_size,
                                      int64_t num_blocks, int64_t max_blocks_per_seq, int64_t cache_block_stride,
                                      int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                                      int64_t q_out_token_stride, int64_t cos_sin_row_stride,
                                      int64_t bt_row_stride, int dtype, int32_t *status, void *stream) {
    NPD_REQUIRE(dtype == NPD_DTYPE_F16 || dtype == NPD_DTYPE_BF16, NPD_ERR_UNSUPPORTED,
                "npd_qk_norm_rope_store: unsupported dtype code %d", dtype);
    NPD_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, NPD_ERR_UNSUPPORTED,
                "npd_qk_norm_rope_store: head_dim %lld not in {64,128,256}", (long long)head_dim);
    NPD_REQUIRE(num_tokens >= 0 && num_q_heads > 0 && num_kv_heads > 0 && block_size > 0 && num_blocks > 0 &&
                    max_blocks_per_seq > 0,
                NPD_ERR_INVALID_ARG, "npd_qk_norm_rope_store: non-positive dimension");
    if (num_tokens == 0) return NPD_OK;
    NPD_REQUIRE(q_out && q && k && v && cos && sin && k_cache && v_cache && block_tables && positions,
                NPD_ERR_INVALID_ARG, "npd_qk_norm_rope_store: NULL pointer");
    NPD_REQUIRE(npd::aligned16(q_out) && npd::aligned16(q) && npd::aligned16(k) && npd::aligned16(v) &&
                    npd::aligned16(cos) && npd::aligned16(sin) && npd::aligned16(k_cache) && npd::aligned16(v_cache) &&
                    (q_norm_weight == nullptr || npd::aligned16(q_norm_weight)) &&
                    (k_norm_weight == nullptr || npd::aligned16(k_norm_weight)),
                NPD_ERR_INVALID_ARG, "npd_qk_norm_rope_store: pointers must be 16-byte aligned");
    NPD_REQUIRE(q_token_stride % 8 == 0 && k_token_stride % 8 == 0 && v_token_stride % 8 == 0 &&
                    q_out_token_stride % 8 == 0 && cos_sin_row_stride % 8 == 0 && cache_block_stride % 8 == 0,
                NPD_ERR_INVALID_ARG, "npd_qk_norm_rope_store: strides must be multiples of 16 bytes");
    NPD_REQUIRE(q_token_stride >= num_q_heads * head_dim && q_out_token_stride >= num_q_heads * head_dim &&
                    k_token_stride >= num_kv_heads * head_dim && v_token_stride >= num_kv_heads * head_dim &&
                    cos_sin_row_stride >= 0,
                NPD_ERR_INVALID_ARG, "npd_qk_norm_rope_store: token stride smaller than one token's heads");
    NPD_REQUIRE(cache_block_stride >= num_kv_heads * block_size * head_dim, NPD_ERR_INVALID_ARG,
                "npd_qk_norm_rope_store: cache block stride smaller than one block");
    NPD_REQUIRE(num_blocks <= INT32_MAX && max_blocks_per_seq <= INT32_MAX && block_size <= INT32_MAX &&
                    num_q_heads <= INT32_MAX / 4 && num_kv_heads <= INT32_MAX / 4,
                NPD_ERR_INVALID_ARG, "npd_qk_norm_rope_store: dimension exceeds int32");
    NPD_REQUIRE(num_tokens * (num_q_heads + 2 * num_kv_heads) < (1LL << 31) - 4096, NPD_ERR_INVALID_ARG,
                "npd_qk_norm_rope_store: more than 2^31 (token, head) rows in one call");

    RopeStoreParams p;
    p.q_out = q_out;
    p.q = q;
    p.k = k;
    p.v = v;
    p.q_w = q_norm_weight;
    p.k_w = k_norm_weight;
    p.cos = cos;
    p.sin = sin;
    p.k_cache = k_cache;
    p.v_cache = v_cache;
    p.block_tables = block_tables;
    p.positions = positions;
    p.status = status;
    p.eps = eps;
    p.num_tokens = num_tokens;
    p.num_q_heads = static_cast<int>(num_q_heads);
    p.num_kv_heads = static_cast<int>(num_kv_heads);
    p.block_size = static_cast<int>(block_size);
    p.num_blocks = static_cast<int>(num_blocks);
    p.max_blocks_per_seq = static_cast<int>(max_blocks_per_seq);
    p.cache_block_stride = cache_block_stride;
    p.q_token_stride = q_token_stride;
    p.k_token_stride = k_token_stride;
    p.v_token_stride = v_token_stride;
    p.q_out_token_stride = q_out_token_stride;
    p.cs_row_stride = cos_sin_row_stride;
    p.bt_row_stride = bt_row_stride;

    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == NPD_DTYPE_BF16 ? launch<__nv_bfloat16>(p, static_cast<int>(head_dim), dev, st)
                                   : launch<__half>(p, static_cast<int>(head_dim), dev, st);
}
