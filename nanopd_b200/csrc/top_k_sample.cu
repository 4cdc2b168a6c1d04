// Batched top-k sampling over the logits of one step (sm_100a).
//
// Replaces the per-sequence sampler of the reference (top_k_sample, nanoPD/engine/model_runner.py:279-284,
// called once per sequence with a device→host read of every token at nanoPD/engine/engine.py:100-106 and
// nanoPD/workers/decode_worker.py:110): nan_to_num, the k largest logits, a softmax over them in the
// logits' dtype, one draw.  Here one launch serves every row of the step and leaves the tokens on the device.
//
// The work is a single pass over T x V logits, so HBM bounds it.  A row is cut into slices of 32 KiB; all slices
// of all rows are dealt, in order, in equal runs to at most two persistent CTAs per SM (a whole number of CTAs per
// row while the rows fit, so that no run crosses a row's end).  A CTA brings its slices into a
// ring of three shared-memory stages by one bulk asynchronous copy each (cp.async.bulk on an mbarrier, no
// multicast) — across the ends of rows, so two copies per CTA are on their way while a slice is examined and no
// register holds data in flight.  The k best of a row (of the CTA's part of it) are found without sorting:
//   * first slice: every group of 2 or 4 threads reduces the maximum of its logits; the k-th largest of the group
//     maxima is a lower bound of the slice's k-th largest logit (k groups hold a logit at least that large).  The
//     logits not below it (about -G ln(1 - k/G) on unordered data, G groups) are gathered into shared memory and
//     ranked by counting; ranks below k are the k best so far and the k-th of them is the running threshold;
//   * later slices: only logits ABOVE the threshold are gathered (their ids are larger than every id seen, so an
//     equal value ranks behind) — about k/(slices seen) of them on unordered data — and ranked together with
//     the k best so far; the scan itself is a packed maximum of each 16 bytes compared with the threshold.
// Data that defeats the threshold (more than 1024 logits past it in one slice: long runs of equal or rising
// values) takes k rounds of a block-wide arg-max over that slice instead — slower, same result.  A row that one
// CTA saw whole is drawn at once; where a run starts or ends inside a row, each CTA writes the k best of its part
// to global memory and the last to arrive (a ticket per row, reset by that CTA) merges them.  One warp computes
// the probabilities and draws.
// Order everywhere: larger value first, equal values by the lower id — which makes the result independent of
// how the rows were cut.
#include <cfloat>
#include <climits>
#include <cstdlib>

#include "npd_common.cuh"

namespace {

constexpr int kThreads = 256;                   // threads that examine the slices (8 warps); one more warp issues the copies
constexpr int kBlockThreads = kThreads + 32;
constexpr int kLoads = 8;                       // 16-byte pieces per thread and slice: 64 (16-bit) or 32 (fp32) logits
constexpr int kSliceBytes = kThreads * kLoads * 16;
constexpr int kStages = 3;                      // ring of slices in shared memory; two CTAs of 96 KiB fit an SM
constexpr long long kWaitLimit = 400000000LL;   // SM clocks a thread waits for a slice before it gives up (~0.2 s)
constexpr int kMaxGroups = 128;
constexpr int kMaxTopK = NPD_SAMPLE_MAX_TOP_K;
constexpr int kSliceCandidates = 1024;          // more logits than this past the bound in one slice: arg-max rounds
constexpr int64_t kTicketBytes = 65536;         // head of the workspace: a status word, then one arrival counter per row
constexpr int64_t kTicketOffset = 256;
constexpr int64_t kRowsPerLaunch = (kTicketBytes - kTicketOffset) / 4;

struct SampleParams {
    const void *logits;
    const float *uniforms;
    int64_t *out;
    float *cand_value;      // [rows of a launch, parts_cap, k]
    int32_t *cand_id;
    uint32_t *tickets;
    int32_t *status;
    int64_t row_stride;
    int64_t first_row;
    int vocab;
    int slices;             // per row
    int parts_cap;          // list slots per row in cand_*: the most CTAs one row is spread over
    int top_k;
    int64_t items;          // rows of this launch x slices, dealt to the CTAs in equal consecutive runs
};

// Barrier among the kThreads examining threads (the copy warp takes no part in it).
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kThreads) : "memory"); }

// (value, id) order: larger value first, equal values by the lower id.  Bitwise on purpose: no branches in the
// counting loops.
__device__ __forceinline__ bool before(float va, int ia, float vb, int ib) {
    return (va > vb) | ((va == vb) & (ia < ib));
}

// nan_to_num(nan = 0, posinf = 1e4, neginf = -1e4), the replacement already rounded to the logits' dtype
__device__ __forceinline__ float replace_special(float x, float replacement) {
    if (x != x) return 0.f;
    if (fabsf(x) > FLT_MAX) return copysignf(replacement, x);
    return x;
}

template <typename T> struct Logit;
template <> struct Logit<float> {
    static constexpr uint32_t kLowestBits = 0xff7fffffu;     // the most negative finite value: pads a ragged row end
    static __device__ __forceinline__ float round(float x) { return x; }
    static __device__ __forceinline__ void widen(const uint4 &raw, float *v) {
        v[0] = __uint_as_float(raw.x); v[1] = __uint_as_float(raw.y);
        v[2] = __uint_as_float(raw.z); v[3] = __uint_as_float(raw.w);
    }
    // The largest of the 16 bytes' logits and `m`; a NaN is passed over.
    static __device__ __forceinline__ float max_of(const uint4 &raw, float m) {
        return fmaxf(fmaxf(fmaxf(m, __uint_as_float(raw.x)), fmaxf(__uint_as_float(raw.y), __uint_as_float(raw.z))),
                     __uint_as_float(raw.w));
    }
    // True when one of the 16 bytes' logits is above `limit` (not below it when `inclusive`) or is a NaN.
    static __device__ __forceinline__ bool any_past(const uint4 &raw, float limit, bool inclusive) {
        const float a = __uint_as_float(raw.x), b = __uint_as_float(raw.y), c = __uint_as_float(raw.z),
                    d = __uint_as_float(raw.w);
        return inclusive ? (!(a < limit) || !(b < limit) || !(c < limit) || !(d < limit))
                         : (!(a <= limit) || !(b <= limit) || !(c <= limit) || !(d <= limit));
    }
};
template <> struct Logit<__half> {
    static constexpr uint32_t kLowestBits = 0xfbffu;
    static __device__ __forceinline__ float round(float x) { return __half2float(__float2half_rn(x)); }
    static __device__ __forceinline__ void widen(const uint4 &raw, float *v) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[i]));
            v[2 * i] = f.x;
            v[2 * i + 1] = f.y;
        }
    }
    static __device__ __forceinline__ float max_of(const uint4 &raw, float m) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        const __half2 a = __hmax2(*reinterpret_cast<const __half2 *>(&w[0]), *reinterpret_cast<const __half2 *>(&w[1]));
        const __half2 b = __hmax2(*reinterpret_cast<const __half2 *>(&w[2]), *reinterpret_cast<const __half2 *>(&w[3]));
        const float2 f = __half22float2(__hmax2(a, b));
        return fmaxf(m, fmaxf(f.x, f.y));
    }
    // The NaN-propagating packed maximum of the eight logits decides: past the limit, or a NaN, or neither.
    static __device__ __forceinline__ bool any_past(const uint4 &raw, float limit, bool inclusive) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        const __half2 a = __hmax2_nan(*reinterpret_cast<const __half2 *>(&w[0]), *reinterpret_cast<const __half2 *>(&w[1]));
        const __half2 b = __hmax2_nan(*reinterpret_cast<const __half2 *>(&w[2]), *reinterpret_cast<const __half2 *>(&w[3]));
        const float2 f = __half22float2(__hmax2_nan(a, b));
        return inclusive ? (!(f.x < limit) || !(f.y < limit)) : (!(f.x <= limit) || !(f.y <= limit));
    }
};
template <> struct Logit<__nv_bfloat16> {
    static constexpr uint32_t kLowestBits = 0xff7fu;
    static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
    static __device__ __forceinline__ void widen(const uint4 &raw, float *v) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            v[2 * i] = __uint_as_float(w[i] << 16);
            v[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ float max_of(const uint4 &raw, float m) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        const __nv_bfloat162 a = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&w[1]));
        const __nv_bfloat162 b = __hmax2(*reinterpret_cast<const __nv_bfloat162 *>(&w[2]),
                                         *reinterpret_cast<const __nv_bfloat162 *>(&w[3]));
        const float2 f = __bfloat1622float2(__hmax2(a, b));
        return fmaxf(m, fmaxf(f.x, f.y));
    }
    static __device__ __forceinline__ bool any_past(const uint4 &raw, float limit, bool inclusive) {
        const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
        const __nv_bfloat162 a = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162 *>(&w[0]),
                                             *reinterpret_cast<const __nv_bfloat162 *>(&w[1]));
        const __nv_bfloat162 b = __hmax2_nan(*reinterpret_cast<const __nv_bfloat162 *>(&w[2]),
                                             *reinterpret_cast<const __nv_bfloat162 *>(&w[3]));
        const __nv_bfloat162 m = __hmax2_nan(a, b);
        const uint32_t bits = *reinterpret_cast<const uint32_t *>(&m);
        const float x = __uint_as_float(bits << 16), y = __uint_as_float(bits & 0xffff0000u);
        return inclusive ? (!(x < limit) || !(y < limit)) : (!(x <= limit) || !(y <= limit));
    }
};

__device__ __forceinline__ void bulk_g2s(uint32_t dst_smem, const void *src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// Piece j of thread t of the slice in `stage`: the 16 bytes at logits base + (j * kThreads + t) * kVec.  The bulk
// copy stops at the last whole 16 bytes of the row; a piece that reaches past the row's end is put together from
// global memory, the most negative finite value standing in for what is not there.
template <typename T>
__device__ __forceinline__ uint4 piece_of(const uint8_t *stage, const T *logits, int vocab, int base, int j, int tid) {
    constexpr int kVec = 16 / sizeof(T);
    const int e0 = base + (j * kThreads + tid) * kVec;
    if (e0 + kVec <= vocab) return *reinterpret_cast<const uint4 *>(stage + (j * kThreads + tid) * 16);
    uint32_t w[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        if (sizeof(T) == 4) {
            w[i] = e0 + i < vocab ? reinterpret_cast<const uint32_t *>(logits)[e0 + i] : Logit<T>::kLowestBits;
        } else {
            const uint16_t *h = reinterpret_cast<const uint16_t *>(logits);
            const uint32_t lo = e0 + 2 * i < vocab ? h[e0 + 2 * i] : Logit<T>::kLowestBits;
            const uint32_t hi = e0 + 2 * i + 1 < vocab ? h[e0 + 2 * i + 1] : Logit<T>::kLowestBits;
            w[i] = lo | (hi << 16);
        }
    }
    return make_uint4(w[0], w[1], w[2], w[3]);
}

// Shared memory beside the ring.
struct Scratch {
    float pool_value[kSliceCandidates];     // logits gathered since the last ranking; the chunks' lists at a merge
    int pool_id[kSliceCandidates];
    alignas(16) float group_max[kMaxGroups];
    float warp_value[kThreads / 32];
    int warp_id[kThreads / 32];
    float top_value[2][kMaxTopK];           // the k best so far, best first; two sides, written in turn
    int top_id[2][kMaxTopK];
    float top_prob[kMaxTopK];
    float bound;
    int gathered[2];
    int is_last;
};

// The paths below run once per row, or a few times, or never; they are kept out of line so that the loop over
// the slices stays a few hundred instructions that the instruction cache holds.

// A lower bound of the slice's k-th largest logit: the k-th largest of the maxima of G groups of threads (k groups
// hold a logit at least that large).  G = 64 for k <= 16, else 128.  The maximum is taken over the logits as they
// are, NaNs passed over, and repaired afterwards: that can only lower a group's maximum below the one nan_to_num
// would give, which keeps the bound valid.
template <typename T>
__device__ __noinline__ float first_bound(Scratch &sh, const uint8_t *stage, const T *logits, int vocab, int base, int k,
                                          float replacement) {
    using L = Logit<T>;
    const int tid = threadIdx.x;
    float m = -INFINITY;
#pragma unroll
    for (int j = 0; j < kLoads; ++j) m = L::max_of(piece_of<T>(stage, logits, vocab, base, j, tid), m);
    if (m != m) m = 0.f;                            // unreachable with fmaxf; kept for a max that returns NaN
    else if (fabsf(m) > FLT_MAX) m = copysignf(replacement, m);
    const int group_shift = k <= 16 ? 2 : 1;        // threads per group: 4 or 2
    const int groups = kThreads >> group_shift;
    for (int o = 1; o < (1 << group_shift); o <<= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((tid & ((1 << group_shift) - 1)) == 0) sh.group_max[tid >> group_shift] = m;
    consumer_sync();
    if (tid < groups) {
        const float mine = sh.group_max[tid];
        int rank = 0;
#pragma unroll 4
        for (int j = 0; j < groups; j += 4) {
            const float4 other = *reinterpret_cast<const float4 *>(&sh.group_max[j]);
            rank += before(other.x, j, mine, tid) + before(other.y, j + 1, mine, tid) +
                    before(other.z, j + 2, mine, tid) + before(other.w, j + 3, mine, tid);
        }
        if (rank == k - 1) sh.bound = mine;
    }
    consumer_sync();
    return sh.bound;
}

// Data that defeats the limit (long runs of equal or rising values): the slice's own k best by k rounds of a
// block-wide arg-max over the slice, placed in the pool behind the `pooled` entries earlier slices left there.
// Returns the pool's new count.
template <typename T>
__device__ __noinline__ int arg_max_rounds(Scratch &sh, const uint8_t *stage, const T *logits, int vocab, int base, int k,
                                           int pooled, float replacement) {
    using L = Logit<T>;
    constexpr int kVec = 16 / sizeof(T);
    const int tid = threadIdx.x;
    uint64_t taken = 0;
    int count = pooled;
    for (int r = 0; r < k; ++r) {
        float bv = -INFINITY;
        int bi = INT_MAX, be = 0;
#pragma unroll
        for (int j = 0; j < kLoads; ++j) {
            float f[kVec];
            L::widen(piece_of<T>(stage, logits, vocab, base, j, tid), f);
            const int e0 = base + (j * kThreads + tid) * kVec;
#pragma unroll
            for (int i = 0; i < kVec; ++i) {
                const float x = replace_special(f[i], replacement);
                if (!((taken >> (j * kVec + i)) & 1ull) && e0 + i < vocab && before(x, e0 + i, bv, bi)) {
                    bv = x;
                    bi = e0 + i;
                    be = j * kVec + i;
                }
            }
        }
        float wv = bv;
        int wi = bi;
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, wv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, wi, off);
            if (before(ov, oi, wv, wi)) {
                wv = ov;
                wi = oi;
            }
        }
        if ((tid & 31) == 0) {
            sh.warp_value[tid >> 5] = wv;
            sh.warp_id[tid >> 5] = wi;
        }
        consumer_sync();
        wv = sh.warp_value[0];
        wi = sh.warp_id[0];
#pragma unroll
        for (int w = 1; w < kThreads / 32; ++w) {
            if (before(sh.warp_value[w], sh.warp_id[w], wv, wi)) {
                wv = sh.warp_value[w];
                wi = sh.warp_id[w];
            }
        }
        if (wi != INT_MAX) {
            if (wi == bi) taken |= 1ull << be;
            if (tid == 0) {
                sh.pool_value[count] = wv;
                sh.pool_id[count] = wi;
            }
            ++count;
        }
        consumer_sync();
    }
    return count;
}

// Ranks the `count` pooled logits together with the `n_top` best so far (side `side`) by counting; ranks below k
// go to the other side.  Entries with a negative id (empty slots of a list) are passed over.  Ends in a barrier.
__device__ __noinline__ void rank_pool(Scratch &sh, int count, int n_top, int side, int k) {
    const int all = count + n_top;
    for (int i = threadIdx.x; i < all; i += kThreads) {
        const float mv = i < count ? sh.pool_value[i] : sh.top_value[side][i - count];
        const int mi = i < count ? sh.pool_id[i] : sh.top_id[side][i - count];
        if (mi < 0) continue;
        int rank = 0;
#pragma unroll 4
        for (int j = 0; j < count; ++j) rank += before(sh.pool_value[j], sh.pool_id[j], mv, mi);     // an empty slot is -inf
#pragma unroll 4
        for (int j = 0; j < n_top; ++j) rank += before(sh.top_value[side][j], sh.top_id[side][j], mv, mi);
        if (rank < k) {
            sh.top_value[side ^ 1][rank] = mv;
            sh.top_id[side ^ 1][rank] = mi;
        }
    }
    consumer_sync();
}

// The k best of a whole row are in side `side`: probabilities (softmax over the k values, rounded to the logits'
// dtype as torch.softmax returns it) and the draw (inverse CDF: the first candidate whose running sum exceeds
// uniform x total), by one warp.
template <typename T>
__device__ __noinline__ void draw_row(Scratch &sh, int side, int k, const float *uniform, int64_t *out) {
    using L = Logit<T>;
    const int tid = threadIdx.x;
    if (tid >= 32) return;
    if (k == 1) {                                   // the arg-max: nothing to draw
        if (tid == 0) *out = sh.top_id[side][0];
        return;
    }
    const float mx = sh.top_value[side][0];
    const float e0 = tid < k ? expf(sh.top_value[side][tid] - mx) : 0.f;
    const float e1 = tid + 32 < k ? expf(sh.top_value[side][tid + 32] - mx) : 0.f;
    float sum = e0 + e1;
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, off);
    if (tid < k) sh.top_prob[tid] = L::round(__fdiv_rn(e0, sum));
    if (tid + 32 < k) sh.top_prob[tid + 32] = L::round(__fdiv_rn(e1, sum));
    __syncwarp();
    if (tid == 0) {
        int pick = 0;
        if (k > 1) {
            float all = 0.f;
            for (int j = 0; j < k; ++j) all += sh.top_prob[j];
            const float target = *uniform * all;
            float run = 0.f;
            pick = k - 1;
            for (int j = 0; j < k; ++j) {
                run += sh.top_prob[j];
                if (run > target) {
                    pick = j;
                    break;
                }
            }
        }
        *out = sh.top_id[side][pick];
    }
    __syncwarp();
}

// End of a CTA's part of a row that several CTAs share: the part's k best (side `side`, n_top of them) go to slot
// `slot` of the row's list in global memory; the last of the `parts` to arrive (a ticket per row, reset by it)
// ranks all lists into the other side and returns true.
__device__ __noinline__ bool hand_over_part(Scratch &sh, float *row_value, int32_t *row_id, uint32_t *ticket, int slot,
                                            int parts, int n_top, int side, int k) {
    const int tid = threadIdx.x;
    for (int r = tid; r < k; r += kThreads) {
        row_value[slot * k + r] = r < n_top ? sh.top_value[side][r] : -INFINITY;
        row_id[slot * k + r] = r < n_top ? sh.top_id[side][r] : -1;
    }
    __threadfence();
    consumer_sync();
    if (tid == 0) sh.is_last = atomicAdd(ticket, 1u) == static_cast<uint32_t>(parts - 1);
    consumer_sync();
    if (!sh.is_last) return false;
    __threadfence();
    const int total = parts * k;                    // at most kSliceCandidates: the pool is idle here
    for (int i = tid; i < total; i += kThreads) {
        sh.pool_value[i] = __ldcg(row_value + i);
        sh.pool_id[i] = __ldcg(row_id + i);
    }
    if (tid == 0) *ticket = 0;                      // every part has arrived: ready for the next launch
    consumer_sync();
    rank_pool(sh, total, 0, side, k);
    return true;
}

template <typename T>
__global__ void __launch_bounds__(kBlockThreads, 2) top_k_sample_kernel(const SampleParams p) {
    using L = Logit<T>;
    constexpr int kVec = 16 / sizeof(T);
    constexpr int kSlice = kThreads * kLoads * kVec;
    extern __shared__ __align__(128) uint8_t ring[];        // kStages slices
    __shared__ uint64_t full[kStages];                      // the slice of a stage has landed
    __shared__ uint64_t empty[kStages];                     // every examining thread is done with the stage
    __shared__ int copies_lost;                             // the copy warp gave up waiting for a stage
    __shared__ Scratch sh;

    const int tid = threadIdx.x;
    const int k = p.top_k;
    const int64_t grid = gridDim.x;
    const int64_t item_begin = blockIdx.x * p.items / grid;
    const int n_items = static_cast<int>((blockIdx.x + 1) * p.items / grid - item_begin);
    const T *const all_logits = static_cast<const T *>(p.logits) + p.first_row * p.row_stride;
    const float replacement = L::round(1e4f);
    if (tid < 2) sh.gathered[tid] = 0;

    // The ring: the copy warp (the last warp of the CTA, one lane) starts the copy of this CTA's t-th slice into
    // stage t % kStages as soon as the slice that was there has been examined — across the ends of rows, so the
    // copies never stop while the CTA has work.  A warp of its own, because fence + expect + issue take a thread
    // ≈850 clocks per slice: done by thread 0 of the examining threads, that chain stood between every two slices
    // of the whole CTA (all wait for thread 0 at the next barrier) and made a slice cost ≈2000 clocks, of which the
    // data was waited for during 400.  Every wait is bounded: a thread that gives up stops waiting, examines
    // whatever the stage holds (all accesses stay inside the ring and the rows) and the launch reports
    // NPD_STATUS_WAIT_TIMEOUT; the copy warp then gives the copies it started a last bounded chance to land.
    const int64_t row_bytes = static_cast<int64_t>(p.vocab) * sizeof(T);
    int64_t copy_row = item_begin / p.slices;           // thread 0: the slice the next copy brings in
    int copy_slice = static_cast<int>(item_begin - copy_row * p.slices);
    auto start_copy = [&](int t) {                      // called for t = 0, 1, 2, ... in order
        const int64_t byte0 = static_cast<int64_t>(copy_slice) * kSliceBytes;
        const int64_t left = row_bytes - byte0;
        const uint32_t bytes = left >= kSliceBytes ? kSliceBytes : static_cast<uint32_t>(left & ~15ll);
        const uint32_t bar = npd::smem_u32(&full[t % kStages]);
        if (bytes) {
            npd::mbar_expect_tx(bar, bytes);
            bulk_g2s(npd::smem_u32(ring + (t % kStages) * kSliceBytes),
                     reinterpret_cast<const uint8_t *>(all_logits + copy_row * p.row_stride) + byte0, bytes, bar);
        } else {
            npd::mbar_arrive(bar);                      // fewer than 16 bytes of the row left: read piecewise
        }
        if (++copy_slice == p.slices) {
            copy_slice = 0;
            ++copy_row;
        }
    };
    // The CTA that owns global slice number i: the g with g * items / grid <= i < (g + 1) * items / grid.
    auto owner_of = [&](int64_t i) { return ((i + 1) * grid - 1) / p.items; };

    if (tid == 0) {
        for (int i = 0; i < kStages; ++i) {
            npd::mbar_init(npd::smem_u32(&full[i]), 1);
            npd::mbar_init(npd::smem_u32(&empty[i]), 1);
        }
        copies_lost = 0;
        npd::mbar_fence_init();
    }
    __syncthreads();                                    // all kBlockThreads: the only barrier the copy warp takes part in
    if (tid >= kThreads) {
        // ---- the copy warp ----
        if (tid == kThreads) {
            npd::fence_proxy_async_smem();
            bool gave_up = false;
            int t = 0;
            for (; t < n_items && !gave_up; ++t) {
                if (t >= kStages) {
                    if (!npd::mbar_wait_bounded(npd::smem_u32(&empty[t % kStages]), ((t / kStages) - 1) & 1, kWaitLimit)) {
                        gave_up = true;
                        break;
                    }
                    npd::fence_proxy_async_smem();
                }
                start_copy(t);
            }
            if (gave_up) {
                *reinterpret_cast<volatile int *>(&copies_lost) = 1;
                if (p.status) atomicOr(p.status, NPD_STATUS_WAIT_TIMEOUT);
            }
            // the copies in flight write into this CTA's shared memory: they must have landed before it is given up
            for (int u = (t > kStages ? t - kStages : 0); u < t; ++u)
                npd::mbar_wait_bounded(npd::smem_u32(&full[u % kStages]), (u / kStages) & 1, kWaitLimit);
        }
        return;
    }

    // This CTA's run of slices may start and end inside a row; a stretch of one row is a "part".  The part's k best
    // so far live in side `side` of the scratch, best first; n_top of them, and `tau` is the k-th.  A later slice of
    // the part only has to look at logits ABOVE tau: its ids are all larger than the ids seen, so an equal value
    // ranks behind.  What it finds collects in the pool (counter gathered[bank]) and is ranked together with the k
    // best so far once there are max(k, 8) of them (enough to move tau), or at the part's end — an older, lower tau
    // only lets a few more logits through.
    int n_top = 0, side = 0, bank = 0, pooled = 0;
    float tau = -INFINITY;
    bool lost = false;
    int row = static_cast<int>(item_begin / p.slices);
    int s = static_cast<int>(item_begin - static_cast<int64_t>(row) * p.slices);
    for (int t = 0; t < n_items; ++t, ++s) {
        if (s == p.slices) {
            s = 0;
            ++row;
        }
        const bool first = t == 0 || s == 0;
        const bool last = t == n_items - 1 || s == p.slices - 1;
        const uint8_t *stage = ring + (t % kStages) * kSliceBytes;
        const T *logits = all_logits + row * p.row_stride;
        const int base = s * kSlice;
        if (!lost && (*reinterpret_cast<volatile int *>(&copies_lost) ||
                      !npd::mbar_wait_bounded(npd::smem_u32(&full[t % kStages]), (t / kStages) & 1, kWaitLimit)))
            lost = true;

        float limit = tau;
        if (first) {
            n_top = 0;
            pooled = 0;
            tau = -INFINITY;
            limit = first_bound<T>(sh, stage, logits, p.vocab, base, k, replacement);
        }

        // ---- gather the logits past the limit (not below it in the first slice, above it later) ---------------
        // -inf only matters when its replacement, -1e4, would pass the limit.  First one bit per 16-byte piece, all
        // eight pieces independent of each other; then the few pieces that hold something.
        const bool careful = limit < -replacement || (first && limit == -replacement);
        unsigned hits = 0;
        if (base + kSlice <= p.vocab) {
#pragma unroll
            for (int j = 0; j < kLoads; ++j) {
                const uint4 raw = *reinterpret_cast<const uint4 *>(stage + (j * kThreads + tid) * 16);
                hits |= static_cast<unsigned>(L::any_past(raw, limit, first)) << j;
            }
        } else {
#pragma unroll
            for (int j = 0; j < kLoads; ++j)
                hits |= static_cast<unsigned>(L::any_past(piece_of<T>(stage, logits, p.vocab, base, j, tid), limit, first)) << j;
        }
        if (careful) hits = (1u << kLoads) - 1;
        while (hits) {
            const int j = __ffs(hits) - 1;
            hits &= hits - 1;
            float f[kVec];
            L::widen(piece_of<T>(stage, logits, p.vocab, base, j, tid), f);
            const int e0 = base + (j * kThreads + tid) * kVec;
#pragma unroll
            for (int i = 0; i < kVec; ++i) {
                const float x = replace_special(f[i], replacement);
                if ((first ? x >= limit : x > limit) && e0 + i < p.vocab) {
                    const int pos = atomicAdd(&sh.gathered[bank], 1);
                    if (pos < kSliceCandidates) {
                        sh.pool_value[pos] = x;
                        sh.pool_id[pos] = e0 + i;
                    }
                }
            }
        }
        consumer_sync();
        int count = sh.gathered[bank];
        if (count > kSliceCandidates)
            count = arg_max_rounds<T>(sh, stage, logits, p.vocab, base, k, pooled, replacement);
        pooled = count;
        // Every read of the stage lies before a barrier all examining threads have passed: the stage can be refilled.
        if (tid == 0) npd::mbar_arrive(npd::smem_u32(&empty[t % kStages]));

        if (count > 0 && (first || count >= (k > 8 ? k : 8) || last)) {
            if (tid == 0) sh.gathered[bank ^ 1] = 0;    // last read before the previous ranking's closing barrier
            rank_pool(sh, count, n_top, side, k);
            n_top = count + n_top < k ? count + n_top : k;
            side ^= 1;
            bank ^= 1;
            pooled = 0;
            if (n_top == k) tau = sh.top_value[side][k - 1];
        }

        if (last) {
            // A row that one CTA saw whole is drawn at once; otherwise the last part to arrive merges and draws.
            const int64_t first_owner = owner_of(static_cast<int64_t>(row) * p.slices);
            const int parts = static_cast<int>(owner_of(static_cast<int64_t>(row + 1) * p.slices - 1) - first_owner) + 1;
            bool whole = true;
            if (parts > 1) {
                whole = hand_over_part(sh, p.cand_value + static_cast<int64_t>(row) * p.parts_cap * k,
                                       p.cand_id + static_cast<int64_t>(row) * p.parts_cap * k, p.tickets + row,
                                       static_cast<int>(blockIdx.x - first_owner), parts, n_top, side, k);
                if (whole) side ^= 1;
            }
            if (whole) draw_row<T>(sh, side, k, p.uniforms ? p.uniforms + p.first_row + row : nullptr, p.out + p.first_row + row);
        }
    }
    if (lost && p.status) atomicOr(p.status, NPD_STATUS_WAIT_TIMEOUT);
}

int slices_of(int64_t vocab, int slice) { return static_cast<int>((vocab + slice - 1) / slice); }

// How one launch is dealt out: rows x slices items in equal consecutive runs, at most two CTAs per SM.  While the
// rows fit, every row gets the same whole number of CTAs, so that no run crosses a row's end (a run that does pays
// a hand-over and a merge for both rows: 27 us against 22.5 us at 256 rows of 151 936 bf16 logits); beyond that
// all 2 x SMs CTAs take equal runs, fewer where a row would otherwise be spread over more parts than the merge
// has room for.
struct Plan {
    int slices;
    int64_t items;
    int grid;
    int parts_cap;
};

Plan plan_for(int64_t rows, int64_t vocab, int elem, int top_k, int sms) {
    Plan plan;
    plan.slices = slices_of(vocab, kThreads * kLoads * (16 / elem));
    plan.items = rows * plan.slices;
    const int max_parts = kSliceCandidates / top_k;
    static const int64_t forced = [] {                                         // for experiments; read once per process
        const char *env = getenv("NPD_SAMPLE_CTAS");
        return env ? atoll(env) : 0LL;
    }();
    if (rows <= 2 * sms && (forced < 1 || forced > plan.items)) {
        int64_t per_row = 2 * sms / rows;
        if (per_row > plan.slices) per_row = plan.slices;
        if (per_row > max_parts) per_row = max_parts;
        plan.grid = static_cast<int>(rows * per_row);
        plan.parts_cap = static_cast<int>(per_row);
        return plan;
    }
    int64_t grid = plan.items < 2 * sms ? plan.items : 2 * sms;
    if (forced >= 1 && forced <= plan.items) grid = forced;
    int parts = 1;
    for (;; --grid) {
        const int64_t shortest = plan.items / grid;                         // a run is at least this long
        parts = static_cast<int>((plan.slices + shortest - 1) / shortest) + 1;
        if (parts > plan.slices) parts = plan.slices;
        if (parts <= max_parts || grid == 1) break;
    }
    plan.grid = static_cast<int>(grid);
    plan.parts_cap = parts;
    return plan;
}

int sms_of_current_device() {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 148;
    const int sms = npd::sm_count(device);
    return sms > 0 ? sms : 148;
}

template <typename T>
cudaError_t launch(const SampleParams &p, unsigned grid, cudaStream_t stream) {
    constexpr int kRingBytes = kStages * kSliceBytes;
    // Set on every call: the attribute is per device and cheap; the maximum carve-out lets two CTAs share an SM.
    cudaError_t e = cudaFuncSetAttribute(top_k_sample_kernel<T>, cudaFuncAttributeMaxDynamicSharedMemorySize, kRingBytes);
    if (e != cudaSuccess) return e;
    e = cudaFuncSetAttribute(top_k_sample_kernel<T>, cudaFuncAttributePreferredSharedMemoryCarveout,
                             cudaSharedmemCarveoutMaxShared);
    if (e != cudaSuccess) return e;
    top_k_sample_kernel<T><<<grid, kBlockThreads, kRingBytes, stream>>>(p);
    return cudaGetLastError();
}

}  // namespace

extern "C" int64_t npd_top_k_sample_workspace_bytes(int64_t num_rows, int64_t vocab, int top_k) {
    if (num_rows <= 0 || vocab <= 0 || top_k <= 0 || top_k > kMaxTopK) return kTicketBytes;
    const int64_t rows = num_rows < kRowsPerLaunch ? num_rows : kRowsPerLaunch;
    const int sms = sms_of_current_device();
    const int a = plan_for(rows, vocab, 2, top_k, sms).parts_cap, b = plan_for(rows, vocab, 4, top_k, sms).parts_cap;
    return kTicketBytes + rows * (a > b ? a : b) * top_k * 8;               // whichever dtype the logits have
}

extern "C" int npd_top_k_sample(int64_t *out_ids, const void *logits, const float *uniforms, int64_t num_rows,
                                int64_t vocab, int64_t row_stride, int top_k, int dtype, void *workspace,
                                int64_t workspace_bytes, void *stream) {
    NPD_REQUIRE(dtype == NPD_DTYPE_F16 || dtype == NPD_DTYPE_BF16 || dtype == NPD_DTYPE_F32, NPD_ERR_UNSUPPORTED,
                "npd_top_k_sample: unsupported dtype code %d", dtype);
    NPD_REQUIRE(num_rows >= 0 && vocab > 0, NPD_ERR_INVALID_ARG, "npd_top_k_sample: non-positive dimension");
    NPD_REQUIRE(top_k >= 1 && top_k <= kMaxTopK, NPD_ERR_UNSUPPORTED, "npd_top_k_sample: top_k %d not in [1, %d]",
                top_k, kMaxTopK);
    NPD_REQUIRE(top_k <= vocab, NPD_ERR_INVALID_ARG, "npd_top_k_sample: top_k %d exceeds the vocabulary %lld", top_k,
                (long long)vocab);
    NPD_REQUIRE(vocab <= (1LL << 30), NPD_ERR_UNSUPPORTED, "npd_top_k_sample: vocabulary %lld too large",
                (long long)vocab);
    if (num_rows == 0) return NPD_OK;
    const int elem = dtype == NPD_DTYPE_F32 ? 4 : 2;
    NPD_REQUIRE(out_ids && logits && workspace, NPD_ERR_INVALID_ARG, "npd_top_k_sample: NULL pointer");
    NPD_REQUIRE(uniforms || top_k == 1, NPD_ERR_INVALID_ARG, "npd_top_k_sample: top_k > 1 needs uniform numbers");
    NPD_REQUIRE(row_stride >= vocab, NPD_ERR_INVALID_ARG, "npd_top_k_sample: row stride smaller than the vocabulary");
    NPD_REQUIRE(npd::aligned16(logits) && (num_rows == 1 || (row_stride * elem) % 16 == 0), NPD_ERR_INVALID_ARG,
                "npd_top_k_sample: rows of logits must start on 16-byte boundaries");
    NPD_REQUIRE(npd::aligned16(workspace), NPD_ERR_INVALID_ARG, "npd_top_k_sample: workspace must be 16-byte aligned");
    NPD_REQUIRE(workspace_bytes >= npd_top_k_sample_workspace_bytes(num_rows, vocab, top_k), NPD_ERR_WORKSPACE,
                "npd_top_k_sample: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                (long long)npd_top_k_sample_workspace_bytes(num_rows, vocab, top_k));
    const int sms = sms_of_current_device();

    SampleParams p;
    p.logits = logits;
    p.uniforms = uniforms;
    p.out = out_ids;
    p.status = static_cast<int32_t *>(workspace);
    p.tickets = reinterpret_cast<uint32_t *>(static_cast<char *>(workspace) + kTicketOffset);
    p.row_stride = row_stride;
    p.vocab = static_cast<int>(vocab);
    p.top_k = top_k;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    for (int64_t first = 0; first < num_rows; first += kRowsPerLaunch) {
        const int64_t rows = num_rows - first < kRowsPerLaunch ? num_rows - first : kRowsPerLaunch;
        const Plan plan = plan_for(rows, vocab, elem, top_k, sms);
        NPD_REQUIRE(plan.parts_cap * top_k <= kSliceCandidates, NPD_ERR_UNSUPPORTED,
                    "npd_top_k_sample: vocabulary %lld x top_k %d needs more than %d candidates per row",
                    (long long)vocab, top_k, kSliceCandidates);
        p.slices = plan.slices;
        p.items = plan.items;
        p.parts_cap = plan.parts_cap;
        p.first_row = first;
        p.cand_value = reinterpret_cast<float *>(static_cast<char *>(workspace) + kTicketBytes);
        p.cand_id = reinterpret_cast<int32_t *>(p.cand_value + rows * plan.parts_cap * top_k);
        const unsigned grid = static_cast<unsigned>(plan.grid);
        if (dtype == NPD_DTYPE_F16) NPD_CUDA_TRY(launch<__half>(p, grid, s));
        else if (dtype == NPD_DTYPE_BF16) NPD_CUDA_TRY(launch<__nv_bfloat16>(p, grid, s));
        else NPD_CUDA_TRY(launch<float>(p, grid, s));
    }
    return NPD_OK;
}
