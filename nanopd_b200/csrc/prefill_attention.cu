// Kernel 3: chunked-prefill causal attention over paged K/V on the 5th-generation tensor cores.
//
// A work item is a PAIR of 128-row query tiles of one chunk and one kv head: the rows of a tile are
// TQ = 128/G consecutive query tokens times the G q heads that share the kv head (token-major), so every
// K/V tile read from the pages serves the whole group and both tiles.  Keys are walked in tiles of 128
// (8 pages of 16 tokens) from position 0 up to the tile's last query position — earlier chunks are read
// from the pages like any other key, which the reference's prefill branch does not do
// (nanoPD/engine/model_runner.py:125-127,152-168 attends to the current chunk only).
//
// Persistent grid, one CTA of 512 threads per SM; items are handed out heaviest first through an atomic
// counter.  Warp roles:
//   warps 0-3 / 4-7  softmax of query tile A / B: thread i owns row i == TMEM lane i (no shuffles)
//   warp  8          TMA producer of the K tiles (a ring of 3 tiles in shared memory; cp.async.bulk.tensor,
//                    128-byte swizzle = the canonical UMMA operand layout); it also draws the next work item,
//                    decodes it and publishes it to the other roles
//   warp  11         TMA producer of the V tiles (a ring of 2 tiles).  Two producer warps, because the rate at
//                    which ONE warp can issue tiled copies (about 100 clocks per 2 KiB box) is what bounded the
//                    kernel when a single warp issued the 32 boxes of a 128-key step
//   warps 9 / 10     issue the tcgen05.mma instructions of tile A / B (one elected lane) and request the tile's
//                    query rows (the next item's as soon as this item's last score MMA has completed)
//   warps 12-15      epilogue of both tiles: O / l -> out, while the softmax groups are already on the next item
// TMEM (512 columns): S_A | S_B | O_A | O_B, 128 columns each.  A query tile walks its keys in HALF-STEPS of 64
// keys; its 128 score columns are a ring of two 64-column buffers, so the scores of half-step c+1 are
// already in TMEM while the softmax group works on half-step c, and those of c+2 are computed while the
// PV product of c+1 waits for its probabilities:
//   S(c) = Q.K(c)^T      tcgen05.mma M128 N64, both operands in shared memory, fp32 scores in buffer c&1
//   P(c) = exp2(S*scale - m), rounded to the input type and written back over the first 32 columns of
//          the buffer (masking only on half-steps that touch the diagonal)
//   O   += P(c).V(c)      tcgen05.mma with P as the TMEM A operand and V as the MN-major B operand; then
//          S(c+2) is issued into the buffer P(c) has just left (MMAs execute in issue order)
// O stays in TMEM and is rescaled only when a row maximum grows by more than 2^8 (after waiting for the
// PV products issued so far), then read once by the epilogue warps.
// Completion of MMAs is tracked with tcgen05.commit on mbarriers; every wait is bounded and an
// abort flag lets all roles leave together, after which TMEM is released.
//
// Algorithmic flops per chunk: 4*Hq*D*(n*start + n(n+1)/2)  (causal; masked work not counted).
#include <algorithm>
#include <vector>

#include "npd_common.cuh"

namespace {

using namespace npd;

constexpr int kMaxChunks = 64;     // chunks per launch (kernel-parameter arrays)
constexpr int kMaxPairs = 2048;    // query-tile pairs per launch (kernel-parameter array, heaviest first)
constexpr int kSchedSlots = 4;     // work items the producer may publish ahead of the slowest consumer
constexpr int kRows = 128;         // UMMA M: rows of one query tile
constexpr int kKeys = 128;         // keys per K/V tile in shared memory (64 at head_dim 256)
constexpr int kHalfKeys = 64;      // keys per half-step (UMMA N of a score MMA, K extent of a PV MMA batch)
constexpr int kThreads = 512;      // warps 0-3 softmax A, 4-7 softmax B, 8 TMA (K), 9 MMA + Q for A, 10 MMA + Q for B, 11 TMA (V),
                                   // 12-15 epilogue
constexpr int kQHalfBytes = kRows * 128;            // one 64-element half of a 128-row query tile
// head_dim kD = 64 * kHalves (64, 128 or 256): a tile is kHalves slabs, each 64 elements wide.  At head_dim 256 an
// item is ONE query tile (two tiles' accumulators, 2 x 256 columns, would not fit the 512 TMEM columns beside the
// scores) and a K/V tile holds 64 keys (one half-step), so that the rings still fit shared memory.
template <int kD> struct TileBytes {
    static constexpr int kHalves = kD / 64;
    static constexpr int kTileKeys = kD == 256 ? 64 : kKeys;
    static constexpr int kQueryTiles = kD == 256 ? 1 : 2;
    static constexpr int kvSlab = kTileKeys * 128;      // one 64-element-wide slab of a K or V tile
    static constexpr int q = kHalves * kQHalfBytes;     // 32 KiB at head_dim 128
    static constexpr int kv = kHalves * kvSlab;         // 32 KiB at head_dim 128 and 256
};
#ifndef NPD_K_STAGES
#define NPD_K_STAGES 3
#endif
#ifndef NPD_V_STAGES
#define NPD_V_STAGES 2
#endif
constexpr int kStagesK = NPD_K_STAGES;              // K ring depth
constexpr int kStagesV = NPD_V_STAGES;              // V ring depth
constexpr int kTmemCols = 512;     // S_A | S_B | O_A | O_B, 128 columns each; a tile's score columns are two buffers of
                                   // 64; the packed probabilities of a half-step overwrite the first 32 of its buffer
constexpr float kRescaleThreshold = 8.f;   // log2 units: O is rescaled only when a row max grows by more
constexpr long long kWaitCycles = 4000000000LL;

struct PrefillParams {
    void *out;
    const int32_t *block_tables;
    int32_t *status;
    float scale_log2;
    int num_chunks;
    int num_q_heads, num_kv_heads, group;
    int tq;                 // query tokens per 128-row tile = 128 / group (floor)
    int block_size;
    int box_rows;           // rows of a K/V TMA box: 16, or the block size when that is 8 or 4
    int query_tiles;        // query tiles per work item (2; 1 at head_dim 256)
    int half_steps_per_tile;   // 64-key half-steps per K/V tile (2; 1 at head_dim 256)
    int max_blocks_per_seq;
    int num_blocks;
    long long bt_row_stride;
    int chunk_q_offset[kMaxChunks];
    int chunk_tokens[kMaxChunks];
    int chunk_start[kMaxChunks];
    int num_pairs;                    // entries of pair_order
    int *work_counter;                // two device int32, zero before the launch and put back to zero by its last
                                      // CTA: [0] items handed out beyond the first gridDim.x, [1] CTAs that have left
    uint32_t pair_order[kMaxPairs];   // (chunk << 16 | pair of query tiles), sorted by key tiles, heaviest first
#ifdef NPD_PREFILL_TRACE
    long long *trace;
#endif
};

// ---- tcgen05 wrappers ---------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols)
                 : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .b32 r;\n\t.reg .pred p;\n\telect.sync r|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] * B[smem]
__device__ __forceinline__ void tc_mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// D[tmem] (+)= A[tmem] * B[smem]   (A: 128 lanes x K/2 columns of packed 16-bit pairs, K-major)
__device__ __forceinline__ void tc_mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc,
                                          uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, {%5, %5, %5, %5}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u)
        : "memory");
}
// 32 lanes x 32 consecutive 32-bit columns: thread i of the warp receives lane (base + i).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
    uint32_t *r = reinterpret_cast<uint32_t *>(v);
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
        "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
    const uint32_t *r = reinterpret_cast<const uint32_t *>(v);
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
        "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]),
          "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]), "r"(r[21]), "r"(r[22]), "r"(r[23]),
          "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]), "r"(r[31])
        : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
          "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
// One 256-bit store (sm_100: st.global.v8.b32); the address must be 32-byte aligned.  The output is written once
// and not read again by this kernel: no L1 allocation (+0.9 % on configuration 3).
__device__ __forceinline__ void st_global_32B(void *ptr, const uint32_t (&w)[8]) {
    asm volatile("st.global.L1::no_allocate.v8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};" ::"l"(ptr), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
                 "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
                 : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Packed fp32x2 arithmetic (__ffma2_rn / __fadd2_rn: two lanes per instruction on sm_100) halves the
// issue slots of the scale-and-subtract and of the row sum.
//
// 2^x for a pair on the FMA pipes instead of the special-function unit.  x = n + f with n = round(x) (taken from
// the low mantissa bits after adding 1.5 * 2^23), f in [-0.5, 0.5]; 2^f by a cubic (max relative error 7.5e-5,
// far below the rounding of P to a 16-bit type); n is added to the exponent field.  x is clamped at -125
// (result ~2e-38, i.e. 0 for every purpose here).  Every kPolyExpEvery-th pair of a half-step's probabilities is
// computed this way: the special-function unit shares its instruction queue with the TMEM, barrier and TMA
// instructions, and a quarter of the exponentials moved off it measured fastest (none: -2.4 %, half: -2.5 %).
#ifndef NPD_POLY_EXP_EVERY
#define NPD_POLY_EXP_EVERY 4
#endif
constexpr int kPolyExpEvery = NPD_POLY_EXP_EVERY;
__device__ __forceinline__ float2 exp2_fma2(float2 x) {
    x.x = fmaxf(x.x, -125.f);
    x.y = fmaxf(x.y, -125.f);
    const float2 t = __fadd2_rn(x, make_float2(12582912.f, 12582912.f));
    const float2 n = __fadd2_rn(t, make_float2(-12582912.f, -12582912.f));
    const float2 f = __ffma2_rn(n, make_float2(-1.f, -1.f), x);
    float2 q = __ffma2_rn(f, make_float2(0.055171460f, 0.055171460f), make_float2(0.24261086f, 0.24261086f));
    q = __ffma2_rn(q, f, make_float2(0.69326097f, 0.69326097f));
    q = __ffma2_rn(q, f, make_float2(0.99992812f, 0.99992812f));
    return make_float2(__int_as_float(__float_as_int(q.x) + (__float_as_int(t.x) << 23)),
                       __int_as_float(__float_as_int(q.y) + (__float_as_int(t.y) << 23)));
}
__device__ __forceinline__ float fmax3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

// Shared-memory matrix descriptors (version 1, 128-byte swizzle, 8-row groups 1024 B apart).
__device__ __forceinline__ uint64_t desc_k_major(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// MN-major operand: 64-element atoms `lbo_bytes` apart along MN, 8-row groups 1024 B apart along K.
__device__ __forceinline__ uint64_t desc_mn_major(uint32_t saddr, uint32_t lbo_bytes) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) | (64ull << 32) | (1ull << 46) |
           (2ull << 61);
}
// Instruction descriptor: fp32 accumulate, A/B of type `fmt` (0 = f16, 1 = bf16), M x N tile.
__host__ __device__ constexpr uint32_t instr_desc(uint32_t fmt, uint32_t b_mn_major, uint32_t M, uint32_t N) {
    return (1u << 4) | (fmt << 7) | (fmt << 10) | (b_mn_major << 16) | ((N >> 3) << 17) | ((M >> 4) << 24);
}

// Bounded, abortable mbarrier wait shared by all roles.
__device__ __forceinline__ bool wait_or_abort(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                              int32_t *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (*abort_flag) return false;
        if (clock64() - t0 > kWaitCycles) {
            *abort_flag = 1;
            atomicOr(status, NPD_STATUS_WAIT_TIMEOUT);
            return false;
        }
    }
    return true;
}

// Optional phase tracing for performance work (compiled out unless NPD_PREFILL_TRACE is defined):
// the CTA with blockIdx.x == 0 appends (tag, key tile, clock) triples to the workspace after its header.
#ifdef NPD_PREFILL_TRACE
#define NPD_TRACE_DECL int trace_n_ = 0;
#define NPD_TRACE(role, tag, j)                                                                   \
    do {                                                                                          \
        if (blockIdx.x == NPD_PREFILL_TRACE && p.trace && trace_n_ < 2040) {                      \
            longlong2 e_;                                                                         \
            e_.x = (static_cast<long long>(tag) << 32) | static_cast<unsigned>(j);               \
            e_.y = clock64();                                                                     \
            reinterpret_cast<longlong2 *>(p.trace + (role) * 4096)[trace_n_++] = e_;              \
        }                                                                                         \
    } while (0)
#else
#define NPD_TRACE_DECL
#define NPD_TRACE(role, tag, j) do { } while (0)
#endif
#ifdef NPD_PREFILL_TRACE_FINE
#define NPD_TRACE_FINE(role, tag, j) NPD_TRACE(role, tag, j)
#else
#define NPD_TRACE_FINE(role, tag, j) do { } while (0)
#endif

// One work item = a pair of 128-row query tiles of one chunk and one kv head.
struct Item {
    int c, h;
    int start, qoff, ctx_end;
    int tok0[2], tq_valid[2];
    int nhalf[2];           // half-steps of 64 keys each query tile takes (keys [0, start + tok0 + tq_valid))
    int ntiles[2];          // K/V tiles of 128 keys they lie in
    int n_kv;
};

struct alignas(8) SmemCtrl {
    uint64_t sched_full[kSchedSlots];   // the producer warp has published the next work item
    int sched_item[kSchedSlots];
    Item sched_desc[kSchedSlots];       // the published item, decoded once by the producer warp: the other roles'
                                        // way from one item to the next stays a few loads (their decoding it
                                        // themselves — divisions, indexed kernel parameters, cold code — took a
                                        // softmax group ~2500 clocks per item)
    uint64_t q_full[2];          // [query tile]: its rows of the current work item have landed
    uint64_t q_empty[2];         // [query tile]: its MMA warp has issued the last score MMA of the item
    uint64_t k_full[kStagesK], v_full[kStagesV];     // the K / V tile of a ring stage has landed
    uint64_t k_empty[kStagesK], v_empty[kStagesV];   // both MMA warps are done with it (2 arrivals)
    uint64_t s_full[2][2];  // [query tile][buffer]: the scores of a half-step are in that buffer (and the PV product
                            // that last read the buffer has completed)
    uint64_t p_ready[2][2]; // [query tile][buffer]: the probabilities of the half-step are in TMEM (128 arrivals)
    uint64_t pv_done[2][2]; // [query tile][buffer]: one completion per PV product that read that buffer, in order.  Two
                            // barriers, because a waiter may find either one or two products still in flight and a
                            // parity wait cannot tell "two behind" from "done"
    uint64_t o_free[2];     // [query tile]: the epilogue has taken O out of TMEM (128 arrivals)
    uint64_t epi_ready[2];  // [query tile]: the softmax group has finished the item and left its row sums (128 arrivals)
    float l_sum[2][kRows];  // [query tile][row]: the row sums of the finished item, for the epilogue warps
    uint32_t tmem_base;
    int abort_flag;
};


// Work item `item` = kv head (item % Hkv) of entry (item / Hkv) of the host-sorted pair list.
__device__ __forceinline__ Item decode_item(const PrefillParams &p, int item) {
    Item it;
    it.h = item % p.num_kv_heads;
    const uint32_t entry = p.pair_order[item / p.num_kv_heads];
    const int c = static_cast<int>(entry >> 16), pair = static_cast<int>(entry & 0xffffu);
    it.c = c;
    const int n_tok = p.chunk_tokens[c];
    it.start = p.chunk_start[c];
    it.qoff = p.chunk_q_offset[c];
    it.ctx_end = it.start + n_tok;                              // keys written so far for this sequence
#pragma unroll
    for (int x = 0; x < 2; ++x) {
        it.tok0[x] = (p.query_tiles * pair + x) * p.tq;
        it.tq_valid[x] = x < p.query_tiles ? max(0, min(p.tq, n_tok - it.tok0[x])) : 0;
        // keys [0, start + tok0 + tq_valid) are visible to the tile
        it.nhalf[x] = it.tq_valid[x] > 0 ? (it.start + it.tok0[x] + it.tq_valid[x] + kHalfKeys - 1) / kHalfKeys : 0;
        it.ntiles[x] = (it.nhalf[x] + p.half_steps_per_tile - 1) / p.half_steps_per_tile;
    }
    it.n_kv = max(it.ntiles[0], it.ntiles[1]);
    return it;
}

// Persistent kernel: one CTA per SM.  Work items are handed out heaviest first through an atomic counter (the
// producer warp fetches the next one and publishes it to the other roles through a small shared-memory ring), so
// ragged chunks balance across the SMs.  All barrier phases are driven by running counters: the producers
// already load the next item's K/V tiles (and the MMA warps, once an item's last score MMA has completed, request
// its query tiles) while the current item drains, and the epilogue of an item overlaps the first MMAs of the next.
// kBoxRows: rows of a K/V TMA box — 16, or the block size when blocks hold 8 or 4 tokens (a 16-key row group of a
// tile is then two or four boxes; the 128-byte swizzle follows the shared-memory address, so the tile in shared
// memory is the same).  A template parameter because the producer warps share their sub-partitions' issue slots
// with two softmax warps each, and every instruction they run per key tile shows in the kernel's time (the
// run-time form of this choice cost 2.3 %).
template <typename T, int kD, int kBoxRows>
__global__ void __launch_bounds__(kThreads, 1)
paged_prefill_kernel(const PrefillParams p, const __grid_constant__ CUtensorMap tm_q,
                     const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t *sbase = smem_raw + pad;
    constexpr int kHalves = TileBytes<kD>::kHalves;
    constexpr int kQTileBytes = TileBytes<kD>::q, kKvTileBytes = TileBytes<kD>::kv;
    constexpr int kTK = TileBytes<kD>::kTileKeys;               // keys per K/V tile
    constexpr int kHPT = kTK / kHalfKeys;                       // half-steps per K/V tile
    constexpr int kKvHalfBytes = TileBytes<kD>::kvSlab;         // one 64-element-wide slab of a K or V tile
    constexpr int kQueryTiles = TileBytes<kD>::kQueryTiles;
    uint8_t *q_tiles = sbase;                                   // query tiles A and B
    uint8_t *k_ring = q_tiles + kQueryTiles * kQTileBytes;      // kStagesK K tiles
    uint8_t *v_ring = k_ring + kStagesK * kKvTileBytes;         // kStagesV V tiles
    SmemCtrl *ctrl = reinterpret_cast<SmemCtrl *>(v_ring + kStagesV * kKvTileBytes);

    const int warp = __shfl_sync(0xffffffffu, static_cast<int>(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int total_items = p.num_pairs * p.num_kv_heads;
    // Consumers read the item the producer published for their k-th iteration (-1 = no more work).
    auto next_item = [&](int k, bool &ok_ref) {
        const int slot = k % kSchedSlots;
        ok_ref = wait_or_abort(smem_u32(&ctrl->sched_full[slot]), (k / kSchedSlots) & 1, &ctrl->abort_flag, p.status);
        return ok_ref ? *reinterpret_cast<volatile int *>(&ctrl->sched_item[slot]) : -1;
    };

    if (threadIdx.x == 0) {
        for (int i = 0; i < kSchedSlots; ++i) mbar_init(smem_u32(&ctrl->sched_full[i]), 1);
        for (int i = 0; i < kStagesK; ++i) {
            mbar_init(smem_u32(&ctrl->k_full[i]), 1);
            mbar_init(smem_u32(&ctrl->k_empty[i]), 2);
        }
        for (int i = 0; i < kStagesV; ++i) {
            mbar_init(smem_u32(&ctrl->v_full[i]), 1);
            mbar_init(smem_u32(&ctrl->v_empty[i]), 2);
        }
        for (int x = 0; x < 2; ++x) {
            mbar_init(smem_u32(&ctrl->q_full[x]), 1);
            mbar_init(smem_u32(&ctrl->q_empty[x]), 1);
            for (int b = 0; b < 2; ++b) {
                mbar_init(smem_u32(&ctrl->s_full[x][b]), 1);
                mbar_init(smem_u32(&ctrl->p_ready[x][b]), 128);
            }
            mbar_init(smem_u32(&ctrl->pv_done[x][0]), 1);
            mbar_init(smem_u32(&ctrl->pv_done[x][1]), 1);
            mbar_init(smem_u32(&ctrl->o_free[x]), 128);
            mbar_init(smem_u32(&ctrl->epi_ready[x]), 128);
        }
        ctrl->abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 9) {
        tmem_alloc(smem_u32(&ctrl->tmem_base), kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = ctrl->tmem_base;
    volatile int *abort_flag = &ctrl->abort_flag;

    // Register re-allocation between warpgroups (first statement of every role).  512 threads start with 128
    // registers each: the two softmax groups, which work on whole score rows in registers, go up to 168; the third
    // group (two TMA warps, two MMA warps) gives up 56 per thread and the epilogue group 24 — 65 536 in all.
    if (warp == 8 || warp == 11) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        // =========================== TMA producers: warp 8 (K tiles), warp 11 (V tiles) ===========================
        // A K or V tile is 16 boxes of 2 KiB (16-key row groups x 64-element slabs; 32 boxes of 1 KiB with blocks
        // of 8 tokens, 64 of 512 B with blocks of 4), one box per lane, issued by ONE instruction of the warp per 32.  Issuing tiled copies costs the
        // issuing warp about 50 clocks per box plus several hundred per instruction, whatever the box holds, while
        // the copy engine itself takes boxes from several warps at once: one warp issuing both tiles of a 128-key
        // step (32 boxes) needed as long as the step's arithmetic, two warps need half of it.  Each lane looks its
        // block id up one tile ahead, so the table reads are off the critical path too.
        const bool k_role = warp == 8;
        const CUtensorMap *tm = k_role ? &tm_k : &tm_v;
        if (lane == 0) {
            if (k_role) tma_prefetch_desc(&tm_q);
            tma_prefetch_desc(tm);
        }
        // box b of a tile = (16-key row group gi, 64-element slab hf, piece `sub` of the group's 16 / kBoxRows boxes when
        // blocks hold fewer than 16 tokens); lane l issues boxes l, l + 32, ... — one instruction per 32 boxes
        constexpr int kSubs = 16 / kBoxRows;
        constexpr int kBoxes = (kTK / 16) * kHalves * kSubs;
        constexpr int kIssues = (kBoxes + 31) / 32;
        int sub[kIssues], hf[kIssues], gi[kIssues];
        bool has_box[kIssues];
        uint32_t off[kIssues];
#pragma unroll
        for (int i = 0; i < kIssues; ++i) {
            const int b = i * 32 + lane, l2 = b / kSubs;
            sub[i] = b % kSubs;
            hf[i] = l2 % kHalves;
            gi[i] = l2 / kHalves;
            has_box[i] = b < kBoxes;
            off[i] = static_cast<uint32_t>(hf[i] * kKvHalfBytes + gi[i] * 2048 + sub[i] * kBoxRows * 128);
        }
        uint8_t *ring = k_role ? k_ring : v_ring;
        uint64_t *full = k_role ? ctrl->k_full : ctrl->v_full, *empty = k_role ? ctrl->k_empty : ctrl->v_empty;
        const int stages = k_role ? kStagesK : kStagesV;
        int stage = 0, round = 0;                               // ring position of the next tile
        NPD_TRACE_DECL
        bool ok = true;
        for (int k = 0; ok; ++k) {
            // Warp 8 fetches and publishes the next work item; warp 11 reads it like the other roles.  A slot is
            // reused kSchedSlots items later; by then every role has long read it (warp 8 cannot run more than
            // two items ahead of the MMA warps, which cannot run ahead of the V tiles or the softmax groups).
            int item = 0;
            if (k_role) {
                if (lane == 0) {
                    // the first item of a CTA is its own index (no round trip to the counter before the first load);
                    // the counter hands out the items behind the first gridDim.x
                    item = k == 0 ? static_cast<int>(blockIdx.x) : static_cast<int>(gridDim.x) + atomicAdd(p.work_counter, 1);
                    if (item >= total_items) item = -1;
                }
                item = __shfl_sync(0xffffffffu, item, 0);
            } else {
                item = next_item(k, ok);
                if (!__all_sync(0xffffffffu, ok)) break;
            }
            Item it;
            if (k_role) {
                if (item >= 0) it = decode_item(p, item);
                if (lane == 0) {
                    if (item >= 0) ctrl->sched_desc[k % kSchedSlots] = it;
                    *reinterpret_cast<volatile int *>(&ctrl->sched_item[k % kSchedSlots]) = item;
                    mbar_arrive(smem_u32(&ctrl->sched_full[k % kSchedSlots]));
                }
                if (item < 0) break;
            } else {
                if (item < 0) break;
                it = ctrl->sched_desc[k % kSchedSlots];
            }
            const int32_t *table = p.block_tables + (long long)it.c * p.bt_row_stride;
            // A box lies in one block: 16 keys of a block of 16 or 32, or all keys of a block of 8 or 4.
            auto lookup = [&](int t, int i) {
                const int key = t * kTK + gi[i] * 16 + sub[i] * kBoxRows;
                int id = 0;
                if (has_box[i] && t < it.n_kv && key < it.ctx_end) {
                    id = __ldg(table + key / p.block_size);
                    if (id < 0 || id >= p.num_blocks) {
                        atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
                        id = p.num_blocks;            // out of bounds for the tensor map: zero fill
                    }
                }
                return id;
            };
            int id_next[kIssues];
#pragma unroll
            for (int i = 0; i < kIssues; ++i) id_next[i] = lookup(0, i);
            for (int t = 0; t < it.n_kv; ++t) {
                const int key0 = t * kTK;
                int id[kIssues];
#pragma unroll
                for (int i = 0; i < kIssues; ++i) {
                    id[i] = id_next[i];
                    id_next[i] = lookup(t + 1, i);
                }
                // 16-key row groups holding at least one written key; the rest is never loaded
                int ngroups = 0;
                for (int g2 = 0; g2 < kTK / 16; ++g2) ngroups += (key0 + g2 * 16 < it.ctx_end) ? 1 : 0;
                const uint32_t bytes = static_cast<uint32_t>(ngroups * kHalves * 16 * 128);
                // the stage is free once the MMAs that read the tile `stages` tiles back are done: the score MMAs
                // for a K tile, the PV MMAs for a V tile
                if (round > 0) ok = wait_or_abort(smem_u32(&empty[stage]), (round - 1) & 1, abort_flag, p.status);
                if (!__all_sync(0xffffffffu, ok)) break;
                if (lane == 0) {
                    if (k_role) NPD_TRACE(0, 1, t);
                    mbar_expect_tx(smem_u32(&full[stage]), bytes);
                }
                __syncwarp();
#pragma unroll
                for (int i = 0; i < kIssues; ++i) {
                    const int row = it.h * p.block_size + ((key0 + gi[i] * 16 + sub[i] * kBoxRows) % p.block_size);
                    if (has_box[i] && gi[i] < ngroups)
                        tma_load_3d(smem_u32(ring + (size_t)stage * kKvTileBytes) + off[i], tm, smem_u32(&full[stage]),
                                    hf[i] * 64, row, id[i]);
                }
                if (++stage == stages) {
                    stage = 0;
                    ++round;
                }
            }
            ok = __all_sync(0xffffffffu, ok);
        }
    } else if (warp == 9 || warp == 10) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 72;");
        // =========================== MMA issuers: warp 9 for query tile A, warp 10 for B ===========================
        // Each warp runs its loop in full (addresses and descriptors stay in uniform registers) and one elected
        // lane issues the tcgen05 instructions.  Two issuers keep the two query tiles from blocking one another.
        {
            const int x = warp - 9;
            constexpr uint32_t fmt = Elem<T>::kDtype == NPD_DTYPE_BF16 ? 1u : 0u;
            constexpr uint32_t idesc_s = instr_desc(fmt, 0u, kRows, kHalfKeys);
            constexpr uint32_t idesc_pv = instr_desc(fmt, 1u, kRows, kD);
            auto wait_all = [&](uint64_t *bar, uint32_t parity) {
                const bool good = wait_or_abort(smem_u32(bar), parity, abort_flag, p.status);
                return __all_sync(0xffffffffu, good);
            };
            auto commit = [&](uint64_t *bar) {
                if (elect_one()) tc_commit(smem_u32(bar));
                __syncwarp();
            };
            // Descriptors are built once; a k-step, a half or a ring stage only adds a constant to the
            // start-address field (16-byte units).
            const uint64_t q_desc = desc_k_major(smem_u32(q_tiles) + x * kQTileBytes);
            const uint64_t k_desc0 = desc_k_major(smem_u32(k_ring));
            const uint64_t v_desc0 = desc_mn_major(smem_u32(v_ring), kKvHalfBytes);
            const uint32_t t_sx = tmem + x * 128, t_o = tmem + 256 + x * 128;
            // S = Q_X . K^T for the 64 keys of half `h` of ring stage `stage`, into score buffer `buf`, then the commit
            // that tells the softmax group (it also covers every MMA issued before): kD/16 k-steps of 16 elements
            // (32 B inside the swizzle atom; the second 64-element half of the head dim starts one half-tile further
            // on); the keys of half h are rows 64h.. of the K tile, 64 rows x 128 B further on.
            auto issue_s = [&](int stage, int h, int buf) {
                const uint64_t kd = k_desc0 + static_cast<uint64_t>((stage * kKvTileBytes + h * kHalfKeys * 128) >> 4);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < kD / 16; ++ks) {
                        const uint64_t a_off = static_cast<uint64_t>(((ks >> 2) * kQHalfBytes + (ks & 3) * 32) >> 4);
                        const uint64_t b_off = static_cast<uint64_t>(((ks >> 2) * kKvHalfBytes + (ks & 3) * 32) >> 4);
                        tc_mma_ss(t_sx + buf * kHalfKeys, q_desc + a_off, kd + b_off, idesc_s, ks > 0 ? 1u : 0u);
                    }
                    tc_commit(smem_u32(&ctrl->s_full[x][buf]));
                }
                __syncwarp();
            };
            // O_X (+)= P . V for the 64 keys of half `h` of ring stage `stage`: P from TMEM (packed pairs over the
            // first 32 columns of score buffer `buf`, 8 columns per 16 keys), V MN-major from shared memory (16 keys
            // = two 8-row groups = 2 KiB further on), then the commit that counts this product as done.
            auto issue_pv = [&](int stage, int h, int buf, bool first) {
                const uint64_t vd = v_desc0 + static_cast<uint64_t>((stage * kKvTileBytes + h * (kHalfKeys / 16) * 2048) >> 4);
                if (elect_one()) {
#pragma unroll
                    for (int ks = 0; ks < kHalfKeys / 16; ++ks)
                        tc_mma_ts(t_o, t_sx + buf * kHalfKeys + ks * 8, vd + static_cast<uint64_t>((ks * 2048) >> 4),
                                  idesc_pv, (!first || ks > 0) ? 1u : 0u);
                    tc_commit(smem_u32(&ctrl->pv_done[x][buf]));
                }
                __syncwarp();
            };

            int g = 0;         // key tiles seen so far (ring position of the item's first key tile)
            int c = 0;         // own half-steps so far: buffer c & 1, phase c >> 1 of that buffer's barriers
            int items_done = 0;   // items in which this query tile had work (phases of q_full and o_free)
            // The query tile's rows are requested by the warp that reads them: box (64 elements, G heads, TQ tokens)
            // per 64-element slab -> rows (token, head) at 128 B pitch.  The rows of the NEXT item can be requested
            // once the last score MMA of this one has completed (q_empty), two half-steps before the item ends; this
            // warp is the one that knows when that is, and it has time — while the producer warp, which used to do
            // it, is held for ~1800 clocks by every K tile it issues and kept the request waiting behind them.
            int q_requests = 0;   // items whose rows have been requested so far (phases of q_empty)
            int q_item = -1;      // index (k) of the last item whose rows have been requested or need none
            // 1 = requested, 0 = the previous rows are still being read (only when !blocking), -1 = abort
            auto request_q = [&](const Item &qi, bool blocking) {
                if (q_requests > 0) {
                    uint64_t *bar = &ctrl->q_empty[x];
                    const uint32_t par = (q_requests - 1) & 1;
                    if (blocking) {
                        if (!wait_all(bar, par)) return -1;
                    } else if (!__all_sync(0xffffffffu, mbar_test_wait(smem_u32(bar), par))) {
                        return 0;
                    }
                }
                ++q_requests;
                if (elect_one()) {
                    const uint32_t qbar = smem_u32(&ctrl->q_full[x]);
                    mbar_expect_tx(qbar, static_cast<uint32_t>(kHalves * p.tq * p.group * 128));
                    for (int h2 = 0; h2 < kHalves; ++h2)
                        tma_load_3d(smem_u32(q_tiles + x * kQTileBytes + h2 * kQHalfBytes), &tm_q, qbar, h2 * 64,
                                    qi.h * p.group, qi.qoff + qi.tok0[x]);
                }
                __syncwarp();
                return 1;
            };
            // The next item's rows, if that item has been published and the rows of this one are no longer read.
            auto request_next_q = [&](int k) {
                const int slot = (k + 1) % kSchedSlots;
                if (!__all_sync(0xffffffffu, mbar_test_wait(smem_u32(&ctrl->sched_full[slot]), ((k + 1) / kSchedSlots) & 1)))
                    return true;
                if (*reinterpret_cast<volatile int *>(&ctrl->sched_item[slot]) < 0 || ctrl->sched_desc[slot].nhalf[x] <= 0) {
                    q_item = k + 1;                                // nothing to request for it
                    return true;
                }
                const int r = request_q(ctrl->sched_desc[slot], false);
                if (r > 0) q_item = k + 1;
                return r >= 0;
            };
            NPD_TRACE_DECL
            bool ok = true;
            for (int k = 0; ok; ++k) {
                const int item = next_item(k, ok);
                if (!__all_sync(0xffffffffu, ok) || item < 0) break;
                const Item it = ctrl->sched_desc[k % kSchedSlots];
                const int U = it.nhalf[x], my_tiles = it.ntiles[x];
                if (U > 0 && q_item < k) {
                    if (request_q(it, true) < 0) {
                        ok = false;
                        break;
                    }
                    q_item = k;
                }
                // Half-step u of the item lies in K/V tile u / kHPT (half u % kHPT of it).  A score batch is followed by
                // the release of its K tile when it was the last one to read it.
                auto scores = [&](int u, int buf) {
                    const int t = u / kHPT, h = u % kHPT, gt = g + t;
                    if (h == 0 && !wait_all(&ctrl->k_full[gt % kStagesK], (gt / kStagesK) & 1)) return false;
                    tc_fence_after();
                    NPD_TRACE(x == 0 ? 1 : 4, 12, u);
                    issue_s(gt % kStagesK, h, buf);
                    NPD_TRACE(x == 0 ? 1 : 4, 13, u);
                    if (h == kHPT - 1 || u == U - 1) commit(&ctrl->k_empty[gt % kStagesK]);
                    if (u == U - 1) commit(&ctrl->q_empty[x]);       // no further score MMA of this item reads Q_X
                    return true;
                };
                if (U > 0) {
                    // the first two half-steps' scores: both buffers are free (the previous item's last PV
                    // products, which read P from them, were issued before these MMAs)
                    if (!(ok = wait_all(&ctrl->q_full[x], items_done & 1))) break;
                    if (!(ok = scores(0, c & 1))) break;
                    if (U > 1 && !(ok = scores(1, (c + 1) & 1))) break;
                }
                for (int u = 0; ok && u < U; ++u) {
                    const int t = u / kHPT, h = u % kHPT, gt = g + t, stage = gt % kStagesV;
                    const int cu = c + u, buf = cu & 1;
                    // O_X is overwritten by the first PV of an item: the previous epilogue must have read it
                    if (u == 0 && items_done > 0 && !(ok = wait_all(&ctrl->o_free[x], (items_done - 1) & 1))) break;
                    if (h == 0 && !(ok = wait_all(&ctrl->v_full[stage], (gt / kStagesV) & 1))) break;
                    NPD_TRACE(x == 0 ? 1 : 4, 10, u);
                    if (!(ok = wait_all(&ctrl->p_ready[x][buf], (cu >> 1) & 1))) break;
                    NPD_TRACE(x == 0 ? 1 : 4, 11, u);
                    tc_fence_after();
                    issue_pv(stage, h, buf, u == 0);
                    NPD_TRACE(x == 0 ? 1 : 4, 14, u);
                    if (h == kHPT - 1 || u == U - 1) commit(&ctrl->v_empty[stage]);
                    // S(u+2) goes into the buffer P(u) sits in; it executes after the PV MMAs above
                    if (u + 2 < U && !(ok = scores(u + 2, buf))) break;
                    // the item's last score MMA has been issued: the next item's rows as soon as it has completed
                    if (u + 3 >= U && q_item <= k && !(ok = request_next_q(k))) break;
                }
                for (int t = my_tiles; ok && t < it.n_kv; ++t) {
                    // a key tile only the other query tile needs: observe it so that ring phases stay in step
                    const int gt = g + t;
                    if (!(ok = wait_all(&ctrl->k_full[gt % kStagesK], (gt / kStagesK) & 1))) break;
                    commit(&ctrl->k_empty[gt % kStagesK]);
                    if (!(ok = wait_all(&ctrl->v_full[gt % kStagesV], (gt / kStagesV) & 1))) break;
                    commit(&ctrl->v_empty[gt % kStagesV]);
                }
                g += it.n_kv;
                c += U;
                items_done += U > 0 ? 1 : 0;
            }
        }
    } else if (warp >= 12) {
        asm volatile("setmaxnreg.dec.sync.aligned.u32 104;");
        // =========================== epilogue (warps 12-15): O / l -> out, for both query tiles ===========================
        // Warp 12 + w reads TMEM lane quarter w, as softmax warps w and 4 + w do.  The softmax group of a tile hands an
        // item over as soon as it has released the last half-step's probabilities (its row sums go through shared
        // memory) and starts on the next item; these warps wait for the item's last PV product, take O out of TMEM —
        // only then may the next item's first PV product overwrite it — and write the normalised rows.  The stores of
        // a tile (32 KiB as 32-byte pieces) take the SM 2-3 thousand clocks, which were 7 % of configuration 3 while
        // the softmax warps did them.
        const int wq = warp & 3;
        const int row = wq * 32 + lane;                          // == TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        const int tq_idx = row / p.group, hg = row - tq_idx * p.group;
        int c[2] = {0, 0};                                       // per query tile: half-steps so far (phases of pv_done)
        int items_done[2] = {0, 0};                              // per query tile: items handed over so far
        bool ok = true;
        for (int k = 0; ok; ++k) {
            const int item = next_item(k, ok);
            if (!ok || item < 0) break;
            const Item it = ctrl->sched_desc[k % kSchedSlots];
#pragma unroll
            for (int x = 0; x < kQueryTiles; ++x) {
                const int U = it.nhalf[x];
                if (U == 0 || !ok) continue;
                if (!(ok = wait_or_abort(smem_u32(&ctrl->epi_ready[x]), items_done[x] & 1, abort_flag, p.status))) continue;
                const float inv = 1.f / ctrl->l_sum[x][row];
                // the item's last PV product (products complete in order, so all of them)
                const int last = c[x] + U - 1;
                if (!(ok = wait_or_abort(smem_u32(&ctrl->pv_done[x][last & 1]), (last >> 1) & 1, abort_flag, p.status))) continue;
                tc_fence_after();
                const uint32_t t_o = tmem + 256 + x * 128 + lane_base;
                const bool store = tq_idx < it.tq_valid[x] && row < p.tq * p.group;
                T *dst = static_cast<T *>(p.out) +
                         ((long long)(it.qoff + it.tok0[x] + tq_idx) * p.num_q_heads + (long long)it.h * p.group + hg) * kD;
                // the accumulator row in groups of 64 columns: both loads of a group in flight, one wait
                constexpr int kChunks = kD / 32, kGroup = kChunks < 2 ? kChunks : 2;
#pragma unroll
                for (int c0 = 0; c0 < kChunks; c0 += kGroup) {
                    float o[kGroup][32];
#pragma unroll
                    for (int cc = 0; cc < kGroup; ++cc) tmem_ld32(t_o + (c0 + cc) * 32, o[cc]);
                    tmem_wait_ld();
                    if (c0 + kGroup == kChunks) {
                        // O is in registers: the next item's first PV may overwrite the accumulator
                        tc_fence_before();
                        mbar_arrive(smem_u32(&ctrl->o_free[x]));
                    }
                    if (store) {
                        // 32 bytes per lane and instruction: a lane's row is contiguous and the lanes of a warp are a
                        // row apart, so every store instruction fills whole 32-byte sectors
#pragma unroll
                        for (int cc = 0; cc < kGroup; ++cc)
#pragma unroll
                            for (int i = 0; i < 32; i += 16) {
                                uint32_t w[8];
#pragma unroll
                                for (int j = 0; j < 8; ++j)
                                    w[j] = Elem<T>::pack2(o[cc][i + 2 * j] * inv, o[cc][i + 2 * j + 1] * inv);
                                st_global_32B(dst + (c0 + cc) * 32 + i, w);
                            }
                    }
                }
                c[x] += U;
                ++items_done[x];
            }
        }
    } else {
        asm volatile("setmaxnreg.inc.sync.aligned.u32 168;");
        // =========================== softmax + correction (warps 0-7) ===========================
        const int x = warp >> 2;                                 // query tile A or B
        const int wq = warp & 3;                                 // TMEM lane quarter this warp may touch
        const int row = wq * 32 + lane;                          // == TMEM lane
        const uint32_t lane_base = static_cast<uint32_t>(wq * 32) << 16;
        const uint32_t t_sx = tmem + x * 128 + lane_base;        // two score buffers of 64 columns
        const uint32_t t_o = tmem + 256 + x * 128 + lane_base;
        const int tq_idx = row / p.group, hg = row - tq_idx * p.group;
        int g = 0, c = 0;                                     // key tiles / own half-steps so far (barrier phases)
        int items_handed = 0;                                 // items handed to the epilogue warps so far
        const int sm_role = wq == 0 ? 2 + x : 5 + x * 3 + (wq - 1);   // trace slot (used only by tracing builds)
        (void)sm_role;
        NPD_TRACE_DECL
        bool ok = true;

        for (int k = 0; ok; ++k) {
            const int item = next_item(k, ok);
            if (!ok || item < 0) break;
            const Item it = ctrl->sched_desc[k % kSchedSlots];
            const int U = it.nhalf[x];
            const int pos = it.start + it.tok0[x] + tq_idx;      // last visible key of this row
            float m_run = -INFINITY, l_run = 0.f;
#pragma unroll 1
            for (int u = 0; ok && u < U; ++u) {
                const int cu = c + u, buf = cu & 1;
                const int t = u / kHPT, gt = g + t, stage = gt % kStagesV;
                const int key0 = u * kHalfKeys;
                // V rows at or past ctx_end were never written (or never loaded): clear them so that P = 0
                // there cannot meet a NaN.  Both softmax groups do it (idempotent), at the first half-step of the
                // key tile, before they release its probabilities.
                if (u % kHPT == 0 && t * kTK + kTK > it.ctx_end) {
                    if (!(ok = wait_or_abort(smem_u32(&ctrl->v_full[stage]), (gt / kStagesV) & 1, abort_flag, p.status))) break;
                    uint8_t *v_tile = v_ring + (size_t)stage * kKvTileBytes;
                    const int first = max(it.ctx_end - t * kTK, 0);
                    constexpr int kPieces = kHalves * 8;           // 16-byte pieces per row
                    const int n16 = (kTK - first) * kPieces;
                    for (int idx = threadIdx.x & 127; idx < n16; idx += 128) {
                        const int r = first + idx / kPieces, piece = idx % kPieces;
                        *reinterpret_cast<uint4 *>(v_tile + (piece >> 3) * kKvHalfBytes + r * 128 + ((piece & 7) << 4)) =
                            make_uint4(0, 0, 0, 0);
                    }
                    fence_proxy_async_smem();
                }
                if (lane == 0) NPD_TRACE_FINE(sm_role, 20, u);
                if (!(ok = wait_or_abort(smem_u32(&ctrl->s_full[x][buf]), (cu >> 1) & 1, abort_flag, p.status))) break;
                if (lane == 0) NPD_TRACE(sm_role, 21, u);
                tc_fence_after();
                // The 64 scores of this half-step move to registers: one TMEM read.
                float sc[2][32];
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) tmem_ld32(t_sx + buf * kHalfKeys + cc * 32, sc[cc]);
                tmem_wait_ld();
                if (lane == 0) NPD_TRACE_FINE(sm_role, 22, u);
                if (key0 + kHalfKeys - 1 > it.start + it.tok0[x]) {  // only half-steps that reach past the first row's diagonal
#pragma unroll
                    for (int cc = 0; cc < 2; ++cc)
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (key0 + cc * 32 + i > pos) sc[cc][i] = -INFINITY;
                }
                // ---- row maximum: four independent chains of three-input max ----
                float mxa[4];
#pragma unroll
                for (int q4 = 0; q4 < 4; ++q4) mxa[q4] = fmaxf(sc[q4 >> 1][(q4 & 1) * 16], sc[q4 >> 1][(q4 & 1) * 16 + 1]);
#pragma unroll
                for (int i = 2; i < 16; i += 2)
#pragma unroll
                    for (int q4 = 0; q4 < 4; ++q4)
                        mxa[q4] = fmax3(mxa[q4], sc[q4 >> 1][(q4 & 1) * 16 + i], sc[q4 >> 1][(q4 & 1) * 16 + i + 1]);
                const float m_new = fmaxf(fmaxf(mxa[0], mxa[1]), fmaxf(mxa[2], mxa[3])) * p.scale_log2;
                if (u == 0) {
                    m_run = m_new;                              // key 0 is visible to every row: finite
                } else {
                    // Lazy correction: O (in TMEM) and l are rescaled only when some row's maximum grew by more
                    // than 2^8; otherwise the stale maximum keeps every probability below 256, exactly cancelled
                    // by the final division.  O may be touched once every PV product issued so far has completed:
                    // PV(u-1) is the last one (PV(u) waits for the probabilities of this half-step); the one before
                    // it on the same barrier, PV(u-3), is known to be complete (s_full of this buffer covers PV(u-2)).
                    const bool grow = m_new > m_run + kRescaleThreshold;
                    if (__any_sync(0xffffffffu, grow)) {
                        if (!(ok = wait_or_abort(smem_u32(&ctrl->pv_done[x][(cu - 1) & 1]), ((cu - 1) >> 1) & 1, abort_flag,
                                                 p.status))) break;
                        tc_fence_after();
                        const float alpha = grow ? fast_exp2(m_run - m_new) : 1.f;
#pragma unroll 1
                        for (int cc = 0; cc < kD / 32; ++cc) {
                            float o[32];
                            tmem_ld32(t_o + cc * 32, o);
                            tmem_wait_ld();
#pragma unroll
                            for (int i = 0; i < 32; ++i) o[i] *= alpha;
                            tmem_st32(t_o + cc * 32, o);
                        }
                        tmem_wait_st();
                        if (grow) {
                            l_run *= alpha;
                            m_run = m_new;
                        }
                    }
                }
                if (lane == 0) NPD_TRACE_FINE(sm_role, 23, u);
                // ---- probabilities (masked scores are -inf -> 0), packed in pairs over the first 32 columns of the
                //      buffer just read ----
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2);
                const float2 negm2 = make_float2(-m_run, -m_run);
                float2 acc2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int cc = 0; cc < 2; ++cc) {
                    uint32_t packed[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 xs = __ffma2_rn(make_float2(sc[cc][2 * i], sc[cc][2 * i + 1]), scale2, negm2);
                        const float2 pr = (kPolyExpEvery > 0 && i % (kPolyExpEvery > 0 ? kPolyExpEvery : 1) == 0)
                                              ? exp2_fma2(xs)
                                              : make_float2(fast_exp2(xs.x), fast_exp2(xs.y));
                        acc2[i & 1] = __fadd2_rn(acc2[i & 1], pr);
                        packed[i] = Elem<T>::pack2(pr.x, pr.y);
                    }
                    tmem_st16(t_sx + buf * kHalfKeys + cc * 16, packed);
                }
                const float psum = (acc2[0].x + acc2[1].x) + (acc2[0].y + acc2[1].y);
                l_run += psum;
                if (lane == 0) NPD_TRACE_FINE(sm_role, 24, u);
                tmem_wait_st();
                tc_fence_before();           // P is in TMEM, S has been read: the MMA warp may go on
                mbar_arrive(smem_u32(&ctrl->p_ready[x][buf]));
                if (lane == 0) NPD_TRACE(sm_role, 25, u);
            }

            // ---- hand the item over to the epilogue warps: the row sums, then the arrival ----
            if (ok && U > 0) {
                if (lane == 0) NPD_TRACE(sm_role, 30, k);
                // The epilogue warps must have taken the previous item's row sums (they arrive on o_free after
                // reading them).  An item of two or more half-steps cannot get here before that — its first PV
                // product waits for o_free — but an item of a single half-step can; the wait also keeps
                // epi_ready at most one phase ahead of its waiters.
                if (items_handed > 0 &&
                    !(ok = wait_or_abort(smem_u32(&ctrl->o_free[x]), (items_handed - 1) & 1, abort_flag, p.status))) break;
                ctrl->l_sum[x][row] = l_run;
                mbar_arrive(smem_u32(&ctrl->epi_ready[x]));
                ++items_handed;
            }
            if (lane == 0) NPD_TRACE(sm_role, 32, k);
            g += it.n_kv;
            c += U;
        }
    }

    // ---- teardown: everyone meets, then the allocating warp releases TMEM ----
    tc_fence_before();
    __syncthreads();
    if (warp == 9) {
        tc_fence_after();
        tmem_dealloc(tmem, kTmemCols);
    }
    // The last CTA to leave puts the two counters back to zero for the next launch on this workspace (every CTA
    // has drawn its last item by now: its producer warp only leaves its loop on an item past the end, or on abort).
    if (threadIdx.x == 0 && atomicAdd(p.work_counter + 1, 1) == static_cast<int>(gridDim.x) - 1) {
        p.work_counter[0] = 0;
        p.work_counter[1] = 0;
    }
}

}  // namespace

extern "C" size_t npd_prefill_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int) { return 256; }

extern "C" int npd_paged_prefill_attention(void *out, const void *q, const void *k_cache, const void *v_cache,
                                           const int32_t *block_tables, const int32_t *chunk_q_offset_host,
                                           const int32_t *chunk_tokens_host, const int32_t *chunk_start_host,
                                           int64_t num_chunks, float scale, int64_t num_q_heads, int64_t num_kv_heads,
                                           int64_t head_dim, int64_t block_size, int64_t max_blocks_per_seq,
                                           int64_t num_blocks, int64_t cache_block_stride, int64_t bt_row_stride,
                                           int dtype, void *workspace, size_t workspace_bytes, int flags,
                                           void *stream) {
    NPD_REQUIRE(dtype == NPD_DTYPE_F16 || dtype == NPD_DTYPE_BF16, NPD_ERR_UNSUPPORTED,
                "prefill attention supports float16 and bfloat16 only (dtype code %d)", dtype);
    NPD_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, NPD_ERR_UNSUPPORTED,
                "prefill attention: head_dim %lld not in {64,128,256}", (long long)head_dim);
    NPD_REQUIRE(block_size == 4 || block_size == 8 || block_size == 16 || block_size == 32, NPD_ERR_UNSUPPORTED,
                "prefill attention: block_size %lld not in {4,8,16,32}", (long long)block_size);
    NPD_REQUIRE(num_chunks >= 0 && num_q_heads > 0 && num_kv_heads > 0 && max_blocks_per_seq > 0 && num_blocks > 0,
                NPD_ERR_INVALID_ARG, "prefill attention: non-positive dimension");
    NPD_REQUIRE(num_q_heads % num_kv_heads == 0, NPD_ERR_INVALID_ARG,
                "prefill attention: num_q_heads is not a multiple of num_kv_heads");
    const int group = static_cast<int>(num_q_heads / num_kv_heads);
    NPD_REQUIRE(group <= 128, NPD_ERR_UNSUPPORTED, "prefill attention: more than 128 q heads per kv head");
    if (num_chunks == 0) return NPD_OK;
    NPD_REQUIRE(out && q && k_cache && v_cache && block_tables && chunk_q_offset_host && chunk_tokens_host &&
                    chunk_start_host,
                NPD_ERR_INVALID_ARG, "prefill attention: NULL pointer");
    NPD_REQUIRE(workspace != nullptr && workspace_bytes >= 256, NPD_ERR_WORKSPACE,
                "prefill attention: workspace of at least 256 bytes needed (status word)");
    NPD_REQUIRE(npd::aligned16(q) && (reinterpret_cast<uintptr_t>(out) & 31u) == 0, NPD_ERR_INVALID_ARG,
                "prefill attention: q must be 16-byte and out 32-byte aligned");
    NPD_REQUIRE(num_blocks < INT32_MAX && max_blocks_per_seq * block_size < INT32_MAX, NPD_ERR_INVALID_ARG,
                "prefill attention: dimension exceeds int32");

    int64_t total_tokens = 0;
    for (int64_t i = 0; i < num_chunks; ++i) {
        NPD_REQUIRE(chunk_tokens_host[i] >= 0 && chunk_start_host[i] >= 0 && chunk_q_offset_host[i] >= 0,
                    NPD_ERR_INVALID_ARG, "prefill attention: negative chunk field");
        NPD_REQUIRE((int64_t)chunk_start_host[i] + chunk_tokens_host[i] <= max_blocks_per_seq * block_size,
                    NPD_ERR_INVALID_ARG, "prefill attention: chunk %lld reaches beyond its block table", (long long)i);
        const int64_t end = (int64_t)chunk_q_offset_host[i] + chunk_tokens_host[i];
        if (end > total_tokens) total_tokens = end;
    }
    if (total_tokens == 0) return NPD_OK;

    const int tq = kRows / group;
    CUtensorMap tq_map, tk, tv;
    {
        const uint64_t dims[3] = {(uint64_t)head_dim, (uint64_t)num_q_heads, (uint64_t)total_tokens};
        const uint64_t strides[2] = {(uint64_t)head_dim * 2u, (uint64_t)num_q_heads * head_dim * 2u};
        const uint32_t box[3] = {64u, (uint32_t)group, (uint32_t)tq};
        const int rc = npd::encode_tiled_3d(&tq_map, q, dtype, dims, strides, box);
        if (rc != NPD_OK) return rc;
    }
    const int box_rows = block_size < 16 ? static_cast<int>(block_size) : 16;
    int rc = npd::encode_cache_tensor_map(&tk, k_cache, dtype, head_dim, num_kv_heads * block_size, num_blocks,
                                          cache_block_stride, box_rows);
    if (rc != NPD_OK) return rc;
    rc = npd::encode_cache_tensor_map(&tv, v_cache, dtype, head_dim, num_kv_heads * block_size, num_blocks,
                                      cache_block_stride, box_rows);
    if (rc != NPD_OK) return rc;

    const size_t halves = static_cast<size_t>(head_dim / 64);
    const int query_tiles = head_dim == 256 ? 1 : 2, tile_keys = head_dim == 256 ? 64 : kKeys;
    const size_t smem = 1024 + query_tiles * halves * kQHalfBytes + (size_t)(kStagesK + kStagesV) * halves * tile_keys * 128 +
                        sizeof(SmemCtrl) + 64;
    const bool f16 = dtype == NPD_DTYPE_F16;
    using Kernel = void (*)(PrefillParams, CUtensorMap, CUtensorMap, CUtensorMap);
    Kernel kern = nullptr;
#define NPD_PICK_B(D_, B_) (f16 ? paged_prefill_kernel<__half, D_, B_> : paged_prefill_kernel<__nv_bfloat16, D_, B_>)
#define NPD_PICK(D_) kern = box_rows == 4 ? NPD_PICK_B(D_, 4) : (box_rows == 8 ? NPD_PICK_B(D_, 8) : NPD_PICK_B(D_, 16))
    if (head_dim == 64) NPD_PICK(64);
    else if (head_dim == 128) NPD_PICK(128);
    else NPD_PICK(256);
#undef NPD_PICK
#undef NPD_PICK_B
    NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));

    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    const long long sms = npd::sm_count(dev);
    for (int64_t c0 = 0; c0 < num_chunks; c0 += kMaxChunks) {
        const int nc = static_cast<int>(num_chunks - c0 < kMaxChunks ? num_chunks - c0 : kMaxChunks);
        PrefillParams p;
        p.out = out;
        p.block_tables = block_tables + c0 * bt_row_stride;
        p.status = static_cast<int32_t *>(workspace);
        p.scale_log2 = scale * 1.4426950408889634f;
        p.num_chunks = nc;
        p.num_q_heads = static_cast<int>(num_q_heads);
        p.num_kv_heads = static_cast<int>(num_kv_heads);
        p.group = group;
        p.tq = tq;
        p.block_size = static_cast<int>(block_size);
        p.box_rows = box_rows;
        p.query_tiles = query_tiles;
        p.half_steps_per_tile = tile_keys / kHalfKeys;
        p.max_blocks_per_seq = static_cast<int>(max_blocks_per_seq);
        p.num_blocks = static_cast<int>(num_blocks);
        p.bt_row_stride = bt_row_stride;
#ifdef NPD_PREFILL_TRACE
        p.trace = workspace_bytes >= 256 + 11 * 4096 * sizeof(long long)
                      ? reinterpret_cast<long long *>(static_cast<uint8_t *>(workspace) + 256) : nullptr;
#endif
        // Pairs of query tiles of the launch, heaviest (most key tiles) first; the kernel hands them out in
        // this order through an atomic counter.
        struct Entry { int weight; uint32_t code; };
        std::vector<Entry> entries;
        for (int i = 0; i < nc; ++i) {
            p.chunk_q_offset[i] = chunk_q_offset_host[c0 + i];
            p.chunk_tokens[i] = chunk_tokens_host[c0 + i];
            p.chunk_start[i] = chunk_start_host[c0 + i];
            const int pairs = (p.chunk_tokens[i] + query_tiles * tq - 1) / (query_tiles * tq);
            NPD_REQUIRE(pairs <= 0xffff, NPD_ERR_INVALID_ARG, "prefill attention: chunk %d is too long", i);
            for (int pr = 0; pr < pairs; ++pr) {
                const int last_tok = std::min(p.chunk_tokens[i], (pr + 1) * query_tiles * tq);
                entries.push_back({(p.chunk_start[i] + last_tok + kKeys - 1) / kKeys,
                                   (static_cast<uint32_t>(i) << 16) | static_cast<uint32_t>(pr)});
            }
        }
        std::stable_sort(entries.begin(), entries.end(), [](const Entry &a, const Entry &b) { return a.weight > b.weight; });
        cudaStream_t launch_stream = st;
        for (size_t e0 = 0; e0 < entries.size(); e0 += kMaxPairs) {
            const int ne = static_cast<int>(std::min<size_t>(kMaxPairs, entries.size() - e0));
            for (int e = 0; e < ne; ++e) p.pair_order[e] = entries[e0 + e].code;
            p.num_pairs = ne;
            p.work_counter = reinterpret_cast<int *>(static_cast<uint8_t *>(workspace) + 64);   // zero: see the kernel's end
            const long long items = (long long)ne * num_kv_heads;
            long long grid = items < sms ? items : sms;           // persistent: one CTA per SM
            const int cta_cap = (flags >> 8) & 0xffff;
            if (cta_cap > 0 && cta_cap < grid) grid = cta_cap;
            kern<<<static_cast<unsigned>(grid), kThreads, smem, launch_stream>>>(p, tq_map, tk, tv);
            NPD_CUDA_TRY(cudaGetLastError());
        }
    }
    return NPD_OK;
}
