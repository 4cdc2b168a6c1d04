// Kernel 2: paged decode attention over ragged block tables (one query token per sequence).
//
// Design (B200, HBM-bound: every K/V byte is read from HBM exactly once):
//   * Work unit = one 16-token TILE of one (sequence, kv head).  All tiles of the batch are
//     laid on one line, ordered (sequence, kv head, tile), and the line is cut into equal
//     contiguous ranges, one per WARP ("worker") of a persistent grid of one CTA per SM.
//     Ragged lengths therefore balance exactly without a host-side plan or a device sync;
//     each CTA rebuilds the tile prefix sum from seq_lens in shared memory.
//   * A worker streams its tiles through a private ring of TMA stages: lane 0 issues
//     cp.async.bulk.tensor loads (128-byte swizzle, one box per 64-element half of a page
//     row block) that complete on a per-stage mbarrier; no CTA-wide barrier in the loop.
//   * All q heads that share the kv head ride along: scores are S^T = K . Q^T with
//     mma.sync m16n8k16 (M = 16 tokens of the tile, N = up to 8 q heads per n-tile),
//     so a page is read once per GROUP, not once per q head as in the reference
//     (nanoPD/paged_attention/csrc/attention/paged_attention_kernel.cu:60-62).
//     fp32 scores, warp-shuffle online softmax in the log2 domain, P^T rebuilt as the B
//     operand with movmatrix, O^T = V^T . P^T accumulated in fp32 registers.
//   * A (sequence, kv head) whose tiles fall into one worker is normalised and written
//     straight to `out`.  One cut by a range boundary leaves fp32 partials (m, l, O) in the
//     workspace — at most two per worker; the worker that delivers the LAST partial of a
//     (sequence, kv head) — found with an atomic ticket, no spinning — merges them in the
//     same kernel (the role of paged_attention_reduce_kernel, csrc/paged_attention_optimized/
//     paged_attention_optimized.cu:173-219, without a second launch, per-call allocations or a sync).
//   * Every mbarrier wait is bounded; on time-out the warp raises NPD_STATUS_WAIT_TIMEOUT
//     and leaves.  Out-of-range block ids are redirected to an out-of-bounds TMA coordinate
//     (zero fill) and flagged — nothing can fault.
//
// Algorithmic bytes per launch: sum(len_s)*2*Hkv*D*e + 2*S*Hq*D*e + sum(ceil(len_s/B))*4 + 4*S.
#include <atomic>
#include <cstdlib>

#include "npd_common.cuh"

namespace {

using namespace npd;

constexpr int kTile = 16;               // tokens per stage
constexpr int kMaxSeqsPerLaunch = 4096; // prefix array lives in shared memory
constexpr int kMaxFloorTilesPerWorker = 16;   // upper end of the floor on tiles per worker (see tiles_per_worker)
constexpr int kStatusBytes = 256;       // workspace header: status word + padding
constexpr int kTicketCapacity = 1 << 18;   // ticket words (1 MiB): a FIXED region right after the header, so that no
                                        // launch shape ever puts partial records where another shape keeps tickets

struct DecodeParams {
    void *out;
    const void *q;
    const int32_t *block_tables;
    const int32_t *seq_lens;
    int32_t *status;
    int32_t *tickets;     // [num_seqs * num_vheads] partials delivered so far; zero between launches
    float *partials;      // [num_workers][2][rec_floats]
    int skip_merge;       // diagnostic: leave cut (sequence, kv head) pairs unmerged
    float scale_log2;
    int num_seqs;
    int num_q_heads;
    int num_vheads;       // virtual kv heads = num_kv_heads * kv_rep
    int kv_rep;           // virtual kv heads per physical kv head (1 unless the group exceeds 16)
    int group;            // q heads per virtual kv head
    int block_size;
    int box_rows;         // min(block_size, 16)
    int max_blocks_per_seq;
    int num_blocks;
    long long bt_row_stride;
    int num_workers;
    int num_stages;
};

__device__ __forceinline__ int clamped_len(const DecodeParams &p, int s) {
    int len = __ldg(p.seq_lens + s);
    const long long cap = (long long)p.max_blocks_per_seq * p.block_size;
    if (len < 0) len = 0;
    if (len > cap) len = static_cast<int>(cap);
    return len;
}

// Tiles per worker: the equal split over all workers, but not below a floor that keeps small batches from
// dissolving into partials.  A worker needs ~0.7 us per tile and the merge of a (sequence, kv head) ~0.45 us per
// four partials, so for `tph` tiles per (sequence, kv head) the time W*0.7 + tph/W/4*0.45 is least near
// W = sqrt(0.16 * tph): 1-2 tiles for the few-hundred-token batches of a micro-benchmark (every SM gets work and
// nobody streams eight tiles in a row), 8-9 for an 8k-token context.
__device__ __forceinline__ long long tiles_per_worker(long long total, int num_workers, long long num_seq_heads) {
    const long long w = (total + num_workers - 1) / num_workers;
    const float tph = static_cast<float>(total) / static_cast<float>(num_seq_heads > 0 ? num_seq_heads : 1);
    long long floor_w = static_cast<long long>(sqrtf(0.16f * tph) + 0.5f);
    floor_w = floor_w < 1 ? 1 : (floor_w > kMaxFloorTilesPerWorker ? kMaxFloorTilesPerWorker : floor_w);
    return w < floor_w ? floor_w : w;
}

// pre[0..S]: exclusive prefix of ceil(len/16) over the sequences, built by the whole CTA.
__device__ void build_tile_prefix(const DecodeParams &p, int *pre) {
    __shared__ int warp_sums[32];
    const int S = p.num_seqs;
    const int tid = threadIdx.x, nthreads = blockDim.x;
    const long long cap = (long long)p.max_blocks_per_seq * p.block_size;
    for (int i = tid; i < S; i += nthreads) {
        const int raw = __ldg(p.seq_lens + i);
        if ((raw < 0 || raw > cap) && blockIdx.x == 0) atomicOr(p.status, NPD_STATUS_BAD_POSITION);
        pre[i + 1] = (clamped_len(p, i) + kTile - 1) / kTile;
    }
    if (tid == 0) pre[0] = 0;
    __syncthreads();
    const int chunk = (S + nthreads - 1) / nthreads;
    const int lo = min(tid * chunk, S), hi = min(lo + chunk, S);
    int sum = 0;
    for (int i = lo; i < hi; ++i) {
        sum += pre[i + 1];
        pre[i + 1] = sum;
    }
    const int lane = tid & 31, warp = tid >> 5;
    int incl = sum;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int v = __shfl_up_sync(0xffffffffu, incl, d);
        if (lane >= d) incl += v;
    }
    if (lane == 31) warp_sums[warp] = incl;
    __syncthreads();
    if (warp == 0) {
        const int nw = nthreads >> 5;
        int v = lane < nw ? warp_sums[lane] : 0;
        int inc = v;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int u = __shfl_up_sync(0xffffffffu, inc, d);
            if (lane >= d) inc += u;
        }
        warp_sums[lane] = inc - v;   // exclusive
    }
    __syncthreads();
    const int offset = warp_sums[warp] + incl - sum;
    for (int i = lo; i < hi; ++i) pre[i + 1] += offset;
    __syncthreads();
}

struct Cursor {
    int s, h, t;   // sequence, virtual kv head, tile
    int n;         // tiles of sequence s
    int len;       // clamped length of sequence s
};

__device__ __forceinline__ void cursor_seek(Cursor &c, long long f, const int *pre, const DecodeParams &p) {
    int lo = 0, hi = p.num_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if ((long long)p.num_vheads * pre[mid] <= f) lo = mid; else hi = mid - 1;
    }
    c.s = lo;
    c.n = pre[lo + 1] - pre[lo];
    const long long r = f - (long long)p.num_vheads * pre[lo];
    c.h = static_cast<int>(r / c.n);
    c.t = static_cast<int>(r - (long long)c.h * c.n);
    c.len = clamped_len(p, lo);
}

// Moves to the next tile of the line; the caller guarantees one exists.
__device__ __forceinline__ void cursor_advance(Cursor &c, const int *pre, const DecodeParams &p) {
    if (++c.t < c.n) return;
    c.t = 0;
    if (++c.h < p.num_vheads) return;
    c.h = 0;
    int s = c.s + 1;
    while (s < p.num_seqs - 1 && pre[s + 1] == pre[s]) ++s;
    c.s = s;
    c.n = pre[s + 1] - pre[s];
    c.len = clamped_len(p, s);
}

// Per-warp register window over one sequence's block-table row: lane i holds entry base+i.
struct TableWindow {
    int s, base, val;
};

__device__ __forceinline__ int table_lookup(TableWindow &w, int s, int page, int npages, int lane,
                                            const DecodeParams &p) {
    if (w.s != s || page < w.base || page >= w.base + 32) {
        w.s = s;
        w.base = page;
        const int idx = page + lane;
        w.val = idx < npages ? __ldg(p.block_tables + (long long)s * p.bt_row_stride + idx) : 0;
    }
    return __shfl_sync(0xffffffffu, w.val, page - w.base);
}

// Byte offset of 16-byte piece `c` of token row `r` inside a K or V tile.  A tile is made of
// 16/box_rows boxes; a box is [half][box_rows][128 B] with the 128-byte swizzle TMA applies
// (piece index XOR the 128-byte row's index within its 1024-byte atom: TMA takes it from the shared-memory
// address, which is row%8 for boxes of 8 or 16 rows and differs for boxes of 4).
template <int D>
__device__ __forceinline__ uint32_t tile_offset(int r, int c, int box_rows) {
    constexpr int NH = D / 64;
    const int box = r / box_rows, rr = r - box * box_rows;
    const int row_off = box * (NH * box_rows * 128) + (c >> 3) * (box_rows * 128) + rr * 128;
    return static_cast<uint32_t>(row_off + (((c & 7) ^ ((row_off >> 7) & 7)) << 4));
}

template <typename T, int D, int NT>
struct AttnState {
    float o[NT][D / 16][4];   // O^T fragments: (d = 16j+g | 16j+g+8) x (head 2t | 2t+1)
    float m[NT][2];           // running max (log2 domain) of heads 2t, 2t+1
    float l[NT][2];           // running sum; per-thread partial until reduce_l()
    __device__ __forceinline__ void reset() {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
            for (int j = 0; j < D / 16; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) o[nt][j][e] = 0.f;
            m[nt][0] = m[nt][1] = -INFINITY;
            l[nt][0] = l[nt][1] = 0.f;
        }
    }
    __device__ __forceinline__ void reduce_l() {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                float v = l[nt][e];
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                l[nt][e] = v;
            }
    }
};

// Normalises and writes the rows of one (sequence, virtual kv head) to `out`.
template <typename T, int D, int NT>
__device__ __forceinline__ void write_output(const AttnState<T, D, NT> &st, const DecodeParams &p, int s, int h,
                                             int lane) {
    const int g = lane >> 2, t = lane & 3;
    T *out = static_cast<T *>(p.out);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        const float inv0 = 1.f / st.l[nt][0], inv1 = 1.f / st.l[nt][1];
        const int head = nt * 8 + g;
        T *row = out + ((long long)s * p.num_q_heads + (long long)h * p.group + head) * D;
#pragma unroll
        for (int j = 0; j < D / 16; ++j) {
            // (d = g, heads 2t..2t+1) -> transpose -> (head g, d = 2t..2t+1)
            const uint32_t u0 = movmatrix_trans(Elem<T>::pack2(st.o[nt][j][0] * inv0, st.o[nt][j][1] * inv1));
            const uint32_t u1 = movmatrix_trans(Elem<T>::pack2(st.o[nt][j][2] * inv0, st.o[nt][j][3] * inv1));
            if (head < p.group) {
                *reinterpret_cast<uint32_t *>(row + 16 * j + 2 * t) = u0;
                *reinterpret_cast<uint32_t *>(row + 16 * j + 8 + 2 * t) = u1;
            }
        }
    }
}

template <int D, int NT>
__host__ __device__ constexpr int rec_floats() {
    return NT * ((D / 16) * 128 + 16);
}

template <typename T, int D, int NT>
__device__ __forceinline__ void write_partial(const AttnState<T, D, NT> &st, float *rec, int lane) {
    float4 *o4 = reinterpret_cast<float4 *>(rec);
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int j = 0; j < D / 16; ++j)
            o4[(nt * (D / 16) + j) * 32 + lane] =
                make_float4(st.o[nt][j][0], st.o[nt][j][1], st.o[nt][j][2], st.o[nt][j][3]);
    float4 *ml4 = reinterpret_cast<float4 *>(rec + NT * (D / 16) * 128);
    if ((lane >> 2) == 0) {
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
            ml4[nt * 4 + (lane & 3)] = make_float4(st.m[nt][0], st.m[nt][1], st.l[nt][0], st.l[nt][1]);
    }
}

// Folds `count` records that lie `stride_floats` apart (shared memory: plain loads) into `st`: the maximum over all
// records first, then the weighted sum.
template <typename T, int D, int NT>
__device__ __forceinline__ void merge_records(AttnState<T, D, NT> &st, const float *first, size_t stride_floats, int count,
                                              int lane) {
    constexpr int KS = D / 16;
    const int t4 = lane & 3;
    float mg[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mg[nt][0] = mg[nt][1] = -INFINITY;
    for (int w = 0; w < count; ++w) {
        const float4 *ml4 = reinterpret_cast<const float4 *>(first + w * stride_floats + NT * KS * 128);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float4 ml = ml4[nt * 4 + t4];
            mg[nt][0] = fmaxf(mg[nt][0], ml.x);
            mg[nt][1] = fmaxf(mg[nt][1], ml.y);
        }
    }
    st.reset();
    for (int w = 0; w < count; ++w) {
        const float *rec = first + w * stride_floats;
        const float4 *o4 = reinterpret_cast<const float4 *>(rec);
        const float4 *ml4 = reinterpret_cast<const float4 *>(rec + NT * KS * 128);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float4 ml = ml4[nt * 4 + t4];
            const float sn0 = ml.x == -INFINITY ? 0.f : fast_exp2(ml.x - mg[nt][0]);
            const float sn1 = ml.y == -INFINITY ? 0.f : fast_exp2(ml.y - mg[nt][1]);
            st.l[nt][0] += ml.z * sn0;
            st.l[nt][1] += ml.w * sn1;
#pragma unroll
            for (int j = 0; j < KS; ++j) {
                const float4 o = o4[(nt * KS + j) * 32 + lane];
                st.o[nt][j][0] += o.x * sn0;
                st.o[nt][j][1] += o.y * sn1;
                st.o[nt][j][2] += o.z * sn0;
                st.o[nt][j][3] += o.w * sn1;
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        st.m[nt][0] = mg[nt][0];
        st.m[nt][1] = mg[nt][1];
    }
}

// Folds the partial records of workers wf..wl (one (sequence, kv head) cut by range boundaries) into `st`.
// Records were written by other SMs during this launch: read them through L2 (ld.global.cg), never L1.
// Two passes, so that no load waits for arithmetic on an earlier one: first the maximum over all records (eight
// records per step, one per lane group), then the weighted sum with four records' loads in flight.  A long
// context in a small batch is cut into a hundred and more partials per kv head; a record-by-record rescaling
// chain made that merge longer than the streaming itself.
template <typename T, int D, int NT>
__device__ __forceinline__ void merge_partials(AttnState<T, D, NT> &st, const DecodeParams &p, int wf, int wl, int lane) {
    constexpr int KS = D / 16;
    const int g = lane >> 2, t4 = lane & 3;
    auto record = [&](int w) { return p.partials + ((size_t)w * 2 + (w == wf ? 1 : 0)) * rec_floats<D, NT>(); };
    float mg[NT][2];
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) mg[nt][0] = mg[nt][1] = -INFINITY;
#pragma unroll 4
    for (int w0 = wf; w0 <= wl; w0 += 8) {
        const int w = w0 + g;
        if (w <= wl) {
            const float4 *ml4 = reinterpret_cast<const float4 *>(record(w) + NT * KS * 128);
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float4 ml = __ldcg(ml4 + nt * 4 + t4);
                mg[nt][0] = fmaxf(mg[nt][0], ml.x);
                mg[nt][1] = fmaxf(mg[nt][1], ml.y);
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
        for (int e = 0; e < 2; ++e)
#pragma unroll
            for (int d = 4; d < 32; d <<= 1) mg[nt][e] = fmaxf(mg[nt][e], __shfl_xor_sync(0xffffffffu, mg[nt][e], d));
    st.reset();
    constexpr int kInFlight = NT * KS >= 16 ? 2 : 4;      // records whose loads are issued together (register budget)
#pragma unroll kInFlight
    for (int w = wf; w <= wl; ++w) {
        const float *rec = record(w);
        const float4 *o4 = reinterpret_cast<const float4 *>(rec);
        const float4 *ml4 = reinterpret_cast<const float4 *>(rec + NT * KS * 128);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
            const float4 ml = __ldcg(ml4 + nt * 4 + t4);
            const float sn0 = ml.x == -INFINITY ? 0.f : fast_exp2(ml.x - mg[nt][0]);
            const float sn1 = ml.y == -INFINITY ? 0.f : fast_exp2(ml.y - mg[nt][1]);
            st.l[nt][0] += ml.z * sn0;
            st.l[nt][1] += ml.w * sn1;
#pragma unroll
            for (int j = 0; j < KS; ++j) {
                const float4 o = __ldcg(o4 + (nt * KS + j) * 32 + lane);
                st.o[nt][j][0] += o.x * sn0;
                st.o[nt][j][1] += o.y * sn1;
                st.o[nt][j][2] += o.z * sn0;
                st.o[nt][j][3] += o.w * sn1;
            }
        }
    }
#pragma unroll
    for (int nt = 0; nt < NT; ++nt) {
        st.m[nt][0] = mg[nt][0];
        st.m[nt][1] = mg[nt][1];
    }
}

// ---------------------------------------------------------------------------
// Streaming kernel
// ---------------------------------------------------------------------------
// IL selects the interleaved cache layouts of the reference's split-K op (K [blocks, Hkv, D/8, B, 8], V
// [blocks, Hkv, D, B]; csrc/paged_attention_optimized/index.h:14-31,60-75): a K tile lands as [d piece][token][8]
// and feeds ldmatrix directly (8 tokens of one piece are 128 contiguous bytes), a V tile lands as [d][token] and is
// already the A operand of O^T = V^T . P^T, so it is read without the transposing ldmatrix.
// MAXW (8 or 12) is the largest number of warps an instance is launched with.  The 8-warp instances are compiled
// for at most 224 registers per thread: enough for the merge of split sequences to keep four records' loads in
// flight, while 8 x 32 x 224 registers leave an eighth of the register file to a small CTA of another stream (the
// page migration kernel) on the same SM.  The 12-warp instances (168 registers) trade registers for warps.
#ifndef NPD_DECODE_MAX_WARPS
#define NPD_DECODE_MAX_WARPS 12
#endif
// SMALL: the form for small batches of short sequences (the reference's operating range: up to 16 sequences of a
// few hundred tokens).  There the equal-work split of the streaming form costs more than it saves — a prefix over
// all sequences, a dozen partial records per (sequence, kv head) written to global memory, a ticket and a merge by
// the last worker: 12-14 us for a launch whose copies take one.  In the small form a CTA owns ONE (sequence, kv
// head): its warps take equal runs of the sequence's tiles, leave their partial records in shared memory (each in
// its own, by then idle, ring) and warp 0 merges them.  No prefix, no workspace traffic, no ticket.
template <typename T, int D, int NT, bool IL, int MAXW, bool SMALL = false>
__global__ void __maxnreg__(MAXW <= 8 ? 224 : 168)
paged_decode_stream_kernel(const DecodeParams p, const __grid_constant__ CUtensorMap tm_k,
                           const __grid_constant__ CUtensorMap tm_v) {
    constexpr int NH = D / 64;
    constexpr int KS = D / 16;
    constexpr int TILE_BYTES = kTile * D * 2;
    constexpr int STAGE_BYTES = 2 * TILE_BYTES;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = smem_u32(smem_raw);
    const uint32_t pad = ((raw_addr + 1023u) & ~1023u) - raw_addr;
    uint8_t *sbase = smem_raw + pad;

    const int nwarps = blockDim.x >> 5;
    const int nst = p.num_stages;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int g = lane >> 2, t4 = lane & 3;

    uint8_t *stage_base = sbase + (size_t)warp * nst * STAGE_BYTES;
    uint64_t *bars = reinterpret_cast<uint64_t *>(sbase + (size_t)nwarps * nst * STAGE_BYTES) + warp * nst;
    int *pre = reinterpret_cast<int *>(sbase + (size_t)nwarps * nst * (STAGE_BYTES + 8));

    if (lane == 0) {
        for (int i = 0; i < nst; ++i) mbar_init(smem_u32(bars + i), 1);
        mbar_fence_init();
    }
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tm_k);
        tma_prefetch_desc(&tm_v);
    }
    long long W = 0;
    int worker = 0, my_tiles = 0;
    Cursor pc, cc;                   // producer / consumer cursors over the same range
    if (SMALL) {
        __syncthreads();             // barriers are initialised for everyone
        const int s0 = blockIdx.x / p.num_vheads, h0 = blockIdx.x - s0 * p.num_vheads;
        const int raw = __ldg(p.seq_lens + s0);
        if ((raw < 0 || raw > (long long)p.max_blocks_per_seq * p.block_size) && h0 == 0 && threadIdx.x == 0)
            atomicOr(p.status, NPD_STATUS_BAD_POSITION);
        const int len0 = clamped_len(p, s0), n0 = (len0 + kTile - 1) / kTile;
        if (n0 == 0) {
            // an empty sequence gets zero rows (see below); this CTA writes those of its own q heads
            uint32_t *row = reinterpret_cast<uint32_t *>(static_cast<T *>(p.out) +
                                                         ((long long)s0 * p.num_q_heads + (long long)h0 * p.group) * D);
            for (int i = threadIdx.x; i < p.group * D / 2; i += blockDim.x) row[i] = 0u;
            return;                  // the whole CTA leaves here: no barrier follows for anyone
        }
        const int per_warp = (n0 + nwarps - 1) / nwarps;
        const int t0 = warp * per_warp;
        W = per_warp;
        worker = warp;
        my_tiles = max(0, min(per_warp, n0 - t0));
        pc.s = s0, pc.h = h0, pc.t = min(t0, n0 - 1), pc.n = n0, pc.len = len0;
    } else {
        build_tile_prefix(p, pre);   // ends with __syncthreads(): barriers are initialised for everyone
        // Empty sequences get zero rows, as the reference's kernel leaves them
        // (nanoPD/paged_attention/csrc/attention/paged_attention_kernel.cu:117-150 with seq_len 0).
        for (int s0 = blockIdx.x; s0 < p.num_seqs; s0 += gridDim.x) {
            if (pre[s0 + 1] != pre[s0]) continue;
            uint32_t *row = reinterpret_cast<uint32_t *>(static_cast<T *>(p.out) + (long long)s0 * p.num_q_heads * D);
            for (int i = threadIdx.x; i < p.num_q_heads * D / 2; i += blockDim.x) row[i] = 0u;
        }

        const long long total = (long long)p.num_vheads * pre[p.num_seqs];
        W = tiles_per_worker(total, p.num_workers, (long long)p.num_vheads * p.num_seqs);
        worker = blockIdx.x * nwarps + warp;
        const long long f_begin = (long long)worker * W;
        if (f_begin >= total) return;
        const long long f_end = min(f_begin + W, total);
        my_tiles = static_cast<int>(f_end - f_begin);
        cursor_seek(pc, f_begin, pre, p);
    }
    cc = pc;

    // ---- per-lane shared-memory offsets of the ldmatrix rows (same for every tile) ----
    const int mi = lane >> 3, mrow = lane & 7;
    const int k_r = (mi & 1) * 8 + mrow;    // K: matrices 0/1 = tokens 0-7 / 8-15, 2/3 = next 8 d
    const int v_r = (mi >> 1) * 8 + mrow;   // V: matrices 0/1 = d pieces, 2/3 = tokens 8-15
    const int k_row_off = (k_r / p.box_rows) * (NH * p.box_rows * 128) + (k_r % p.box_rows) * 128;
    const int v_row_off = (v_r / p.box_rows) * (NH * p.box_rows * 128) + (v_r % p.box_rows) * 128;
    const int half_bytes = p.box_rows * 128;
    // swizzle phase of this lane's row in each 64-element slab: the row's 128-byte index within its 1024-byte atom
    int k_phase[NH], v_phase[NH];
#pragma unroll
    for (int hf = 0; hf < NH; ++hf) {
        k_phase[hf] = ((k_row_off + hf * half_bytes) >> 7) & 7;
        v_phase[hf] = ((v_row_off + hf * half_bytes) >> 7) & 7;
    }
    // interleaved layouts: a box holds box_rows tokens; K box = [D/8 pieces][box_rows][16 B], V box = [D][box_rows x 2 B]
    const int box_bytes = p.box_rows * D * 2;
    const int il_k_off = (k_r / p.box_rows) * box_bytes + (k_r % p.box_rows) * 16;       // + piece * box_rows * 16
    const int il_v_tok = (mi >> 1) * 8;                                                  // token piece of this lane's matrix
    const int il_v_off = (il_v_tok / p.box_rows) * box_bytes + (il_v_tok % p.box_rows) * 2 +
                         ((mi & 1) * 8 + mrow) * (p.box_rows * 2);                         // + 16 j rows

    TableWindow win{-1, 0, 0};

    int issued = 0;
    auto issue_tile = [&](int stage) {
        // Executed by the whole warp (uniform), the copies by lane 0.
        const int tok0 = pc.t * kTile;
        const int npages = (pc.len + p.block_size - 1) / p.block_size;
        const int nbox_total = kTile / p.box_rows;
        int nbox = 0;
        for (int k = 0; k < nbox_total; ++k) nbox += (tok0 + k * p.box_rows < pc.len) ? 1 : 0;
        const uint32_t bar = smem_u32(bars + stage);
        const uint32_t kdst = smem_u32(stage_base + (size_t)stage * STAGE_BYTES);
        const uint32_t vdst = kdst + TILE_BYTES;
        const int phys_head = pc.h / p.kv_rep;
        if (lane == 0) {
            fence_proxy_async_smem();
            mbar_expect_tx(bar, static_cast<uint32_t>(nbox * 2 * NH * p.box_rows * 128));
        }
        for (int k = 0; k < nbox; ++k) {
            const int token = tok0 + k * p.box_rows;
            const int page = token / p.block_size;
            const int row_in_page = token - page * p.block_size;
            int id = table_lookup(win, pc.s, page, npages, lane, p);
            if (id < 0 || id >= p.num_blocks) {
                if (lane == 0) atomicOr(p.status, NPD_STATUS_BAD_BLOCK_ID);
                id = p.num_blocks;   // out of bounds for the tensor map: the box is zero-filled
            }
            if (lane == 0) {
                if (IL) {
                    const uint32_t off = static_cast<uint32_t>(k * box_bytes);
                    tma_load_3d(kdst + off, &tm_k, bar, row_in_page * 8, phys_head * (D / 8), id);
                    tma_load_3d(vdst + off, &tm_v, bar, row_in_page, phys_head * D, id);
                } else {
                    const int row = phys_head * p.block_size + row_in_page;
#pragma unroll
                    for (int hf = 0; hf < NH; ++hf) {
                        const uint32_t off = static_cast<uint32_t>(k * (NH * half_bytes) + hf * half_bytes);
                        tma_load_3d(kdst + off, &tm_k, bar, hf * 64, row, id);
                        tma_load_3d(vdst + off, &tm_v, bar, hf * 64, row, id);
                    }
                }
            }
        }
        ++issued;
        if (issued < my_tiles) cursor_advance(pc, pre, p);
    };

    const int prologue = min(nst, my_tiles);
    for (int i = 0; i < prologue; ++i) issue_tile(i);

    AttnState<T, D, NT> st;
    uint32_t qf[NT][KS][2];
    bool dead = false;
    int stage = 0;
    uint32_t parity = 0;
    int done = 0;

    while (done < my_tiles && !dead) {
        // ---- one segment: the tiles of (cc.s, cc.h) that lie inside this worker's range ----
        const int seg_s = cc.s, seg_h = cc.h, seg_len = cc.len;
        const int t_first = cc.t;
        const int seg_tiles = min(cc.n - cc.t, my_tiles - done);
        const bool head_cut = t_first > 0;
        const bool tail_cut = t_first + seg_tiles < cc.n;

        // Q as the B operand: b0b1 = Q[head g][16ks+2t..], b2b3 = Q[head g][16ks+8+2t..]
        {
            const T *qbase = static_cast<const T *>(p.q) +
                             ((long long)seg_s * p.num_q_heads + (long long)seg_h * p.group) * D;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const int head = nt * 8 + g;
                const uint32_t *qrow = reinterpret_cast<const uint32_t *>(qbase + (long long)head * D);
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    qf[nt][ks][0] = head < p.group ? __ldg(qrow + 8 * ks + t4) : 0u;
                    qf[nt][ks][1] = head < p.group ? __ldg(qrow + 8 * ks + 4 + t4) : 0u;
                }
            }
        }
        st.reset();

        for (int it = 0; it < seg_tiles; ++it) {
            const uint32_t bar = smem_u32(bars + stage);
            if (!mbar_wait_bounded(bar, parity)) {
                if (lane == 0) atomicOr(p.status, NPD_STATUS_WAIT_TIMEOUT);
                dead = true;
            }
            dead = __any_sync(0xffffffffu, dead);
            if (dead) break;

            uint8_t *kt = stage_base + (size_t)stage * STAGE_BYTES;
            uint8_t *vt = kt + TILE_BYTES;
            const uint32_t ks_addr = smem_u32(kt), vs_addr = smem_u32(vt);
            const int tok0 = (t_first + it) * kTile;
            const int valid = min(kTile, seg_len - tok0);

            if (valid < kTile) {
                // V rows past the sequence end may hold anything (NaN included): P is exactly 0
                // there, and 0 * NaN would still poison O, so clear them.
                if (IL) {
                    const int dead_toks = kTile - valid;
                    for (int idx = lane; idx < dead_toks * D; idx += 32) {
                        const int d = idx / dead_toks, tk = valid + idx % dead_toks;
                        *reinterpret_cast<uint16_t *>(vt + (tk / p.box_rows) * box_bytes + d * (p.box_rows * 2) +
                                                      (tk % p.box_rows) * 2) = 0;
                    }
                } else {
                    const int cnt = (kTile - valid) * NH * 8;
                    for (int idx = lane; idx < cnt; idx += 32) {
                        const int r = valid + idx / (NH * 8);
                        const int c = idx % (NH * 8);
                        *reinterpret_cast<uint4 *>(vt + tile_offset<D>(r, c, p.box_rows)) = make_uint4(0, 0, 0, 0);
                    }
                }
                __syncwarp();
            }

            // ---- S^T = K . Q^T  (two accumulator chains) ----
            float sa[NT][4], sb[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int e = 0; e < 4; ++e) sa[nt][e] = sb[nt][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                uint32_t a[4];
                const int c = 2 * ks + (mi >> 1);
                if (IL) ldmatrix_x4(a, ks_addr + il_k_off + c * (p.box_rows * 16));
                else ldmatrix_x4(a, ks_addr + k_row_off + (ks >> 2) * half_bytes + (((c & 7) ^ k_phase[ks >> 2]) << 4));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                    if (ks & 1) Elem<T>::mma16816(sb[nt], a, qf[nt][ks][0], qf[nt][ks][1]);
                    else        Elem<T>::mma16816(sa[nt], a, qf[nt][ks][0], qf[nt][ks][1]);
                }
            }

            // ---- online softmax (log2 domain), P^T as B operand ----
            uint32_t pb[NT][2];
            const bool va = tok0 + g < seg_len, vb = tok0 + g + 8 < seg_len;
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
                const float x0 = va ? (sa[nt][0] + sb[nt][0]) * p.scale_log2 : -INFINITY;
                const float x1 = va ? (sa[nt][1] + sb[nt][1]) * p.scale_log2 : -INFINITY;
                const float x2 = vb ? (sa[nt][2] + sb[nt][2]) * p.scale_log2 : -INFINITY;
                const float x3 = vb ? (sa[nt][3] + sb[nt][3]) * p.scale_log2 : -INFINITY;
                float mx0 = fmaxf(x0, x2), mx1 = fmaxf(x1, x3);
#pragma unroll
                for (int d = 4; d < 32; d <<= 1) {
                    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, d));
                    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, d));
                }
                const float mn0 = fmaxf(st.m[nt][0], mx0), mn1 = fmaxf(st.m[nt][1], mx1);
                const float p0 = fast_exp2(x0 - mn0), p1 = fast_exp2(x1 - mn1);
                const float p2 = fast_exp2(x2 - mn0), p3 = fast_exp2(x3 - mn1);
                // O and l are rescaled only in tiles where some head's maximum grew (warp-uniform test): deep
                // into a sequence that is the exception, and the 4*KS multiplies are the bulk of the softmax code
                if (__any_sync(0xffffffffu, mn0 != st.m[nt][0] || mn1 != st.m[nt][1])) {
                    const float a0 = fast_exp2(st.m[nt][0] - mn0), a1 = fast_exp2(st.m[nt][1] - mn1);
                    st.l[nt][0] *= a0;
                    st.l[nt][1] *= a1;
                    st.m[nt][0] = mn0;
                    st.m[nt][1] = mn1;
#pragma unroll
                    for (int j = 0; j < KS; ++j) {
                        st.o[nt][j][0] *= a0;
                        st.o[nt][j][1] *= a1;
                        st.o[nt][j][2] *= a0;
                        st.o[nt][j][3] *= a1;
                    }
                }
                st.l[nt][0] += p0 + p2;
                st.l[nt][1] += p1 + p3;
                pb[nt][0] = movmatrix_trans(Elem<T>::pack2(p0, p1));
                pb[nt][1] = movmatrix_trans(Elem<T>::pack2(p2, p3));
            }

            // ---- O^T += V^T . P^T ----
#pragma unroll
            for (int j = 0; j < KS; ++j) {
                uint32_t a[4];
                const int c = 2 * j + (mi & 1);
                if (IL) ldmatrix_x4(a, vs_addr + il_v_off + j * 16 * (p.box_rows * 2));
                else ldmatrix_x4_trans(a, vs_addr + v_row_off + (j >> 2) * half_bytes + (((c & 7) ^ v_phase[j >> 2]) << 4));
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) Elem<T>::mma16816(st.o[nt][j], a, pb[nt][0], pb[nt][1]);
            }

            // ---- the stage is free: refill it ----
            __syncwarp();
            if (issued < my_tiles) issue_tile(stage);
            if (++stage == nst) {
                stage = 0;
                parity ^= 1u;
            }
            ++done;
            if (done < my_tiles) cursor_advance(cc, pre, p);
        }
        if (dead) break;

        st.reduce_l();
        if (SMALL) {
            // this warp's run is done and nothing is in flight into its ring: the record goes there
            write_partial<T, D, NT>(st, reinterpret_cast<float *>(stage_base), lane);
        } else if (!head_cut && !tail_cut) {
            write_output<T, D, NT>(st, p, seg_s, seg_h, lane);
        } else {
            float *rec = p.partials + ((size_t)worker * 2 + (head_cut ? 0 : 1)) * rec_floats<D, NT>();
            write_partial<T, D, NT>(st, rec, lane);
            if (!p.skip_merge) {
                // Which workers share this (sequence, kv head)?  The one whose ticket is the last merges.
                const int n_s = pre[seg_s + 1] - pre[seg_s];
                const long long fb = (long long)p.num_vheads * pre[seg_s] + (long long)seg_h * n_s;
                const int wf = static_cast<int>(fb / W), wl = static_cast<int>((fb + n_s - 1) / W);
                __threadfence();                       // every lane: my part of the record is visible device-wide
                __syncwarp();
                int ticket = 0;
                int *slot = p.tickets + seg_s * p.num_vheads + seg_h;
                if (lane == 0) ticket = atomicAdd(slot, 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket == wl - wf) {
                    __threadfence();                   // the other workers' records are visible to me
                    merge_partials<T, D, NT>(st, p, wf, wl, lane);
                    write_output<T, D, NT>(st, p, seg_s, seg_h, lane);
                    if (lane == 0) *slot = 0;          // ready for the next launch
                }
            }
        }
    }

    if (SMALL) {
        __syncthreads();             // every warp's record is in shared memory (all warps of the CTA get here)
        if (warp == 0) {
            const int n_records = (pc.n + static_cast<int>(W) - 1) / static_cast<int>(W);     // warps that had tiles
            AttnState<T, D, NT> merged;
            merge_records<T, D, NT>(merged, reinterpret_cast<const float *>(sbase), (size_t)nst * STAGE_BYTES / sizeof(float),
                                    n_records, lane);
            write_output<T, D, NT>(merged, p, pc.s, pc.h, lane);
        }
    }
    if (dead) {
        // Give copies still in flight one more bounded chance to land before the CTA's shared
        // memory can be handed to another CTA.
        const int outstanding = issued - done;
        for (int i = 0; i < outstanding && i < nst; ++i) {
            (void)mbar_wait_bounded(smem_u32(bars + stage), parity, 200000000LL);
            if (++stage == nst) {
                stage = 0;
                parity ^= 1u;
            }
        }
    }
}

// ---------------------------------------------------------------------------
// Host side
// ---------------------------------------------------------------------------
struct LaunchShape {
    int nwarps, nstages, grid;
    bool small;     // the small-batch form: one CTA per (sequence, virtual kv head)
};

int env_int(const char *name, int fallback) {
    const char *v = std::getenv(name);
    if (!v || !*v) return fallback;
    const int x = std::atoi(v);
    return x > 0 ? x : fallback;
}

// Warps per CTA and ring depth.  A warp is bound by the latency of its own instruction chain (a tile every
// ~1.4 us), so the SM's bandwidth comes from the number of warps, not from deeper rings: two stages do as well as
// three.  Measured on a B200 (microseconds per launch; configuration 2 unless noted):
//   D=128, full grid:   8 warps 238-240, 12 warps 249 (more request streams than HBM serves well)
//   D=128, 100 CTAs:    8 warps 323,     12 warps 243 -> a capped grid (a mixed step sharing the SMs) takes 12
//   D=128, block 8:     8 warps 263,     12 warps 235
//   D=64:               8 warps 107,     12 warps 81
//   D=256:              4 warps x 3 stages 135, 8 warps x 1 stage 122
//   D=128, one sequence of 8k / 64k tokens: 3 stages 29 / 76, 2 stages 36 / 86
LaunchShape launch_shape(int head_dim, int block_size, int cta_cap, long long num_seq_heads, int device) {
    LaunchShape ls;
    const int stage_bytes = 2 * kTile * head_dim * 2;
    const int sms = npd::sm_count(device);
    // tuning knobs from the environment, read once per process
    static const int knob_ctas = env_int("NPD_DECODE_CTAS", 0), knob_warps = env_int("NPD_DECODE_WARPS", 0),
                     knob_stages = env_int("NPD_DECODE_STAGES", 0);
    ls.grid = knob_ctas > 0 ? knob_ctas : sms;
    if (cta_cap > 0 && cta_cap < ls.grid) ls.grid = cta_cap;
    int warps = 8, stages = 2;
    if (head_dim == 256) stages = 1;
    // a handful of long sequences: every worker has few tiles and the launch is latency-bound, a deeper ring helps
    if (head_dim == 128 && num_seq_heads < 64) stages = 3;
    if (head_dim == 64 || (head_dim == 128 && (block_size < 16 || ls.grid * 100 < sms * 85))) warps = 12;
    ls.nwarps = knob_warps > 0 ? knob_warps : warps;
    if (ls.nwarps > NPD_DECODE_MAX_WARPS) ls.nwarps = NPD_DECODE_MAX_WARPS;   // the kernel's launch bound
    int nst = knob_stages > 0 ? knob_stages : stages;
    while (nst > 1 && (long long)ls.nwarps * nst * stage_bytes > 192 * 1024) --nst;
    ls.nstages = nst;
    ls.small = false;
    return ls;
}

// The small-batch form is taken when no sequence can be longer than kSmallMaxTokens (the table's width bounds it:
// the reference's caller pads its tables to the longest sequence of the batch, nanoPD/engine/model_runner.py:176-187)
// and every (sequence, virtual kv head) gets an SM of its own.  Standard layout, uncapped grid.  Device time per
// launch on a B200, small form / streaming form (Qwen3-8B shape, bf16): 1 sequence of up to 512 tokens 6.3 / 10.0 us,
// 8 x 512: 9.6 / 14.9, 16 x 256: 7.6 / 15.0, 16 x 1024: 16.0 / 19.5, 16 x 2048: 26.6 / 26.7, 4 x 2048: 22.6 / 18.4 —
// beyond a thousand tokens a CTA's eight warps stream too long for the saved merge to pay.
constexpr long long kSmallMaxTokens = 1024;
void consider_small_form(LaunchShape &ls, int head_dim, long long max_tokens, long long seq_heads, int cta_cap,
                         bool interleaved, int flags, int device) {
    static const int knob = env_int("NPD_DECODE_SMALL", 1);      // 2 = off (for experiments; read once per process)
    if (knob == 2 || (flags & NPD_DECODE_NO_SMALL) || interleaved || cta_cap > 0) return;
    if (max_tokens > kSmallMaxTokens || seq_heads < 1 || seq_heads > npd::sm_count(device)) return;
    const int stage_bytes = 2 * kTile * head_dim * 2;
    ls.small = true;
    ls.grid = static_cast<int>(seq_heads);
    ls.nwarps = 8;
    ls.nstages = head_dim == 256 ? 1 : (head_dim == 128 ? 3 : 4);
    while (ls.nstages > 1 && (long long)ls.nwarps * ls.nstages * stage_bytes > 192 * 1024) --ls.nstages;
}

// Smallest split of the group into virtual kv heads whose q-head count fits the n-tiles.
int choose_kv_rep(int group, int max_heads) {
    for (int r = 1; r <= group; ++r)
        if (group % r == 0 && group / r <= max_heads) return r;
    return group;
}

size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

template <typename T, int D, int NT, bool IL>
int launch_decode(const DecodeParams &p, const CUtensorMap &tk, const CUtensorMap &tv, const LaunchShape &ls,
                  cudaStream_t stream) {
    constexpr int STAGE_BYTES = 2 * kTile * D * 2;
    const size_t smem = 1024 + (size_t)ls.nwarps * ls.nstages * (STAGE_BYTES + 8) + ((size_t)p.num_seqs + 1) * 4 + 16;
    // Largest shared-memory carve-out on both instances: the SM then has room for a small CTA of another stream
    // (the page migration kernel asks for the same), instead of being configured for this CTA alone.
    if (ls.small) {
        if constexpr (!IL) {
            auto kern = paged_decode_stream_kernel<T, D, NT, false, 8, true>;
            NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
            NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
            kern<<<ls.grid, ls.nwarps * 32, smem, stream>>>(p, tk, tv);
        }
    } else if (ls.nwarps <= 8) {
        auto kern = paged_decode_stream_kernel<T, D, NT, IL, 8>;
        NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        kern<<<ls.grid, ls.nwarps * 32, smem, stream>>>(p, tk, tv);
    } else {
        auto kern = paged_decode_stream_kernel<T, D, NT, IL, NPD_DECODE_MAX_WARPS>;
        NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        NPD_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared));
        kern<<<ls.grid, ls.nwarps * 32, smem, stream>>>(p, tk, tv);
    }
    NPD_CUDA_TRY(cudaGetLastError());
    return NPD_OK;
}

template <typename T, bool IL>
int dispatch_decode(int head_dim, int nt, const DecodeParams &p, const CUtensorMap &tk, const CUtensorMap &tv,
                    const LaunchShape &ls, cudaStream_t stream) {
    if (head_dim == 64 && nt == 1) return launch_decode<T, 64, 1, IL>(p, tk, tv, ls, stream);
    if (head_dim == 64 && nt == 2) return launch_decode<T, 64, 2, IL>(p, tk, tv, ls, stream);
    if (head_dim == 128 && nt == 1) return launch_decode<T, 128, 1, IL>(p, tk, tv, ls, stream);
    if (head_dim == 128 && nt == 2) return launch_decode<T, 128, 2, IL>(p, tk, tv, ls, stream);
    if (head_dim == 256 && nt == 1) return launch_decode<T, 256, 1, IL>(p, tk, tv, ls, stream);
    return npd::fail(NPD_ERR_UNSUPPORTED, "decode attention: no kernel for head_dim %d with %d head tiles", head_dim, nt);
}

struct WorkspacePlan {
    size_t ticket_off, partial_off, total;
    int kv_rep, nt, group;
};

WorkspacePlan plan_workspace(int64_t num_seqs, int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim,
                             const LaunchShape &ls) {
    WorkspacePlan w;
    const int group_full = static_cast<int>(num_q_heads / (num_kv_heads > 0 ? num_kv_heads : 1));
    const int max_heads = head_dim == 256 ? 8 : 16;
    w.kv_rep = choose_kv_rep(group_full > 0 ? group_full : 1, max_heads);
    w.group = (group_full > 0 ? group_full : 1) / w.kv_rep;
    w.nt = w.group <= 8 ? 1 : 2;
    const size_t seqs = static_cast<size_t>(num_seqs < kMaxSeqsPerLaunch ? num_seqs : kMaxSeqsPerLaunch);
    const size_t rec = (size_t)w.nt * ((size_t)(head_dim / 16) * 128 + 16) * sizeof(float);
    (void)seqs;
    w.ticket_off = kStatusBytes;
    w.partial_off = align_up(w.ticket_off + (size_t)kTicketCapacity * sizeof(int32_t), 256);
    w.total = w.partial_off + (size_t)ls.grid * ls.nwarps * 2 * rec;
    return w;
}

}  // namespace

extern "C" size_t npd_decode_workspace_bytes(int64_t num_seqs, int64_t num_q_heads, int64_t num_kv_heads,
                                             int64_t head_dim, int device) {
    if (num_seqs < 0 || num_q_heads <= 0 || num_kv_heads <= 0 || head_dim <= 0) return 0;
    // Sized for the largest grid/warp shape the launcher may pick, so tuning knobs never outgrow it.
    LaunchShape ls = launch_shape(static_cast<int>(head_dim), 16, 0, 1 << 20, device);
    if (ls.nwarps < NPD_DECODE_MAX_WARPS) ls.nwarps = NPD_DECODE_MAX_WARPS;
    return plan_workspace(num_seqs, num_q_heads, num_kv_heads, head_dim, ls).total;
}

extern "C" int npd_paged_decode_attention(void *out, const void *q, const void *k_cache, const void *v_cache,
                                          const int32_t *block_tables, const int32_t *seq_lens, float scale,
                                          int64_t num_seqs, int64_t num_q_heads, int64_t num_kv_heads,
                                          int64_t head_dim, int64_t block_size, int64_t max_blocks_per_seq,
                                          int64_t num_blocks, int64_t cache_block_stride, int64_t bt_row_stride,
                                          int dtype, void *workspace, size_t workspace_bytes, int flags,
                                          void *stream) {
    NPD_REQUIRE(dtype == NPD_DTYPE_F16 || dtype == NPD_DTYPE_BF16, NPD_ERR_UNSUPPORTED,
                "decode attention supports float16 and bfloat16 only (dtype code %d)", dtype);
    NPD_REQUIRE(head_dim == 64 || head_dim == 128 || head_dim == 256, NPD_ERR_UNSUPPORTED,
                "decode attention: head_dim %lld not in {64,128,256}", (long long)head_dim);
    NPD_REQUIRE(block_size == 4 || block_size == 8 || block_size == 16 || block_size == 32, NPD_ERR_UNSUPPORTED,
                "decode attention: block_size %lld not in {4,8,16,32}", (long long)block_size);
    NPD_REQUIRE(num_seqs >= 0 && num_q_heads > 0 && num_kv_heads > 0 && max_blocks_per_seq > 0 && num_blocks > 0,
                NPD_ERR_INVALID_ARG, "decode attention: non-positive dimension");
    NPD_REQUIRE(num_q_heads % num_kv_heads == 0, NPD_ERR_INVALID_ARG,
                "decode attention: num_q_heads %lld is not a multiple of num_kv_heads %lld", (long long)num_q_heads,
                (long long)num_kv_heads);
    if (num_seqs == 0) return NPD_OK;
    NPD_REQUIRE(out && q && k_cache && v_cache && block_tables && seq_lens, NPD_ERR_INVALID_ARG,
                "decode attention: NULL pointer");
    NPD_REQUIRE(npd::aligned16(out) && npd::aligned16(q), NPD_ERR_INVALID_ARG,
                "decode attention: q/out must be 16-byte aligned");
    NPD_REQUIRE(cache_block_stride >= num_kv_heads * block_size * head_dim, NPD_ERR_INVALID_ARG,
                "decode attention: cache block stride smaller than one block");
    NPD_REQUIRE(num_blocks < INT32_MAX && max_blocks_per_seq * block_size < INT32_MAX &&
                    num_seqs * num_q_heads < INT32_MAX,
                NPD_ERR_INVALID_ARG, "decode attention: dimension exceeds int32");

    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    LaunchShape ls = launch_shape(static_cast<int>(head_dim), static_cast<int>(block_size), (flags >> 8) & 0xffff,
                                  (long long)num_seqs * num_kv_heads, dev);
    const WorkspacePlan wp = plan_workspace(num_seqs, num_q_heads, num_kv_heads, head_dim, ls);
    NPD_REQUIRE(workspace != nullptr && workspace_bytes >= wp.total, NPD_ERR_WORKSPACE,
                "decode attention: workspace of %zu bytes given, %zu needed", workspace_bytes, wp.total);
    consider_small_form(ls, static_cast<int>(head_dim), (long long)max_blocks_per_seq * block_size,
                        (long long)num_seqs * num_kv_heads * wp.kv_rep, (flags >> 8) & 0xffff,
                        (flags & NPD_DECODE_KV_INTERLEAVED) != 0, flags, dev);
    NPD_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, NPD_ERR_WORKSPACE,
                "decode attention: workspace must be 256-byte aligned");

    CUtensorMap tk, tv;
    const int box_rows = block_size < 16 ? static_cast<int>(block_size) : 16;
    const bool interleaved = (flags & NPD_DECODE_KV_INTERLEAVED) != 0;
    int rc;
    if (interleaved) {
        NPD_REQUIRE(block_size >= 8, NPD_ERR_UNSUPPORTED,
                    "decode attention: the interleaved layouts need block_size >= 8 (a V row of a block is "
                    "block_size * 2 bytes, and a TMA box row is at least 16)");
        // K [blocks, Hkv, D/8, B, 8]: rows of B*8 elements, one per (kv head, 8-element piece of the head dim);
        // V [blocks, Hkv, D, B]: rows of B elements, one per (kv head, head-dim element).  No swizzle.
        const uint64_t kdims[3] = {(uint64_t)block_size * 8, (uint64_t)(num_kv_heads * head_dim / 8), (uint64_t)num_blocks};
        const uint64_t kstr[2] = {(uint64_t)block_size * 16, (uint64_t)cache_block_stride * 2};
        const uint32_t kbox[3] = {(uint32_t)box_rows * 8, (uint32_t)(head_dim / 8), 1u};
        rc = npd::encode_tiled_3d(&tk, k_cache, dtype, kdims, kstr, kbox, false);
        if (rc != NPD_OK) return rc;
        const uint64_t vdims[3] = {(uint64_t)block_size, (uint64_t)(num_kv_heads * head_dim), (uint64_t)num_blocks};
        const uint64_t vstr[2] = {(uint64_t)block_size * 2, (uint64_t)cache_block_stride * 2};
        const uint32_t vbox[3] = {(uint32_t)box_rows, (uint32_t)head_dim, 1u};
        rc = npd::encode_tiled_3d(&tv, v_cache, dtype, vdims, vstr, vbox, false);
        if (rc != NPD_OK) return rc;
    } else {
        rc = npd::encode_cache_tensor_map(&tk, k_cache, dtype, head_dim, num_kv_heads * block_size, num_blocks,
                                          cache_block_stride, box_rows);
        if (rc != NPD_OK) return rc;
        rc = npd::encode_cache_tensor_map(&tv, v_cache, dtype, head_dim, num_kv_heads * block_size, num_blocks,
                                          cache_block_stride, box_rows);
        if (rc != NPD_OK) return rc;
    }

    uint8_t *ws = static_cast<uint8_t *>(workspace);
    DecodeParams p;
    p.status = reinterpret_cast<int32_t *>(ws);
    p.tickets = reinterpret_cast<int32_t *>(ws + wp.ticket_off);
    p.partials = reinterpret_cast<float *>(ws + wp.partial_off);
    p.scale_log2 = scale * 1.4426950408889634f;
    p.num_q_heads = static_cast<int>(num_q_heads);
    p.kv_rep = wp.kv_rep;
    p.num_vheads = static_cast<int>(num_kv_heads) * wp.kv_rep;
    p.group = wp.group;
    p.block_size = static_cast<int>(block_size);
    p.box_rows = box_rows;
    p.max_blocks_per_seq = static_cast<int>(max_blocks_per_seq);
    p.num_blocks = static_cast<int>(num_blocks);
    p.bt_row_stride = bt_row_stride;
    p.num_workers = ls.grid * ls.nwarps;
    p.num_stages = ls.nstages;

    const size_t elem = 2;
    p.skip_merge = (flags & NPD_DECODE_SKIP_MERGE) != 0;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // Batches beyond the shared-memory prefix capacity run as consecutive sub-batches; the
    // stream orders their use of the workspace.
    int64_t batch_cap = kTicketCapacity / p.num_vheads;
    if (batch_cap > kMaxSeqsPerLaunch) batch_cap = kMaxSeqsPerLaunch;
    NPD_REQUIRE(batch_cap >= 1, NPD_ERR_UNSUPPORTED, "decode attention: too many kv heads (%d virtual heads)", p.num_vheads);
    for (int64_t s0 = 0; s0 < num_seqs; s0 += batch_cap) {
        const int64_t ns = num_seqs - s0 < batch_cap ? num_seqs - s0 : batch_cap;
        p.num_seqs = static_cast<int>(ns);
        p.out = static_cast<uint8_t *>(out) + (size_t)s0 * num_q_heads * head_dim * elem;
        p.q = static_cast<const uint8_t *>(q) + (size_t)s0 * num_q_heads * head_dim * elem;
        p.block_tables = block_tables + s0 * bt_row_stride;
        p.seq_lens = seq_lens + s0;
        const int hd = static_cast<int>(head_dim);
        if (interleaved)
            rc = dtype == NPD_DTYPE_F16 ? dispatch_decode<__half, true>(hd, wp.nt, p, tk, tv, ls, st)
                                        : dispatch_decode<__nv_bfloat16, true>(hd, wp.nt, p, tk, tv, ls, st);
        else
            rc = dtype == NPD_DTYPE_F16 ? dispatch_decode<__half, false>(hd, wp.nt, p, tk, tv, ls, st)
                                        : dispatch_decode<__nv_bfloat16, false>(hd, wp.nt, p, tk, tv, ls, st);
        if (rc != NPD_OK) return rc;
    }
    return NPD_OK;
}

// ---------------------------------------------------------------------------
// Decode attention for callers that must not allocate device memory
// ---------------------------------------------------------------------------
// Some hosts of this library cannot hand it a workspace: a decode worker that gave all free
// HBM to the KV block pool and the weights at start-up, a step loop with a "no allocation
// after initialisation" rule, or a foreign-language runtime binding the C ABI without a device
// allocator of its own (and cudaMalloc / cudaFree would stall every stream of the device
// anyway).  For them the scratch below is part of the library image: every GPU that loads the
// library holds these 32 MiB until the process exits.  It is large enough for every supported
// shape on a B200 (148 SMs x 12 workers x 2 partial records of at most 8320 B, plus the ticket region and header).
#define NPD_STATIC_SCRATCH_BYTES (32u << 20)
static __device__ __align__(256) unsigned char g_decode_static_scratch[NPD_STATIC_SCRATCH_BYTES];

namespace {

// In host code `g_decode_static_scratch` is only a stand-in for the device array; the device
// address has to be asked for, once per device, with that device current.
int static_scratch_address(void **ptr_out) {
    static std::atomic<void *> resolved[64];
    int dev = -1;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    NPD_REQUIRE(dev >= 0 && dev < 64, NPD_ERR_UNSUPPORTED, "static scratch: device index %d out of range", dev);
    void *ptr = resolved[dev].load(std::memory_order_acquire);
    if (ptr == nullptr) {
        NPD_CUDA_TRY(cudaGetSymbolAddress(&ptr, g_decode_static_scratch));
        NPD_REQUIRE(ptr != nullptr, NPD_ERR_CUDA, "static scratch: cudaGetSymbolAddress returned NULL");
        resolved[dev].store(ptr, std::memory_order_release);
    }
    *ptr_out = ptr;
    return NPD_OK;
}

}  // namespace

extern "C" size_t npd_decode_static_scratch_bytes(void) { return NPD_STATIC_SCRATCH_BYTES; }

extern "C" int npd_paged_decode_attention_static(void *out, const void *q, const void *k_cache,
                                                 const void *v_cache, const int32_t *block_tables,
                                                 const int32_t *seq_lens, float scale, int64_t num_seqs,
                                                 int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim,
                                                 int64_t block_size, int64_t max_blocks_per_seq,
                                                 int64_t num_blocks, int64_t cache_block_stride,
                                                 int64_t bt_row_stride, int dtype, int32_t *status_out,
                                                 int flags, void *stream) {
    int dev = 0;
    NPD_CUDA_TRY(cudaGetDevice(&dev));
    const size_t need = npd_decode_workspace_bytes(num_seqs, num_q_heads, num_kv_heads, head_dim, dev);
    NPD_REQUIRE(need != 0, NPD_ERR_INVALID_ARG, "decode attention (static scratch): non-positive dimension");
    NPD_REQUIRE(need <= NPD_STATIC_SCRATCH_BYTES, NPD_ERR_WORKSPACE,
                "decode attention (static scratch): this shape needs %zu bytes of scratch, the built-in array "
                "holds %u; use npd_paged_decode_attention with a caller-owned workspace",
                need, (unsigned)NPD_STATIC_SCRATCH_BYTES);
    void *scratch = nullptr;
    const int rc_addr = static_scratch_address(&scratch);   // first call on a device: resolves the symbol
    if (rc_addr != NPD_OK) return rc_addr;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // The array keeps whatever the previous call left.  The status word must start at zero, and so must the
    // arrival tickets: the kernel leaves them at zero itself, except when an earlier launch gave up on a bounded
    // wait — and this caller has no pointer to clean up with.  The partial records are written before they are read.
    // Only the tickets one launch can touch are cleared: one per (sequence of a sub-batch, virtual kv head).
    const LaunchShape ls = launch_shape(static_cast<int>(head_dim), static_cast<int>(block_size), (flags >> 8) & 0xffff,
                                        (long long)num_seqs * num_kv_heads, dev);
    const WorkspacePlan wp = plan_workspace(num_seqs, num_q_heads, num_kv_heads, head_dim, ls);
    const int64_t vheads = num_kv_heads * wp.kv_rep;
    int64_t batch_cap = vheads > 0 ? kTicketCapacity / vheads : 0;
    if (batch_cap > kMaxSeqsPerLaunch) batch_cap = kMaxSeqsPerLaunch;
    const int64_t tickets = (num_seqs < batch_cap ? num_seqs : batch_cap) * vheads;
    NPD_CUDA_TRY(cudaMemsetAsync(scratch, 0, kStatusBytes + (size_t)tickets * sizeof(int32_t), st));
    const int rc = npd_paged_decode_attention(out, q, k_cache, v_cache, block_tables, seq_lens, scale, num_seqs,
                                              num_q_heads, num_kv_heads, head_dim, block_size, max_blocks_per_seq,
                                              num_blocks, cache_block_stride, bt_row_stride, dtype, scratch,
                                              NPD_STATIC_SCRATCH_BYTES, flags, st);
    if (rc != NPD_OK) return rc;
    if (status_out != nullptr)
        NPD_CUDA_TRY(cudaMemcpyAsync(status_out, scratch, sizeof(int32_t), cudaMemcpyDeviceToDevice, st));
    return NPD_OK;
}
