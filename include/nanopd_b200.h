/*
 * nanopd_b200 — C ABI of the paged-attention hot path for NVIDIA B200 (sm_100a).
 *
 * Every entry point takes plain device pointers, 64-bit sizes/strides counted in
 * ELEMENTS, a dtype code and a CUDA stream handle (cudaStream_t passed as void*;
 * NULL = the legacy default stream).  Calls are asynchronous on that stream, never
 * synchronise the device, allocate nothing, and return NPD_OK or an NPD_ERR_* code;
 * npd_last_error() then gives a message for the calling thread.  Nothing here
 * terminates the process (the reference's CHECK_KERNEL does:
 * nanoPD/paged_attention/csrc/utils/cuda_utils.h:18-29).
 *
 * The Python module `paged_kernels` shipped with this library binds these symbols
 * with ctypes and exposes the reference's op signatures on top of them.
 */
#ifndef NANOPD_B200_H
#define NANOPD_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- codes ------------------------------------------------------------------ */
#define NPD_OK               0
#define NPD_ERR_INVALID_ARG  1   /* shape / alignment / NULL pointer                      */
#define NPD_ERR_UNSUPPORTED  2   /* dtype, head_dim, block_size or group outside the set  */
#define NPD_ERR_CUDA         3   /* a CUDA runtime / driver call failed                   */
#define NPD_ERR_WORKSPACE    4   /* workspace missing or smaller than *_workspace_bytes   */

#define NPD_DTYPE_F16   0
#define NPD_DTYPE_BF16  1
#define NPD_DTYPE_F32   2   /* accepted by npd_kv_store only (the payload is opaque there) */

/* Bits of the device-side status word (first int32 of a decode/prefill workspace, or
 * the `status` argument of npd_kv_store / npd_kv_migrate).  Kernels OR bits in; they
 * never fault or spin without bound.  Read and clear it with npd_read_status().      */
#define NPD_STATUS_BAD_BLOCK_ID   1   /* a block-table entry outside [0, num_blocks); the access was skipped */
#define NPD_STATUS_BAD_POSITION   2   /* a position / seq_len beyond the table's capacity; clamped or skipped */
#define NPD_STATUS_WAIT_TIMEOUT   4   /* a bounded wait on an in-kernel barrier ran out                       */

/* Flags of npd_paged_decode_attention and npd_paged_prefill_attention.  Both kernels are persistent, one CTA per
 * SM; NPD_FLAG_MAX_CTAS(n) caps the grid at n CTAs (0 = no cap) so that two of them — a prompt chunk and the
 * decode batch of the same scheduler step — can run side by side on two streams, each on its share of the SMs. */
#define NPD_FLAG_MAX_CTAS(n)      (((n) & 0xffff) << 8)

#define NPD_DECODE_KV_INTERLEAVED 2   /* caches in the layouts of the reference's split-K op and of its kernel tests
                                       * (csrc/paged_attention_optimized/index.h:14-31,60-75; tests/test_paged_kernels.py:39-56):
                                       * K [num_blocks, num_kv_heads, head_dim/8, block_size, 8],
                                       * V [num_blocks, num_kv_heads, head_dim, block_size]                           */

int         npd_version(void);
const char *npd_last_error(void);

/* Copies the int32 status word at `status_dev` to the host, clears it on the device,
 * and waits for `stream`.  Returns the word in *out.                                  */
int npd_read_status(int32_t *status_dev, int32_t *out, void *stream);

/* ---- (1) paged KV store ---------------------------------------------------------
 * Replaces paged_kv_store (nanoPD/paged_attention/csrc/kvstore/paged_kv_store.h:23-27,
 * paged_kv_store_ops.cu:7-50, paged_kv_store_kernel.cu:16-58).
 * For token t and kv head h:
 *   cache[block_tables[t*bt_row_stride + positions[t]/block_size], h, positions[t]%block_size, :]
 *       = src[h, t, :]                        for K and for V.
 * k_cache/v_cache: [num_blocks, num_kv_heads, block_size, head_dim], the last three
 * dims contiguous, blocks `cache_block_stride` elements apart.
 * k_src/v_src: element (h, t, d) at h*src_head_stride + t*src_token_stride + d.
 * block_tables: int32, one row per token (bt_row_stride may be 0 for a shared row).
 * head_dim*elem must be a multiple of 16 bytes; all base pointers 16-byte aligned.
 * `status` (device int32, may be NULL) receives NPD_STATUS_* bits.                     */
int npd_kv_store(void *k_cache, void *v_cache, const void *k_src, const void *v_src,
                 const int32_t *block_tables, const int32_t *positions,
                 int64_t num_tokens, int64_t num_kv_heads, int64_t head_dim,
                 int64_t block_size, int64_t num_blocks, int64_t max_blocks_per_seq,
                 int64_t cache_block_stride, int64_t src_head_stride,
                 int64_t src_token_stride, int64_t bt_row_stride,
                 int dtype, int32_t *status, void *stream);

/* ---- (2) paged decode attention -------------------------------------------------
 * Replaces paged_attention_forward (nanoPD/paged_attention/csrc/attention/paged_attention.h:24-34,
 * paged_attention_ops.cu:7-59, paged_attention_kernel.cu:39-151) and the split-K pair
 * (csrc/paged_attention_optimized/paged_attention_optimized_ops.cu:20-112).
 *   out[s, h, :] = softmax(scale * q[s, h, :] . K_s^T) . V_s
 * over the first seq_lens[s] tokens of the pages block_tables[s, :]; the kv head of
 * q head h is h / (num_q_heads / num_kv_heads).  out, q: [num_seqs, num_q_heads,
 * head_dim] contiguous.  Caches as in npd_kv_store.  fp32 accumulation throughout.
 * Supported: dtype f16/bf16, head_dim in {64,128,256}, block_size in {4,8,16,32} (8 and up with
 * NPD_DECODE_KV_INTERLEAVED),
 * num_q_heads/num_kv_heads <= 32.  A sequence with seq_lens[s] == 0 gets a zero row.
 * `workspace` is caller-owned device memory of at least
 * npd_decode_workspace_bytes(...) bytes, 256-byte aligned, ZEROED ONCE before first
 * use and then only touched by this library; its first int32 is the status word.
 * Two calls that may overlap on the GPU need two workspaces.  After a call that reported
 * NPD_STATUS_WAIT_TIMEOUT zero the workspace again before reusing it.                  */
size_t npd_decode_workspace_bytes(int64_t num_seqs, int64_t num_q_heads,
                                  int64_t num_kv_heads, int64_t head_dim, int device);
int npd_paged_decode_attention(void *out, const void *q, const void *k_cache,
                               const void *v_cache, const int32_t *block_tables,
                               const int32_t *seq_lens, float scale,
                               int64_t num_seqs, int64_t num_q_heads, int64_t num_kv_heads,
                               int64_t head_dim, int64_t block_size,
                               int64_t max_blocks_per_seq, int64_t num_blocks,
                               int64_t cache_block_stride, int64_t bt_row_stride,
                               int dtype, void *workspace, size_t workspace_bytes,
                               int flags, void *stream);

/* ---- (2b) decode attention without a caller workspace ----------------------------
 * No counterpart in the reference.  Same arithmetic and arguments as
 * npd_paged_decode_attention, for hosts that cannot allocate device memory when they call:
 * a worker whose HBM went entirely to the KV pool and weights at start-up, a step loop
 * that forbids allocation after initialisation, a foreign runtime binding this ABI with no
 * device allocator (cudaMalloc/cudaFree would also stall the whole device).  The scratch is a
 * 32 MiB device array inside the library image (npd_decode_static_scratch_bytes()); every
 * GPU that loads the library holds it until the process exits.  The call allocates and
 * frees nothing.  Shapes whose scratch need (npd_decode_workspace_bytes) exceeds the array
 * are refused with NPD_ERR_WORKSPACE; on a B200 every supported shape fits.
 * The FIRST call on each device looks up the array's device address (one
 * cudaGetSymbolAddress, with that device current) — make that call before any stream
 * capture begins.  All calls on a device share the one array, which keeps the previous
 * call's contents; the status word and the arrival tickets are cleared at the start of each
 * call, the rest is written before it is read.  Two calls that can overlap on the GPU (different streams)
 * race on it: serialise them, or give the concurrent ones the workspace variant.
 * `status_out` (device int32, may be NULL) receives this call's NPD_STATUS_* bits.         */
size_t npd_decode_static_scratch_bytes(void);
int npd_paged_decode_attention_static(void *out, const void *q, const void *k_cache,
                                      const void *v_cache, const int32_t *block_tables,
                                      const int32_t *seq_lens, float scale,
                                      int64_t num_seqs, int64_t num_q_heads, int64_t num_kv_heads,
                                      int64_t head_dim, int64_t block_size,
                                      int64_t max_blocks_per_seq, int64_t num_blocks,
                                      int64_t cache_block_stride, int64_t bt_row_stride,
                                      int dtype, int32_t *status_out, int flags, void *stream);

/* ---- (3) chunked-prefill causal attention over paged K/V ------------------------
 * Replaces the prefill branch of ModelRunner.paged_forward
 * (nanoPD/engine/model_runner.py:152-169: dense -inf mask + repeat_interleave +
 * scaled_dot_product_attention) and, unlike it, reads earlier chunks from the pages.
 * For chunk c (c < num_chunks) with n = chunk_tokens[c] queries starting at row
 * chunk_q_offset[c] of q/out and absolute position chunk_start[c]:
 *   query i attends to keys 0 .. chunk_start[c] + i of the pages
 *   block_tables[c*bt_row_stride + ...]; the chunk's own K/V must already be stored.
 * q, out: [total_q_tokens, num_q_heads, head_dim] contiguous.  The three chunk arrays
 * are HOST int32 arrays (the scheduler knows them; nanoPD/engine/engine.py:68-90).
 * Supported: f16/bf16, head_dim 64/128/256, block_size 4/8/16/32; out 32-byte aligned.
 * `workspace`: device memory of at least npd_prefill_workspace_bytes(...) bytes, ZEROED
 * ONCE before first use (status word, then two counters every launch leaves at zero);
 * two calls that may overlap on the GPU need two workspaces.                              */
size_t npd_prefill_workspace_bytes(int64_t total_q_tokens, int64_t num_q_heads,
                                   int64_t num_kv_heads, int64_t head_dim, int device);
int npd_paged_prefill_attention(void *out, const void *q, const void *k_cache,
                                const void *v_cache, const int32_t *block_tables,
                                const int32_t *chunk_q_offset_host,
                                const int32_t *chunk_tokens_host,
                                const int32_t *chunk_start_host,
                                int64_t num_chunks, float scale,
                                int64_t num_q_heads, int64_t num_kv_heads, int64_t head_dim,
                                int64_t block_size, int64_t max_blocks_per_seq,
                                int64_t num_blocks, int64_t cache_block_stride,
                                int64_t bt_row_stride, int dtype,
                                void *workspace, size_t workspace_bytes,
                                int flags, void *stream);

/* ---- (4) KV page migration ------------------------------------------------------
 * Replaces transfer_kv's per-block copy_ loop (nanoPD/workers/kv_transfer.py:69-83):
 *   for i < num_pairs, for every layer l:
 *     dst_k[l, dst_blocks[i]] = src_k[l, src_blocks[i]]     (and the same for V)
 * Pools are [num_layers, num_blocks, block_elems] with `*_layer_stride` and
 * `*_block_stride` in elements; block_elems*elem_bytes must be a multiple of 16.
 * src_blocks/dst_blocks are DEVICE int32 arrays resident on the device the kernel runs
 * on (the current device).  Either pool may live on a peer GPU whose memory is mapped
 * into the current device (peer access enabled, or an IPC mapping); the copy is done by
 * the kernel itself (bulk asynchronous copies through shared memory, no multicast), so no
 * copy engine or NCCL call is involved.
 * `max_ctas` > 0 sets the grid (one warp and 64 KiB of shared memory per CTA, small enough to
 * share an SM with a decode-attention CTA of the compute stream; 0 = 64 CTAs, which fill an
 * NVLink); `max_ctas` < 0 selects the plain load/store variant with -max_ctas CTAs of 256 threads. */
int npd_kv_migrate(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                   const int32_t *src_blocks, const int32_t *dst_blocks, int64_t num_pairs,
                   int64_t num_layers, int64_t block_elems, int elem_bytes,
                   int64_t src_layer_stride, int64_t src_block_stride, int64_t src_num_blocks,
                   int64_t dst_layer_stride, int64_t dst_block_stride, int64_t dst_num_blocks,
                   int max_ctas, int32_t *status, void *stream);

/* ---- (5) fused QK-norm + rotary embedding + KV store ------------------------------
 * Replaces the chain of element-wise passes the caller runs between the projections and
 * the store (nanoPD/engine/model_runner.py:97-115: q_norm, k_norm, transposes, rotary
 * embedding of Q and K) together with paged_kv_store (model_runner.py:142-149, 188-194).
 * For token t: q_out[t, h, :] = rope(norm(q[t, h, :])), the K page slot of the token gets
 * rope(norm(k[t, h, :])) and the V page slot v[t, h, :]; slots as in npd_kv_store.
 *   norm(x) = w * T(float(x) * rsqrt(mean(float(x)^2) + eps))      (skipped when w is NULL)
 *   rope(y) = T(y * cos[t]) + T(rotate_half(y) * sin[t]),  rotate_half(y) = (-y[D/2:], y[:D/2])
 * with T(.) the rounding to the 16-bit dtype the Hugging Face modules apply at each step
 * (Qwen3RMSNorm and apply_rotary_pos_emb of transformers, which the reference calls).
 * q, k, v are token-major: element (t, h, d) at t*token_stride + h*head_dim + d, so views
 * into one fused projection output are accepted; q_out may alias q.  cos/sin: [T, head_dim]
 * rows `cos_sin_row_stride` elements apart (0 broadcasts one row).  head_dim in {64,128,256},
 * dtype f16/bf16; strides multiples of 8 elements, pointers 16-byte aligned.              */
int npd_qk_norm_rope_store(void *q_out, const void *q, const void *k, const void *v,
                           const void *q_norm_weight, const void *k_norm_weight,
                           const void *cos, const void *sin, float eps,
                           void *k_cache, void *v_cache, const int32_t *block_tables,
                           const int32_t *positions, int64_t num_tokens, int64_t num_q_heads,
                           int64_t num_kv_heads, int64_t head_dim, int64_t block_size,
                           int64_t num_blocks, int64_t max_blocks_per_seq, int64_t cache_block_stride,
                           int64_t q_token_stride, int64_t k_token_stride, int64_t v_token_stride,
                           int64_t q_out_token_stride, int64_t cos_sin_row_stride,
                           int64_t bt_row_stride, int dtype, int32_t *status, void *stream);

/* ---- (6) batched top-k sampling -------------------------------------------------------
 * Replaces top_k_sample (nanoPD/engine/model_runner.py:279-284), which the reference calls
 * once per sequence and reads back with .item() (nanoPD/engine/engine.py:100-106,
 * nanoPD/workers/decode_worker.py:110, nanoPD/workers/prefill_worker.py:79).  One launch
 * serves all `num_rows` rows of `logits` ([num_rows, vocab], rows `row_stride` elements
 * apart, f16 / bf16 / f32) and writes one token id per row to `out_ids` (device int64):
 *   x = nan_to_num(row, nan = 0, posinf = 1e4, neginf = -1e4)          (in the logits' dtype)
 *   the top_k largest x, larger first, equal values by the lower id first
 *   p = softmax over those values, computed in fp32 and rounded to the logits' dtype
 *   the draw: the first candidate whose running fp32 sum of p exceeds uniforms[row] * sum(p)
 * `uniforms` (device float32 [num_rows], values in [0, 1)) supplies the randomness, so a
 * caller's generator decides the stream; it may be NULL when top_k == 1 (the arg-max,
 * the reference's default).  top_k in [1, NPD_SAMPLE_MAX_TOP_K], top_k <= vocab <= 2^30;
 * rows must start on 16-byte boundaries.
 * `workspace`: device memory of at least npd_top_k_sample_workspace_bytes(...), zeroed once
 * by the caller and then reusable by any later call on the same stream (the kernel leaves
 * its arrival counters at zero).  Its first int32 collects NPD_STATUS_* bits: the only one
 * this kernel raises is NPD_STATUS_WAIT_TIMEOUT (a bounded wait for a bulk copy ran out;
 * the tokens of that launch are then undefined — zero the workspace before reusing it).   */
#define NPD_SAMPLE_MAX_TOP_K 64
int64_t npd_top_k_sample_workspace_bytes(int64_t num_rows, int64_t vocab, int top_k);
int npd_top_k_sample(int64_t *out_ids, const void *logits, const float *uniforms, int64_t num_rows,
                     int64_t vocab, int64_t row_stride, int top_k, int dtype, void *workspace,
                     int64_t workspace_bytes, void *stream);

/* Enables peer access from the current device to `peer_device` (idempotent).
 * Stands in for the driver-side mapping torch's copy_ sets up in the reference
 * (nanoPD/workers/kv_transfer.py:6-14 only probes can_device_access_peer).              */
int npd_enable_peer_access(int peer_device);

#ifdef __cplusplus
}
#endif
#endif /* NANOPD_B200_H */
