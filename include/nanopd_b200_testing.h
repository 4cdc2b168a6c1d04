/*
 * nanopd_b200 — entry points for the library's own tests.  Not part of the stable ABI and of no
 * use to a caller: they exist so that error paths which never run in normal operation can be
 * exercised without faulting, trapping or hanging a GPU.
 */
#ifndef NANOPD_B200_TESTING_H
#define NANOPD_B200_TESTING_H

#include "nanopd_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

/* The bounded-wait path of the page-migration kernel (no counterpart in the reference, whose
 * copy_ loop has no waits of its own: nanoPD/workers/kv_transfer.py:73-79).
 * Same arguments and copy as npd_kv_migrate on its bulk path (max_ctas > 0 required), except that
 * the load of piece number `withhold_piece` (pieces are numbered unit-major: (pair, layer, K|V),
 * then 16 KiB pieces of a unit; -1 = none) is announced to its barrier but never issued, and a
 * wait for a load gives up after `wait_limit_clocks` SM clocks (at most 2e9, about a second).
 * The CTA that owns the piece therefore runs out of patience, ORs NPD_STATUS_WAIT_TIMEOUT into
 * `status`, waits (bounded) for its other loads in flight, and returns; pieces behind the
 * withheld one in that CTA's sequence stay uncopied, every other CTA finishes its share.  The
 * kernel always returns and the context stays usable.                                         */
int npd_testing_kv_migrate_withheld(const void *src_k, const void *src_v, void *dst_k, void *dst_v,
                                    const int32_t *src_blocks, const int32_t *dst_blocks, int64_t num_pairs,
                                    int64_t num_layers, int64_t block_elems, int elem_bytes,
                                    int64_t src_layer_stride, int64_t src_block_stride, int64_t src_num_blocks,
                                    int64_t dst_layer_stride, int64_t dst_block_stride, int64_t dst_num_blocks,
                                    int max_ctas, int32_t *status, void *stream, int64_t withhold_piece,
                                    int64_t wait_limit_clocks);

#ifdef __cplusplus
}
#endif
#endif /* NANOPD_B200_TESTING_H */
