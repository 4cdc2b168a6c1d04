// Kernel 3 placeholder so the library exports every declared symbol while the kernel is built.
#include "npd_common.cuh"

extern "C" size_t npd_prefill_workspace_bytes(int64_t, int64_t, int64_t, int64_t, int) { return 256; }

extern "C" int npd_paged_prefill_attention(void *, const void *, const void *, const void *, const int32_t *,
                                           const int32_t *, const int32_t *, const int32_t *, int64_t, float,
                                           int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t, int64_t,
                                           int, void *, size_t, int, void *) {
    return npd::fail(NPD_ERR_UNSUPPORTED, "npd_paged_prefill_attention: not built yet");
}
