// Host-side helpers shared by every entry point: error text, device queries, the
// tensor-map encoder, the status-word reader and peer-access set-up.
#include <cudaTypedefs.h>

#include <atomic>

#include "npd_common.cuh"

namespace npd {

std::string &last_error_ref() {
    thread_local std::string msg;
    return msg;
}

int sm_count(int device) {
    // Small fixed table, written once per device; a benign race writes the same value.
    static std::atomic<int> cache[64];
    if (device >= 0 && device < 64) {
        int v = cache[device].load(std::memory_order_relaxed);
        if (v > 0) return v;
    }
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) {
        (void)cudaGetLastError();
        n = 148;  // B200; only reached when no device answers (size queries on a CPU-only host)
    }
    if (device >= 0 && device < 64) cache[device].store(n, std::memory_order_relaxed);
    return n;
}

using EncodeTiledFn = CUresult (*)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                   const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                   const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                   CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn resolve_encode_tiled() {
    static std::atomic<void *> cached{nullptr};
    void *fn = cached.load(std::memory_order_acquire);
    if (fn) return reinterpret_cast<EncodeTiledFn>(fn);
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fn == nullptr) {
        (void)cudaGetLastError();
        return nullptr;
    }
    cached.store(fn, std::memory_order_release);
    return reinterpret_cast<EncodeTiledFn>(fn);
}

int encode_tiled_3d(CUtensorMap *map, const void *base, int dtype, const uint64_t dims[3],
                    const uint64_t strides_bytes[2], const uint32_t box[3], bool swizzle128) {
    EncodeTiledFn encode = resolve_encode_tiled();
    NPD_REQUIRE(encode != nullptr, NPD_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    NPD_REQUIRE(aligned16(base), NPD_ERR_INVALID_ARG, "tensor base pointer must be 16-byte aligned");
    NPD_REQUIRE(strides_bytes[0] % 16 == 0 && strides_bytes[1] % 16 == 0, NPD_ERR_INVALID_ARG,
                "tensor strides must be multiples of 16 bytes");
    const cuuint64_t gdims[3] = {dims[0], dims[1], dims[2]};
    const cuuint64_t gstrides[2] = {strides_bytes[0], strides_bytes[1]};
    const cuuint32_t gbox[3] = {box[0], box[1], box[2]};
    const cuuint32_t estr[3] = {1u, 1u, 1u};
    const CUtensorMapDataType dt =
        dtype == NPD_DTYPE_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    CUresult r = encode(map, dt, 3, const_cast<void *>(base), gdims, gstrides, gbox, estr,
                        CU_TENSOR_MAP_INTERLEAVE_NONE,
                        swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    NPD_REQUIRE(r == CUDA_SUCCESS, NPD_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return NPD_OK;
}

int encode_cache_tensor_map(CUtensorMap *map, const void *base, int dtype, int64_t head_dim,
                            int64_t rows_per_block, int64_t num_blocks,
                            int64_t block_stride_elems, int box_rows) {
    const uint64_t dims[3] = {static_cast<uint64_t>(head_dim), static_cast<uint64_t>(rows_per_block),
                              static_cast<uint64_t>(num_blocks)};
    const uint64_t strides[2] = {static_cast<uint64_t>(head_dim) * 2u,
                                 static_cast<uint64_t>(block_stride_elems) * 2u};
    const uint32_t box[3] = {64u, static_cast<uint32_t>(box_rows), 1u};
    return encode_tiled_3d(map, base, dtype, dims, strides, box);
}

}  // namespace npd

extern "C" {

int npd_version(void) { return 100; }

const char *npd_last_error(void) { return npd::last_error_ref().c_str(); }

int npd_read_status(int32_t *status_dev, int32_t *out, void *stream) {
    NPD_REQUIRE(status_dev != nullptr && out != nullptr, NPD_ERR_INVALID_ARG, "npd_read_status: NULL pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    NPD_CUDA_TRY(cudaMemcpyAsync(out, status_dev, sizeof(int32_t), cudaMemcpyDeviceToHost, st));
    NPD_CUDA_TRY(cudaMemsetAsync(status_dev, 0, sizeof(int32_t), st));
    NPD_CUDA_TRY(cudaStreamSynchronize(st));
    return NPD_OK;
}

int npd_enable_peer_access(int peer_device) {
    int cur = -1;
    NPD_CUDA_TRY(cudaGetDevice(&cur));
    if (cur == peer_device) return NPD_OK;
    int can = 0;
    NPD_CUDA_TRY(cudaDeviceCanAccessPeer(&can, cur, peer_device));
    NPD_REQUIRE(can != 0, NPD_ERR_UNSUPPORTED, "device %d cannot access peer device %d", cur, peer_device);
    cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e == cudaErrorPeerAccessAlreadyEnabled) {
        (void)cudaGetLastError();
        return NPD_OK;
    }
    NPD_CUDA_TRY(e);
    return NPD_OK;
}

}  // extern "C"
