// Shared host/device helpers for the nanopd_b200 kernels (sm_100a only).
#pragma once

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <string>

#include "../../include/nanopd_b200.h"

// Internal diagnostic flag of the decode launcher (bit 0 of `flags`): sequences split across workers stay
// unmerged, which leaves wrong rows for those.  Not part of the public ABI.
#define NPD_DECODE_SKIP_MERGE 1
// Bit 2: always take the streaming form, also where the small-batch form would be chosen (for tests of the former).
#define NPD_DECODE_NO_SMALL 4

// ---------------------------------------------------------------------------
// Host-side error plumbing: every entry point returns a code and leaves a message.
// ---------------------------------------------------------------------------
namespace npd {

std::string &last_error_ref();

inline int fail(int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof(buf), fmt, ap);
    va_end(ap);
    last_error_ref() = buf;
    return code;
}

#define NPD_CUDA_TRY(expr)                                                              \
    do {                                                                                \
        cudaError_t _e = (expr);                                                        \
        if (_e != cudaSuccess)                                                          \
            return ::npd::fail(NPD_ERR_CUDA, "%s failed: %s (%s:%d)", #expr,            \
                               cudaGetErrorString(_e), __FILE__, __LINE__);             \
    } while (0)

#define NPD_REQUIRE(cond, code, ...)                                                    \
    do {                                                                                \
        if (!(cond)) return ::npd::fail(code, __VA_ARGS__);                             \
    } while (0)

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per device id, read-only after first use).
int sm_count(int device);

// Encodes a rank-3 tiled tensor map over a paged cache [num_blocks, Hkv*B rows, D] of
// 2-byte elements with 128-byte swizzle; box = 64 elements x box_rows rows x 1 block.
// Resolved through cudaGetDriverEntryPoint so the library has no link-time dependency
// on libcuda and loads on machines without a driver.
// General rank-3 tiled map of 2-byte elements; with the 128-byte swizzle (box[0] must be 64) or without.
int encode_tiled_3d(CUtensorMap *map, const void *base, int dtype, const uint64_t dims[3],
                    const uint64_t strides_bytes[2], const uint32_t box[3], bool swizzle128 = true);
int encode_cache_tensor_map(CUtensorMap *map, const void *base, int dtype, int64_t head_dim,
                            int64_t rows_per_block, int64_t num_blocks,
                            int64_t block_stride_elems, int box_rows);

}  // namespace npd

// ---------------------------------------------------------------------------
// Device-side PTX wrappers
// ---------------------------------------------------------------------------
#if defined(__CUDACC__)

namespace npd {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier ---------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Non-blocking test of a phase (try_wait may suspend the thread for a while before it answers "not yet").
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after ~`limit_cycles` SM clocks and returns false, so a lost
// completion can never hang the GPU.  Two seconds at 2 GHz by default.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity,
                                                  long long limit_cycles = 4000000000LL) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    while (!mbar_try_wait(bar, parity)) {
        if (clock64() - t0 > limit_cycles) return false;
    }
    return true;
}

// Orders earlier generic-proxy accesses to shared memory before later async-proxy
// (TMA) accesses issued by this thread.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- TMA: rank-3 tiled load, global -> shared, completion on an mbarrier ----
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap *map, uint32_t bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
        "[%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(bar), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *map) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

// ---- warp-level matrix ops ----------------------------------------------------
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(addr));
}
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
    uint32_t d;
    asm("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
    return d;
}

template <typename T> struct Elem;
template <> struct Elem<__half> {
    static constexpr int kDtype = NPD_DTYPE_F16;
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
        __half2 h = __floats2half2_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __device__ static __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4],
                                                    uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};
template <> struct Elem<__nv_bfloat16> {
    static constexpr int kDtype = NPD_DTYPE_BF16;
    __device__ static __forceinline__ uint32_t pack2(float lo, float hi) {
        __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
        return *reinterpret_cast<uint32_t *>(&h);
    }
    __device__ static __forceinline__ void mma16816(float (&d)[4], const uint32_t (&a)[4],
                                                    uint32_t b0, uint32_t b1) {
        asm("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 "
            "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
            : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
            : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
};

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

}  // namespace npd
#endif  // __CUDACC__
