// Small device and host helpers shared by the kernels that use the 5th-generation tensor cores:
// mbarrier waits with an iteration limit, shared-memory matrix descriptors, commit, and the
// driver entry point that encodes TMA tensor maps.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <mutex>
#include "common.h"

namespace tc {

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;\n" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;\n" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n.reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

// Bounded wait.  Returns false (after raising the CTA-wide abort flag and recording `code` in
// `error_word`) when the barrier did not complete within the limit or another role already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag,
                                          int *error_word, int code, uint32_t limit = 1u << 22) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *abort_flag) return false;
    }
    *abort_flag = 1;
    atomicCAS(error_word, 0, code);
    return false;
}

// Shared-memory matrix descriptor: start address, leading and stride byte offsets (all in
// 16-byte units), descriptor version 1, layout type (0 = no swizzle, 2 = 128-byte swizzle).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo, uint32_t layout) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)((lbo >> 4) & 0x3fffu) << 16) |
           ((uint64_t)((sbo >> 4) & 0x3fffu) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                        uint32_t accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate));
}
__device__ __forceinline__ void commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n"
                 ::"r"(bar) : "memory");
}

// 16 accumulator columns of this thread's tensor-memory lane; waits for the data.
__device__ __forceinline__ void ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];\n"
        "tcgen05.wait::ld.sync.aligned;\n"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

// cuTensorMapEncodeTiled through the runtime's driver entry point query (no link against libcuda).
inline int get_encode_fn(EncodeTiledFn *out) {
    static EncodeTiledFn cached = nullptr;
    static std::mutex m;
    std::lock_guard<std::mutex> lock(m);
    if (!cached) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        MORTAR_CUDA_CHECK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres));
        if (!fn || qres != cudaDriverEntryPointSuccess) {
            mortar_set_cuda_error("cudaGetDriverEntryPoint", "cuTensorMapEncodeTiled unavailable");
            return MORTAR_ERR_CUDA;
        }
        cached = reinterpret_cast<EncodeTiledFn>(fn);
    }
    *out = cached;
    return MORTAR_OK;
}

// [rows][cols] bf16 row-major with row stride ld (elements) as a 2-D map with a [box_rows][box_cols]
// box and the 128-byte swizzle (box_cols * 2 bytes must be 128).
inline int encode_bf16_2d(CUtensorMap *map, const void *base, int64_t cols, int64_t rows, int64_t ld,
                          uint32_t box_cols, uint32_t box_rows) {
    EncodeTiledFn encode;
    const int rc = get_encode_fn(&encode);
    if (rc != MORTAR_OK) return rc;
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstride[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {box_cols, box_rows};
    const cuuint32_t estride[2] = {1, 1};
    const CUresult cr = encode(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void *>(base), gdim, gstride, box,
                               estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS) {
        mortar_set_cuda_error("cuTensorMapEncodeTiled", "failed to encode a tensor map");
        return MORTAR_ERR_CUDA;
    }
    return MORTAR_OK;
}

}  // namespace tc
