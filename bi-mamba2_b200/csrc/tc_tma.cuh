// TMA (cp.async.bulk.tensor) plumbing for the tcgen05 kernels: host-side tensor-map construction and the device-side
// load / expect-tx primitives.  Every load targets this CTA's own shared memory only (no cluster-wide variants).
// Tiles land in the same 128-byte-swizzled layouts the engine's thread-written stages use, so a TMA-loaded tile can be
// handed to tcgen05.mma directly:
//   * box [64 elements x R rows] of a row-major matrix, swizzle 128B  ->  K-major slab (row r at byte r*128)
//   * the same box read as [K rows x 64 MN elements]                  ->  one MN-major block of 64
#pragma once
#include <cuda.h>

#include "tc_engine.cuh"

namespace bissd {
namespace tc {

// ---- host -----------------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                  const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = [] {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

// Rank-4 map over a 16-bit tensor: dims[0] is the contiguous one; strides_bytes[i] is the stride of dims[i+1].
// Out-of-range parts of a box read as zero.  Returns false if the driver refuses the description.
inline bool make_map4(CUtensorMap *m, int dtype, const void *ptr, const unsigned long long (&dims)[4],
                      const unsigned long long (&strides_bytes)[3], const unsigned (&box)[4]) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t gd[4] = {dims[0], dims[1], dims[2], dims[3]};
    cuuint64_t gs[3] = {strides_bytes[0], strides_bytes[1], strides_bytes[2]};
    cuuint32_t bx[4] = {box[0], box[1], box[2], box[3]};
    cuuint32_t es[4] = {1, 1, 1, 1};
    const CUtensorMapDataType dt = dtype == BISSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return fn(m, dt, 4, const_cast<void *>(ptr), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}
inline bool make_map2(CUtensorMap *m, int dtype, const void *ptr, unsigned long long inner, unsigned long long rows,
                      unsigned box_inner, unsigned box_rows) {
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return false;
    cuuint64_t gd[2] = {inner, rows};
    cuuint64_t gs[1] = {inner * 2};
    cuuint32_t bx[2] = {box_inner, box_rows};
    cuuint32_t es[2] = {1, 1};
    const CUtensorMapDataType dt = dtype == BISSD_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
    return fn(m, dt, 2, const_cast<void *>(ptr), gd, gs, bx, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) ==
           CUDA_SUCCESS;
}

// ---- device ---------------------------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(m) : "memory");
}
// x = innermost coordinate (elements; x * 2 bytes must be a multiple of 16)
__device__ __forceinline__ void tma_load4(void *dst, const CUtensorMap *m, int x, int y, int z, int w, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y), "r"(z), "r"(w)
        : "memory");
}
__device__ __forceinline__ void tma_load2(void *dst, const CUtensorMap *m, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(dst)), "l"(m), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}
__device__ __forceinline__ float ex2_approx(float v) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

}  // namespace tc
}  // namespace bissd
