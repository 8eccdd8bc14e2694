// Tensor-map (TMA) helpers: host-side descriptor encoding and the device-side bulk tensor load.
//
// The activation tensors are (B, L, C) with arbitrary batch and row strides and a unit-stride
// channel dimension, which is exactly a 3-D tiled tensor map {C, L, B}.  A CTA fetches a
// (channels x timesteps) box of one batch row with a single instruction issued by one thread;
// the copy completes on a CTA-local mbarrier, needs no registers, and zero-fills whatever part
// of the box lies outside the tensor (ragged L and ragged channel tiles need no special code).
// Only plain (non-multicast) loads of this GPU's own memory are used.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace mb200 {

// cuTensorMapEncodeTiled is a driver entry point; it is looked up at run time so the library
// has no link-time dependency on libcuda (it must load on machines without a GPU).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*,
                                  const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn tma_encoder() {
  static EncodeTiledFn fn = [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess)
      p = nullptr;
    (void)cudaGetLastError();
    return reinterpret_cast<EncodeTiledFn>(p);
  }();
  return fn;
}

// True when `base` with the given element strides can be described by a tiled tensor map.
inline bool tma_compatible(const void* base, int64_t sb, int64_t sl, int64_t C, int elem_bytes,
                           int box_c) {
  if (!base || (reinterpret_cast<uintptr_t>(base) & 15)) return false;
  if ((sl * elem_bytes) % 16 || (sb * elem_bytes) % 16) return false;
  if ((box_c * elem_bytes) % 16) return false;
  return C > 0 && sl >= C;
}

// Encode {C, L, B} with strides (1, sl, sb) elements and box {box_c, box_l, 1}.
inline bool tma_encode(CUtensorMap* map, const void* base, bool bf16, int64_t B, int64_t L, int64_t C,
                       int64_t sb, int64_t sl, int box_c, int box_l) {
  EncodeTiledFn enc = tma_encoder();
  if (!enc) return false;
  const int es = bf16 ? 2 : 4;
  // a batch of 1 may come with any batch stride; give the unused dimension a legal one
  const int64_t sb_eff = (B > 1) ? sb : L * sl;
  cuuint64_t dims[3] = {cuuint64_t(C), cuuint64_t(L), cuuint64_t(B)};
  cuuint64_t strides[2] = {cuuint64_t(sl) * es, cuuint64_t(sb_eff) * es};
  cuuint32_t box[3] = {cuuint32_t(box_c), cuuint32_t(box_l), 1};
  cuuint32_t estr[3] = {1, 1, 1};
  return enc(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3,
             const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
             CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

#ifdef __CUDACC__
// Arm `bar` for `bytes` of incoming copy data (one arrival by the calling thread).
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.expect_tx.shared::cta.b64 st, [%0], %1;\n\t}" ::"r"(
                   static_cast<uint32_t>(__cvta_generic_to_shared(bar))),
               "r"(bytes)
               : "memory");
}
// Box at element coordinates (c, l, b) of the mapped tensor -> shared memory at dst.
__device__ __forceinline__ void tma_load_3d(void* dst, const CUtensorMap* map, int c, int l, int b,
                                            uint64_t* bar) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes "
      "[%0], [%1, {%2, %3, %4}], [%5];" ::"r"(static_cast<uint32_t>(__cvta_generic_to_shared(dst))),
      "l"(reinterpret_cast<uint64_t>(map)), "r"(c), "r"(l), "r"(b),
      "r"(static_cast<uint32_t>(__cvta_generic_to_shared(bar)))
      : "memory");
}
#endif

}  // namespace mb200
