// RMSNorm over the last dimension, forward and backward:
//     y = x * rsqrt(mean(x^2) + eps) * weight          (mambapy/mamba.py:416-433; weight absent with muP)
// This is the normalisation in front of every MambaBlock (ResidualBlock.forward, mambapy/mamba.py:111)
// and the optional inner normalisation of delta, B, C.  The reference builds it from five elementwise
// and reduction ops; here a row is read once and written once (HBM streaming).
//
// Mapping: one warp per row, rows taken with a grid stride.  The row is read twice, the second time out
// of L1/L2 (a row is a few KB), so nothing about D limits the register count.  All arithmetic is
// float32 whatever the I/O type.  The backward needs sum_d g*xhat per row (warp shuffle) and
// dweight[d] = sum_rows dy*xhat, which the CTA accumulates in shared memory (one shared-memory
// reduction per element, conflict-free inside a warp) before one atomic per column and CTA adds to
// global memory.
#include <initializer_list>
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;

template <typename T, int V> struct alignas(sizeof(T) * V) NVec {
  T v[V];
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int s = 16; s >= 1; s >>= 1) v += __shfl_xor_sync(0xffffffffu, v, s);
  return v;
}

template <typename T, int V>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, T* __restrict__ y,
                   float* __restrict__ rstd, int64_t rows, int64_t D, int64_t x_rs, int64_t y_rs, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = int64_t(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
  const int64_t nwarps = int64_t(gridDim.x) * kNormWarps;
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* xp = x + r * x_rs;
    T* yp = y + r * y_rs;
    float ss = 0.f;
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      const NVec<T, V> v = *reinterpret_cast<const NVec<T, V>*>(xp + d);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float f = Elem<T>::to_f(v.v[i]);
        ss = fmaf(f, f, ss);
      }
    }
    const float rs = rsqrtf(warp_sum(ss) / float(D) + eps);
    if (rstd && lane == 0) rstd[r] = rs;
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      const NVec<T, V> v = *reinterpret_cast<const NVec<T, V>*>(xp + d);
      NVec<T, V> o;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        float f = Elem<T>::to_f(v.v[i]) * rs;
        if (w) f *= w[d + i];
        o.v[i] = Elem<T>::from_f(f);
      }
      *reinterpret_cast<NVec<T, V>*>(yp + d) = o;
    }
  }
}

// dx = (g - xhat * mean(g * xhat)) * rstd with g = dy * weight, xhat = x * rstd;  dweight = sum_rows dy * xhat.
template <typename T, int V, bool kAccW>
__global__ void __launch_bounds__(kNormThreads)
rmsnorm_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ rstd,
                   const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ dw, int64_t rows, int64_t D,
                   int64_t x_rs, int64_t dy_rs, int64_t dx_rs) {
  extern __shared__ float s_dw[];               // [D] when kAccW
  const int lane = threadIdx.x & 31;
  const int64_t warp = int64_t(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
  const int64_t nwarps = int64_t(gridDim.x) * kNormWarps;
  if constexpr (kAccW) {
    for (int64_t d = threadIdx.x; d < D; d += kNormThreads) s_dw[d] = 0.f;
    __syncthreads();
  }
  for (int64_t r = warp; r < rows; r += nwarps) {
    const T* xp = x + r * x_rs;
    const T* gp = dy + r * dy_rs;
    T* op = dx + r * dx_rs;
    const float rs = rstd[r];
    float dot = 0.f;
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      const NVec<T, V> xv = *reinterpret_cast<const NVec<T, V>*>(xp + d);
      const NVec<T, V> gv = *reinterpret_cast<const NVec<T, V>*>(gp + d);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float xh = Elem<T>::to_f(xv.v[i]) * rs;
        const float gy = Elem<T>::to_f(gv.v[i]);
        if constexpr (kAccW) atomicAdd(&s_dw[d + i], gy * xh);
        dot = fmaf(w ? gy * w[d + i] : gy, xh, dot);
      }
    }
    const float m = warp_sum(dot) / float(D);
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      const NVec<T, V> xv = *reinterpret_cast<const NVec<T, V>*>(xp + d);
      const NVec<T, V> gv = *reinterpret_cast<const NVec<T, V>*>(gp + d);
      NVec<T, V> o;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float xh = Elem<T>::to_f(xv.v[i]) * rs;
        float g = Elem<T>::to_f(gv.v[i]);
        if (w) g *= w[d + i];
        o.v[i] = Elem<T>::from_f((g - xh * m) * rs);
      }
      *reinterpret_cast<NVec<T, V>*>(op + d) = o;
    }
  }
  if constexpr (kAccW) {
    __syncthreads();
    for (int64_t d = threadIdx.x; d < D; d += kNormThreads) atomicAdd(dw + d, s_dw[d]);
  }
}

int norm_grid(int64_t rows) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (rows + kNormWarps - 1) / kNormWarps;
  const int64_t cap = int64_t(sms) * 8;                    // 8 CTAs of 256 threads per SM
  return int(want < cap ? (want > 0 ? want : 1) : cap);
}

}  // namespace
}  // namespace mb200

using namespace mb200;

static int norm_vec(int64_t D, int es, std::initializer_list<const void*> ptrs, std::initializer_list<int64_t> strides) {
  const int v = 16 / es;
  if (D % v) return 1;
  for (const void* p : ptrs) if (!aligned16(p)) return 1;
  for (int64_t s : strides) if (s % v) return 1;
  return v;
}

extern "C" int mb200_rmsnorm_fwd(const void* x, const float* weight, void* y, float* rstd, int64_t rows,
                                 int64_t D, int64_t x_rs, int64_t y_rs, float eps, int dtype, void* stream) {
  if (rows < 0 || D < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (rows == 0 || D == 0) return MB200_OK;
  if (!x || !y) return MB200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = dtype == MB200_F32 ? 4 : 2;
  const int v = norm_vec(D, es, {x, y}, {x_rs, y_rs});
  const int grid = norm_grid(rows);
#define MB200_NORM_FWD(TT, VV) \
  rmsnorm_fwd_kernel<TT, VV><<<grid, kNormThreads, 0, st>>>((const TT*)x, weight, (TT*)y, rstd, rows, D, x_rs, y_rs, eps)
  if (dtype == MB200_F32) { if (v > 1) MB200_NORM_FWD(float, 4); else MB200_NORM_FWD(float, 1); }
  else { if (v > 1) MB200_NORM_FWD(__nv_bfloat16, 8); else MB200_NORM_FWD(__nv_bfloat16, 1); }
#undef MB200_NORM_FWD
  return check_launch();
}

extern "C" int mb200_rmsnorm_bwd(const void* x, const float* weight, const float* rstd, const void* dy, void* dx,
                                 float* dweight, int64_t rows, int64_t D, int64_t x_rs, int64_t dy_rs,
                                 int64_t dx_rs, int dtype, void* stream) {
  if (rows < 0 || D < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (rows == 0 || D == 0) return MB200_OK;
  if (!x || !rstd || !dy || !dx) return MB200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = dtype == MB200_F32 ? 4 : 2;
  const int v = norm_vec(D, es, {x, dy, (const void*)dx}, {x_rs, dy_rs, dx_rs});
  if (dweight && D > 12288) return MB200_ETOOBIG;                    // the CTA's dweight buffer is D floats of static-limit shared memory
  const int grid = norm_grid(rows);
  const size_t smem = dweight ? size_t(D) * sizeof(float) : 0;
#define MB200_NORM_BWD(TT, VV)                                                                             \
  {                                                                                                        \
    if (dweight)                                                                                           \
      rmsnorm_bwd_kernel<TT, VV, true><<<grid, kNormThreads, smem, st>>>((const TT*)x, weight, rstd,      \
          (const TT*)dy, (TT*)dx, dweight, rows, D, x_rs, dy_rs, dx_rs);                                   \
    else                                                                                                   \
      rmsnorm_bwd_kernel<TT, VV, false><<<grid, kNormThreads, 0, st>>>((const TT*)x, weight, rstd,        \
          (const TT*)dy, (TT*)dx, dweight, rows, D, x_rs, dy_rs, dx_rs);                                   \
  }
  if (dtype == MB200_F32) { if (v > 1) MB200_NORM_BWD(float, 4) else MB200_NORM_BWD(float, 1) }
  else { if (v > 1) MB200_NORM_BWD(__nv_bfloat16, 8) else MB200_NORM_BWD(__nv_bfloat16, 1) }
#undef MB200_NORM_BWD
  return check_launch();
}
