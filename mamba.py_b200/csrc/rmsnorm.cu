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

// ---- residual add fused with the normalisation that follows it -----------------------------------------
// A stack of blocks computes x_{l+1} = mixer(norm(x_l)) + x_l (mambapy/mamba.py:106-112).  Written per
// layer that is an add kernel (read two tensors, write one) followed by the norm (read one, write one);
// fused, the sum is formed in registers:   s = x + res_in;  res_out = s;  y = s * rsqrt(mean(s^2) + eps) * w.
// x (the previous mixer's output), the residual stream and y may have different element types (under
// autocast the mixer's output and y are bfloat16 while the residual stream stays float32).
template <typename T, int V>
__device__ __forceinline__ void load_vec(const T* p, float (&f)[V]) {
  const NVec<T, V> v = *reinterpret_cast<const NVec<T, V>*>(p);
#pragma unroll
  for (int i = 0; i < V; ++i) f[i] = Elem<T>::to_f(v.v[i]);
}
template <typename T, int V>
__device__ __forceinline__ void store_vec(T* p, const float (&f)[V]) {
  NVec<T, V> v;
#pragma unroll
  for (int i = 0; i < V; ++i) v.v[i] = Elem<T>::from_f(f[i]);
  *reinterpret_cast<NVec<T, V>*>(p) = v;
}

template <typename TX, typename TR, typename TY, int V>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_fwd_kernel(const TX* __restrict__ x, const TR* __restrict__ res_in, const float* __restrict__ w,
                       TR* __restrict__ res_out, TY* __restrict__ y, float* __restrict__ rstd, int64_t rows,
                       int64_t D, int64_t x_rs, int64_t ri_rs, int64_t ro_rs, int64_t y_rs, float eps) {
  const int lane = threadIdx.x & 31;
  const int64_t warp = int64_t(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
  const int64_t nwarps = int64_t(gridDim.x) * kNormWarps;
  for (int64_t r = warp; r < rows; r += nwarps) {
    float ss = 0.f;
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      float a[V], c[V];
      load_vec<TX, V>(x + r * x_rs + d, a);
      if (res_in) {
        load_vec<TR, V>(res_in + r * ri_rs + d, c);
#pragma unroll
        for (int i = 0; i < V; ++i) a[i] += c[i];
      }
      // the sum is rounded to the residual stream's type BEFORE it is normalised, as the reference's
      // separate add would have rounded it
#pragma unroll
      for (int i = 0; i < V; ++i) { a[i] = Elem<TR>::to_f(Elem<TR>::from_f(a[i])); ss = fmaf(a[i], a[i], ss); }
      store_vec<TR, V>(res_out + r * ro_rs + d, a);
    }
    const float rs = rsqrtf(warp_sum(ss) / float(D) + eps);
    if (rstd && lane == 0) rstd[r] = rs;
    __syncwarp();
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {       // second pass out of L1/L2: this lane's own stores
      float a[V];
      load_vec<TR, V>(res_out + r * ro_rs + d, a);
#pragma unroll
      for (int i = 0; i < V; ++i) a[i] = w ? a[i] * rs * w[d + i] : a[i] * rs;
      store_vec<TY, V>(y + r * y_rs + d, a);
    }
  }
}

// ds = (g - shat * mean(g * shat)) * rstd + dres_out, with g = dy * weight and shat = s * rstd: the gradient of
// the sum s, which is the gradient of both x and res_in.  dweight as in rmsnorm_bwd_kernel.
template <typename TR, typename TY, int V, bool kAccW>
__global__ void __launch_bounds__(kNormThreads)
add_rmsnorm_bwd_kernel(const TR* __restrict__ s, const float* __restrict__ w, const float* __restrict__ rstd,
                       const TY* __restrict__ dy, const TR* __restrict__ dres, TR* __restrict__ ds,
                       float* __restrict__ dw, int64_t rows, int64_t D, int64_t s_rs, int64_t dy_rs,
                       int64_t dr_rs, int64_t ds_rs) {
  extern __shared__ float s_dw[];               // [D] when kAccW
  const int lane = threadIdx.x & 31;
  const int64_t warp = int64_t(blockIdx.x) * kNormWarps + (threadIdx.x >> 5);
  const int64_t nwarps = int64_t(gridDim.x) * kNormWarps;
  if constexpr (kAccW) {
    for (int64_t d = threadIdx.x; d < D; d += kNormThreads) s_dw[d] = 0.f;
    __syncthreads();
  }
  for (int64_t r = warp; r < rows; r += nwarps) {
    const float rs = rstd[r];
    float dot = 0.f;
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      float sv[V], gv[V];
      load_vec<TR, V>(s + r * s_rs + d, sv);
      load_vec<TY, V>(dy + r * dy_rs + d, gv);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float sh = sv[i] * rs;
        if constexpr (kAccW) atomicAdd(&s_dw[d + i], gv[i] * sh);
        dot = fmaf(w ? gv[i] * w[d + i] : gv[i], sh, dot);
      }
    }
    const float m = warp_sum(dot) / float(D);
    for (int64_t d = int64_t(lane) * V; d < D; d += 32 * V) {
      float sv[V], gv[V], o[V];
      load_vec<TR, V>(s + r * s_rs + d, sv);
      load_vec<TY, V>(dy + r * dy_rs + d, gv);
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float g = w ? gv[i] * w[d + i] : gv[i];
        o[i] = (g - sv[i] * rs * m) * rs;
      }
      if (dres) {
        float rv[V];
        load_vec<TR, V>(dres + r * dr_rs + d, rv);
#pragma unroll
        for (int i = 0; i < V; ++i) o[i] += rv[i];
      }
      store_vec<TR, V>(ds + r * ds_rs + d, o);
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

// Element-type triple of the fused add + norm: (x, residual stream, y), each MB200_F32 or MB200_BF16.
template <typename TX, typename TR, typename TY>
static int add_norm_fwd_launch(const void* x, const void* res_in, const float* weight, void* res_out, void* y,
                               float* rstd, int64_t rows, int64_t D, int64_t x_rs, int64_t ri_rs, int64_t ro_rs,
                               int64_t y_rs, float eps, bool vec, cudaStream_t st) {
  const int grid = norm_grid(rows);
  if (vec)
    add_rmsnorm_fwd_kernel<TX, TR, TY, 4><<<grid, kNormThreads, 0, st>>>((const TX*)x, (const TR*)res_in, weight,
        (TR*)res_out, (TY*)y, rstd, rows, D, x_rs, ri_rs, ro_rs, y_rs, eps);
  else
    add_rmsnorm_fwd_kernel<TX, TR, TY, 1><<<grid, kNormThreads, 0, st>>>((const TX*)x, (const TR*)res_in, weight,
        (TR*)res_out, (TY*)y, rstd, rows, D, x_rs, ri_rs, ro_rs, y_rs, eps);
  return check_launch();
}

extern "C" int mb200_add_rmsnorm_fwd(const void* x, const void* res_in, const float* weight, void* res_out, void* y,
                                     float* rstd, int64_t rows, int64_t D, int64_t x_rs, int64_t ri_rs, int64_t ro_rs,
                                     int64_t y_rs, float eps, int dtype_x, int dtype_res, int dtype_y, void* stream) {
  if (rows < 0 || D < 0) return MB200_EINVAL;
  for (int dt : {dtype_x, dtype_res, dtype_y})
    if (dt != MB200_F32 && dt != MB200_BF16) return MB200_EDTYPE;
  if (rows == 0 || D == 0) return MB200_OK;
  if (!x || !res_out || !y) return MB200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // 4 elements per access: 16 bytes in float32, 8 in bfloat16; every pointer and stride must allow it
  bool vec = D % 4 == 0;
  for (const void* q : {x, res_in, (const void*)res_out, (const void*)y}) vec = vec && aligned16(q);
  for (int64_t sd : {x_rs, ri_rs, ro_rs, y_rs}) vec = vec && sd % 8 == 0;
  const int key = dtype_x * 4 + dtype_res * 2 + dtype_y;
#define MB200_ADDNORM(TX, TR, TY) \
  return add_norm_fwd_launch<TX, TR, TY>(x, res_in, weight, res_out, y, rstd, rows, D, x_rs, ri_rs, ro_rs, y_rs, eps, vec, st)
  switch (key) {
    case 0: MB200_ADDNORM(float, float, float);
    case 1: MB200_ADDNORM(float, float, __nv_bfloat16);
    case 4: MB200_ADDNORM(__nv_bfloat16, float, float);
    case 5: MB200_ADDNORM(__nv_bfloat16, float, __nv_bfloat16);
    case 7: MB200_ADDNORM(__nv_bfloat16, __nv_bfloat16, __nv_bfloat16);
    default: return MB200_EUNSUPPORTED;     // a residual stream narrower than what is added to it
  }
#undef MB200_ADDNORM
}

template <typename TR, typename TY>
static int add_norm_bwd_launch(const void* s, const float* weight, const float* rstd, const void* dy, const void* dres,
                               void* ds, float* dweight, int64_t rows, int64_t D, int64_t s_rs, int64_t dy_rs,
                               int64_t dr_rs, int64_t ds_rs, bool vec, cudaStream_t st) {
  const int grid = norm_grid(rows);
  const size_t smem = dweight ? size_t(D) * sizeof(float) : 0;
#define MB200_GO(VV, ACC)                                                                                         \
  add_rmsnorm_bwd_kernel<TR, TY, VV, ACC><<<grid, kNormThreads, smem, st>>>((const TR*)s, weight, rstd, (const TY*)dy, \
      (const TR*)dres, (TR*)ds, dweight, rows, D, s_rs, dy_rs, dr_rs, ds_rs)
  if (vec) { if (dweight) MB200_GO(4, true); else MB200_GO(4, false); }
  else { if (dweight) MB200_GO(1, true); else MB200_GO(1, false); }
#undef MB200_GO
  return check_launch();
}

extern "C" int mb200_add_rmsnorm_bwd(const void* s, const float* weight, const float* rstd, const void* dy,
                                     const void* dres, void* ds, float* dweight, int64_t rows, int64_t D,
                                     int64_t s_rs, int64_t dy_rs, int64_t dr_rs, int64_t ds_rs, int dtype_res,
                                     int dtype_y, void* stream) {
  if (rows < 0 || D < 0) return MB200_EINVAL;
  for (int dt : {dtype_res, dtype_y})
    if (dt != MB200_F32 && dt != MB200_BF16) return MB200_EDTYPE;
  if (rows == 0 || D == 0) return MB200_OK;
  if (!s || !rstd || !dy || !ds) return MB200_EINVAL;
  if (dweight && D > 12288) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  bool vec = D % 4 == 0;
  for (const void* q : {s, dy, dres, (const void*)ds}) vec = vec && aligned16(q);
  for (int64_t sd : {s_rs, dy_rs, dr_rs, ds_rs}) vec = vec && sd % 8 == 0;
  if (dtype_res == MB200_F32 && dtype_y == MB200_F32)
    return add_norm_bwd_launch<float, float>(s, weight, rstd, dy, dres, ds, dweight, rows, D, s_rs, dy_rs, dr_rs, ds_rs, vec, st);
  if (dtype_res == MB200_F32 && dtype_y == MB200_BF16)
    return add_norm_bwd_launch<float, __nv_bfloat16>(s, weight, rstd, dy, dres, ds, dweight, rows, D, s_rs, dy_rs, dr_rs, ds_rs, vec, st);
  if (dtype_res == MB200_BF16 && dtype_y == MB200_BF16)
    return add_norm_bwd_launch<__nv_bfloat16, __nv_bfloat16>(s, weight, rstd, dy, dres, ds, dweight, rows, D, s_rs, dy_rs, dr_rs, ds_rs, vec, st);
  return MB200_EUNSUPPORTED;
}
