// Depthwise causal conv1d + SiLU on (B, L, ED) tensors, forward and backward, for d_conv = 4:
//     y[b,t,e] = silu( bias[e] + sum_k w[e,k] * x[b, t-3+k, e] ),   x[b, t<0, e] = 0.
// This is the step in front of the selective scan in MambaBlock.forward (mambapy/mamba.py:217-221),
// done there as transpose -> nn.Conv1d(padding=3) -> slice -> transpose -> F.silu.  Here it runs in the
// (B, L, ED) layout the block already has: one read of x and one write of y (HBM-bound streaming).
//
// Mapping: a thread owns one 16-byte vector of channels and walks a chunk of kConvChunk timesteps with
// the 4-wide window of each channel in registers; a warp reads 512 contiguous bytes per timestep.
// The backward walks the chunk in reverse with two windows (x behind, d(pre) ahead), recomputing the
// pre-activation, and adds its per-thread sums for dw and dbias with atomics.
#include <initializer_list>
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kConvK = 4;
constexpr int kConvChunk = 64;
constexpr int kConvThreads = 128;

template <typename T, int V> struct CVec {
  T v[V];
};
template <typename T, int V>
__device__ __forceinline__ CVec<T, V> cload(const T* p, bool ok) {
  CVec<T, V> r;
  if (!ok) {
#pragma unroll
    for (int i = 0; i < V; ++i) r.v[i] = Elem<T>::from_f(0.f);
  } else if constexpr (V == 1) {
    r.v[0] = __ldg(p);
  } else {
    *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  }
  return r;
}
template <typename T, int V>
__device__ __forceinline__ void cstore(T* p, const CVec<T, V>& r) {
  if constexpr (V == 1) *p = r.v[0];
  else *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
}

template <typename T, int V>
__global__ void __launch_bounds__(kConvThreads)
conv1d_silu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       T* __restrict__ y, int64_t L, int64_t ED, int64_t x_sb, int64_t x_sl,
                       int64_t y_sb, int64_t y_sl) {
  const int64_t e = (int64_t(blockIdx.x) * kConvThreads + threadIdx.x) * V;
  if (e >= ED) return;
  const int64_t b = blockIdx.y;
  const int64_t t0 = int64_t(blockIdx.z) * kConvChunk, t1 = min64(L, t0 + kConvChunk);
  float wk[V][kConvK], bv[V], win[V][kConvK - 1];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    bv[i] = bias ? bias[e + i] : 0.f;
#pragma unroll
    for (int k = 0; k < kConvK; ++k) wk[i][k] = w[(e + i) * kConvK + k];
  }
  const T* xp = x + b * x_sb + e;
  T* yp = y + b * y_sb + e;
#pragma unroll
  for (int k = 0; k < kConvK - 1; ++k) {                  // x[t0-3 .. t0-1]
    const int64_t t = t0 - (kConvK - 1) + k;
    const CVec<T, V> v = cload<T, V>(xp + t * x_sl, t >= 0);
#pragma unroll
    for (int i = 0; i < V; ++i) win[i][k] = Elem<T>::to_f(v.v[i]);
  }
#pragma unroll 4
  for (int64_t t = t0; t < t1; ++t) {
    const CVec<T, V> v = cload<T, V>(xp + t * x_sl, true);
    CVec<T, V> o;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float xn = Elem<T>::to_f(v.v[i]);
      float acc = bv[i];
      acc = fmaf(wk[i][0], win[i][0], acc);
      acc = fmaf(wk[i][1], win[i][1], acc);
      acc = fmaf(wk[i][2], win[i][2], acc);
      acc = fmaf(wk[i][3], xn, acc);
      win[i][0] = win[i][1]; win[i][1] = win[i][2]; win[i][2] = xn;
      o.v[i] = Elem<T>::from_f(acc * sigmoid_fast(acc));
    }
    cstore<T, V>(yp + t * y_sl, o);
  }
}

// dx[t] = sum_k w[k] * dpre[t+3-k];  dw[k] = sum_{b,t} dpre[t] * x[t-3+k];  dbias = sum dpre;
// dpre[t] = dy[t] * silu'(pre[t]),  pre recomputed from x.
template <typename T, int V>
__global__ void __launch_bounds__(kConvThreads)
conv1d_silu_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ dw,
                       float* __restrict__ dbias, int64_t L, int64_t ED, int64_t x_sb, int64_t x_sl,
                       int64_t dy_sb, int64_t dy_sl, int64_t dx_sb, int64_t dx_sl) {
  const int64_t e = (int64_t(blockIdx.x) * kConvThreads + threadIdx.x) * V;
  if (e >= ED) return;
  const int64_t b = blockIdx.y;
  const int64_t t0 = int64_t(blockIdx.z) * kConvChunk, t1 = min64(L, t0 + kConvChunk);
  float wk[V][kConvK], bv[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    bv[i] = bias ? bias[e + i] : 0.f;
#pragma unroll
    for (int k = 0; k < kConvK; ++k) wk[i][k] = w[(e + i) * kConvK + k];
  }
  const T* xp = x + b * x_sb + e;
  const T* gp = dy + b * dy_sb + e;
  T* op = dx + b * dx_sb + e;
  // xw[i][k] = x[t-3+k] for the timestep t whose dpre is being formed; starts at t = t1 + 2
  float xw[V][kConvK], dq[V][kConvK - 1], dwacc[V][kConvK], dbacc[V];
#pragma unroll
  for (int i = 0; i < V; ++i) {
    dbacc[i] = 0.f;
#pragma unroll
    for (int k = 0; k < kConvK; ++k) dwacc[i][k] = 0.f;
#pragma unroll
    for (int k = 0; k < kConvK - 1; ++k) dq[i][k] = 0.f;
  }
  auto load_x = [&](int64_t t, float (&dst)[V]) {
    const CVec<T, V> v = cload<T, V>(xp + t * x_sl, t >= 0 && t < L);
#pragma unroll
    for (int i = 0; i < V; ++i) dst[i] = Elem<T>::to_f(v.v[i]);
  };
  {
    const int64_t ts = t1 + kConvK - 2;                  // first timestep processed (a halo step)
#pragma unroll
    for (int k = 0; k < kConvK; ++k) {
      float tmp[V];
      load_x(ts - (kConvK - 1) + k, tmp);
#pragma unroll
      for (int i = 0; i < V; ++i) xw[i][k] = tmp[i];
    }
  }
  // t runs from t1+2 down to t0; steps with t >= t1 only feed dq (their dx, dw belong to the next chunk)
  for (int64_t t = t1 + kConvK - 2; t >= t0; --t) {
    const bool own = t < t1;
    const CVec<T, V> g = cload<T, V>(gp + t * dy_sl, t < L);
    float xnew[V];
    load_x(t - kConvK, xnew);                            // x entering the window for the next step
    CVec<T, V> o;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float pre = bv[i];
#pragma unroll
      for (int k = 0; k < kConvK; ++k) pre = fmaf(wk[i][k], xw[i][k], pre);
      const float s = sigmoid_fast(pre);
      const float dp = (t < L) ? Elem<T>::to_f(g.v[i]) * s * (1.f + pre * (1.f - s)) : 0.f;
      if (own) {
        // dx[t] = w3*dpre[t] + w2*dpre[t+1] + w1*dpre[t+2] + w0*dpre[t+3]
        float acc = wk[i][3] * dp;
        acc = fmaf(wk[i][2], dq[i][0], acc);
        acc = fmaf(wk[i][1], dq[i][1], acc);
        acc = fmaf(wk[i][0], dq[i][2], acc);
        o.v[i] = Elem<T>::from_f(acc);
        dbacc[i] += dp;
#pragma unroll
        for (int k = 0; k < kConvK; ++k) dwacc[i][k] = fmaf(dp, xw[i][k], dwacc[i][k]);
      }
      dq[i][2] = dq[i][1]; dq[i][1] = dq[i][0]; dq[i][0] = dp;
      xw[i][3] = xw[i][2]; xw[i][2] = xw[i][1]; xw[i][1] = xw[i][0]; xw[i][0] = xnew[i];
    }
    if (own) cstore<T, V>(op + t * dx_sl, o);
  }
#pragma unroll
  for (int i = 0; i < V; ++i) {
    if (dbias) atomicAdd(dbias + e + i, dbacc[i]);
#pragma unroll
    for (int k = 0; k < kConvK; ++k) atomicAdd(dw + (e + i) * kConvK + k, dwacc[i][k]);
  }
}

}  // namespace
}  // namespace mb200

using namespace mb200;

static bool conv_vec_ok(int64_t ED, int kv, std::initializer_list<const void*> ptrs,
                        std::initializer_list<int64_t> strides) {
  if (ED % kv) return false;
  for (const void* p : ptrs) if (!aligned16(p)) return false;
  for (int64_t s : strides) if (s % kv) return false;
  return true;
}

extern "C" int mb200_conv1d_silu_fwd(const void* x, const float* w, const float* bias, void* y,
                                     int64_t B, int64_t L, int64_t ED, int K, int64_t x_sb, int64_t x_sl,
                                     int64_t y_sb, int64_t y_sl, int dtype, void* stream) {
  if (B < 0 || L < 0 || ED < 0) return MB200_EINVAL;
  if (K != kConvK) return MB200_ETOOBIG;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (B == 0 || L == 0 || ED == 0) return MB200_OK;
  if (!x || !w || !y) return MB200_EINVAL;
  const int64_t nchunk = (L + kConvChunk - 1) / kConvChunk;
  if (B > 65535 || nchunk > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv = dtype == MB200_F32 ? 4 : 8;
  const bool vec = conv_vec_ok(ED, kv, {x, y}, {x_sb, x_sl, y_sb, y_sl});
  const int v = vec ? kv : 1;
  dim3 grid(unsigned((ED + int64_t(v) * kConvThreads - 1) / (int64_t(v) * kConvThreads)), unsigned(B), unsigned(nchunk));
#define MB200_CONV_FWD(TT, VV) \
  conv1d_silu_fwd_kernel<TT, VV><<<grid, kConvThreads, 0, st>>>((const TT*)x, w, bias, (TT*)y, L, ED, x_sb, x_sl, y_sb, y_sl)
  if (dtype == MB200_F32) { if (vec) MB200_CONV_FWD(float, 4); else MB200_CONV_FWD(float, 1); }
  else { if (vec) MB200_CONV_FWD(__nv_bfloat16, 8); else MB200_CONV_FWD(__nv_bfloat16, 1); }
#undef MB200_CONV_FWD
  return check_launch();
}

extern "C" int mb200_conv1d_silu_bwd(const void* x, const float* w, const float* bias, const void* dy,
                                     void* dx, float* dw, float* dbias, int64_t B, int64_t L, int64_t ED,
                                     int K, int64_t x_sb, int64_t x_sl, int64_t dy_sb, int64_t dy_sl,
                                     int64_t dx_sb, int64_t dx_sl, int dtype, void* stream) {
  if (B < 0 || L < 0 || ED < 0) return MB200_EINVAL;
  if (K != kConvK) return MB200_ETOOBIG;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (B == 0 || L == 0 || ED == 0) return MB200_OK;
  if (!x || !w || !dy || !dx || !dw) return MB200_EINVAL;
  const int64_t nchunk = (L + kConvChunk - 1) / kConvChunk;
  if (B > 65535 || nchunk > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv = dtype == MB200_F32 ? 4 : 8;
  const bool vec = conv_vec_ok(ED, kv, {x, dy, (const void*)dx}, {x_sb, x_sl, dy_sb, dy_sl, dx_sb, dx_sl});
  const int v = vec ? kv : 1;
  dim3 grid(unsigned((ED + int64_t(v) * kConvThreads - 1) / (int64_t(v) * kConvThreads)), unsigned(B), unsigned(nchunk));
#define MB200_CONV_BWD(TT, VV)                                                                          \
  conv1d_silu_bwd_kernel<TT, VV><<<grid, kConvThreads, 0, st>>>((const TT*)x, w, bias, (const TT*)dy, \
      (TT*)dx, dw, dbias, L, ED, x_sb, x_sl, dy_sb, dy_sl, dx_sb, dx_sl)
  if (dtype == MB200_F32) { if (vec) MB200_CONV_BWD(float, 4); else MB200_CONV_BWD(float, 1); }
  else { if (vec) MB200_CONV_BWD(__nv_bfloat16, 8); else MB200_CONV_BWD(__nv_bfloat16, 1); }
#undef MB200_CONV_BWD
  return check_launch();
}
