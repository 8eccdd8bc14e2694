// Depthwise causal conv1d + SiLU on (B, L, ED) tensors, forward and backward, for d_conv = 4:
//     y[b,t,e] = silu( bias[e] + sum_k w[e,k] * x[b, t-3+k, e] ),   x[b, t<0, e] = 0.
// This is the step in front of the selective scan in MambaBlock.forward (mambapy/mamba.py:217-221),
// done there as transpose -> nn.Conv1d(padding=3) -> slice -> transpose -> F.silu.  Here it runs in the
// (B, L, ED) layout the block already has: one read of x and one write of y (HBM-bound streaming).
//
// Mapping: a thread owns a vector of V channels and walks a chunk of kConvChunk timesteps with the
// 4-wide window of each channel in registers; a warp covers 32 neighbouring vectors of one chunk, so
// it reads whole contiguous rows.  Chunks are short (32 steps): the tensors are only (B, L, ED), and
// HBM bandwidth needs tens of thousands of independent 16-byte loads in flight, which only many short
// chunks provide; the 3-step halo each chunk re-reads comes out of L2.  Loads of a group of timesteps
// are issued together, ahead of the arithmetic.
// The backward walks a chunk in reverse with two windows (x behind, d(pre) ahead), recomputing the
// pre-activation; the 8 warps of a CTA take 8 consecutive chunks of the same channels and add their
// sums for dw and dbias in shared memory first, so global memory sees one atomic per CTA and value.
#include <initializer_list>
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kConvK = 4;
constexpr int kConvChunk = 32;
constexpr int kConvThreads = 256;
constexpr int kConvGroup = 4;                 // timesteps whose loads are in flight together (forward)

template <typename T, int V> struct alignas(sizeof(T) * V) CVec {
  T v[V];
};
template <typename T, int V>
__device__ __forceinline__ CVec<T, V> cload(const T* p, bool ok) {
  CVec<T, V> r;
  if (!ok) {
#pragma unroll
    for (int i = 0; i < V; ++i) r.v[i] = Elem<T>::from_f(0.f);
  } else if constexpr (sizeof(T) * V == 16) {
    *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  } else if constexpr (sizeof(T) * V == 8) {
    *reinterpret_cast<uint2*>(&r) = __ldg(reinterpret_cast<const uint2*>(p));
  } else {
#pragma unroll
    for (int i = 0; i < V; ++i) r.v[i] = __ldg(p + i);
  }
  return r;
}
template <typename T, int V>
__device__ __forceinline__ void cstore(T* p, const CVec<T, V>& r) {
  if constexpr (sizeof(T) * V == 16) *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
  else if constexpr (sizeof(T) * V == 8) *reinterpret_cast<uint2*>(p) = *reinterpret_cast<const uint2*>(&r);
  else {
#pragma unroll
    for (int i = 0; i < V; ++i) p[i] = r.v[i];
  }
}

// grid: x = ceil(nvec / 32) channel groups, y = ceil(nchunk / 8), z = batch; warp w of a CTA takes chunk 8*y + w
template <typename T, int V>
__global__ void __launch_bounds__(kConvThreads, 4)
conv1d_silu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       T* __restrict__ y, int64_t L, int64_t ED, int64_t x_sb, int64_t x_sl,
                       int64_t y_sb, int64_t y_sl) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t e = (int64_t(blockIdx.x) * 32 + lane) * V;
  const int64_t t0 = (int64_t(blockIdx.y) * (kConvThreads / 32) + warp) * kConvChunk;
  if (e >= ED || t0 >= L) return;
  const int64_t b = blockIdx.z;
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
#pragma unroll
  for (int g = 0; g < kConvChunk / kConvGroup; ++g) {
    CVec<T, V> v[kConvGroup];
#pragma unroll
    for (int j = 0; j < kConvGroup; ++j) {
      const int64_t t = t0 + g * kConvGroup + j;
      v[j] = cload<T, V>(xp + t * x_sl, t < L);
    }
#pragma unroll
    for (int j = 0; j < kConvGroup; ++j) {
      const int64_t t = t0 + g * kConvGroup + j;
      CVec<T, V> o;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float xn = Elem<T>::to_f(v[j].v[i]);
        float acc = bv[i];
        acc = fmaf(wk[i][0], win[i][0], acc);
        acc = fmaf(wk[i][1], win[i][1], acc);
        acc = fmaf(wk[i][2], win[i][2], acc);
        acc = fmaf(wk[i][3], xn, acc);
        win[i][0] = win[i][1]; win[i][1] = win[i][2]; win[i][2] = xn;
        o.v[i] = Elem<T>::from_f(acc * sigmoid_fast(acc));
      }
      if (t < L) cstore<T, V>(yp + t * y_sl, o);
    }
  }
}

// dx[t] = sum_k w[k] * dpre[t+3-k];  dw[k] = sum_{b,t} dpre[t] * x[t-3+k];  dbias = sum dpre;
// dpre[t] = dy[t] * silu'(pre[t]),  pre recomputed from x.
template <typename T, int V>
__global__ void __launch_bounds__(kConvThreads, 2)
conv1d_silu_bwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       const T* __restrict__ dy, T* __restrict__ dx, float* __restrict__ dw,
                       float* __restrict__ dbias, int64_t L, int64_t ED, int64_t x_sb, int64_t x_sl,
                       int64_t dy_sb, int64_t dy_sl, int64_t dx_sb, int64_t dx_sl) {
  __shared__ float s_acc[32 * V * (kConvK + 1)];          // per channel of the CTA: dw[0..3], dbias
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * V * (kConvK + 1); i += kConvThreads) s_acc[i] = 0.f;
  __syncthreads();
  const int64_t e = (int64_t(blockIdx.x) * 32 + lane) * V;
  const int64_t t0 = (int64_t(blockIdx.y) * (kConvThreads / 32) + warp) * kConvChunk;
  const int64_t t1 = min64(L, t0 + kConvChunk);
  const int64_t b = blockIdx.z;
  if (e < ED && t0 < L) {
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
    // Both windows are circular buffers of 4 slots indexed by (steps taken) mod 4, and 4 steps are
    // unrolled per loop iteration, so every slot index is a compile-time constant and nothing is moved:
    // x[tau] and dpre[tau] live in slot (ts - tau) mod 4, ts = t1 + 2 being the first timestep processed.
    float xr[V][kConvK], dr[V][kConvK], dwacc[V][kConvK], dbacc[V];
#pragma unroll
    for (int i = 0; i < V; ++i) {
      dbacc[i] = 0.f;
#pragma unroll
      for (int k = 0; k < kConvK; ++k) { dwacc[i][k] = 0.f; dr[i][k] = 0.f; }
    }
    const int64_t ts = t1 + kConvK - 2;
#pragma unroll
    for (int k = 0; k < kConvK; ++k) {                     // x[ts-3 .. ts] -> slots 3-k
      const int64_t t = ts - (kConvK - 1) + k;
      const CVec<T, V> v = cload<T, V>(xp + t * x_sl, t >= 0 && t < L);
#pragma unroll
      for (int i = 0; i < V; ++i) xr[i][kConvK - 1 - k] = Elem<T>::to_f(v.v[i]);
    }
    // steps c = 0, 1, 2 (t >= t1) only produce dpre for the chunk's last outputs: their dx, dw belong
    // to the next chunk.  Steps below t0 (a short last chunk, padding of the last group) do nothing.
    const int nsteps = int(ts - t0) + 1;
#pragma unroll 1
    for (int c0 = 0; c0 < nsteps; c0 += kConvK) {
      CVec<T, V> gv[kConvK], xv[kConvK];
#pragma unroll
      for (int j = 0; j < kConvK; ++j) {
        const int64_t t = ts - (c0 + j);
        gv[j] = cload<T, V>(gp + t * dy_sl, t >= t0 && t < L);
        xv[j] = cload<T, V>(xp + (t - kConvK) * x_sl, t >= t0 && t - kConvK >= 0);
      }
#pragma unroll
      for (int j = 0; j < kConvK; ++j) {
        const int c = c0 + j;
        const int64_t t = ts - c;
        const bool own = c >= kConvK - 1 && t >= t0;
        CVec<T, V> o;
#pragma unroll
        for (int i = 0; i < V; ++i) {
          // window of step t: x[t-3+k] is in slot (j + 3 - k) mod 4
          float pre = bv[i];
#pragma unroll
          for (int k = 0; k < kConvK; ++k) pre = fmaf(wk[i][k], xr[i][(j + 3 - k) & 3], pre);
          const float s = sigmoid_fast(pre);
          const float dp = Elem<T>::to_f(gv[j].v[i]) * s * (1.f + pre * (1.f - s));   // dy is 0 outside [t0, L)
          // dx[t] = w3*dpre[t] + w2*dpre[t+1] + w1*dpre[t+2] + w0*dpre[t+3]; dpre[t+m] is in slot (j - m) mod 4
          float acc = wk[i][3] * dp;
          acc = fmaf(wk[i][2], dr[i][(j + 3) & 3], acc);
          acc = fmaf(wk[i][1], dr[i][(j + 2) & 3], acc);
          acc = fmaf(wk[i][0], dr[i][(j + 1) & 3], acc);
          o.v[i] = Elem<T>::from_f(acc);
          if (own) {
            dbacc[i] += dp;
#pragma unroll
            for (int k = 0; k < kConvK; ++k) dwacc[i][k] = fmaf(dp, xr[i][(j + 3 - k) & 3], dwacc[i][k]);
          }
          dr[i][j] = dp;
          xr[i][j] = Elem<T>::to_f(xv[j].v[i]);              // x[t-4] takes the slot of x[t]
        }
        if (own) cstore<T, V>(op + t * dx_sl, o);
      }
    }
#pragma unroll
    for (int i = 0; i < V; ++i) {
      float* a = s_acc + (lane * V + i) * (kConvK + 1);
#pragma unroll
      for (int k = 0; k < kConvK; ++k) atomicAdd(a + k, dwacc[i][k]);
      atomicAdd(a + kConvK, dbacc[i]);
    }
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 32 * V * (kConvK + 1); i += kConvThreads) {
    const int64_t ch = int64_t(blockIdx.x) * 32 * V + i / (kConvK + 1);
    const int k = i % (kConvK + 1);
    if (ch >= ED) continue;
    if (k < kConvK) atomicAdd(dw + ch * kConvK + k, s_acc[i]);
    else if (dbias) atomicAdd(dbias + ch, s_acc[i]);
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
  const int64_t ngroup = (nchunk + kConvThreads / 32 - 1) / (kConvThreads / 32);
  if (B > 65535 || ngroup > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv = 4;                                      // 4 channels per thread: 8-byte (bf16) or 16-byte (f32) accesses
  const bool vec = conv_vec_ok(ED, kv, {x, y}, {x_sb, x_sl, y_sb, y_sl});
  const int v = vec ? kv : 1;
  dim3 grid(unsigned((ED + 32 * int64_t(v) - 1) / (32 * int64_t(v))), unsigned(ngroup), unsigned(B));
#define MB200_CONV_FWD(TT, VV) \
  conv1d_silu_fwd_kernel<TT, VV><<<grid, kConvThreads, 0, st>>>((const TT*)x, w, bias, (TT*)y, L, ED, x_sb, x_sl, y_sb, y_sl)
  if (dtype == MB200_F32) { if (vec) MB200_CONV_FWD(float, 4); else MB200_CONV_FWD(float, 1); }
  else { if (vec) MB200_CONV_FWD(__nv_bfloat16, 4); else MB200_CONV_FWD(__nv_bfloat16, 1); }
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
  const int64_t ngroup = (nchunk + kConvThreads / 32 - 1) / (kConvThreads / 32);
  if (B > 65535 || ngroup > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv = 4;                                      // 4 channels per thread: 8-byte (bf16) or 16-byte (f32) accesses
  const bool vec = conv_vec_ok(ED, kv, {x, dy, (const void*)dx}, {x_sb, x_sl, dy_sb, dy_sl, dx_sb, dx_sl});
  const int v = vec ? kv : 1;
  dim3 grid(unsigned((ED + 32 * int64_t(v) - 1) / (32 * int64_t(v))), unsigned(ngroup), unsigned(B));
#define MB200_CONV_BWD(TT, VV)                                                                          \
  conv1d_silu_bwd_kernel<TT, VV><<<grid, kConvThreads, 0, st>>>((const TT*)x, w, bias, (const TT*)dy, \
      (TT*)dx, dw, dbias, L, ED, x_sb, x_sl, dy_sb, dy_sl, dx_sb, dx_sl)
  if (dtype == MB200_F32) { if (vec) MB200_CONV_BWD(float, 4); else MB200_CONV_BWD(float, 1); }
  else { if (vec) MB200_CONV_BWD(__nv_bfloat16, 4); else MB200_CONV_BWD(__nv_bfloat16, 1); }
#undef MB200_CONV_BWD
  return check_launch();
}
