// Depthwise causal conv1d + SiLU on (B, L, ED) tensors, forward and backward, for d_conv = 4:
//     y[b,t,e] = silu( bias[e] + sum_k w[e,k] * x[b, t-3+k, e] ),   x[b, t<0, e] = 0.
// This is the step in front of the selective scan in MambaBlock.forward (mambapy/mamba.py:217-221),
// done there as transpose -> nn.Conv1d(padding=3) -> slice -> transpose -> F.silu.  Here it runs in the
// (B, L, ED) layout the block already has: one read of x and one write of y (HBM-bound streaming).
//
// Mapping: a thread owns a vector of V channels and walks a chunk of `chunk` timesteps with the
// 4-wide window of each channel in registers; a warp covers 32 neighbouring vectors of one chunk, so
// it reads whole contiguous rows.  Chunks are short: the tensors are only (B, L, ED), and HBM bandwidth
// needs tens of thousands of independent loads in flight, which only many short chunks provide; the
// 3-step halo each chunk re-reads comes out of L2.  For the backward the host picks the chunk length
// (a multiple of 4) so that the warps fill the GPU in whole waves.  Loads of a group of timesteps
// are issued together, ahead of the arithmetic.
// The backward walks a chunk in reverse with two windows (x behind, d(pre) ahead), recomputing the
// pre-activation; the 8 warps of a CTA take 8 consecutive chunks of the same channels and add their
// sums for dw and dbias in shared memory first, so global memory sees one atomic per CTA and value.
#include <initializer_list>
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kConvK = 4;
constexpr int kConvThreads = 256;
constexpr int kConvChunkFwd = 32;             // forward chunk (compile time: its loop is fully unrolled)
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

// W channels of float arithmetic in one value: W = 2 uses the packed f32x2 instructions (one issue
// slot for two channels; these kernels would otherwise be bound by instruction issue, not by HBM).
template <int W> struct Pk;
template <> struct Pk<1> {
  float v;
  __device__ __forceinline__ static Pk splat(float a) { return {a}; }
  __device__ __forceinline__ static Pk load(const float* p, int stride) { return {p[0]}; }
  __device__ __forceinline__ float sum() const { return v; }
};
template <> struct Pk<2> {
  float2 v;
  __device__ __forceinline__ static Pk splat(float a) { return {make_float2(a, a)}; }
  __device__ __forceinline__ static Pk load(const float* p, int stride) { return {make_float2(p[0], p[stride])}; }
};
__device__ __forceinline__ Pk<1> pfma(Pk<1> a, Pk<1> b, Pk<1> c) { return {fmaf(a.v, b.v, c.v)}; }
__device__ __forceinline__ Pk<1> pmul(Pk<1> a, Pk<1> b) { return {a.v * b.v}; }
__device__ __forceinline__ Pk<1> padd(Pk<1> a, Pk<1> b) { return {a.v + b.v}; }
__device__ __forceinline__ Pk<1> psigmoid(Pk<1> a) { return {sigmoid_fast(a.v)}; }
__device__ __forceinline__ Pk<2> pfma(Pk<2> a, Pk<2> b, Pk<2> c) { return {__ffma2_rn(a.v, b.v, c.v)}; }
__device__ __forceinline__ Pk<2> pmul(Pk<2> a, Pk<2> b) { return {__fmul2_rn(a.v, b.v)}; }
__device__ __forceinline__ Pk<2> padd(Pk<2> a, Pk<2> b) { return {__fadd2_rn(a.v, b.v)}; }
__device__ __forceinline__ Pk<2> psigmoid(Pk<2> a) {
  const float2 m = __fmul2_rn(a.v, make_float2(-kLog2e, -kLog2e));
  const float2 d = __fadd2_rn(make_float2(ex2f(m.x), ex2f(m.y)), make_float2(1.f, 1.f));
  return {make_float2(__fdividef(1.f, d.x), __fdividef(1.f, d.y))};
}
// V raw elements <-> V/W packs
template <typename T, int V, int W>
__device__ __forceinline__ void unpack(const CVec<T, V>& r, Pk<W> (&o)[V / W]) {
#pragma unroll
  for (int i = 0; i < V / W; ++i) {
    if constexpr (W == 1) o[i].v = Elem<T>::to_f(r.v[i]);
    else o[i].v = make_float2(Elem<T>::to_f(r.v[2 * i]), Elem<T>::to_f(r.v[2 * i + 1]));
  }
}
template <typename T, int V, int W>
__device__ __forceinline__ CVec<T, V> pack(const Pk<W> (&o)[V / W]) {
  CVec<T, V> r;
#pragma unroll
  for (int i = 0; i < V / W; ++i) {
    if constexpr (W == 1) r.v[i] = Elem<T>::from_f(o[i].v);
    else if constexpr (sizeof(T) == 2) {
      *reinterpret_cast<__nv_bfloat162*>(&r.v[2 * i]) = __floats2bfloat162_rn(o[i].v.x, o[i].v.y);
    } else { r.v[2 * i] = o[i].v.x; r.v[2 * i + 1] = o[i].v.y; }
  }
  return r;
}

// grid: x = ceil(nvec / 32) channel groups, y = ceil(nchunk / 8), z = batch; warp w of a CTA takes chunk 8*y + w
template <typename T, int V>
__global__ void __launch_bounds__(kConvThreads, 4)
conv1d_silu_fwd_kernel(const T* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                       T* __restrict__ y, int64_t L, int64_t ED, int64_t x_sb, int64_t x_sl,
                       int64_t y_sb, int64_t y_sl) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t e = (int64_t(blockIdx.x) * 32 + lane) * V;
  const int64_t t0 = (int64_t(blockIdx.y) * (kConvThreads / 32) + warp) * kConvChunkFwd;
  if (e >= ED || t0 >= L) return;
  const int64_t b = blockIdx.z;
  constexpr int W = (V % 2 == 0) ? 2 : 1, P = V / W;
  using F = Pk<W>;
  F wk[P][kConvK], bv[P], win[P][kConvK - 1];
#pragma unroll
  for (int i = 0; i < P; ++i) {
    bv[i] = bias ? F::load(bias + e + W * i, 1) : F::splat(0.f);
#pragma unroll
    for (int k = 0; k < kConvK; ++k) wk[i][k] = F::load(w + (e + W * i) * kConvK + k, kConvK);
  }
  const T* xp = x + b * x_sb + e;
  T* yp = y + b * y_sb + e;
#pragma unroll
  for (int k = 0; k < kConvK - 1; ++k) {                  // x[t0-3 .. t0-1]
    const int64_t t = t0 - (kConvK - 1) + k;
    F xv[P];
    unpack<T, V, W>(cload<T, V>(xp + t * x_sl, t >= 0), xv);
#pragma unroll
    for (int i = 0; i < P; ++i) win[i][k] = xv[i];
  }
  // fully unrolled: the compiler hoists the loads of later groups over the arithmetic of earlier ones
#pragma unroll
  for (int g = 0; g < kConvChunkFwd / kConvGroup; ++g) {
    CVec<T, V> v[kConvGroup];
#pragma unroll
    for (int j = 0; j < kConvGroup; ++j) {
      const int64_t t = t0 + g * kConvGroup + j;
      v[j] = cload<T, V>(xp + t * x_sl, t < L);
    }
#pragma unroll
    for (int j = 0; j < kConvGroup; ++j) {
      const int64_t t = t0 + g * kConvGroup + j;
      F xn[P], o[P];
      unpack<T, V, W>(v[j], xn);
#pragma unroll
      for (int i = 0; i < P; ++i) {
        F acc = pfma(wk[i][0], win[i][0], bv[i]);
        acc = pfma(wk[i][1], win[i][1], acc);
        acc = pfma(wk[i][2], win[i][2], acc);
        acc = pfma(wk[i][3], xn[i], acc);
        win[i][0] = win[i][1]; win[i][1] = win[i][2]; win[i][2] = xn[i];
        o[i] = pmul(acc, psigmoid(acc));
      }
      if (t < L) cstore<T, V>(yp + t * y_sl, pack<T, V, W>(o));
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
                       int64_t dy_sb, int64_t dy_sl, int64_t dx_sb, int64_t dx_sl, int chunk) {
  __shared__ float s_acc[32 * V * (kConvK + 1)];          // per channel of the CTA: dw[0..3], dbias
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 32 * V * (kConvK + 1); i += kConvThreads) s_acc[i] = 0.f;
  __syncthreads();
  const int64_t e = (int64_t(blockIdx.x) * 32 + lane) * V;
  const int64_t t0 = (int64_t(blockIdx.y) * (kConvThreads / 32) + warp) * chunk;
  const int64_t t1 = min64(L, t0 + chunk);
  const int64_t b = blockIdx.z;
  if (e < ED && t0 < L) {
    constexpr int W = (V % 2 == 0) ? 2 : 1, P = V / W;
    using F = Pk<W>;
    F wk[P][kConvK], bv[P];
#pragma unroll
    for (int i = 0; i < P; ++i) {
      bv[i] = bias ? F::load(bias + e + W * i, 1) : F::splat(0.f);
#pragma unroll
      for (int k = 0; k < kConvK; ++k) wk[i][k] = F::load(w + (e + W * i) * kConvK + k, kConvK);
    }
    const T* xp = x + b * x_sb + e;
    const T* gp = dy + b * dy_sb + e;
    T* op = dx + b * dx_sb + e;
    // Both windows are circular buffers of 4 slots indexed by (steps taken) mod 4, and 4 steps are
    // unrolled per loop iteration, so every slot index is a compile-time constant and nothing is moved:
    // x[tau] and dpre[tau] live in slot (ts - tau) mod 4, ts = t1 + 2 being the first timestep processed.
    F xr[P][kConvK], dr[P][kConvK], dwacc[P][kConvK], dbacc[P];
#pragma unroll
    for (int i = 0; i < P; ++i) {
      dbacc[i] = F::splat(0.f);
#pragma unroll
      for (int k = 0; k < kConvK; ++k) { dwacc[i][k] = F::splat(0.f); dr[i][k] = F::splat(0.f); }
    }
    const int64_t ts = t1 + kConvK - 2;
#pragma unroll
    for (int k = 0; k < kConvK; ++k) {                     // x[ts-3 .. ts] -> slots 3-k
      const int64_t t = ts - (kConvK - 1) + k;
      F xv[P];
      unpack<T, V, W>(cload<T, V>(xp + t * x_sl, t >= 0 && t < L), xv);
#pragma unroll
      for (int i = 0; i < P; ++i) xr[i][kConvK - 1 - k] = xv[i];
    }
    // steps c = 0, 1, 2 (t >= t1) only produce dpre for the chunk's last outputs: their dx, dw belong
    // to the next chunk.  Steps below t0 (a short last chunk, padding of the last group) do nothing.
    const int nsteps = int(ts - t0) + 1;
    const F one = F::splat(1.f), mone = F::splat(-1.f);
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
        F g[P], xn[P], o[P];
        unpack<T, V, W>(gv[j], g);
        unpack<T, V, W>(xv[j], xn);
#pragma unroll
        for (int i = 0; i < P; ++i) {
          // window of step t: x[t-3+k] is in slot (j + 3 - k) mod 4
          F pre = bv[i];
#pragma unroll
          for (int k = 0; k < kConvK; ++k) pre = pfma(wk[i][k], xr[i][(j + 3 - k) & 3], pre);
          const F sg = psigmoid(pre);
          // dpre = dy * s * (1 + pre * (1 - s));  dy is 0 outside [t0, L)
          const F dp = pmul(pmul(g[i], sg), pfma(pre, pfma(sg, mone, one), one));
          // dx[t] = w3*dpre[t] + w2*dpre[t+1] + w1*dpre[t+2] + w0*dpre[t+3]; dpre[t+m] is in slot (j - m) mod 4
          F acc = pmul(wk[i][3], dp);
          acc = pfma(wk[i][2], dr[i][(j + 3) & 3], acc);
          acc = pfma(wk[i][1], dr[i][(j + 2) & 3], acc);
          acc = pfma(wk[i][0], dr[i][(j + 1) & 3], acc);
          o[i] = acc;
          if (own) {
            dbacc[i] = padd(dbacc[i], dp);
#pragma unroll
            for (int k = 0; k < kConvK; ++k) dwacc[i][k] = pfma(dp, xr[i][(j + 3 - k) & 3], dwacc[i][k]);
          }
          dr[i][j] = dp;
          xr[i][j] = xn[i];                                  // x[t-4] takes the slot of x[t]
        }
        if (own) cstore<T, V>(op + t * dx_sl, pack<T, V, W>(o));
      }
    }
#pragma unroll
    for (int i = 0; i < P; ++i) {
#pragma unroll
      for (int u = 0; u < W; ++u) {
        float* a = s_acc + (lane * V + i * W + u) * (kConvK + 1);
#pragma unroll
        for (int k = 0; k < kConvK; ++k) {
          float val;
          if constexpr (W == 1) val = dwacc[i][k].v; else val = u ? dwacc[i][k].v.y : dwacc[i][k].v.x;
          atomicAdd(a + k, val);
        }
        float dbv;
        if constexpr (W == 1) dbv = dbacc[i].v; else dbv = u ? dbacc[i].v.y : dbacc[i].v.x;
        atomicAdd(a + kConvK, dbv);
      }
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

// Chunk length (multiple of 4 in [16, 256]) that minimises waves x (chunk + halo): `cols` warps per
// (row, chunk), `warps_per_sm` resident warps per SM.
static int pick_conv_chunk(int64_t B, int64_t L, int64_t cols, int warps_per_sm) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const double cap = double(sms) * warps_per_sm;
  int best = 32;
  double best_cost = 1e300;
  for (int c = 16; c <= 256; c += 4) {
    const double warps = double(cols) * double((L + c - 1) / c) * double(B);
    const double waves = warps <= cap ? 1.0 : double(int64_t((warps + cap - 1) / cap));
    // a wave that is not full still runs for a whole chunk; very few warps cannot keep HBM busy
    const double fill = warps < cap ? cap / (warps > 1 ? warps : 1) : 1.0;
    const double cost = waves * (c + 3) * (fill > 4 ? fill / 4 : 1.0);
    if (cost < best_cost) { best_cost = cost; best = c; }
  }
  return best;
}

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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv = 4;                                      // 4 channels per thread: 8-byte (bf16) or 16-byte (f32) accesses
  const bool vec = conv_vec_ok(ED, kv, {x, y}, {x_sb, x_sl, y_sb, y_sl});
  const int v = vec ? kv : 1;
  const int64_t cols = (ED + 32 * int64_t(v) - 1) / (32 * int64_t(v));
  const int chunk = kConvChunkFwd;
  const int64_t nchunk = (L + chunk - 1) / chunk;
  const int64_t ngroup = (nchunk + kConvThreads / 32 - 1) / (kConvThreads / 32);
  if (B > 65535 || ngroup > 65535) return MB200_ETOOBIG;
  const dim3 grid(static_cast<unsigned>(cols), static_cast<unsigned>(ngroup), static_cast<unsigned>(B));
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
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int kv = 4;                                      // 4 channels per thread: 8-byte (bf16) or 16-byte (f32) accesses
  const bool vec = conv_vec_ok(ED, kv, {x, dy, (const void*)dx}, {x_sb, x_sl, dy_sb, dy_sl, dx_sb, dx_sl});
  const int v = vec ? kv : 1;
  const int64_t cols = (ED + 32 * int64_t(v) - 1) / (32 * int64_t(v));
  const int chunk = pick_conv_chunk(B, L, cols, 16);
  const int64_t nchunk = (L + chunk - 1) / chunk;
  const int64_t ngroup = (nchunk + kConvThreads / 32 - 1) / (kConvThreads / 32);
  if (B > 65535 || ngroup > 65535) return MB200_ETOOBIG;
  const dim3 grid(static_cast<unsigned>(cols), static_cast<unsigned>(ngroup), static_cast<unsigned>(B));
#define MB200_CONV_BWD(TT, VV)                                                                          \
  conv1d_silu_bwd_kernel<TT, VV><<<grid, kConvThreads, 0, st>>>((const TT*)x, w, bias, (const TT*)dy, \
      (TT*)dx, dw, dbias, L, ED, x_sb, x_sl, dy_sb, dy_sl, dx_sb, dx_sl, chunk)
  if (dtype == MB200_F32) { if (vec) MB200_CONV_BWD(float, 4); else MB200_CONV_BWD(float, 1); }
  else { if (vec) MB200_CONV_BWD(__nv_bfloat16, 4); else MB200_CONV_BWD(__nv_bfloat16, 1); }
#undef MB200_CONV_BWD
  return check_launch();
}
