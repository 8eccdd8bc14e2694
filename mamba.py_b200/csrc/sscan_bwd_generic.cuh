// GENERIC path of the fused selective scan backward (any alignment, any strides; sscan_bwd.cu
// holds the tensor-map path used whenever the tensors allow it).
//
// Fused selective scan, backward.  One pass over x, delta, z, B, C, dy (read once) that
// writes dx, ddelta, dz and accumulates dB, dC, dA, dD; the hidden states are recomputed
// chunk by chunk from the states the forward saved every kChunk timesteps.
//
// Mapping: the same as the forward (a thread owns 4 states n of one channel e and walks time
// serially), but time runs from the last chunk to the first.  For each chunk of kChunk timesteps
//   phase R  recomputes a[t] = exp(delta[t] A) and h[t] forwards from the saved state and keeps
//            both in registers (2 x 16 x 4 floats), so the exponential is evaluated once;
//   phase B  walks the chunk backwards:  g[t] = dy'[t] C[t] + a[t+1] g[t+1]  and from g, h, a
//            forms every gradient term.
// Two kinds of sums leave a thread:
//   over n (dx, ddelta, and y for dz): the N/4 lanes of a channel exchange three partial sums
//            per timestep through shared memory; one lane per timestep finishes it;
//   over e (dB, dC): a warp's channels are summed through a per-warp shared-memory transpose,
//            warps are merged with shared-memory atomics, and the CTA adds its 16 x 2N block to
//            global memory with one atomic per value.
#pragma once
#include "common.cuh"
#include "tile.cuh"
#include "sscan.cuh"

namespace mb200 {
namespace {

constexpr int kGenWin = 4;                       // timesteps per reduction window
constexpr int kGenWarps = kThreadsPerCta / 32;

template <typename T, int N> struct GenBwdSmem {
  using G = SscanGeom<N>;
  static constexpr int kTE = G::kTE, kLPE = G::kLPE, kEPW = 32 / G::kLPE;
  // float offsets of each region inside the dynamic shared memory block
  static constexpr int kIn = 0;                                   // float4 [2][kChunk][kTE] {delta, delta*x, dy', x}
  static constexpr int kEp = kIn + 2 * kChunk * kTE * 4;          // float4 [2][kChunk][kTE] {z, dy, dsoftplus, -}
  static constexpr int kB = kEp + 2 * kChunk * kTE * 4;           // float [2][kChunk][N]
  static constexpr int kC = kB + 2 * kChunk * N;                  // float [2][kChunk][N]
  static constexpr int kNred = kC + 2 * kChunk * N;               // float4 [kGenWin][kThreads+1]
  static constexpr int kEredB = kNred + kGenWin * (kThreadsPerCta + 1) * 4;   // float [kGenWarps][kGenWin][kEPW][N]
  static constexpr int kEredStride = kGenWin * kEPW * N + 16;        // per warp, B part; C part follows
  static constexpr int kAcc = kEredB + kGenWarps * 2 * kEredStride;  // float [2][kChunk][N]
  static constexpr int kOut = kAcc + 2 * kChunk * N;              // float [3][kChunk][kTE]
  static constexpr int kFloats = kOut + 3 * kChunk * kTE;
  static constexpr int kBytes = kFloats * 4;
};

template <typename T, int N, int KV>
__global__ void __launch_bounds__(kThreadsPerCta)
sscan_bwd_generic_kernel(const SscanBwdParams p) {
  using G = SscanGeom<N>;
  using S = GenBwdSmem<T, N>;
  constexpr int kLPE = G::kLPE, kTE = G::kTE, kEPW = S::kEPW;
  constexpr int KVB = (N % KV == 0) ? KV : 1;
  using ActRegs = TileRegs<T, kChunk, kTE, KV>;
  using BcRegs = TileRegs<T, kChunk, N, KVB>;

  extern __shared__ __align__(16) float smem[];
  float4* s_in = reinterpret_cast<float4*>(smem + S::kIn);
  float4* s_ep = reinterpret_cast<float4*>(smem + S::kEp);
  float* s_B = smem + S::kB;
  float* s_C = smem + S::kC;
  float4* s_nred = reinterpret_cast<float4*>(smem + S::kNred);
  float* s_acc = smem + S::kAcc;
  float* s_out = smem + S::kOut;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int e_l = tid / kLPE, q = tid % kLPE, e_w = lane / kLPE;
  float* s_eB = smem + S::kEredB + warp * 2 * S::kEredStride;
  float* s_eC = s_eB + S::kEredStride;
  const int64_t e0 = int64_t(blockIdx.x) * kTE;
  const int64_t e = e0 + e_l;
  const int64_t b = blockIdx.y;
  const bool e_ok = e < p.ED;
  const int cols_ok = int(min64(kTE, p.ED - e0));
  const bool has_z = p.z != nullptr;
  const bool softplus = (p.flags & MB200_DELTA_SOFTPLUS) != 0;

  const T* gx = static_cast<const T*>(p.x) + b * p.x_sb + e0;
  const T* gd = static_cast<const T*>(p.delta) + b * p.d_sb + e0;
  const T* gz = has_z ? static_cast<const T*>(p.z) + b * p.z_sb + e0 : nullptr;
  const T* gdy = static_cast<const T*>(p.dy) + b * p.dy_sb + e0;
  const T* gB = static_cast<const T*>(p.Bm) + b * p.b_sb;
  const T* gC = static_cast<const T*>(p.Cm) + b * p.c_sb;
  T* odx = static_cast<T*>(p.dx) + b * p.dx_sb + e0;
  T* odd = static_cast<T*>(p.ddelta) + b * p.dd_sb + e0;
  T* odz = has_z ? static_cast<T*>(p.dz) + b * p.dz_sb + e0 : nullptr;

  float A2[4], gc[4], dAacc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    A2[j] = e_ok ? p.A[e * N + 4 * q + j] * kLog2e : 0.f;
    gc[j] = (e_ok && p.g_in) ? p.g_in[(b * p.ED + e) * N + 4 * q + j] : 0.f;
    dAacc[j] = 0.f;
  }
  const float Dv = (e_ok && p.D) ? p.D[e] : 0.f;
  float dDacc = 0.f, dbias_acc = 0.f;

  ActRegs rx, rd, rz, rdy;
  BcRegs rB, rC;
  const int64_t nchunks = (p.L + kChunk - 1) / kChunk;

  auto fetch = [&](int64_t t0) {
    const int rows_ok = int(min64(kChunk, p.L - t0));
    rx.load(gx + t0 * p.x_sl, p.x_sl, rows_ok, cols_ok, tid);
    rd.load(gd + t0 * p.d_sl, p.d_sl, rows_ok, cols_ok, tid);
    rdy.load(gdy + t0 * p.dy_sl, p.dy_sl, rows_ok, cols_ok, tid);
    if (has_z) rz.load(gz + t0 * p.z_sl, p.z_sl, rows_ok, cols_ok, tid);
    rB.load(gB + t0 * p.b_sl, p.b_sl, rows_ok, N, tid);
    rC.load(gC + t0 * p.c_sl, p.c_sl, rows_ok, N, tid);
  };
  auto commit = [&](int buf, int64_t t0) {
    const int rows_ok = int(min64(kChunk, p.L - t0));
#pragma unroll
    for (int i = 0; i < ActRegs::Map::kPerThread; ++i) {
      if (!ActRegs::Map::owns(i, tid)) continue;
      const int rr = ActRegs::Map::row(i, tid), cc = ActRegs::Map::col(i, tid);
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        const bool ok = rr < rows_ok && cc + k < cols_ok;
        float dv = Elem<T>::to_f(rd.r[i].v[k]);
        const float xv = Elem<T>::to_f(rx.r[i].v[k]);
        const float dyv = Elem<T>::to_f(rdy.r[i].v[k]);
        const float zv = has_z ? Elem<T>::to_f(rz.r[i].v[k]) : 0.f;
        float spg = 1.f;
        if (softplus) {
          const float raw = ok ? dv + p.delta_bias[e0 + cc + k] : 0.f;
          dv = ok ? softplusf(raw) : 0.f;
          spg = sigmoidf(raw);
        }
        const float dyg = has_z ? dyv * zv * sigmoidf(zv) : dyv;
        s_in[(buf * kChunk + rr) * kTE + cc + k] = make_float4(dv, dv * xv, dyg, xv);
        s_ep[(buf * kChunk + rr) * kTE + cc + k] = make_float4(zv, dyv, spg, 0.f);
      }
    }
#pragma unroll
    for (int i = 0; i < BcRegs::Map::kPerThread; ++i) {
      if (!BcRegs::Map::owns(i, tid)) continue;
      const int rr = BcRegs::Map::row(i, tid), cc = BcRegs::Map::col(i, tid);
#pragma unroll
      for (int k = 0; k < KVB; ++k) {
        s_B[(buf * kChunk + rr) * N + cc + k] = Elem<T>::to_f(rB.r[i].v[k]);
        s_C[(buf * kChunk + rr) * N + cc + k] = Elem<T>::to_f(rC.r[i].v[k]);
      }
    }
  };
  auto load_carry = [&](int64_t c, float (&hp)[4]) {
    if (e_ok) {
      const float4 v = *reinterpret_cast<const float4*>(
          p.carries + ((b * nchunks + c) * p.ED + e) * N + 4 * q);
      hp[0] = v.x; hp[1] = v.y; hp[2] = v.z; hp[3] = v.w;
    } else {
      hp[0] = hp[1] = hp[2] = hp[3] = 0.f;
    }
  };

  for (int i = tid; i < 2 * kChunk * N; i += kThreadsPerCta) s_acc[i] = 0.f;
  float hp_next[4];
  fetch((nchunks - 1) * kChunk);
  load_carry(nchunks - 1, hp_next);
  commit(0, (nchunks - 1) * kChunk);
  __syncthreads();

  int buf = 0;
  for (int64_t c = nchunks - 1; c >= 0; --c, buf ^= 1) {
    const int64_t t0 = c * kChunk;
    float hp[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) hp[j] = hp_next[j];
    if (c > 0) {
      fetch(t0 - kChunk);
      load_carry(c - 1, hp_next);
    }

    // ---- phase R: decay factors and states of the chunk, kept in registers
    float a[kChunk][4], hh[kChunk][4];
#pragma unroll
    for (int t = 0; t < kChunk; ++t) {
      const float4 in = s_in[(buf * kChunk + t) * kTE + e_l];
      const float4 Bq = *reinterpret_cast<const float4*>(&s_B[(buf * kChunk + t) * N + 4 * q]);
      const float bq[4] = {Bq.x, Bq.y, Bq.z, Bq.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a[t][j] = ex2f(in.x * A2[j]);
        hh[t][j] = fmaf(a[t][j], t ? hh[t - 1][j] : hp[j], in.y * bq[j]);
      }
    }

    // ---- phase B: reverse walk, one reduction window of kGenWin timesteps at a time
#pragma unroll
    for (int w = kChunk / kGenWin - 1; w >= 0; --w) {
#pragma unroll
      for (int i = kGenWin - 1; i >= 0; --i) {
        const int t = w * kGenWin + i;
        const float4 in = s_in[(buf * kChunk + t) * kTE + e_l];
        const float4 Bq = *reinterpret_cast<const float4*>(&s_B[(buf * kChunk + t) * N + 4 * q]);
        const float4 Cq = *reinterpret_cast<const float4*>(&s_C[(buf * kChunk + t) * N + 4 * q]);
        const float bq[4] = {Bq.x, Bq.y, Bq.z, Bq.w};
        const float cq[4] = {Cq.x, Cq.y, Cq.z, Cq.w};
        float ypart = 0.f, gBpart = 0.f, wApart = 0.f;
        float dBp[4], dCp[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float g = fmaf(in.z, cq[j], gc[j]);
          ypart = fmaf(hh[t][j], cq[j], ypart);
          dCp[j] = in.z * hh[t][j];
          dBp[j] = g * in.y;
          gBpart = fmaf(g, bq[j], gBpart);
          const float hprev = t ? hh[t - 1][j] : hp[j];
          const float wv = g * hprev * a[t][j];
          dAacc[j] = fmaf(wv, in.x, dAacc[j]);
          wApart = fmaf(wv, A2[j], wApart);
          gc[j] = a[t][j] * g;
        }
        s_nred[i * (kThreadsPerCta + 1) + tid] = make_float4(ypart, gBpart, wApart, 0.f);
        *reinterpret_cast<float4*>(&s_eB[(i * kEPW + e_w) * N + 4 * q]) =
            make_float4(dBp[0], dBp[1], dBp[2], dBp[3]);
        *reinterpret_cast<float4*>(&s_eC[(i * kEPW + e_w) * N + 4 * q]) =
            make_float4(dCp[0], dCp[1], dCp[2], dCp[3]);
      }
      __syncwarp();
      // sums over n: lane q finishes the timesteps i == q (mod kLPE) of the window
      for (int i = q; i < kGenWin; i += kLPE) {
        const int t = w * kGenWin + i;
        float ys = 0.f, gBs = 0.f, wAs = 0.f;
#pragma unroll
        for (int k = 0; k < kLPE; ++k) {
          const float4 v = s_nred[i * (kThreadsPerCta + 1) + tid - q + k];
          ys += v.x; gBs += v.y; wAs += v.z;
        }
        const float4 in = s_in[(buf * kChunk + t) * kTE + e_l];     // delta, delta*x, dy', x
        const float4 ep = s_ep[(buf * kChunk + t) * kTE + e_l];     // z, dy, dsoftplus
        const float dxv = fmaf(in.z, Dv, in.x * gBs);
        float ddv = fmaf(in.w, gBs, wAs * (1.f / kLog2e));
        ddv *= ep.z;
        dDacc = fmaf(in.z, in.w, dDacc);
        dbias_acc += ddv;
        s_out[(0 * kChunk + t) * kTE + e_l] = dxv;
        s_out[(1 * kChunk + t) * kTE + e_l] = ddv;
        if (has_z) {
          const float sg = sigmoidf(ep.x);
          const float yv = fmaf(Dv, in.w, ys);
          s_out[(2 * kChunk + t) * kTE + e_l] = ep.y * yv * sg * (1.f + ep.x * (1.f - sg));
        }
      }
      // sums over the warp's channels: one float4 group (timestep, B|C, n/4) per step
      for (int g = lane; g < kGenWin * 2 * (N / 4); g += 32) {
        const int i = g / (2 * (N / 4)), r = g % (2 * (N / 4));
        const bool isC = r >= N / 4;
        const int n4 = isC ? r - N / 4 : r;
        const float* src = (isC ? s_eC : s_eB) + i * kEPW * N + 4 * n4;
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int k = 0; k < kEPW; ++k) {
          const float4 v = *reinterpret_cast<const float4*>(src + k * N);
          acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
        }
        float* dst = s_acc + ((isC ? 1 : 0) * kChunk + w * kGenWin + i) * N + 4 * n4;
        atomicAdd(dst + 0, acc.x); atomicAdd(dst + 1, acc.y);
        atomicAdd(dst + 2, acc.z); atomicAdd(dst + 3, acc.w);
      }
      __syncwarp();
    }
    __syncthreads();

    // ---- write the chunk's dx, ddelta, dz tiles and flush its dB, dC block
    {
      const int rows_ok = int(min64(kChunk, p.L - t0));
#pragma unroll
      for (int i = 0; i < ActRegs::Map::kPerThread; ++i) {
        if (!ActRegs::Map::owns(i, tid)) continue;
        const int rr = ActRegs::Map::row(i, tid), cc = ActRegs::Map::col(i, tid);
        if (rr >= rows_ok || cc >= cols_ok) continue;
        TVec<T, KV> vx, vd, vz;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
          vx.v[k] = Elem<T>::from_f(s_out[(0 * kChunk + rr) * kTE + cc + k]);
          vd.v[k] = Elem<T>::from_f(s_out[(1 * kChunk + rr) * kTE + cc + k]);
          if (has_z) vz.v[k] = Elem<T>::from_f(s_out[(2 * kChunk + rr) * kTE + cc + k]);
        }
        tvec_store<T, KV>(odx + (t0 + rr) * p.dx_sl + cc, vx);
        tvec_store<T, KV>(odd + (t0 + rr) * p.dd_sl + cc, vd);
        if (has_z) tvec_store<T, KV>(odz + (t0 + rr) * p.dz_sl + cc, vz);
      }
      for (int i = tid; i < 2 * kChunk * N; i += kThreadsPerCta) {
        const int which = i / (kChunk * N), rr = (i / N) % kChunk, n = i % N;
        const float v = s_acc[i];
        s_acc[i] = 0.f;
        if (rr < rows_ok)
          atomicAdd((which ? p.dC : p.dB) + (b * p.L + t0 + rr) * N + n, v);
      }
    }
    if (c > 0) commit(buf ^ 1, t0 - kChunk);
    __syncthreads();
  }

  // ---- sums over (b, t) kept per thread: dA, dD, d(delta_bias); and the outgoing carry
  if (e_ok) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      atomicAdd(p.dA + e * N + 4 * q + j, dAacc[j]);
    if (p.g_out) {
      *reinterpret_cast<float4*>(p.g_out + (b * p.ED + e) * N + 4 * q) =
          make_float4(gc[0], gc[1], gc[2], gc[3]);
    }
  }
#pragma unroll
  for (int s = kLPE / 2; s >= 1; s >>= 1) {
    dDacc += __shfl_xor_sync(0xffffffffu, dDacc, s);
    dbias_acc += __shfl_xor_sync(0xffffffffu, dbias_acc, s);
  }
  if (e_ok && q == 0) {
    if (p.dD) atomicAdd(p.dD + e, dDacc);
    if (p.ddelta_bias) atomicAdd(p.ddelta_bias + e, dbias_acc);
  }
}

template <typename T, int N>
int bwd_generic_launch_n(const SscanBwdParams& p, bool vec, cudaStream_t st) {
  using G = SscanGeom<N>;
  using S = GenBwdSmem<T, N>;
  dim3 grid(unsigned((p.ED + G::kTE - 1) / G::kTE), unsigned(p.B));
  constexpr int KV = Elem<T>::kVec;
  auto kv = sscan_bwd_generic_kernel<T, N, KV>;
  auto k1 = sscan_bwd_generic_kernel<T, N, 1>;
  auto k = vec ? kv : k1;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes) != cudaSuccess)
    return MB200_ELAUNCH;
  k<<<grid, kThreadsPerCta, S::kBytes, st>>>(p);
  return check_launch();
}

template <typename T>
int bwd_generic_launch_t(const SscanBwdParams& p, int N, bool vec, cudaStream_t st) {
  switch (N) {
    case 8: return bwd_generic_launch_n<T, 8>(p, vec, st);
    case 16: return bwd_generic_launch_n<T, 16>(p, vec, st);
    case 32: return bwd_generic_launch_n<T, 32>(p, vec, st);
    case 64: return bwd_generic_launch_n<T, 64>(p, vec, st);
    default: return MB200_ENSTATE;
  }
}

}  // namespace
}  // namespace mb200

