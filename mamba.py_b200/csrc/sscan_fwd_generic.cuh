// GENERIC path of the fused selective scan forward (any alignment, any strides; see
// sscan_fwd.cu for the tensor-map path that is used whenever the tensors allow it).
//
// Fused selective scan, forward: discretisation, recurrence, C-contraction, D skip and
// SiLU(z) gate in one pass.  Reads x, delta, z, B, C once; writes y (and, for training,
// the scan state every kChunk timesteps).  The (B, L, ED, N) tensors never exist.
//
// What bounds it.  Per (b, t, e, n) element the kernel needs one ex2 (16/clk/SM on the MUFU
// pipe), four FP32 operations, and its B and C operands out of shared memory; HBM traffic is
// 0.5 byte per element.  Measured on B200 the recurrence loop alone runs at the shared-memory
// return bandwidth (128 B/clk/SM), ahead of the MUFU pipe, and far ahead of HBM.  So the kernel
// does no redundant arithmetic (every recurrence is walked serially along L by exactly one
// thread) and keeps everything that is not the recurrence off the threads that run it.
//
// Structure: warp-specialised CTA of 192 threads owning a tile of channels of one batch row.
//   - 4 consumer warps run the recurrence.  A thread owns 4 consecutive states n of one channel
//     (N/4 lanes share a channel).  Per timestep: 3 shared loads ({delta, delta*x}, B quad,
//     C quad), 4 ex2, 8 packed f32x2 operations, and one 4-byte store of its partial
//     C-contraction.  Nothing else.
//   - 2 producer warps stream time in tiles of kTT timesteps: 128-bit coalesced global loads one
//     tile ahead, conversion to float32 operands (softplus(delta+bias), delta*x) into a swizzled
//     double-buffered shared tile, and, two tiles behind, the epilogue: sum the N/4 partials of
//     each channel, add D*x, apply the SiLU(z) gate, and store y with 128-bit vectors.
//   - Hand-off through four CTA-local mbarriers (full/empty per buffer).  Every wait is bounded;
//     a wait that gives up records MB200_DEV_WAIT_TIMEOUT and the thread leaves the kernel.
#pragma once
#include "common.cuh"
#include "tile.cuh"
#include "sscan.cuh"

namespace mb200 {
namespace {

constexpr int kConsumers = kThreadsPerCta;      // 128
constexpr int kGenProducers = 64;
constexpr int kGenThreads = kConsumers + kGenProducers;

__device__ int g_fwd_status = MB200_DEV_OK;

template <typename T, int N> struct GenFwdSmem {
  using G = SscanGeom<N>;
  static constexpr int kTE = G::kTE, kTT = G::kTT;
  // offsets in floats
  static constexpr int kBars = 0;                                   // 4 x uint64
  static constexpr int kOp = 8;                                     // float2 [2][kTT][kTE]
  static constexpr int kB = kOp + 2 * kTT * kTE * 2;                // float  [2][kTT][N]
  static constexpr int kC = kB + 2 * kTT * N;                       // float  [2][kTT][N]
  static constexpr int kYp = kC + 2 * kTT * N;                      // float  [2][kTT][128]
  static constexpr int kX = kYp + 2 * kTT * kConsumers;             // T      [2][kTT][kTE]
  static constexpr int kRawFloats = (kTT * kTE * int(sizeof(T)) + 3) / 4;
  static constexpr int kZ = kX + 2 * kRawFloats;                    // T      [2][kTT][kTE]
  static constexpr int kD = kZ + 2 * kRawFloats;                    // float  [kTE]
  static constexpr int kBias = kD + kTE;                            // float  [kTE]
  static constexpr int kFloats = kBias + kTE;
  static constexpr int kBytes = kFloats * 4;
};

// slot of channel e_l's partial sums inside a row of the partial-sum tile; the XOR keeps the
// epilogue's 128-bit reads of 8 neighbouring channels per lane free of bank conflicts
template <int kLPE, int kTE>
__device__ __forceinline__ int yp_slot(int t, int e_l) {
  if constexpr (kLPE == 4 && kTE == 32) return e_l ^ ((e_l >> 3) & 3) ^ ((t & 1) << 2);
  return e_l;
}

template <typename T, int N, int KV>
__global__ void __launch_bounds__(kGenThreads, 3)
sscan_fwd_generic_kernel(const SscanFwdParams p) {
  using G = SscanGeom<N>;
  using S = GenFwdSmem<T, N>;
  constexpr int kLPE = G::kLPE, kTE = G::kTE, kTT = G::kTT;

  extern __shared__ __align__(16) float smem[];
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBars);   // full[0], full[1], empty[0], empty[1]
  float2* s_op = reinterpret_cast<float2*>(smem + S::kOp);
  float* s_B = smem + S::kB;
  float* s_C = smem + S::kC;
  float* s_yp = smem + S::kYp;
  T* s_x = reinterpret_cast<T*>(smem + S::kX);
  T* s_z = reinterpret_cast<T*>(smem + S::kZ);
  float* s_D = smem + S::kD;
  float* s_bias = smem + S::kBias;

  const int tid = threadIdx.x;
  const int64_t e0 = int64_t(blockIdx.x) * kTE;
  const int64_t b = blockIdx.y;
  const int cols_ok = int(min64(kTE, p.ED - e0));
  const bool softplus = (p.flags & MB200_DELTA_SOFTPLUS) != 0;
  const bool has_y = p.y != nullptr;
  const bool has_z = p.z != nullptr;
  const int64_t ntiles = (p.L + kTT - 1) / kTT;

  if (tid == 0) {
    mbar_init(&bars[0], kGenProducers); mbar_init(&bars[1], kGenProducers);
    mbar_init(&bars[2], kConsumers); mbar_init(&bars[3], kConsumers);
  }
  for (int i = tid; i < kTE; i += kGenThreads) {
    const bool ok = i < cols_ok;
    s_D[i] = (ok && p.D) ? p.D[e0 + i] : 0.f;
    s_bias[i] = (ok && softplus) ? p.delta_bias[e0 + i] : 0.f;
  }
  __syncthreads();

  if (tid < kConsumers) {
    // ------------------------------------------------------------------ consumers
    const int e_l = tid / kLPE, q = tid % kLPE;
    const int64_t e = e0 + e_l;
    const bool e_ok = e < p.ED;
    const int64_t nchunks = (p.L + kChunk - 1) / kChunk;
    float2 A2lo, A2hi, hlo, hhi;
    {
      float a4[4], h4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a4[j] = e_ok ? p.A[e * N + 4 * q + j] * kLog2e : 0.f;
        h4[j] = (e_ok && p.h0) ? p.h0[(b * p.ED + e) * N + 4 * q + j] : 0.f;
      }
      A2lo = make_float2(a4[0], a4[1]); A2hi = make_float2(a4[2], a4[3]);
      hlo = make_float2(h4[0], h4[1]); hhi = make_float2(h4[2], h4[3]);
    }
    const int op_off0 = op_index(0, e_l, kTE), op_off1 = op_index(1, e_l, kTE) - kTE;
    const int yp_off0 = yp_slot<kLPE, kTE>(0, e_l) * kLPE + q;
    const int yp_off1 = yp_slot<kLPE, kTE>(1, e_l) * kLPE + q;

    for (int64_t kt = 0; kt < ntiles; ++kt) {
      const int buf = int(kt & 1);
      const int64_t t0 = kt * kTT;
      if (!mbar_wait(&bars[buf], int((kt >> 1) & 1))) {
        atomicExch(&g_fwd_status, MB200_DEV_WAIT_TIMEOUT);
        return;
      }
      const float2* op = s_op + buf * kTT * kTE;
      const float* sB = s_B + buf * kTT * N + 4 * q;
      const float* sC = s_C + buf * kTT * N + 4 * q;
      float* yp = s_yp + buf * kTT * kConsumers;
#pragma unroll
      for (int t = 0; t < kTT; ++t) {
        if ((t % kChunk) == 0 && p.carries && e_ok && t0 + t < p.L) {
          float4* dst = reinterpret_cast<float4*>(
              p.carries + ((b * nchunks + (t0 + t) / kChunk) * p.ED + e) * N + 4 * q);
          *dst = make_float4(hlo.x, hlo.y, hhi.x, hhi.y);
        }
        const float2 o = op[t * kTE + ((t & 1) ? op_off1 : op_off0)];   // {delta, delta*x}
        const float4 Bq = *reinterpret_cast<const float4*>(sB + t * N);
        const float4 Cq = *reinterpret_cast<const float4*>(sC + t * N);
        const float2 dd = make_float2(o.x, o.x), dxx = make_float2(o.y, o.y);
        const float2 e_lo = __fmul2_rn(dd, A2lo), e_hi = __fmul2_rn(dd, A2hi);
        const float2 a_lo = make_float2(ex2f(e_lo.x), ex2f(e_lo.y));
        const float2 a_hi = make_float2(ex2f(e_hi.x), ex2f(e_hi.y));
        const float2 u_lo = __fmul2_rn(dxx, make_float2(Bq.x, Bq.y));
        const float2 u_hi = __fmul2_rn(dxx, make_float2(Bq.z, Bq.w));
        hlo = __ffma2_rn(a_lo, hlo, u_lo);
        hhi = __ffma2_rn(a_hi, hhi, u_hi);
        float2 acc = __fmul2_rn(hlo, make_float2(Cq.x, Cq.y));
        acc = __ffma2_rn(hhi, make_float2(Cq.z, Cq.w), acc);
        if (has_y) yp[t * kConsumers + ((t & 1) ? yp_off1 : yp_off0)] = acc.x + acc.y;
      }
      mbar_arrive(&bars[2 + buf]);
    }
    if (p.hT && e_ok) {
      float4* dst = reinterpret_cast<float4*>(p.hT + (b * p.ED + e) * N + 4 * q);
      *dst = make_float4(hlo.x, hlo.y, hhi.x, hhi.y);
    }
  } else {
    // ------------------------------------------------------------------ producers
    const int pt = tid - kConsumers;
    constexpr int KVB = (N % KV == 0) ? KV : 1;
    using ActRegs = TileRegs<T, kTT, kTE, KV, kGenProducers>;
    using BcRegs = TileRegs<T, kTT, N, KVB, kGenProducers>;
    using AMap = typename ActRegs::Map;
    constexpr int kPT = AMap::kPerThread;

    const T* gx = static_cast<const T*>(p.x) + b * p.x_sb + e0;
    const T* gd = static_cast<const T*>(p.delta) + b * p.d_sb + e0;
    const T* gz = has_z ? static_cast<const T*>(p.z) + b * p.z_sb + e0 : nullptr;
    const T* gB = static_cast<const T*>(p.Bm) + b * p.b_sb;
    const T* gC = static_cast<const T*>(p.Cm) + b * p.c_sb;
    T* gy = has_y ? static_cast<T*>(p.y) + b * p.y_sb + e0 : nullptr;

    ActRegs rx, rd, rz;
    BcRegs rB, rC;
    auto fetch = [&](int64_t kt) {
      const int64_t t0 = kt * kTT;
      const int rows_ok = int(min64(kTT, p.L - t0));
      rx.load(gx + t0 * p.x_sl, p.x_sl, rows_ok, cols_ok, pt);
      rd.load(gd + t0 * p.d_sl, p.d_sl, rows_ok, cols_ok, pt);
      if (has_z) rz.load(gz + t0 * p.z_sl, p.z_sl, rows_ok, cols_ok, pt);
      rB.load(gB + t0 * p.b_sl, p.b_sl, rows_ok, N, pt);
      rC.load(gC + t0 * p.c_sl, p.c_sl, rows_ok, N, pt);
    };
    // convert the fetched tile and publish it in buffer kt & 1
    auto commit = [&](int64_t kt) {
      const int buf = int(kt & 1);
      const int rows_ok = int(min64(kTT, p.L - kt * kTT));
      float2* tile = s_op + buf * kTT * kTE;
#pragma unroll
      for (int i = 0; i < kPT; ++i) {
        if (!AMap::owns(i, pt)) continue;
        const int rr = AMap::row(i, pt), cc = AMap::col(i, pt);
        float2 v[KV];
#pragma unroll
        for (int k = 0; k < KV; ++k) {
          const bool ok = rr < rows_ok && cc + k < cols_ok;
          float dv = Elem<T>::to_f(rd.r[i].v[k]);
          const float xv = Elem<T>::to_f(rx.r[i].v[k]);
          if (softplus) dv = ok ? softplus_fast(dv + s_bias[cc + k]) : 0.f;
          v[k] = make_float2(dv, dv * xv);
        }
        if constexpr (KV % 2 == 0) {
#pragma unroll
          for (int k = 0; k < KV; k += 2)
            *reinterpret_cast<float4*>(tile + op_index(rr, cc + k, kTE)) =
                make_float4(v[k].x, v[k].y, v[k + 1].x, v[k + 1].y);
        } else {
          tile[op_index(rr, cc, kTE)] = v[0];
        }
        if (has_y) {                              // raw x and z, for this tile's epilogue
          tvec_store<T, KV>(s_x + (buf * kTT + rr) * kTE + cc, rx.r[i]);
          if (has_z) tvec_store<T, KV>(s_z + (buf * kTT + rr) * kTE + cc, rz.r[i]);
        }
      }
      commit_bc<T, N, KVB>(rB, rC, s_B + buf * kTT * N, s_C + buf * kTT * N, pt);
      mbar_arrive(&bars[buf]);
    };
    // finish tile kt: partial sums -> y.  Caller has waited for the consumers of tile kt.
    auto epilogue = [&](int64_t kt) {
      const int buf = int(kt & 1);
      const int64_t t0 = kt * kTT;
      const int rows_ok = int(min64(kTT, p.L - t0));
      const float* yp = s_yp + buf * kTT * kConsumers;
#pragma unroll
      for (int i = 0; i < kPT; ++i) {
        if (!AMap::owns(i, pt)) continue;
        const int rr = AMap::row(i, pt), cc = AMap::col(i, pt);
        if (rr >= rows_ok || cc >= cols_ok) continue;
        const TVec<T, KV> xv = *reinterpret_cast<const TVec<T, KV>*>(s_x + (buf * kTT + rr) * kTE + cc);
        TVec<T, KV> zv = xv;
        if (has_z) zv = *reinterpret_cast<const TVec<T, KV>*>(s_z + (buf * kTT + rr) * kTE + cc);
        TVec<T, KV> out;
#pragma unroll
        for (int k = 0; k < KV; ++k) {
          const float s = sum_lanes<kLPE>(yp + rr * kConsumers + yp_slot<kLPE, kTE>(rr, cc + k) * kLPE);
          float yv = fmaf(s_D[cc + k], Elem<T>::to_f(xv.v[k]), s);
          if (has_z) {
            const float zf = Elem<T>::to_f(zv.v[k]);
            yv *= zf * sigmoid_fast(zf);
          }
          out.v[k] = Elem<T>::from_f(yv);
        }
        tvec_store<T, KV>(gy + (t0 + rr) * p.y_sl + cc, out);
      }
    };
    auto wait_consumed = [&](int64_t kt) {            // consumers are done with tile kt
      if (mbar_wait(&bars[2 + int(kt & 1)], int((kt >> 1) & 1))) return true;
      atomicExch(&g_fwd_status, MB200_DEV_WAIT_TIMEOUT);
      return false;
    };

    fetch(0);
    for (int64_t kt = 0; kt < ntiles; ++kt) {
      if (kt >= 2) {                                  // buffer kt & 1 still holds tile kt - 2
        if (!wait_consumed(kt - 2)) return;
        if (has_y) epilogue(kt - 2);
      }
      commit(kt);
      if (kt + 1 < ntiles) fetch(kt + 1);
    }
    for (int64_t kt = ntiles >= 2 ? ntiles - 2 : 0; kt < ntiles; ++kt) {
      if (!wait_consumed(kt)) return;
      if (has_y) epilogue(kt);
    }
  }
}

template <typename T, int N>
int generic_launch_n(const SscanFwdParams& p, bool vec, cudaStream_t st) {
  using G = SscanGeom<N>;
  using S = GenFwdSmem<T, N>;
  dim3 grid(unsigned((p.ED + G::kTE - 1) / G::kTE), unsigned(p.B));
  constexpr int KV = Elem<T>::kVec;
  auto kv = sscan_fwd_generic_kernel<T, N, KV>;
  auto k1 = sscan_fwd_generic_kernel<T, N, 1>;
  auto k = vec ? kv : k1;
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes) != cudaSuccess)
    return MB200_ELAUNCH;
  k<<<grid, kGenThreads, S::kBytes, st>>>(p);
  return check_launch();
}

template <typename T>
int generic_launch_t(const SscanFwdParams& p, int N, bool vec, cudaStream_t st) {
  switch (N) {
    case 8: return generic_launch_n<T, 8>(p, vec, st);
    case 16: return generic_launch_n<T, 16>(p, vec, st);
    case 32: return generic_launch_n<T, 32>(p, vec, st);
    case 64: return generic_launch_n<T, 64>(p, vec, st);
    default: return MB200_ENSTATE;
  }
}

}  // namespace
}  // namespace mb200

