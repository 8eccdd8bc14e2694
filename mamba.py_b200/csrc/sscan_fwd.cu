// Fused selective scan, forward: discretisation, recurrence, C-contraction, D skip and
// SiLU(z) gate in one pass.  Reads x, delta, z, B, C once; writes y (and, for training,
// the scan state every kChunk timesteps).  The (B, L, ED, N) tensors never exist.
//
// Mapping.  The kernel is bound by the exponential (one ex2 per (b, t, e, n)) and the FP32
// pipe, not by HBM, so it does no redundant arithmetic: every recurrence is walked serially
// along L by exactly one thread.  A thread owns 4 consecutive states n of one channel e
// (N/4 lanes share a channel), a CTA owns a tile of channels of one batch row and streams
// over time in tiles of kTT timesteps staged in shared memory with register prefetch of the
// next tile.  The partial C-contractions of kLPE consecutive timesteps are transposed across
// the kLPE lanes of a channel, so each lane finishes (D skip, gate, store) one timestep.
#include "common.cuh"
#include "tile.cuh"
#include "sscan.cuh"

namespace mb200 {
namespace {

template <typename T, int N, int KV>
__global__ void __launch_bounds__(kThreadsPerCta)
sscan_fwd_kernel(const SscanFwdParams p) {
  using G = SscanGeom<N>;
  constexpr int kLPE = G::kLPE, kTE = G::kTE, kTT = G::kTT;
  constexpr int KVB = (N % KV == 0) ? KV : 1;
  using ActRegs = TileRegs<T, kTT, kTE, KV>;
  using BcRegs = TileRegs<T, kTT, N, KVB>;

  __shared__ __align__(16) float2 s_dd[2][kTT][kTE];   // {delta, delta*x}
  __shared__ __align__(16) float2 s_xz[2][kTT][kTE];   // {x, z}
  __shared__ __align__(16) float s_B[2][kTT][N];
  __shared__ __align__(16) float s_C[2][kTT][N];
  __shared__ __align__(16) T s_y[kTT][kTE];

  const int tid = threadIdx.x;
  const int e_l = tid / kLPE, q = tid % kLPE;
  const int64_t e0 = int64_t(blockIdx.x) * kTE;
  const int64_t e = e0 + e_l;
  const int64_t b = blockIdx.y;
  const bool e_ok = e < p.ED;
  const int cols_ok = int(min64(kTE, p.ED - e0));

  const T* gx = static_cast<const T*>(p.x) + b * p.x_sb + e0;
  const T* gd = static_cast<const T*>(p.delta) + b * p.d_sb + e0;
  const T* gz = p.z ? static_cast<const T*>(p.z) + b * p.z_sb + e0 : nullptr;
  const T* gB = static_cast<const T*>(p.Bm) + b * p.b_sb;
  const T* gC = static_cast<const T*>(p.Cm) + b * p.c_sb;
  T* gy = p.y ? static_cast<T*>(p.y) + b * p.y_sb + e0 : nullptr;

  float A2[4], h[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    A2[j] = e_ok ? p.A[e * N + 4 * q + j] * kLog2e : 0.f;
    h[j] = (e_ok && p.h0) ? p.h0[(b * p.ED + e) * N + 4 * q + j] : 0.f;
  }
  const float Dv = (e_ok && p.D) ? p.D[e] : 0.f;
  const bool softplus = (p.flags & MB200_DELTA_SOFTPLUS) != 0;

  ActRegs rx, rd, rz;
  BcRegs rB, rC;

  auto fetch = [&](int64_t t0) {
    const int rows_ok = int(min64(kTT, p.L - t0));
    rx.load(gx + t0 * p.x_sl, p.x_sl, rows_ok, cols_ok, tid);
    rd.load(gd + t0 * p.d_sl, p.d_sl, rows_ok, cols_ok, tid);
    if (gz) rz.load(gz + t0 * p.z_sl, p.z_sl, rows_ok, cols_ok, tid);
    rB.load(gB + t0 * p.b_sl, p.b_sl, rows_ok, N, tid);
    rC.load(gC + t0 * p.c_sl, p.c_sl, rows_ok, N, tid);
  };
  auto commit = [&](int buf, int64_t t0) {
    const int rows_ok = int(min64(kTT, p.L - t0));
#pragma unroll
    for (int i = 0; i < ActRegs::Map::kPerThread; ++i) {
      if (!ActRegs::Map::owns(i, tid)) continue;
      const int rr = ActRegs::Map::row(i, tid), cc = ActRegs::Map::col(i, tid);
#pragma unroll
      for (int k = 0; k < KV; ++k) {
        const bool ok = rr < rows_ok && cc + k < cols_ok;
        float dv = Elem<T>::to_f(rd.r[i].v[k]);
        const float xv = Elem<T>::to_f(rx.r[i].v[k]);
        if (softplus) dv = ok ? softplusf(dv + p.delta_bias[e0 + cc + k]) : 0.f;
        s_dd[buf][rr][cc + k] = make_float2(dv, dv * xv);
        s_xz[buf][rr][cc + k] = make_float2(xv, gz ? Elem<T>::to_f(rz.r[i].v[k]) : 0.f);
      }
    }
#pragma unroll
    for (int i = 0; i < BcRegs::Map::kPerThread; ++i) {
      if (!BcRegs::Map::owns(i, tid)) continue;
      const int rr = BcRegs::Map::row(i, tid), cc = BcRegs::Map::col(i, tid);
#pragma unroll
      for (int k = 0; k < KVB; ++k) {
        s_B[buf][rr][cc + k] = Elem<T>::to_f(rB.r[i].v[k]);
        s_C[buf][rr][cc + k] = Elem<T>::to_f(rC.r[i].v[k]);
      }
    }
  };

  const int64_t ntiles = (p.L + kTT - 1) / kTT;
  const int64_t nchunks = (p.L + kChunk - 1) / kChunk;
  fetch(0);
  commit(0, 0);
  __syncthreads();

  for (int64_t k = 0; k < ntiles; ++k) {
    const int buf = int(k & 1);
    const int64_t t0 = k * kTT;
    if (k + 1 < ntiles) fetch(t0 + kTT);

#pragma unroll 1
    for (int w = 0; w < kTT / kLPE; ++w) {
      float yp[kLPE];
#pragma unroll
      for (int i = 0; i < kLPE; ++i) {
        const int t = w * kLPE + i;
        if (p.carries && (t % kChunk) == 0 && t0 + t < p.L && e_ok) {
          float4* dst = reinterpret_cast<float4*>(
              p.carries + ((b * nchunks + (t0 + t) / kChunk) * p.ED + e) * N + 4 * q);
          *dst = make_float4(h[0], h[1], h[2], h[3]);
        }
        const float2 dd = s_dd[buf][t][e_l];
        const float4 Bq = *reinterpret_cast<const float4*>(&s_B[buf][t][4 * q]);
        const float4 Cq = *reinterpret_cast<const float4*>(&s_C[buf][t][4 * q]);
        const float bq[4] = {Bq.x, Bq.y, Bq.z, Bq.w};
        const float cq[4] = {Cq.x, Cq.y, Cq.z, Cq.w};
        float acc = 0.f;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float a = ex2f(dd.x * A2[j]);
          h[j] = fmaf(a, h[j], dd.y * bq[j]);
          acc = fmaf(h[j], cq[j], acc);
        }
        yp[i] = acc;
      }
      if (gy) {
        // transpose-reduce: lane q ends with the full sum of timestep w*kLPE + q
#pragma unroll
        for (int s = kLPE / 2; s >= 1; s >>= 1) {
          const bool up = (q & s) != 0;
#pragma unroll
          for (int i = 0; i < s; ++i) {
            const float send = up ? yp[i] : yp[i + s];
            const float keep = up ? yp[i + s] : yp[i];
            yp[i] = keep + __shfl_xor_sync(0xffffffffu, send, s);
          }
        }
        const int t = w * kLPE + q;
        const float2 xz = s_xz[buf][t][e_l];
        float yv = fmaf(Dv, xz.x, yp[0]);
        if (gz) yv *= xz.y * sigmoidf(xz.y);
        s_y[t][e_l] = Elem<T>::from_f(yv);
      }
    }
    __syncthreads();
    if (gy) {
      // coalesced write of the finished tile (same vector split as the loads)
      ActRegs ry;
      const int rows_ok = int(min64(kTT, p.L - t0));
#pragma unroll
      for (int i = 0; i < ActRegs::Map::kPerThread; ++i)
        if (ActRegs::Map::owns(i, tid))
          ry.r[i] = *reinterpret_cast<const TVec<T, KV>*>(
              &s_y[ActRegs::Map::row(i, tid)][ActRegs::Map::col(i, tid)]);
      ry.store(gy + t0 * p.y_sl, p.y_sl, rows_ok, cols_ok, tid);
    }
    if (k + 1 < ntiles) commit(buf ^ 1, t0 + kTT);
    __syncthreads();
  }

  if (p.hT && e_ok) {
    float4* dst = reinterpret_cast<float4*>(p.hT + (b * p.ED + e) * N + 4 * q);
    *dst = make_float4(h[0], h[1], h[2], h[3]);
  }
}

template <typename T, int N>
int launch_n(const SscanFwdParams& p, bool vec, cudaStream_t st) {
  using G = SscanGeom<N>;
  dim3 grid(unsigned((p.ED + G::kTE - 1) / G::kTE), unsigned(p.B));
  constexpr int KV = Elem<T>::kVec;
  if (vec) sscan_fwd_kernel<T, N, KV><<<grid, kThreadsPerCta, 0, st>>>(p);
  else sscan_fwd_kernel<T, N, 1><<<grid, kThreadsPerCta, 0, st>>>(p);
  return check_launch();
}

template <typename T>
int launch_t(const SscanFwdParams& p, int N, bool vec, cudaStream_t st) {
  switch (N) {
    case 8: return launch_n<T, 8>(p, vec, st);
    case 16: return launch_n<T, 16>(p, vec, st);
    case 32: return launch_n<T, 32>(p, vec, st);
    case 64: return launch_n<T, 64>(p, vec, st);
    default: return MB200_ENSTATE;
  }
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" int mb200_sscan_chunk(void) { return kChunk; }

extern "C" int mb200_sscan_fwd(const void* x, const void* delta, const void* z, const float* A,
                               const void* Bm, const void* Cm, const float* D,
                               const float* delta_bias, const float* h0, void* y, float* hT,
                               float* carries, int64_t B, int64_t L, int64_t ED, int N,
                               int64_t x_sb, int64_t x_sl, int64_t d_sb, int64_t d_sl,
                               int64_t z_sb, int64_t z_sl, int64_t b_sb, int64_t b_sl,
                               int64_t c_sb, int64_t c_sl, int64_t y_sb, int64_t y_sl,
                               int dtype, int flags, void* stream) {
  if (B < 0 || L < 0 || ED < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (N != 8 && N != 16 && N != 32 && N != 64) return MB200_ENSTATE;
  if (B == 0 || ED == 0) return MB200_OK;
  if (L == 0) {                                   // empty sequence: the state passes through
    if (hT) {
      cudaStream_t st = static_cast<cudaStream_t>(stream);
      if (h0) cudaMemcpyAsync(hT, h0, sizeof(float) * B * ED * N, cudaMemcpyDeviceToDevice, st);
      else cudaMemsetAsync(hT, 0, sizeof(float) * B * ED * N, st);
    }
    return check_launch();
  }
  if (!x || !delta || !A || !Bm || !Cm) return MB200_EINVAL;
  if ((flags & MB200_DELTA_SOFTPLUS) && !delta_bias) return MB200_EINVAL;
  if (B > 65535) return MB200_ETOOBIG;
  if (!aligned16(h0) || !aligned16(hT) || !aligned16(carries)) return MB200_EALIGN;
  SscanFwdParams p;
  p.x = x; p.delta = delta; p.z = z; p.A = A; p.Bm = Bm; p.Cm = Cm; p.D = D;
  p.delta_bias = delta_bias; p.h0 = h0; p.y = y; p.hT = hT; p.carries = carries;
  p.B = B; p.L = L; p.ED = ED;
  p.x_sb = x_sb; p.x_sl = x_sl; p.d_sb = d_sb; p.d_sl = d_sl; p.z_sb = z_sb; p.z_sl = z_sl;
  p.b_sb = b_sb; p.b_sl = b_sl; p.c_sb = c_sb; p.c_sl = c_sl; p.y_sb = y_sb; p.y_sl = y_sl;
  p.flags = flags;
  const int kv = dtype == MB200_F32 ? 4 : 8;
  bool vec = ED % kv == 0 && aligned16(x) && aligned16(delta) && aligned16(z) && aligned16(y) &&
             aligned16(Bm) && aligned16(Cm);
  for (int64_t s : {x_sb, x_sl, d_sb, d_sl, y_sb, y_sl, b_sb, b_sl, c_sb, c_sl}) vec = vec && s % kv == 0;
  if (z) vec = vec && z_sb % kv == 0 && z_sl % kv == 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MB200_F32 ? launch_t<float>(p, N, vec, st)
                            : launch_t<__nv_bfloat16>(p, N, vec, st);
}
