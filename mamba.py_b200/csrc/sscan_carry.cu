// Reverse carry pass of the sequence-sharded backward: for a shard of the sequence, the gradient
// carry that leaves its first timestep when no carry enters its last one,
//     gc <- a[t] * (dy'[t] * C[t] + gc),   t = L-1 ... 0,   a = exp(delta * A),  dy' = dy * silu(z).
// It needs no hidden states, reads delta, z, dy, C once and writes (B, ED, N) floats.  Thread and tile
// mapping are those of the forward kernel, walked from the last tile to the first.
#include "common.cuh"
#include "tile.cuh"
#include "sscan.cuh"

namespace mb200 {
namespace {

struct CarryParams {
  const void *delta, *z, *dy, *Cm;
  const float *A, *delta_bias;
  float* g_out;
  int64_t B, L, ED;
  int64_t d_sb, d_sl, z_sb, z_sl, dy_sb, dy_sl, c_sb, c_sl;
  int flags;
};

template <typename T, int N, int KV>
__global__ void __launch_bounds__(kThreadsPerCta)
sscan_bwd_carry_kernel(const CarryParams p) {
  using G = SscanGeom<N>;
  constexpr int kLPE = G::kLPE, kTE = G::kTE, kTT = G::kTT;
  constexpr int KVB = (N % KV == 0) ? KV : 1;
  using ActRegs = TileRegs<T, kTT, kTE, KV>;
  using BcRegs = TileRegs<T, kTT, N, KVB>;

  __shared__ __align__(16) float2 s_dv[2][kTT][kTE];   // {delta, dy'}
  __shared__ __align__(16) float s_C[2][kTT][N];

  const int tid = threadIdx.x;
  const int e_l = tid / kLPE, q = tid % kLPE;
  const int64_t e0 = int64_t(blockIdx.x) * kTE;
  const int64_t e = e0 + e_l;
  const int64_t b = blockIdx.y;
  const bool e_ok = e < p.ED;
  const int cols_ok = int(min64(kTE, p.ED - e0));
  const bool has_z = p.z != nullptr;
  const bool softplus = (p.flags & MB200_DELTA_SOFTPLUS) != 0;

  const T* gd = static_cast<const T*>(p.delta) + b * p.d_sb + e0;
  const T* gz = has_z ? static_cast<const T*>(p.z) + b * p.z_sb + e0 : nullptr;
  const T* gdy = static_cast<const T*>(p.dy) + b * p.dy_sb + e0;
  const T* gC = static_cast<const T*>(p.Cm) + b * p.c_sb;

  float A2[4], gc[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    A2[j] = e_ok ? p.A[e * N + 4 * q + j] * kLog2e : 0.f;
    gc[j] = 0.f;
  }

  ActRegs rd, rz, rdy;
  BcRegs rC;
  auto fetch = [&](int64_t t0) {
    const int rows_ok = int(min64(kTT, p.L - t0));
    rd.load(gd + t0 * p.d_sl, p.d_sl, rows_ok, cols_ok, tid);
    rdy.load(gdy + t0 * p.dy_sl, p.dy_sl, rows_ok, cols_ok, tid);
    if (has_z) rz.load(gz + t0 * p.z_sl, p.z_sl, rows_ok, cols_ok, tid);
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
        if (softplus) dv = ok ? softplusf(dv + p.delta_bias[e0 + cc + k]) : 0.f;
        float dyv = Elem<T>::to_f(rdy.r[i].v[k]);
        if (has_z) {
          const float zv = Elem<T>::to_f(rz.r[i].v[k]);
          dyv *= zv * sigmoidf(zv);
        }
        s_dv[buf][rr][cc + k] = make_float2(dv, dyv);
      }
    }
#pragma unroll
    for (int i = 0; i < BcRegs::Map::kPerThread; ++i) {
      if (!BcRegs::Map::owns(i, tid)) continue;
      const int rr = BcRegs::Map::row(i, tid), cc = BcRegs::Map::col(i, tid);
#pragma unroll
      for (int k = 0; k < KVB; ++k) s_C[buf][rr][cc + k] = Elem<T>::to_f(rC.r[i].v[k]);
    }
  };

  const int64_t ntiles = (p.L + kTT - 1) / kTT;
  fetch((ntiles - 1) * kTT);
  commit(0, (ntiles - 1) * kTT);
  __syncthreads();
  int buf = 0;
  for (int64_t k = ntiles - 1; k >= 0; --k, buf ^= 1) {
    if (k > 0) fetch((k - 1) * kTT);
#pragma unroll 8
    for (int t = kTT - 1; t >= 0; --t) {
      const float2 dv = s_dv[buf][t][e_l];
      const float4 Cq = *reinterpret_cast<const float4*>(&s_C[buf][t][4 * q]);
      const float cq[4] = {Cq.x, Cq.y, Cq.z, Cq.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) gc[j] = ex2f(dv.x * A2[j]) * fmaf(dv.y, cq[j], gc[j]);
    }
    if (k > 0) commit(buf ^ 1, (k - 1) * kTT);
    __syncthreads();
  }
  if (e_ok)
    *reinterpret_cast<float4*>(p.g_out + (b * p.ED + e) * N + 4 * q) =
        make_float4(gc[0], gc[1], gc[2], gc[3]);
}

template <typename T, int N>
int launch_n(const CarryParams& p, bool vec, cudaStream_t st) {
  using G = SscanGeom<N>;
  dim3 grid(unsigned((p.ED + G::kTE - 1) / G::kTE), unsigned(p.B));
  constexpr int KV = Elem<T>::kVec;
  if (vec) sscan_bwd_carry_kernel<T, N, KV><<<grid, kThreadsPerCta, 0, st>>>(p);
  else sscan_bwd_carry_kernel<T, N, 1><<<grid, kThreadsPerCta, 0, st>>>(p);
  return check_launch();
}

template <typename T>
int launch_t(const CarryParams& p, int N, bool vec, cudaStream_t st) {
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

extern "C" int mb200_sscan_bwd_carry(const void* delta, const void* z, const void* dy, const void* Cm,
                                     const float* A, const float* delta_bias, float* g_out,
                                     int64_t B, int64_t L, int64_t ED, int N,
                                     int64_t d_sb, int64_t d_sl, int64_t z_sb, int64_t z_sl,
                                     int64_t dy_sb, int64_t dy_sl, int64_t c_sb, int64_t c_sl,
                                     int dtype, int flags, void* stream) {
  if (B < 0 || L < 0 || ED < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (N != 8 && N != 16 && N != 32 && N != 64) return MB200_ENSTATE;
  if (B == 0 || ED == 0) return MB200_OK;
  if (!g_out) return MB200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (L == 0) {
    cudaMemsetAsync(g_out, 0, sizeof(float) * B * ED * N, st);
    return check_launch();
  }
  if (!delta || !dy || !Cm || !A) return MB200_EINVAL;
  if ((flags & MB200_DELTA_SOFTPLUS) && !delta_bias) return MB200_EINVAL;
  if (B > 65535) return MB200_ETOOBIG;
  if (!aligned16(g_out)) return MB200_EALIGN;
  CarryParams p;
  p.delta = delta; p.z = z; p.dy = dy; p.Cm = Cm; p.A = A; p.delta_bias = delta_bias; p.g_out = g_out;
  p.B = B; p.L = L; p.ED = ED;
  p.d_sb = d_sb; p.d_sl = d_sl; p.z_sb = z_sb; p.z_sl = z_sl; p.dy_sb = dy_sb; p.dy_sl = dy_sl;
  p.c_sb = c_sb; p.c_sl = c_sl; p.flags = flags;
  {
    // tensor-map path: the forward kernel in its carry mode (dy in the place of x, C in the place of B)
    SscanFwdParams f;
    f.x = dy; f.delta = delta; f.z = z; f.Bm = Cm; f.Cm = Cm; f.A = A; f.D = nullptr;
    f.delta_bias = delta_bias; f.h0 = nullptr; f.y = nullptr; f.hT = g_out; f.carries = nullptr;
    f.B = B; f.L = L; f.ED = ED;
    f.x_sb = dy_sb; f.x_sl = dy_sl; f.d_sb = d_sb; f.d_sl = d_sl; f.z_sb = z_sb; f.z_sl = z_sl;
    f.b_sb = c_sb; f.b_sl = c_sl; f.c_sb = c_sb; f.c_sl = c_sl; f.y_sb = 0; f.y_sl = 0;
    f.flags = (flags & MB200_DELTA_SOFTPLUS) | MB200_REVERSE | kFlagCarryPass;
    const int rc = mb200_fwd_tma_try(f, N, dtype, st);
    if (rc <= 0) return rc;                                  // launched, or failed hard
  }
  const int kv = dtype == MB200_F32 ? 4 : 8;
  bool vec = ED % kv == 0 && aligned16(delta) && aligned16(z) && aligned16(dy) && aligned16(Cm);
  for (int64_t s : {d_sb, d_sl, dy_sb, dy_sl, c_sb, c_sl}) vec = vec && s % kv == 0;
  if (z) vec = vec && z_sb % kv == 0 && z_sl % kv == 0;
  return dtype == MB200_F32 ? launch_t<float>(p, N, vec, st) : launch_t<__nv_bfloat16>(p, N, vec, st);
}
