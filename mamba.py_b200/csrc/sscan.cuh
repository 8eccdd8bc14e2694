// Geometry and parameter blocks shared by the fused selective-scan kernels.
#pragma once
#include "common.cuh"
#include "tile.cuh"

namespace mb200 {

// Timesteps between two saved states.  The backward kernels keep the states of one chunk in
// registers while they walk it in reverse (kChunk * 4 floats per thread), which fixes this at 8:
// the saved states cost kChunk times less memory than the full state tensor the reference keeps.
constexpr int kChunk = 8;

// A thread owns 4 states of one channel, so N/4 lanes share a channel and a 128-thread CTA
// covers 128/(N/4) channels.  kTT is the number of timesteps staged per shared-memory tile.
template <int N> struct SscanGeom {
  static_assert(N % 4 == 0 && N >= 8 && N <= 64, "d_state must be 8, 16, 32 or 64");
  static constexpr int kLPE = N / 4;                       // lanes per channel
  static constexpr int kTE = kThreadsPerCta / kLPE;        // channels per CTA
  static constexpr int kTT = (N == 16 || N == 32) ? 32 : 16;   // timesteps per tile (fits 48 KB static smem)
};

// The operand tile holds one float2 {delta, delta*x} per (timestep, channel).  Two channels share
// a 16-byte slot; slot s of row t is stored at physical slot swz(t, s).  The XOR spreads the
// slots that one quarter-warp of the commit writes together (and odd/even rows) over different
// banks, so the commit's 128-bit stores and the hot loop's 64-bit loads are conflict free.
__device__ __forceinline__ int swz(int t, int s) {
  return s ^ ((s >> 3) & 1) ^ ((t & 1) << 1);
}
// float2 index of channel column c in row t of a tile that is `te` channels wide
__device__ __forceinline__ int op_index(int t, int c, int te) {
  return t * te + swz(t, c >> 1) * 2 + (c & 1);
}

// four consecutive channels of one timestep, moved with one 8- or 16-byte access
template <typename T> struct alignas(sizeof(T) * 4) Vec4 {
  T v[4];
};

// Sum of the kLPE partial sums the lanes of one channel left in shared memory.
template <int kLPE>
__device__ __forceinline__ float sum_lanes(const float* p) {
  if constexpr (kLPE == 2) {
    const float2 v = *reinterpret_cast<const float2*>(p);
    return v.x + v.y;
  } else {
    float s = 0.f;
#pragma unroll
    for (int l = 0; l < kLPE; l += 4) {
      const float4 v = *reinterpret_cast<const float4*>(p + l);
      s += (v.x + v.y) + (v.z + v.w);
    }
    return s;
  }
}

// Commit the fetched B and C tiles (kTT-or-kChunk rows of N values) to shared memory as float32.
template <typename T, int N, int KVB, typename Regs>
__device__ __forceinline__ void commit_bc(const Regs& rB, const Regs& rC, float* sB, float* sC, int tid) {
  using Map = typename Regs::Map;
#pragma unroll
  for (int i = 0; i < Map::kPerThread; ++i) {
    if (!Map::owns(i, tid)) continue;
    const int rr = Map::row(i, tid), cc = Map::col(i, tid);
    float* db = sB + rr * N + cc;
    float* dc = sC + rr * N + cc;
    if constexpr (KVB % 4 == 0) {
#pragma unroll
      for (int k = 0; k < KVB; k += 4) {
        *reinterpret_cast<float4*>(db + k) =
            make_float4(Elem<T>::to_f(rB.r[i].v[k]), Elem<T>::to_f(rB.r[i].v[k + 1]),
                        Elem<T>::to_f(rB.r[i].v[k + 2]), Elem<T>::to_f(rB.r[i].v[k + 3]));
        *reinterpret_cast<float4*>(dc + k) =
            make_float4(Elem<T>::to_f(rC.r[i].v[k]), Elem<T>::to_f(rC.r[i].v[k + 1]),
                        Elem<T>::to_f(rC.r[i].v[k + 2]), Elem<T>::to_f(rC.r[i].v[k + 3]));
      }
    } else {
#pragma unroll
      for (int k = 0; k < KVB; ++k) {
        db[k] = Elem<T>::to_f(rB.r[i].v[k]);
        dc[k] = Elem<T>::to_f(rC.r[i].v[k]);
      }
    }
  }
}

struct SscanFwdParams {
  const void *x, *delta, *z, *Bm, *Cm;
  const float *A, *D, *delta_bias, *h0;
  void* y;
  float *hT, *carries;
  float* pT = nullptr;         // (B, ED, N) decay product of the whole span; written by the state-only pass
  int64_t B, L, ED;
  int64_t x_sb, x_sl, d_sb, d_sl, z_sb, z_sl, b_sb, b_sl, c_sb, c_sl, y_sb, y_sl;
  int flags;
};

struct SscanBwdParams {
  const void *x, *delta, *z, *Bm, *Cm, *dy;
  const float *A, *D, *delta_bias, *carries, *g_in;
  void *dx, *ddelta, *dz;
  float *dB, *dC, *dA, *dD, *ddelta_bias, *g_out;
  int64_t B, L, ED;
  int64_t x_sb, x_sl, d_sb, d_sl, z_sb, z_sl, b_sb, b_sl, c_sb, c_sl, dy_sb, dy_sl;
  int64_t dx_sb, dx_sl, dd_sb, dd_sl, dz_sb, dz_sl;
  int flags;
};

}  // namespace mb200

// Internal flag (never part of the public flags): run the forward kernel as the reverse carry pass.
namespace mb200 { constexpr int kFlagCarryPass = 1 << 16; }
int mb200_fwd_tma_try(const mb200::SscanFwdParams& p, int N, int dtype, cudaStream_t st);

// Device-side status words of the kernels that contain bounded waits (host functions; each reads
// and clears its kernel's word, synchronising the device).
int mb200_fwd_device_status();
int mb200_bwd_device_status();
