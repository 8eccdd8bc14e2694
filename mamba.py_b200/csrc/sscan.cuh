// Geometry and parameter blocks shared by the fused selective-scan kernels.
#pragma once
#include "common.cuh"
#include "tile.cuh"

namespace mb200 {

// Timesteps between two saved states.  The backward kernel keeps one chunk of decay factors
// and states in registers (2 * kChunk * 4 floats per thread), which fixes this at 16.
constexpr int kChunk = 16;

// A thread owns 4 states of one channel, so N/4 lanes share a channel and a 128-thread CTA
// covers 128/(N/4) channels.  kTT is the number of timesteps staged per shared-memory tile.
template <int N> struct SscanGeom {
  static_assert(N % 4 == 0 && N >= 8 && N <= 64, "d_state must be 8, 16, 32 or 64");
  static constexpr int kLPE = N / 4;                       // lanes per channel
  static constexpr int kTE = kThreadsPerCta / kLPE;        // channels per CTA
  static constexpr int kTT = N >= 16 ? 32 : 16;            // timesteps per tile
};

struct SscanFwdParams {
  const void *x, *delta, *z, *Bm, *Cm;
  const float *A, *D, *delta_bias, *h0;
  void* y;
  float *hT, *carries;
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
