// Fused selective scan, backward.  One pass over x, delta, z, B, C, dy (read once) that writes
// dx, ddelta, dz and accumulates dB, dC, dA, dD; the hidden states are recomputed chunk by chunk
// from the states the forward saved every kChunk (8) timesteps.
//
// The kernel is bound by shared-memory traffic, instruction issue and the latency of each warp's
// dependent chain, not by HBM, so the recurrences run on warps that do nothing else (tensor-map
// path, d_state 16; the register-staged kernel in sscan_bwd_generic.cuh covers every other case).
//
// A CTA of 256 threads owns 32 channels of one batch row and walks time BACKWARDS in tiles of 16
// (two saved states per tile):
//   - warp 4 issues TMA loads of the raw x, delta, z, dy, B, C boxes a few tiles ahead into a
//     shared-memory ring and converts each landed tile into float32 operands
//     ({softplus(delta+bias), delta*x}, dy*silu(z), B, C; double-buffered).
//   - warps 0-3 (consumers; a thread owns 4 states of one channel) recompute the 8 states of a
//     chunk forwards from its saved state into registers and walk them backwards:
//     g[t] = dy'[t] C[t] + a[t+1] g[t+1],  da = g h[t-1].  Operands of the walk are fetched two
//     timesteps ahead.  Per timestep a thread leaves three partial sums over its 4 states (for y,
//     dx, ddelta) and its 8 products for dB, dC in shared memory, in windows of 2 timesteps.
//   - warps 5 and 7 finish alternate windows: sum the 4 partials of each channel, form dx, ddelta,
//     dz (and the running sums for dD and d(delta_bias)), store them.  delta and dy' come from the
//     operand tile, so only sigmoid(z) and 1 - exp(-delta) are evaluated here.
//   - warp 6 sums the dB, dC products of each window over the CTA's 32 channels and adds the
//     result to global memory with vector atomics.
//   - Hand-off through CTA-local mbarriers; every wait is bounded (see mbar_wait).  A barrier's
//     round trip through the busy shared-memory pipe costs a few hundred cycles, so the consumers
//     ask for a window's buffer with a non-blocking test before the arithmetic of the window and
//     only block if the answer was "not yet".
#include "sscan_bwd_generic.cuh"
#include "tma.cuh"

namespace mb200 {
namespace {

constexpr int kBN = 16;                      // d_state of this path
constexpr int kBTE = 32;                     // channels per CTA
constexpr int kBTile = 2 * kChunk;           // timesteps per tile (two saved states per tile)
constexpr int kHalf = kChunk;                // states kept in registers at a time
constexpr int kBWin = 2;                     // timesteps per reduction window
constexpr int kWinsPerTile = kBTile / kBWin;
constexpr int kBwdThreads = 256;
constexpr int kEpStride = 34;                // float4 per (t, which, q) row of the dB/dC products

__device__ int g_bwd_status = MB200_DEV_OK;

template <typename T> struct alignas(sizeof(T) * 2) Vec2 {
  T v[2];
};

struct BwdMaps {
  CUtensorMap x, d, z, dy, B, C;
};

template <typename T> struct TmaBwdSmem {
  static constexpr int kStages = sizeof(T) == 2 ? 6 : 3;
  static constexpr int kActBytes = kBTile * kBTE * int(sizeof(T));
  static constexpr int kBcBytes = kBTile * kBN * int(sizeof(T));
  static constexpr int kStageBytes = 4 * kActBytes + 2 * kBcBytes;       // x, delta, z, dy, B, C
  static constexpr int kRaw = 0;
  static constexpr int kOp = kRaw + kStages * kStageBytes;                // float2 [2][16][32]
  static constexpr int kDyp = kOp + 2 * kBTile * kBTE * 8;                // float  [2][16][32]
  static constexpr int kB = kDyp + 2 * kBTile * kBTE * 4;                 // float  [2][16][16]
  static constexpr int kC = kB + 2 * kBTile * kBN * 4;
  static constexpr int kNp = kC + 2 * kBTile * kBN * 4;                   // float  [2][kBWin][3][128]
  static constexpr int kEp = kNp + 2 * kBWin * 3 * 128 * 4;                  // float4 [2][kBWin][2][4][kEpStride]
  static constexpr int kD = kEp + 2 * kBWin * 2 * 4 * kEpStride * 16;     // float [32]
  static constexpr int kBias = kD + kBTE * 4;
  static constexpr int kBars = kBias + kBTE * 4;                          // 2*kStages + 8 mbarriers
  static constexpr int kBytes = kBars + (2 * kStages + 8) * 8;
};

// The partial sums over a thread's 4 states (for y, dx, ddelta) go to three planes of 128 floats per
// timestep; the 4 lanes of a channel are neighbours, so a finishing thread fetches one sum of one
// channel with a single 16-byte load.  np_chan(c) is the float4 position of channel c in a plane: the
// XOR keeps the finishing warps' loads (channels 2l, 2l+1 per lane) free of bank conflicts.
__device__ __forceinline__ int np_chan(int c) { return c ^ ((c >> 3) & 1); }

__device__ __forceinline__ void red_add_v4(float* addr, float a, float b, float c, float d) {
  asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(a), "f"(b), "f"(c), "f"(d) : "memory");
}

// The softplus option and the presence of the gate are template parameters too: as run-time flags they
// cost the converter and finishing warps (the busiest ones) branches and selects, 6 % of the launch.
template <typename T, bool kRev, bool kSoftplus, bool kHasZ>
__global__ void __launch_bounds__(kBwdThreads, 3)
sscan_bwd_tma_kernel(const __grid_constant__ BwdMaps maps, const SscanBwdParams p) {
  using S = TmaBwdSmem<T>;
  constexpr int kStages = S::kStages, kAhead = S::kStages - 2;
  constexpr int N = kBN;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  float2* s_op = reinterpret_cast<float2*>(smem_raw + S::kOp);
  float* s_dyp = reinterpret_cast<float*>(smem_raw + S::kDyp);
  float* s_B = reinterpret_cast<float*>(smem_raw + S::kB);
  float* s_C = reinterpret_cast<float*>(smem_raw + S::kC);
  float* s_np = reinterpret_cast<float*>(smem_raw + S::kNp);
  float4* s_ep = reinterpret_cast<float4*>(smem_raw + S::kEp);
  float* s_D = reinterpret_cast<float*>(smem_raw + S::kD);
  float* s_bias = reinterpret_cast<float*>(smem_raw + S::kBias);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + S::kBars);
  uint64_t* raw_full = bars;                      // [kStages] copy landed
  uint64_t* raw_free = bars + kStages;            // [kStages] warps 4, 5, 7 are done with the stage
  uint64_t* op_full = bars + 2 * kStages;         // [2] operands committed (warp 4)
  uint64_t* op_empty = op_full + 2;               // [2] consumers are done with the operand buffer
  uint64_t* win_full = op_full + 4;               // [2] consumers filled a window of partials
  uint64_t* win_empty = op_full + 6;              // [2] finishing warps drained it

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int64_t e0 = int64_t(blockIdx.x) * kBTE;
  const int64_t b = blockIdx.y;
  const int cols_ok = int(min64(kBTE, p.ED - e0));
  constexpr bool softplus = kSoftplus;
  constexpr bool has_z = kHasZ;
  const int64_t ntiles = (p.L + kBTile - 1) / kBTile;
  // Direction of the scan being differentiated (MB200_REVERSE: it ran from t = L-1 down to 0).  Tiles
  // are taken in the opposite order of that scan: iteration j works on the tile that starts at
  // tile_t0(j); step s of a tile in the scan's own order is its row `row(s)`.  Saved states are
  // indexed by time chunk: entry c is the state entering chunk c in the scan direction.
  constexpr bool rev = kRev;
  auto tile_t0 = [&](int64_t j) { return (rev ? j : ntiles - 1 - j) * kBTile; };
  auto row = [](int s) { return rev ? kBTile - 1 - s : s; };

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < kStages; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_free[i], 96); }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mbar_init(&op_full[i], 32); mbar_init(&op_empty[i], 128 + 64);
      mbar_init(&win_full[i], 128); mbar_init(&win_empty[i], 64);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < kBTE; i += kBwdThreads) {
    const bool ok = i < cols_ok;
    s_D[i] = (ok && p.D) ? p.D[e0 + i] : 0.f;
    s_bias[i] = (ok && softplus) ? p.delta_bias[e0 + i] : 0.f;
  }
  __syncthreads();
  auto fail = [&]() { atomicExch(&g_bwd_status, MB200_DEV_WAIT_TIMEOUT); };

  // The recurrence warps need far more registers than the others: hand 32 registers per thread of
  // warps 4-7 over to warps 0-3 (the kernel is compiled for 80; 128 * 48 + 128 * 112 = 256 * 80).
  if (warp < 4) {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 112;");
  } else {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 48;");
  }
  if (warp < 4) {
    // ================================================================== consumers
    const int e_l = tid >> 2, q = tid & 3;
    const int64_t e = e0 + e_l;
    const bool e_ok = e < p.ED;
    float2 A2[2], gc[2], dAacc[2];
    {
      float a4[4], g4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a4[j] = e_ok ? p.A[e * N + 4 * q + j] * kLog2e : 0.f;
        g4[j] = (e_ok && p.g_in) ? p.g_in[(b * p.ED + e) * N + 4 * q + j] : 0.f;
      }
      A2[0] = make_float2(a4[0], a4[1]); A2[1] = make_float2(a4[2], a4[3]);
      gc[0] = make_float2(g4[0], g4[1]); gc[1] = make_float2(g4[2], g4[3]);
      dAacc[0] = dAacc[1] = make_float2(0.f, 0.f);
    }
    const int op_off0 = op_index(0, e_l, kBTE), op_off1 = op_index(1, e_l, kBTE) - kBTE;
    const int npo = np_chan(e_l) * 4 + q;
    const int64_t nchunks = (p.L + kHalf - 1) / kHalf;
    const float* carry_base = p.carries + (b * nchunks * p.ED + e) * N + 4 * q;
    auto load_carry = [&](int64_t c) {
      return (e_ok && c < nchunks) ? *reinterpret_cast<const float4*>(carry_base + c * p.ED * N)
                                   : make_float4(0.f, 0.f, 0.f, 0.f);
    };
    // states entering the first / second half (in scan order) of iteration j's tile
    // (time chunk 2*tile + 1 is the first half in scan order when reversed, chunk 2*tile otherwise)
    float4 carry_next = load_carry(rev ? 1 : 2 * (ntiles - 1)), carry_next_mid = load_carry(rev ? 0 : 2 * (ntiles - 1) + 1);

    for (int64_t j = 0; j < ntiles; ++j) {
      const int buf = int(j & 1);
      const float4 cv = carry_next, cm = carry_next_mid;
      if (j + 1 < ntiles) {                               // the next tile's two states, a tile ahead
        const int64_t c = rev ? 2 * j + 2 : 2 * (ntiles - 2 - j);
        carry_next = load_carry(rev ? c + 1 : c);
        carry_next_mid = load_carry(rev ? c : c + 1);
      }
      if (!mbar_wait(&op_full[buf], int((j >> 1) & 1))) { fail(); return; }
      const float2* op = s_op + buf * kBTile * kBTE;
      const float* dyp = s_dyp + buf * kBTile * kBTE + e_l;
      const float* sB = s_B + buf * kBTile * N + 4 * q;
      const float* sC = s_C + buf * kBTile * N + 4 * q;
      const float2 hp[2] = {make_float2(cv.x, cv.y), make_float2(cv.z, cv.w)};   // state entering the tile

      // one forward step of the recurrence from operands in shared memory
      auto step = [&](int s, float2 (&h)[2]) {
        const int t = row(s);
        const float2 o = op[t * kBTE + ((t & 1) ? op_off1 : op_off0)];
        const float4 Bq = *reinterpret_cast<const float4*>(sB + t * N);
        const float2 dd = make_float2(o.x, o.x), dxx = make_float2(o.y, o.y);
        const float2 e0v = __fmul2_rn(dd, A2[0]), e1v = __fmul2_rn(dd, A2[1]);
        const float2 a0 = make_float2(ex2f(e0v.x), ex2f(e0v.y)), a1 = make_float2(ex2f(e1v.x), ex2f(e1v.y));
        h[0] = __ffma2_rn(a0, h[0], __fmul2_rn(dxx, make_float2(Bq.x, Bq.y)));
        h[1] = __ffma2_rn(a1, h[1], __fmul2_rn(dxx, make_float2(Bq.z, Bq.w)));
      };
      const float2 hmid[2] = {make_float2(cm.x, cm.y), make_float2(cm.z, cm.w)};   // state entering the second half

#pragma unroll 1
      for (int half = 1; half >= 0; --half) {
        // states after each step of this half, in registers
        float2 hh[kHalf][2];
        {
          float2 h[2] = {half ? hmid[0] : hp[0], half ? hmid[1] : hp[1]};
#pragma unroll
          for (int i = 0; i < kHalf; ++i) {
            step(half * kHalf + i, h);
            hh[i][0] = h[0]; hh[i][1] = h[1];
          }
        }
        // operands of the reverse walk are fetched one timestep ahead, so that their trip through the
        // shared-memory pipe overlaps the previous timestep's arithmetic, stores and barrier traffic
        struct Opnd { float2 o; float dy; float4 B, C; };
        auto fetch = [&](int s) {
          const int t = row(s);
          Opnd r;
          r.o = op[t * kBTE + ((t & 1) ? op_off1 : op_off0)];
          r.dy = dyp[t * kBTE];
          r.B = *reinterpret_cast<const float4*>(sB + t * N);
          r.C = *reinterpret_cast<const float4*>(sC + t * N);
          return r;
        };
        Opnd nx = fetch(half * kHalf + kHalf - 1), nx2 = fetch(half * kHalf + kHalf - 2);
#pragma unroll
        for (int wi = kHalf / kBWin - 1; wi >= 0; --wi) {
          // window sequence number: tiles in processing order, windows from the tile's end
          const int64_t wseq = j * kWinsPerTile + (1 - half) * (kHalf / kBWin) + (kHalf / kBWin - 1 - wi);
          const int wb = int(wseq & 1);
          // asked now, needed only before the first store of the window
          const bool slot_free = wseq < 2 || mbar_test(&win_empty[wb], int(((wseq - 2) >> 1) & 1));
          float* np = s_np + wb * kBWin * 3 * 128;
          float4* ep = s_ep + wb * kBWin * 2 * 4 * kEpStride;
#pragma unroll
          for (int ti = kBWin - 1; ti >= 0; --ti) {
            const int i = wi * kBWin + ti;                    // index inside the half
            const int t = half * kHalf + i;                   // index inside the tile
            const Opnd cu = nx;
            nx = nx2;
            if (i > 1) nx2 = fetch(t - 2);
            const float2 o = cu.o;
            const float dyv = cu.dy;
            const float4 Bq = cu.B, Cq = cu.C;
            const float2 dd = make_float2(o.x, o.x), dxx = make_float2(o.y, o.y), dy2 = make_float2(dyv, dyv);
            const float2 Bv[2] = {make_float2(Bq.x, Bq.y), make_float2(Bq.z, Bq.w)};
            const float2 Cv[2] = {make_float2(Cq.x, Cq.y), make_float2(Cq.z, Cq.w)};
            float2 ysum = make_float2(0.f, 0.f), gBs = ysum, wAs = ysum;
            float2 dBp[2], dCp[2];
#pragma unroll
            for (int k = 0; k < 2; ++k) {
              const float2 hcur = hh[i][k];
              const float2 hprev = i ? hh[i - 1][k] : (half ? hmid[k] : hp[k]);
              const float2 g = __ffma2_rn(dy2, Cv[k], gc[k]);
              ysum = __ffma2_rn(hcur, Cv[k], ysum);
              dCp[k] = __fmul2_rn(dy2, hcur);
              dBp[k] = __fmul2_rn(g, dxx);
              gBs = __ffma2_rn(g, Bv[k], gBs);
              const float2 ev = __fmul2_rn(dd, A2[k]);
              gc[k] = __fmul2_rn(make_float2(ex2f(ev.x), ex2f(ev.y)), g);
              const float2 w = __fmul2_rn(gc[k], hprev);
              dAacc[k] = __ffma2_rn(w, dd, dAacc[k]);
              wAs = __ffma2_rn(w, A2[k], wAs);
            }
            if (ti == kBWin - 1 && !slot_free && !mbar_wait(&win_empty[wb], int(((wseq - 2) >> 1) & 1))) { fail(); return; }
            np[(ti * 3 + 0) * 128 + npo] = ysum.x + ysum.y;
            np[(ti * 3 + 1) * 128 + npo] = gBs.x + gBs.y;
            np[(ti * 3 + 2) * 128 + npo] = wAs.x + wAs.y;
            ep[((ti * 2 + 0) * 4 + q) * kEpStride + e_l] = make_float4(dBp[0].x, dBp[0].y, dBp[1].x, dBp[1].y);
            ep[((ti * 2 + 1) * 4 + q) * kEpStride + e_l] = make_float4(dCp[0].x, dCp[0].y, dCp[1].x, dCp[1].y);
          }
          mbar_arrive(&win_full[wb]);
        }
      }
      mbar_arrive(&op_empty[buf]);
    }
    if (e_ok) {
      float* dA = p.dA + e * N + 4 * q;
      atomicAdd(dA + 0, dAacc[0].x); atomicAdd(dA + 1, dAacc[0].y);
      atomicAdd(dA + 2, dAacc[1].x); atomicAdd(dA + 3, dAacc[1].y);
      if (p.g_out)
        *reinterpret_cast<float4*>(p.g_out + (b * p.ED + e) * N + 4 * q) =
            make_float4(gc[0].x, gc[0].y, gc[1].x, gc[1].y);
    }
    return;
  }
  auto stage_ptr = [&](int64_t j) { return smem_raw + S::kRaw + int(j % kStages) * S::kStageBytes; };
  // window wl (0..7, in processing order) of a tile covers timesteps win_t(wl) and win_t(wl) + 1
  auto win_t = [](int wl) { return (wl < 4 ? kHalf : 0) + 2 * (3 - (wl & 3)); };

  if (warp == 4) {
    // ================================================================== loader + converter
    const uint32_t stage_tx = uint32_t((has_z ? 4 : 3) * S::kActBytes + 2 * S::kBcBytes);
    auto issue = [&](int64_t j) -> bool {                       // lane 0 only
      const int r = int(j % kStages);
      if (j >= kStages && !mbar_wait(&raw_free[r], int((j / kStages - 1) & 1))) return false;
      unsigned char* st = stage_ptr(j);
      const int t0 = int(tile_t0(j));
      mbar_expect_tx(&raw_full[r], stage_tx);
      tma_load_3d(st, &maps.x, int(e0), t0, int(b), &raw_full[r]);
      tma_load_3d(st + S::kActBytes, &maps.d, int(e0), t0, int(b), &raw_full[r]);
      if (has_z) tma_load_3d(st + 2 * S::kActBytes, &maps.z, int(e0), t0, int(b), &raw_full[r]);
      tma_load_3d(st + 3 * S::kActBytes, &maps.dy, int(e0), t0, int(b), &raw_full[r]);
      tma_load_3d(st + 4 * S::kActBytes, &maps.B, 0, t0, int(b), &raw_full[r]);
      tma_load_3d(st + 4 * S::kActBytes + S::kBcBytes, &maps.C, 0, t0, int(b), &raw_full[r]);
      return true;
    };
    if (lane == 0) {
      for (int64_t j = 0; j < kAhead && j < ntiles; ++j)
        if (!issue(j)) { fail(); return; }
    }
    for (int64_t j = 0; j < ntiles; ++j) {
      const int buf = int(j & 1);
      const int rows_ok = int(min64(kBTile, p.L - tile_t0(j)));
      if (j >= 2 && !mbar_wait(&op_empty[buf], int(((j - 2) >> 1) & 1))) { fail(); return; }
      if (!mbar_wait(&raw_full[j % kStages], int((j / kStages) & 1))) { fail(); return; }
      const unsigned char* st = stage_ptr(j);
      const T* rx = reinterpret_cast<const T*>(st);
      const T* rd = reinterpret_cast<const T*>(st + S::kActBytes);
      const T* rz = reinterpret_cast<const T*>(st + 2 * S::kActBytes);
      const T* rdy = reinterpret_cast<const T*>(st + 3 * S::kActBytes);
      float2* tile = s_op + buf * kBTile * kBTE;
      float* dyt = s_dyp + buf * kBTile * kBTE;
      const float4 bq = *reinterpret_cast<const float4*>(s_bias + (lane & 7) * 4);   // this lane's 4 channels
      const float bias4[4] = {bq.x, bq.y, bq.z, bq.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int v = lane + 32 * i;
        const int rr = v >> 3, cc = (v & 7) * 4;
        const Vec4<T> xv = *reinterpret_cast<const Vec4<T>*>(rx + rr * kBTE + cc);
        const Vec4<T> dv4 = *reinterpret_cast<const Vec4<T>*>(rd + rr * kBTE + cc);
        const Vec4<T> yv4 = *reinterpret_cast<const Vec4<T>*>(rdy + rr * kBTE + cc);
        Vec4<T> zv4 = yv4;
        if (has_z) zv4 = *reinterpret_cast<const Vec4<T>*>(rz + rr * kBTE + cc);
        float2 o[4];
        float dyo[4];
#pragma unroll
        for (int k = 0; k < 4; k += 2) {                   // two channels at a time (packed arithmetic)
          float2 dv = make_float2(Elem<T>::to_f(dv4.v[k]), Elem<T>::to_f(dv4.v[k + 1]));
          if (softplus) dv = softplus_fast2(__fadd2_rn(dv, make_float2(bias4[k], bias4[k + 1])));
          if (rr >= rows_ok) dv = make_float2(0.f, 0.f);
          const float2 dx2 = __fmul2_rn(dv, make_float2(Elem<T>::to_f(xv.v[k]), Elem<T>::to_f(xv.v[k + 1])));
          o[k] = make_float2(dv.x, dx2.x);
          o[k + 1] = make_float2(dv.y, dx2.y);
          float2 g = make_float2(Elem<T>::to_f(yv4.v[k]), Elem<T>::to_f(yv4.v[k + 1]));
          if (has_z) {
            const float2 zf = make_float2(Elem<T>::to_f(zv4.v[k]), Elem<T>::to_f(zv4.v[k + 1]));
            g = __fmul2_rn(g, __fmul2_rn(zf, sigmoid_fast2(zf)));
          }
          dyo[k] = g.x;
          dyo[k + 1] = g.y;
        }
        *reinterpret_cast<float4*>(tile + op_index(rr, cc, kBTE)) = make_float4(o[0].x, o[0].y, o[1].x, o[1].y);
        *reinterpret_cast<float4*>(tile + op_index(rr, cc + 2, kBTE)) = make_float4(o[2].x, o[2].y, o[3].x, o[3].y);
        *reinterpret_cast<float4*>(dyt + rr * kBTE + cc) = make_float4(dyo[0], dyo[1], dyo[2], dyo[3]);
      }
      const T* rB = reinterpret_cast<const T*>(st + 4 * S::kActBytes);      // B box then C box
      float* dstB = s_B + buf * kBTile * N;
      float* dstC = s_C + buf * kBTile * N;
      constexpr int kBcVecs = kBTile * N / 4;                                // 64
#pragma unroll
      for (int i = 0; i < 2 * kBcVecs / 32; ++i) {
        const int v = lane + 32 * i;
        const Vec4<T> r4 = *reinterpret_cast<const Vec4<T>*>(rB + v * 4);
        float* dst = (v < kBcVecs) ? dstB + v * 4 : dstC + (v - kBcVecs) * 4;
        *reinterpret_cast<float4*>(dst) = make_float4(Elem<T>::to_f(r4.v[0]), Elem<T>::to_f(r4.v[1]),
                                                      Elem<T>::to_f(r4.v[2]), Elem<T>::to_f(r4.v[3]));
      }
      mbar_arrive(&op_full[buf]);
      mbar_arrive(&raw_free[j % kStages]);
      if (lane == 0 && j + kAhead < ntiles && !issue(j + kAhead)) { fail(); return; }
    }
    return;
  }

  if (warp == 6) {
    // ================================================================== dB, dC: sums over channels
    // A lane owns one row of products (timestep of the window, dB | dC, state quad: 16 rows) and one half
    // of the CTA's 32 channels; it adds its 16 float4 and sends the four sums to global memory with one
    // vector atomic.  Rows are kEpStride = 34 float4 apart, which puts rows r and r + 4 into the same
    // banks: the lanes of rows 4..7 and 12..15 therefore take each pair of neighbouring channels in the
    // opposite order (index c ^ 1), through two base pointers, so that no index is computed in the loop.
    const int hf = lane >> 4, r = lane & 15;
    const int ti = r >> 3, which = (r >> 2) & 1, qq = r & 3;       // r = (ti * 2 + which) * 4 + qq
    float* gbase = (which ? p.dC : p.dB) + b * p.L * N + 4 * qq;
    const int nt = int(ntiles);
    for (int j = 0; j < nt; ++j) {
      const int64_t t0 = tile_t0(j);
#pragma unroll 1
      for (int wl = 0; wl < kWinsPerTile; ++wl) {
        const int wseq = j * kWinsPerTile + wl;
        const int wb = wseq & 1;
        if (!mbar_wait(&win_full[wb], (wseq >> 1) & 1)) { fail(); return; }
        const float4* rowp = s_ep + wb * kBWin * 2 * 4 * kEpStride + r * kEpStride + hf * 16;
        const float4* pe = rowp + which;                          // even channels: c ^ which = c + which
        const float4* po = rowp - which;                          // odd channels:  c ^ which = c - which
        float2 acc0 = make_float2(0.f, 0.f), acc1 = acc0;
#pragma unroll
        for (int c = 0; c < kBTE / 2; ++c) {
          const float4 v = (c & 1) ? po[c] : pe[c];
          acc0 = __fadd2_rn(acc0, make_float2(v.x, v.y));
          acc1 = __fadd2_rn(acc1, make_float2(v.z, v.w));
        }
        mbar_arrive(&win_empty[wb]);
        const int64_t t = t0 + row(win_t(wl) + ti);
        if (t < p.L) red_add_v4(gbase + t * N, acc0.x, acc0.y, acc1.x, acc1.y);
      }
    }
    return;
  }

  // ==================================================================== warps 5, 7: dx, ddelta, dz
  {
    const int par = (warp == 5) ? 0 : 1;                 // parity of the windows this warp finishes
    const int ti = lane >> 4, c0 = (lane & 15) * 2;
    T* odx = static_cast<T*>(p.dx) + b * p.dx_sb + e0 + c0;
    T* odd = static_cast<T*>(p.ddelta) + b * p.dd_sb + e0 + c0;
    T* odz = has_z ? static_cast<T*>(p.dz) + b * p.dz_sb + e0 + c0 : nullptr;
    const float Dv[2] = {s_D[c0], s_D[c0 + 1]};
    float dDacc[2] = {0.f, 0.f}, dbacc[2] = {0.f, 0.f};
    for (int64_t j = 0; j < ntiles; ++j) {
      const int64_t t0 = tile_t0(j);
      if (!mbar_wait(&raw_full[j % kStages], int((j / kStages) & 1))) { fail(); return; }
      const unsigned char* st = stage_ptr(j);
      const T* rx = reinterpret_cast<const T*>(st);
      const T* rz = reinterpret_cast<const T*>(st + 2 * S::kActBytes);
      const T* rdy = reinterpret_cast<const T*>(st + 3 * S::kActBytes);
      // delta and dy' come from the operand tile the consumers are reading (still held: this warp
      // is one of the arrivals the converter waits for before it reuses the buffer)
      const int buf = int(j & 1);
      const float2* opt = s_op + buf * kBTile * kBTE;
      const float* dyt = s_dyp + buf * kBTile * kBTE;
#pragma unroll 1
      for (int wl = par; wl < kWinsPerTile; wl += 2) {
        const int64_t wseq = j * kWinsPerTile + wl;
        if (!mbar_wait(&win_full[par], int((wseq >> 1) & 1))) { fail(); return; }
        const float4* np = reinterpret_cast<const float4*>(s_np + (par * kBWin + ti) * 3 * 128);
        float ys[2], gBs[2], wAs[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
          const int cs = np_chan(c0 + k);
          const float4 v0 = np[cs], v1 = np[32 + cs], v2 = np[64 + cs];
          ys[k] = (v0.x + v0.y) + (v0.z + v0.w);
          gBs[k] = (v1.x + v1.y) + (v1.z + v1.w);
          wAs[k] = (v2.x + v2.y) + (v2.z + v2.w);
        }
        mbar_arrive(&win_empty[par]);
        const int tt = row(win_t(wl) + ti);              // row inside the tile
        const int64_t t = t0 + tt;
        if (t < p.L && c0 < cols_ok) {
          const Vec2<T> xv = *reinterpret_cast<const Vec2<T>*>(rx + tt * kBTE + c0);
          const float4 o4 = *reinterpret_cast<const float4*>(opt + op_index(tt, c0, kBTE));   // {delta, delta*x} x 2
          const float2 dyg2 = *reinterpret_cast<const float2*>(dyt + tt * kBTE + c0);
          const float dvs[2] = {o4.x, o4.z}, dygs[2] = {dyg2.x, dyg2.y};
          const Vec2<T> yv2 = *reinterpret_cast<const Vec2<T>*>(rdy + tt * kBTE + c0);
          Vec2<T> zv2 = yv2;
          if (has_z) zv2 = *reinterpret_cast<const Vec2<T>*>(rz + tt * kBTE + c0);
          Vec2<T> ox, od, oz;
#pragma unroll
          for (int k = 0; k < 2; ++k) {
            const float xf = Elem<T>::to_f(xv.v[k]), dyf = Elem<T>::to_f(yv2.v[k]);
            const float dv = dvs[k], dyg = dygs[k];
            // d softplus = sigmoid(raw) = 1 - exp(-softplus(raw)); series where the difference cancels
            float spg = 1.f;
            if (softplus) spg = dv < 1e-2f ? dv * (1.f - dv * (0.5f - dv * (1.f / 6.f))) : 1.f - __expf(-dv);
            float dzv = 0.f;
            if (has_z) {
              const float zf = Elem<T>::to_f(zv2.v[k]);
              const float sg = sigmoid_fast(zf);
              dzv = dyf * fmaf(Dv[k], xf, ys[k]) * sg * (1.f + zf * (1.f - sg));
            }
            const float dxv = fmaf(dyg, Dv[k], dv * gBs[k]);
            const float ddv = fmaf(xf, gBs[k], wAs[k] * (1.f / kLog2e)) * spg;
            if (c0 + k < cols_ok) {
              dDacc[k] = fmaf(dyg, xf, dDacc[k]);
              dbacc[k] += ddv;
            }
            ox.v[k] = Elem<T>::from_f(dxv);
            od.v[k] = Elem<T>::from_f(ddv);
            oz.v[k] = Elem<T>::from_f(dzv);
          }
          if (c0 + 2 <= cols_ok) {
            *reinterpret_cast<Vec2<T>*>(odx + t * p.dx_sl) = ox;
            *reinterpret_cast<Vec2<T>*>(odd + t * p.dd_sl) = od;
            if (has_z) *reinterpret_cast<Vec2<T>*>(odz + t * p.dz_sl) = oz;
          } else {
            odx[t * p.dx_sl] = ox.v[0];
            odd[t * p.dd_sl] = od.v[0];
            if (has_z) odz[t * p.dz_sl] = oz.v[0];
          }
        }
      }
      mbar_arrive(&op_empty[buf]);
      mbar_arrive(&raw_free[j % kStages]);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      if (c0 + k < cols_ok) {
        if (p.dD) atomicAdd(p.dD + e0 + c0 + k, dDacc[k]);
        if (p.ddelta_bias) atomicAdd(p.ddelta_bias + e0 + c0 + k, dbacc[k]);
      }
    }
  }
}

}  // namespace
}  // namespace mb200

namespace mb200 {
namespace {

template <typename T>
int bwd_tma_launch(const SscanBwdParams& p, cudaStream_t st) {
  using S = TmaBwdSmem<T>;
  constexpr bool bf = sizeof(T) == 2;
  BwdMaps m;
  bool ok = tma_encode(&m.x, p.x, bf, p.B, p.L, p.ED, p.x_sb, p.x_sl, kBTE, kBTile) &&
            tma_encode(&m.d, p.delta, bf, p.B, p.L, p.ED, p.d_sb, p.d_sl, kBTE, kBTile) &&
            tma_encode(&m.dy, p.dy, bf, p.B, p.L, p.ED, p.dy_sb, p.dy_sl, kBTE, kBTile) &&
            tma_encode(&m.B, p.Bm, bf, p.B, p.L, kBN, p.b_sb, p.b_sl, kBN, kBTile) &&
            tma_encode(&m.C, p.Cm, bf, p.B, p.L, kBN, p.c_sb, p.c_sl, kBN, kBTile);
  if (ok && p.z) ok = tma_encode(&m.z, p.z, bf, p.B, p.L, p.ED, p.z_sb, p.z_sl, kBTE, kBTile);
  else if (ok) m.z = m.x;
  if (!ok) return 1;                                   // caller falls back to the generic path
  const bool rv = (p.flags & MB200_REVERSE) != 0, sp = (p.flags & MB200_DELTA_SOFTPLUS) != 0, hz = p.z != nullptr;
  void (*k)(const BwdMaps, const SscanBwdParams) = nullptr;
#define MB200_BWD_PICK(R, S, Z) if (rv == R && sp == S && hz == Z) k = sscan_bwd_tma_kernel<T, R, S, Z>;
  MB200_BWD_PICK(false, false, false) MB200_BWD_PICK(false, false, true)
  MB200_BWD_PICK(false, true, false) MB200_BWD_PICK(false, true, true)
  MB200_BWD_PICK(true, false, false) MB200_BWD_PICK(true, false, true)
  MB200_BWD_PICK(true, true, false) MB200_BWD_PICK(true, true, true)
#undef MB200_BWD_PICK
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes) != cudaSuccess)
    return MB200_ELAUNCH;
  dim3 grid(unsigned((p.ED + kBTE - 1) / kBTE), unsigned(p.B));
  k<<<grid, kBwdThreads, S::kBytes, st>>>(m, p);
  return check_launch();
}

bool bwd_tma_path_ok(const SscanBwdParams& p, int N, int es) {
  if (N != kBN || p.L >= (int64_t(1) << 31) || p.ED >= (int64_t(1) << 31)) return false;
  bool ok = tma_compatible(p.x, p.x_sb, p.x_sl, p.ED, es, kBTE) &&
            tma_compatible(p.delta, p.d_sb, p.d_sl, p.ED, es, kBTE) &&
            tma_compatible(p.dy, p.dy_sb, p.dy_sl, p.ED, es, kBTE) &&
            tma_compatible(p.Bm, p.b_sb, p.b_sl, N, es, N) &&
            tma_compatible(p.Cm, p.c_sb, p.c_sl, N, es, N);
  if (p.z) ok = ok && tma_compatible(p.z, p.z_sb, p.z_sl, p.ED, es, kBTE) && aligned16(p.dz) &&
                (p.dz_sl * es) % 16 == 0 && (p.dz_sb * es) % 16 == 0;
  ok = ok && aligned16(p.dx) && aligned16(p.ddelta) && (p.dx_sl * es) % 16 == 0 && (p.dx_sb * es) % 16 == 0 &&
       (p.dd_sl * es) % 16 == 0 && (p.dd_sb * es) % 16 == 0 && aligned16(p.dB) && aligned16(p.dC);
  return ok && tma_encoder() != nullptr;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

// Reads (and clears) the device-side status word of the backward kernel.  Synchronises the device.
int mb200_bwd_device_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_bwd_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_bwd_status, &zero, sizeof(int));
  return v;
}

extern "C" int mb200_sscan_bwd(const void* x, const void* delta, const void* z, const float* A,
                               const void* Bm, const void* Cm, const float* D,
                               const float* delta_bias, const void* dy, const float* carries,
                               const float* g_in, void* dx, void* ddelta, void* dz, float* dB,
                               float* dC, float* dA, float* dD, float* ddelta_bias, float* g_out,
                               int64_t B, int64_t L, int64_t ED, int N,
                               int64_t x_sb, int64_t x_sl, int64_t d_sb, int64_t d_sl,
                               int64_t z_sb, int64_t z_sl, int64_t b_sb, int64_t b_sl,
                               int64_t c_sb, int64_t c_sl, int64_t dy_sb, int64_t dy_sl,
                               int64_t dx_sb, int64_t dx_sl, int64_t dd_sb, int64_t dd_sl,
                               int64_t dz_sb, int64_t dz_sl, int dtype, int flags, void* stream) {
  if (B < 0 || L < 0 || ED < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (N != 8 && N != 16 && N != 32 && N != 64) return MB200_ENSTATE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (B == 0 || ED == 0) return MB200_OK;
  if (L == 0) {                                   // nothing to differentiate; the carry passes through
    if (g_out) {
      if (g_in) cudaMemcpyAsync(g_out, g_in, sizeof(float) * B * ED * N, cudaMemcpyDeviceToDevice, st);
      else cudaMemsetAsync(g_out, 0, sizeof(float) * B * ED * N, st);
    }
    return check_launch();
  }
  if (!x || !delta || !A || !Bm || !Cm || !dy || !carries || !dx || !ddelta || !dB || !dC || !dA)
    return MB200_EINVAL;
  if (z && !dz) return MB200_EINVAL;
  if ((flags & MB200_DELTA_SOFTPLUS) && !delta_bias) return MB200_EINVAL;
  if (B > 65535) return MB200_ETOOBIG;
  if (!aligned16(carries) || !aligned16(g_in) || !aligned16(g_out)) return MB200_EALIGN;
  SscanBwdParams p;
  p.x = x; p.delta = delta; p.z = z; p.Bm = Bm; p.Cm = Cm; p.dy = dy; p.A = A; p.D = D;
  p.delta_bias = delta_bias; p.carries = carries; p.g_in = g_in;
  p.dx = dx; p.ddelta = ddelta; p.dz = dz; p.dB = dB; p.dC = dC; p.dA = dA; p.dD = dD;
  p.ddelta_bias = ddelta_bias; p.g_out = g_out;
  p.B = B; p.L = L; p.ED = ED;
  p.x_sb = x_sb; p.x_sl = x_sl; p.d_sb = d_sb; p.d_sl = d_sl; p.z_sb = z_sb; p.z_sl = z_sl;
  p.b_sb = b_sb; p.b_sl = b_sl; p.c_sb = c_sb; p.c_sl = c_sl; p.dy_sb = dy_sb; p.dy_sl = dy_sl;
  p.dx_sb = dx_sb; p.dx_sl = dx_sl; p.dd_sb = dd_sb; p.dd_sl = dd_sl; p.dz_sb = dz_sb; p.dz_sl = dz_sl;
  p.flags = flags;
  const int es = dtype == MB200_F32 ? 4 : 2;
  if (bwd_tma_path_ok(p, N, es)) {
    const int rc = dtype == MB200_F32 ? bwd_tma_launch<float>(p, st) : bwd_tma_launch<__nv_bfloat16>(p, st);
    if (rc <= 0) return rc;
  }
  if (flags & MB200_REVERSE) return MB200_EUNSUPPORTED;   // the reverse direction exists on the tensor-map path only
  const int kv = dtype == MB200_F32 ? 4 : 8;
  bool vec = ED % kv == 0;
  for (const void* q : {x, delta, z, Bm, Cm, dy, (const void*)dx, (const void*)ddelta, (const void*)dz})
    vec = vec && aligned16(q);
  for (int64_t s : {x_sb, x_sl, d_sb, d_sl, b_sb, b_sl, c_sb, c_sl, dy_sb, dy_sl, dx_sb, dx_sl, dd_sb, dd_sl})
    vec = vec && s % kv == 0;
  if (z) vec = vec && z_sb % kv == 0 && z_sl % kv == 0 && dz_sb % kv == 0 && dz_sl % kv == 0;
  return dtype == MB200_F32 ? bwd_generic_launch_t<float>(p, N, vec, st)
                            : bwd_generic_launch_t<__nv_bfloat16>(p, N, vec, st);
}
