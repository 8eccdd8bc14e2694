// Fused selective scan, forward: discretisation, recurrence, C-contraction, D skip and
// SiLU(z) gate in one pass.  Reads x, delta, z, B, C once; writes y (and, for training,
// the scan state every kChunk timesteps).  The (B, L, ED, N) tensors never exist.
//
// What bounds it.  Per (b, t, e, n) element the kernel needs one ex2 (16/clk/SM on the MUFU
// pipe), four FP32 operations, and its B and C operands out of shared memory; HBM traffic is
// 0.5 byte per element.  Measured on B200 no single unit is the limit (shared-memory pipe ~75 %, issue
// ~65 %, FMA ~40 %, MUFU ~38 %, DRAM ~20 %): the time is that of the in-order recurrence warps, whose
// dependent chain only overlaps with the other resident warps.  So: no redundant arithmetic (every
// recurrence is walked serially along L by exactly one thread), everything that is not the recurrence
// (softplus, delta*x, D skip, gate, conversions: 70 % as many instructions again) runs on other warps,
// and the recurrence is software-pipelined by hand.
//
// Structure (this file, used whenever the tensors satisfy the tensor-map alignment rules;
// sscan_fwd_generic.cuh holds the register-staged path for everything else):
// a CTA of 288 threads owns a tile of 32 channels (d_state 16) of one batch row and walks time in tiles of 16.
//   - One warp does nothing but issue TMA loads (cp.async.bulk.tensor, 3-D maps {channels, L, B}) of the
//     raw x, delta, z, B, C boxes into a shared-memory ring, as far ahead as the ring has free stages;
//     ragged L and ragged channel tiles are zero-filled by the copy engine.
//   - 4 producer warps turn a raw tile into float32 operands ({softplus(delta+bias), delta*x},
//     B, C; swizzled, double-buffered) and, two tiles later, finish it: sum the N/4 partial
//     C-contractions per channel, add D*x, apply the SiLU(z) gate, store y.
//   - 4 recurrence warps run nothing but the recurrence: a thread owns 4 consecutive states of one
//     channel, a warp the same 4 states of 32 neighbouring channels; per timestep 3 shared loads, 4 ex2
//     (2 when A has the S4D-real structure), 8 packed f32x2 operations and one 4-byte store of its partial
//     C-contraction, with the loads and decays of later timesteps written next to the recurrence of
//     the current one (the warp issues in order).
//   - Hand-off through CTA-local mbarriers.  Every wait is bounded: a wait that gives up records
//     MB200_DEV_WAIT_TIMEOUT and the thread leaves the kernel, so nothing can spin forever.
#include <type_traits>
#include "sscan_fwd_generic.cuh"
#include "tma.cuh"

namespace mb200 {
namespace {

// Raw-tile ring depth.  Copies are issued kStages - 2 tiles ahead: a box takes a few microseconds
// to land, several times the ~1 us a tile is worked on, so the ring must hold that many in flight.
template <typename T> struct Ring { static constexpr int kStages = sizeof(T) == 2 ? 8 : 5; };
constexpr int kTile = 2 * kChunk;          // timesteps per tile (two saved states per tile)

// Geometry of one CTA: kCW consumer warps whose threads each own 4 consecutive states of kCPT
// neighbouring channels, and kPW producer warps.  What a consumer thread pulls out of shared memory per
// element is 8/kCPT bytes of B and C plus 2 bytes of {delta, delta*x}, so two channels per thread (d_state
// 16) cut the recurrence's shared-memory traffic from 11 to 7 bytes per element -- and halve the number of
// warps that run it.  Measured on the 130m layer shape (B 8, L 2048, ED 1536, bf16), forward with saved
// states: 4 warps x 1 channel, 3 CTAs/SM 0.226 ms; 3 warps x 2 channels (48-channel CTAs, 2 per SM)
// 0.246 ms; 4 x 2 (64-channel CTAs) 0.283 ms; 2 x 2 (32-channel CTAs, 4 per SM) 0.263 ms.  The recurrence
// warps are in-order and wait on the loaded shared-memory pipe's round trip, so the count of resident
// warps matters more than the bytes: one channel per thread stays the default.
#ifndef MB200_FWD_CW
#define MB200_FWD_CW 4
#endif
#ifndef MB200_FWD_CPT
#define MB200_FWD_CPT 1
#endif
#ifndef MB200_FWD_PW
#define MB200_FWD_PW 4
#endif
#ifndef MB200_FWD_OCC
#define MB200_FWD_OCC 3
#endif
#ifndef MB200_FWD_DEFER
#define MB200_FWD_DEFER 1
#endif
#ifndef MB200_FWD_LA
#define MB200_FWD_LA 2
#endif
#ifndef MB200_FWD_EA
#define MB200_FWD_EA 1
#endif
constexpr int kLoadAhead = MB200_FWD_LA, kDecayAhead = MB200_FWD_EA;   // software-pipeline depths of the recurrence warps
constexpr int kDefer = MB200_FWD_DEFER;     // timesteps of partial sums a recurrence thread holds before storing them
template <int N> struct FwdGeom {
  static constexpr int kCPT = (N == 16) ? MB200_FWD_CPT : 1;
  static constexpr int kCW = (N == 16) ? MB200_FWD_CW : 4;
  static constexpr int kPW = (N == 16) ? MB200_FWD_PW : 4;
  static constexpr int kOcc = (N == 16) ? MB200_FWD_OCC : 3;          // CTAs per SM the kernel is compiled for
  static constexpr int kLPE = N / 4;                                   // lanes per channel group
  static constexpr int kConsumers = 32 * kCW;
  static constexpr int kProducers = 32 * kPW;
  static constexpr int kThreads = kConsumers + kProducers + 32;      // + the warp that issues the TMA copies
  static constexpr int kTE = kConsumers / kLPE * kCPT;                 // channels per CTA
  static_assert(kCPT == 1 || (kCPT == 2 && N == 16), "two channels per thread are laid out for d_state 16");
  static_assert(kTE % 8 == 0, "a tile row is a whole number of 16-byte vectors in bf16");
};

struct FwdMaps {
  CUtensorMap x, d, z, B, C;
};

template <typename T, int N> struct TmaFwdSmem {
  using G = FwdGeom<N>;
  static constexpr int kStages = Ring<T>::kStages;
  static constexpr int kTE = G::kTE;
  static constexpr int kYpRow = kTE * G::kLPE;                          // partial sums per timestep
  static constexpr int kActBytes = kTile * kTE * int(sizeof(T));       // one raw x / delta / z box
  static constexpr int kBcBytes = kTile * N * int(sizeof(T));          // one raw B / C box
  static constexpr int kStageBytes = 3 * kActBytes + 2 * kBcBytes;
  static_assert(kActBytes % 128 == 0 && kBcBytes % 128 == 0, "TMA destinations stay 128-byte aligned");
  // byte offsets
  static constexpr int kRaw = 0;
  static constexpr int kOp = kRaw + kStages * kStageBytes;              // float2 [2][kTile][kTE]
  static constexpr int kB = kOp + 2 * kTile * kTE * 8;                  // float  [2][kTile][N]
  static constexpr int kC = kB + 2 * kTile * N * 4;
  static constexpr int kYp = kC + 2 * kTile * N * 4;                    // float  [2][kTile][kYpRow]
  static constexpr int kD = kYp + 2 * kTile * kYpRow * 4;               // float  [kTE]
  static constexpr int kBias = kD + kTE * 4;
  static constexpr int kBars = kBias + kTE * 4;                         // (2*kStages + 4) x uint64
  static constexpr int kBytes = kBars + (2 * kStages + 4) * 8;
};

// The decays a[j] = exp(delta * A[4q + j]), j = 0..3, of one channel.  General form: four ex2.
// With the S4D-real structure A[e, n] = (n + 1) A[e, 0] (the reference's initialisation,
// mambapy/mamba.py:168-169) they are p, p r, p r^2, p r^3 with r = exp(delta A[e, 0]) and
// p = exp(delta A[e, 4q]): two ex2 and three multiplies, which halves the load on the MUFU pipe.
template <bool kStruct>
__device__ __forceinline__ void decay4(float dl, const float2& A2lo, const float2& A2hi, float A0, float2& a_lo,
                                       float2& a_hi) {
  const float2 dd = make_float2(dl, dl);
  if constexpr (!kStruct) {
    const float2 e_lo = __fmul2_rn(dd, A2lo), e_hi = __fmul2_rn(dd, A2hi);
    a_lo = make_float2(ex2f(e_lo.x), ex2f(e_lo.y));
    a_hi = make_float2(ex2f(e_hi.x), ex2f(e_hi.y));
  } else {
    const float2 e = __fmul2_rn(dd, make_float2(A0, A2lo.x));
    const float r = ex2f(e.x), p1 = ex2f(e.y);
    const float r2 = r * r;
    a_lo = make_float2(p1, p1 * r);
    a_hi = __fmul2_rn(a_lo, make_float2(r2, r2));
  }
}

// True when the 4 states 4q .. 4q+3 of a row of A (scaled by log2 e or not) follow A[n] = (n + 1) A[0]
// to within 2^-20 relative: a perturbation of the decay RATE of at most 1e-6, below the error of
// ex2.approx on the general path (libm's exp(log(n)) is not exactly n, so exact equality never holds).
__device__ __forceinline__ bool s4d_structured(const float* a4, float a0, int q) {
  bool ok = true;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float want = float(4 * q + j + 1) * a0;
    ok = ok && fabsf(a4[j] - want) <= 9.5367431640625e-7f * fabsf(want);
  }
  return ok;
}

// kCarry turns the kernel into the reverse carry pass of the sequence-sharded backward
// (gc <- a[t] * (dy'[t] * C[t] + gc), t = L-1 ... 0): the caller passes dy as `x` and C as `Bm`, the
// converter forms dy' = dy * silu(z) instead of delta * x, and the recurrence multiplies by the decay
// after adding the input.  It has no y and saves no states; the result leaves through hT.
// kHasY = false is the pass that only wants states (no C-contraction, no epilogue).
template <typename T, int N, bool kRev, bool kCarry, bool kHasY>
__global__ void __launch_bounds__(FwdGeom<N>::kThreads, FwdGeom<N>::kOcc)
sscan_fwd_tma_kernel(const __grid_constant__ FwdMaps maps, const SscanFwdParams p) {
  using G = FwdGeom<N>;
  using S = TmaFwdSmem<T, N>;
  constexpr int kLPE = G::kLPE, kTE = G::kTE, kStages = S::kStages;
  constexpr int kCPT = G::kCPT, kNC = G::kConsumers, kNP = G::kProducers, kYpRow = S::kYpRow;

  extern __shared__ __align__(128) unsigned char smem_raw[];
  float2* s_op = reinterpret_cast<float2*>(smem_raw + S::kOp);
  float* s_B = reinterpret_cast<float*>(smem_raw + S::kB);
  float* s_C = reinterpret_cast<float*>(smem_raw + S::kC);
  float* s_yp = reinterpret_cast<float*>(smem_raw + S::kYp);
  float* s_D = reinterpret_cast<float*>(smem_raw + S::kD);
  float* s_bias = reinterpret_cast<float*>(smem_raw + S::kBias);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem_raw + S::kBars);
  uint64_t* raw_full = bars;            // [kStages] copy landed
  uint64_t* raw_free = bars + kStages;  // [kStages] producers are done with the stage
  uint64_t* op_full = bars + 2 * kStages;       // [2] operands committed
  uint64_t* op_empty = bars + 2 * kStages + 2;  // [2] consumers are done with the buffer

  const int tid = threadIdx.x;
  const int64_t e0 = int64_t(blockIdx.x) * kTE;
  const int64_t b = blockIdx.y;
  const int cols_ok = int(min64(kTE, p.ED - e0));
  const bool softplus = (p.flags & MB200_DELTA_SOFTPLUS) != 0;
  constexpr bool has_y = kHasY;
  const bool has_z = p.z != nullptr;
  const int64_t ntiles = (p.L + kTile - 1) / kTile;
  // Direction.  With MB200_REVERSE time is walked from L-1 down to 0: processing tile kt is the
  // tile of timesteps starting at tile_t0(kt), and processing step s of a tile is its row 15 - s.
  // Saved states are indexed by TIME chunk either way: entry c is the state entering chunk c in the
  // scan direction.
  constexpr bool rev = kRev;
  auto tile_t0 = [&](int64_t kt) { return (rev ? ntiles - 1 - kt : kt) * kTile; };

  if (tid == 0) {
#pragma unroll
    for (int i = 0; i < kStages; ++i) { mbar_init(&raw_full[i], 1); mbar_init(&raw_free[i], kNP); }
    mbar_init(&op_full[0], kNP); mbar_init(&op_full[1], kNP);
    mbar_init(&op_empty[0], kNC); mbar_init(&op_empty[1], kNC);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  for (int i = tid; i < kTE; i += G::kThreads) {
    const bool ok = i < cols_ok;
    s_D[i] = (ok && p.D) ? p.D[e0 + i] : 0.f;
    s_bias[i] = (ok && softplus) ? p.delta_bias[e0 + i] : 0.f;
  }
  __syncthreads();

  if (tid < kNC) {
    // ------------------------------------------------------------------ consumers
    // One channel per thread: the lanes of a warp are neighbouring CHANNELS with the same state quad q, so
    // the warp's B and C loads have a single address.  Shared memory delivers a 16-byte load with four
    // distinct addresses (lanes = 8 channels x 4 quads) in 4 wavefronts, one with a single address in 2.
    const int grp = (kCPT == 1) ? tid % kTE : tid / kLPE;
    const int q = (kCPT == 1) ? tid / kTE : tid % kLPE;   // state quad
    const int e_l = grp * kCPT;                        // first channel of this thread inside the tile
    float2 A2lo[kCPT], A2hi[kCPT], hlo[kCPT], hhi[kCPT];
    float A0[kCPT];
    bool e_ok[kCPT];
    bool structured = (p.flags & MB200_GENERAL_DECAY) == 0;
#pragma unroll
    for (int i = 0; i < kCPT; ++i) {
      const int64_t e = e0 + e_l + i;
      e_ok[i] = e < p.ED;
      float a4[4], h4[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        a4[j] = e_ok[i] ? p.A[e * N + 4 * q + j] * kLog2e : 0.f;
        h4[j] = (e_ok[i] && p.h0) ? p.h0[(b * p.ED + e) * N + 4 * q + j] : 0.f;
      }
      A0[i] = e_ok[i] ? p.A[e * N] * kLog2e : 0.f;
      structured = structured && s4d_structured(a4, A0[i], q);
      A2lo[i] = make_float2(a4[0], a4[1]); A2hi[i] = make_float2(a4[2], a4[3]);
      hlo[i] = make_float2(h4[0], h4[1]); hhi[i] = make_float2(h4[2], h4[3]);
    }
    structured = __all_sync(0xffffffffu, structured);          // one code path per warp
    const int op_off0 = op_index(0, e_l, kTE), op_off1 = op_index(1, e_l, kTE) - kTE;
    // where this thread leaves its partial C-contractions inside a timestep's row of partial sums
    int yp_off0, yp_off1;
    if constexpr (kCPT == 1) {
      yp_off0 = yp_off1 = q * kTE + e_l;                          // [quad][channel]: a warp stores one contiguous row
    } else {
      yp_off0 = yp_off1 = ((e_l >> 2) * 4 + q) * 4 + (e_l & 3);   // [channel quad][q][channel in quad]
    }
    const int64_t nchunks = (p.L + kChunk - 1) / kChunk;
    float* carry_base = p.carries ? p.carries + (b * nchunks * p.ED + e0 + e_l) * N + 4 * q : nullptr;
    // row of processing step t is rb0 + t * rstep (in operand-tile rows); odd rows use the other swizzle offset
    constexpr int rb0 = rev ? kTile - 1 : 0, rstep = rev ? -1 : 1;
    const int off_even = rev ? op_off1 : op_off0, off_odd = rev ? op_off0 : op_off1;

    // The pass that only wants states (the carry pass of a split sequence) also returns the decay product of
    // the whole span, exp(A * sum_t delta[t]): the sum costs one add per timestep here, and a pass of its own
    // over delta otherwise.
    constexpr bool kWantP = !kHasY && !kCarry;
    float dsum[kCPT], dcomp[kCPT];
#pragma unroll
    for (int i = 0; i < kCPT; ++i) dsum[i] = dcomp[i] = 0.f;
    auto run_tiles = [&](auto struct_tag) {
      constexpr bool kStruct = decltype(struct_tag)::value;
      for (int64_t kt = 0; kt < ntiles; ++kt) {
        const int buf = int(kt & 1);
        if (!mbar_wait(&op_full[buf], int((kt >> 1) & 1))) {
          atomicExch(&g_fwd_status, MB200_DEV_WAIT_TIMEOUT);
          return false;
        }
        const int64_t t0a = tile_t0(kt);
        const float2* op = s_op + buf * kTile * kTE;
        const float* sB = s_B + buf * kTile * N + 4 * q;
        const float* sC = s_C + buf * kTile * N + 4 * q;
        float* yp = s_yp + buf * kTile * kYpRow;
        float ypend[kTile][kCPT];                                            // partial sums not stored yet
        // One timestep is three stages -- operand loads, decays and inputs (ex2), recurrence and contraction --
        // and only the last one depends on the previous timestep.  The stages of three consecutive timesteps
        // are written side by side (loads of t+2, decays of t+1, recurrence of t), so that this in-order warp
        // always has independent work between an instruction and the first use of its result.
        struct Loaded { float2 o[kCPT]; float4 Bq, Cq; };
        struct Ready { float2 a_lo[kCPT], a_hi[kCPT], dxx[kCPT]; float4 Bq, Cq; };
        auto load = [&](int t) {
          Loaded l;
          const int r = rb0 + t * rstep;
          if constexpr (kCPT == 1) {
            l.o[0] = op[r * kTE + ((t & 1) ? off_odd : off_even)];
          } else {
            const float4 o4 = *reinterpret_cast<const float4*>(op + r * kTE + ((t & 1) ? off_odd : off_even));
            l.o[0] = make_float2(o4.x, o4.y); l.o[1] = make_float2(o4.z, o4.w);
          }
          l.Bq = *reinterpret_cast<const float4*>(sB + r * N);
          l.Cq = l.Bq;
          if constexpr (kHasY) l.Cq = *reinterpret_cast<const float4*>(sC + r * N);
          return l;
        };
        auto prepare = [&](const Loaded& l) {
          Ready e;
#pragma unroll
          for (int i = 0; i < kCPT; ++i) {
            e.dxx[i] = make_float2(l.o[i].y, l.o[i].y);
            decay4<kStruct>(l.o[i].x, A2lo[i], A2hi[i], A0[i], e.a_lo[i], e.a_hi[i]);
          }
          e.Bq = l.Bq; e.Cq = l.Cq;
          return e;
        };
        Loaded ld[kTile];
        Ready rd[kTile];
        float dtile[kCPT];                                                   // sum of delta over this tile
#pragma unroll
        for (int i = 0; i < kCPT; ++i) dtile[i] = 0.f;
#pragma unroll
        for (int t = 0; t < kLoadAhead; ++t) ld[t] = load(t);
#pragma unroll
        for (int t = 0; t < kDecayAhead; ++t) rd[t] = prepare(ld[t]);
#pragma unroll
        for (int t = 0; t < kTile; ++t) {
          if (t % kChunk == 0 && carry_base) {                              // state entering this chunk
            const int64_t c = t0a / kChunk + (rev ? 1 - t / kChunk : t / kChunk);
            if (c < nchunks) {
#pragma unroll
              for (int i = 0; i < kCPT; ++i)
                if (e_ok[i])
                  *reinterpret_cast<float4*>(carry_base + (c * p.ED + i) * N) =
                      make_float4(hlo[i].x, hlo[i].y, hhi[i].x, hhi[i].y);
            }
          }
          if (t + kLoadAhead < kTile) ld[t + kLoadAhead] = load(t + kLoadAhead);
          if (t + kDecayAhead < kTile) rd[t + kDecayAhead] = prepare(ld[t + kDecayAhead]);
          const Ready cur = rd[t];
          if constexpr (kWantP) {
#pragma unroll
            for (int i = 0; i < kCPT; ++i) dtile[i] += ld[t].o[i].x;
          }
          const float4 Bq = cur.Bq, Cq = cur.Cq;
          float ysum[kCPT];
#pragma unroll
          for (int i = 0; i < kCPT; ++i) {
            const float2 dxx = cur.dxx[i], a_lo = cur.a_lo[i], a_hi = cur.a_hi[i];
            if constexpr (kCarry) {
              hlo[i] = __fmul2_rn(a_lo, __ffma2_rn(dxx, make_float2(Bq.x, Bq.y), hlo[i]));
              hhi[i] = __fmul2_rn(a_hi, __ffma2_rn(dxx, make_float2(Bq.z, Bq.w), hhi[i]));
            } else {
              const float2 u_lo = __fmul2_rn(dxx, make_float2(Bq.x, Bq.y));
              const float2 u_hi = __fmul2_rn(dxx, make_float2(Bq.z, Bq.w));
              hlo[i] = __ffma2_rn(a_lo, hlo[i], u_lo);
              hhi[i] = __ffma2_rn(a_hi, hhi[i], u_hi);
              if constexpr (kHasY) {
                float2 acc = __fmul2_rn(hlo[i], make_float2(Cq.x, Cq.y));
                acc = __ffma2_rn(hhi[i], make_float2(Cq.z, Cq.w), acc);
                ysum[i] = acc.x + acc.y;
              }
            }
          }
          if constexpr (kHasY && !kCarry) {
            // A shared-memory store between two timesteps' operand loads pins the loads behind it (the
            // compiler cannot tell that they do not alias); the partial sums are therefore held in
            // registers and stored kDefer timesteps at a time.
#pragma unroll
            for (int i = 0; i < kCPT; ++i) ypend[t][i] = ysum[i];
            if ((t + 1) % kDefer == 0) {
#pragma unroll
              for (int u = t + 1 - kDefer; u <= t; ++u) {
                float* dst = yp + u * kYpRow + ((u & 1) ? yp_off1 : yp_off0);
                if constexpr (kCPT == 1) *dst = ypend[u][0];
                else *reinterpret_cast<float2*>(dst) = make_float2(ypend[u][0], ypend[u][1]);
              }
            }
          }
        }
        if constexpr (kWantP) {                     // compensated sum over the tiles: L can be 10^5 and it feeds an exponent
#pragma unroll
          for (int i = 0; i < kCPT; ++i) {
            const float yk = dtile[i] - dcomp[i];
            const float tk = dsum[i] + yk;
            dcomp[i] = (tk - dsum[i]) - yk;
            dsum[i] = tk;
          }
        }
        mbar_arrive(&op_empty[buf]);
      }
      return true;
    };
    const bool ok = structured ? run_tiles(std::true_type{}) : run_tiles(std::false_type{});
    if (!ok) return;
    if (p.hT) {
#pragma unroll
      for (int i = 0; i < kCPT; ++i)
        if (e_ok[i])
          *reinterpret_cast<float4*>(p.hT + (b * p.ED + e0 + e_l + i) * N + 4 * q) =
              make_float4(hlo[i].x, hlo[i].y, hhi[i].x, hhi[i].y);
    }
    if constexpr (kWantP) {
      if (p.pT) {
#pragma unroll
        for (int i = 0; i < kCPT; ++i)
          if (e_ok[i])
            *reinterpret_cast<float4*>(p.pT + (b * p.ED + e0 + e_l + i) * N + 4 * q) =
                make_float4(ex2f(A2lo[i].x * dsum[i]), ex2f(A2lo[i].y * dsum[i]), ex2f(A2hi[i].x * dsum[i]),
                            ex2f(A2hi[i].y * dsum[i]));
      }
    }
  } else if (tid >= kNC + kNP) {
    // ------------------------------------------------------------------ loader
    // One lane issues the TMA copies, as far ahead as the ring has free stages.  Issuing the five copies of
    // a tile takes the issuing thread over a thousand cycles (clock64 stamps); done by a producer thread,
    // as it used to be, that made its warp the last one to hand every tile to the recurrence warps.
    if (tid != kNC + kNP) return;
    const uint32_t stage_tx = uint32_t((has_z ? 3 : 2) * S::kActBytes + 2 * S::kBcBytes);
    for (int64_t kt = 0; kt < ntiles; ++kt) {
      const int r = int(kt % kStages);
      if (kt >= kStages && !mbar_wait(&raw_free[r], int((kt / kStages - 1) & 1))) {
        atomicExch(&g_fwd_status, MB200_DEV_WAIT_TIMEOUT);
        return;
      }
      unsigned char* st = smem_raw + S::kRaw + r * S::kStageBytes;
      const int t0 = int(tile_t0(kt));
      mbar_expect_tx(&raw_full[r], stage_tx);
      tma_load_3d(st, &maps.x, int(e0), t0, int(b), &raw_full[r]);
      tma_load_3d(st + S::kActBytes, &maps.d, int(e0), t0, int(b), &raw_full[r]);
      if (has_z) tma_load_3d(st + 2 * S::kActBytes, &maps.z, int(e0), t0, int(b), &raw_full[r]);
      tma_load_3d(st + 3 * S::kActBytes, &maps.B, 0, t0, int(b), &raw_full[r]);
      tma_load_3d(st + 3 * S::kActBytes + S::kBcBytes, &maps.C, 0, t0, int(b), &raw_full[r]);
    }
  } else {
    // ------------------------------------------------------------------ producers
    const int pt = tid - kNC;
    constexpr int kVecs = kTile * kTE / 4;                 // 4-channel vectors per activation tile
    constexpr int kVecPerRow = kTE / 4;
    T* gy = has_y ? static_cast<T*>(p.y) + b * p.y_sb + e0 : nullptr;

    auto stage_ptr = [&](int64_t kt) { return smem_raw + S::kRaw + int(kt % kStages) * S::kStageBytes; };
    auto fail = [&]() { atomicExch(&g_fwd_status, MB200_DEV_WAIT_TIMEOUT); };

    // raw tile kt -> float32 operands in buffer kt & 1
    auto convert = [&](int64_t kt) {
      const int buf = int(kt & 1);
      const int rows_ok = int(min64(kTile, p.L - tile_t0(kt)));
      const unsigned char* st = stage_ptr(kt);
      const T* rx = reinterpret_cast<const T*>(st);
      const T* rd = reinterpret_cast<const T*>(st + S::kActBytes);
      float2* tile = s_op + buf * kTile * kTE;
      for (int v = pt; v < kVecs; v += kNP) {
        const int rr = v / kVecPerRow, cc = (v % kVecPerRow) * 4;
        const Vec4<T> xv = *reinterpret_cast<const Vec4<T>*>(rx + rr * kTE + cc);
        const Vec4<T> dv4 = *reinterpret_cast<const Vec4<T>*>(rd + rr * kTE + cc);
        Vec4<T> zv4 = xv;
        if constexpr (kCarry) {
          if (has_z) zv4 = *reinterpret_cast<const Vec4<T>*>(reinterpret_cast<const T*>(st + 2 * S::kActBytes) + rr * kTE + cc);
        }
        float2 o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float dv = Elem<T>::to_f(dv4.v[k]);
          if (softplus) dv = softplus_fast(dv + s_bias[cc + k]);
          if (rr >= rows_ok) dv = 0.f;                      // past the end of the sequence
          if constexpr (kCarry) {
            float g = Elem<T>::to_f(xv.v[k]);               // dy in the place of x
            if (has_z) {
              const float zf = Elem<T>::to_f(zv4.v[k]);
              g *= zf * sigmoid_fast(zf);
            }
            o[k] = make_float2(dv, g);
          } else {
            o[k] = make_float2(dv, dv * Elem<T>::to_f(xv.v[k]));
          }
        }
        *reinterpret_cast<float4*>(tile + op_index(rr, cc, kTE)) = make_float4(o[0].x, o[0].y, o[1].x, o[1].y);
        *reinterpret_cast<float4*>(tile + op_index(rr, cc + 2, kTE)) = make_float4(o[2].x, o[2].y, o[3].x, o[3].y);
      }
      const T* rB = reinterpret_cast<const T*>(st + 3 * S::kActBytes);     // B box then C box, contiguous
      float* dstB = s_B + buf * kTile * N;
      float* dstC = s_C + buf * kTile * N;
      constexpr int kBcVecs = kTile * N / 4;
      for (int v = pt; v < 2 * kBcVecs; v += kNP) {
        const Vec4<T> r4 = *reinterpret_cast<const Vec4<T>*>(rB + v * 4);
        float* dst = (v < kBcVecs) ? dstB + v * 4 : dstC + (v - kBcVecs) * 4;
        *reinterpret_cast<float4*>(dst) = make_float4(Elem<T>::to_f(r4.v[0]), Elem<T>::to_f(r4.v[1]),
                                                      Elem<T>::to_f(r4.v[2]), Elem<T>::to_f(r4.v[3]));
      }
    };
    // finish tile kt: partial sums -> y (the consumers of tile kt have been waited for)
    auto epilogue = [&](int64_t kt) {
      const int buf = int(kt & 1);
      const int64_t t0 = tile_t0(kt);
      const int rows_ok = int(min64(kTile, p.L - t0));
      const unsigned char* st = stage_ptr(kt);
      const T* rx = reinterpret_cast<const T*>(st);
      const T* rz = reinterpret_cast<const T*>(st + 2 * S::kActBytes);
      const float* yp = s_yp + buf * kTile * kYpRow;
      for (int v = pt; v < kVecs; v += kNP) {
        const int rr = v / kVecPerRow, cc = (v % kVecPerRow) * 4;
        if (rr >= rows_ok || cc >= cols_ok) continue;
        const Vec4<T> xv = *reinterpret_cast<const Vec4<T>*>(rx + rr * kTE + cc);
        Vec4<T> zv = xv;
        if (has_z) zv = *reinterpret_cast<const Vec4<T>*>(rz + rr * kTE + cc);
        const int ps = rev ? kTile - 1 - rr : rr;            // processing step that produced row rr
        float s4[4];
        if constexpr (kCPT == 1) {
          // one 16-byte vector per state quad holds that quad's partial sums of channels cc .. cc+3
          const float4* quad = reinterpret_cast<const float4*>(yp + ps * kYpRow + cc);
          float4 acc = quad[0];
#pragma unroll
          for (int j = 1; j < kLPE; ++j) {
            const float4 w = quad[j * (kTE / 4)];
            acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;
          }
          s4[0] = acc.x; s4[1] = acc.y; s4[2] = acc.z; s4[3] = acc.w;
        } else {
          // the four state quads' partials of channels cc .. cc+3 are four 16-byte vectors; lanes start at
          // different ones so that a quarter-warp's loads fall into different banks
          const float4* quad = reinterpret_cast<const float4*>(yp + ps * kYpRow + cc * 4);
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 w = quad[(j + (pt >> 1)) & 3];
            acc.x += w.x; acc.y += w.y; acc.z += w.z; acc.w += w.w;
          }
          s4[0] = acc.x; s4[1] = acc.y; s4[2] = acc.z; s4[3] = acc.w;
        }
        Vec4<T> out;
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          float yv = fmaf(s_D[cc + k], Elem<T>::to_f(xv.v[k]), s4[k]);
          if (has_z) {
            const float zf = Elem<T>::to_f(zv.v[k]);
            yv *= zf * sigmoid_fast(zf);
          }
          out.v[k] = Elem<T>::from_f(yv);
        }
        T* dst = gy + (t0 + rr) * p.y_sl + cc;
        if (cc + 4 <= cols_ok) {
          *reinterpret_cast<Vec4<T>*>(dst) = out;
        } else {
#pragma unroll
          for (int k = 0; k < 4; ++k)
            if (cc + k < cols_ok) dst[k] = out.v[k];
        }
      }
    };

    for (int64_t kt = 0; kt < ntiles; ++kt) {
      if (kt >= 2) {
        if (!mbar_wait(&op_empty[kt & 1], int(((kt - 2) >> 1) & 1))) { fail(); return; }
        if (has_y) epilogue(kt - 2);
        mbar_arrive(&raw_free[(kt - 2) % kStages]);
      }
      if (!mbar_wait(&raw_full[kt % kStages], int((kt / kStages) & 1))) { fail(); return; }
      convert(kt);
      mbar_arrive(&op_full[kt & 1]);
    }
    for (int64_t kt = ntiles >= 2 ? ntiles - 2 : 0; kt < ntiles; ++kt) {
      if (!mbar_wait(&op_empty[kt & 1], int((kt >> 1) & 1))) { fail(); return; }
      if (has_y) epilogue(kt);
    }
  }
}

template <typename T, int N>
int tma_launch_n(const SscanFwdParams& p, cudaStream_t st) {
  using G = FwdGeom<N>;
  using S = TmaFwdSmem<T, N>;
  constexpr bool bf = sizeof(T) == 2;
  FwdMaps m;
  bool ok = tma_encode(&m.x, p.x, bf, p.B, p.L, p.ED, p.x_sb, p.x_sl, G::kTE, kTile) &&
            tma_encode(&m.d, p.delta, bf, p.B, p.L, p.ED, p.d_sb, p.d_sl, G::kTE, kTile) &&
            tma_encode(&m.B, p.Bm, bf, p.B, p.L, N, p.b_sb, p.b_sl, N, kTile) &&
            tma_encode(&m.C, p.Cm, bf, p.B, p.L, N, p.c_sb, p.c_sl, N, kTile);
  if (ok && p.z) ok = tma_encode(&m.z, p.z, bf, p.B, p.L, p.ED, p.z_sb, p.z_sl, G::kTE, kTile);
  else if (ok) m.z = m.x;
  if (!ok) return 1;                                   // caller falls back to the generic path
  const bool rv = (p.flags & MB200_REVERSE) != 0, hy = p.y != nullptr;
  auto k = (p.flags & kFlagCarryPass) ? sscan_fwd_tma_kernel<T, N, true, true, false>
           : rv ? (hy ? sscan_fwd_tma_kernel<T, N, true, false, true> : sscan_fwd_tma_kernel<T, N, true, false, false>)
                : (hy ? sscan_fwd_tma_kernel<T, N, false, false, true> : sscan_fwd_tma_kernel<T, N, false, false, false>);
  if (cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kBytes) != cudaSuccess)
    return MB200_ELAUNCH;
  dim3 grid(unsigned((p.ED + G::kTE - 1) / G::kTE), unsigned(p.B));
  k<<<grid, G::kThreads, S::kBytes, st>>>(m, p);
  return check_launch();
}

template <typename T>
int tma_launch_t(const SscanFwdParams& p, int N, cudaStream_t st) {
  switch (N) {
    case 8: return tma_launch_n<T, 8>(p, st);
    case 16: return tma_launch_n<T, 16>(p, st);
    case 32: return tma_launch_n<T, 32>(p, st);
    case 64: return tma_launch_n<T, 64>(p, st);
    default: return MB200_ENSTATE;
  }
}

// The tensor-map path needs 16-byte aligned bases and byte strides, and 8-byte aligned y rows.
bool tma_path_ok(const SscanFwdParams& p, int N, int es) {
  const int te = N == 8 ? FwdGeom<8>::kTE : N == 16 ? FwdGeom<16>::kTE : N == 32 ? FwdGeom<32>::kTE : FwdGeom<64>::kTE;
  if (p.L >= (int64_t(1) << 31) || p.ED >= (int64_t(1) << 31)) return false;
  bool ok = tma_compatible(p.x, p.x_sb, p.x_sl, p.ED, es, te) &&
            tma_compatible(p.delta, p.d_sb, p.d_sl, p.ED, es, te) &&
            tma_compatible(p.Bm, p.b_sb, p.b_sl, N, es, N) &&
            tma_compatible(p.Cm, p.c_sb, p.c_sl, N, es, N);
  if (p.z) ok = ok && tma_compatible(p.z, p.z_sb, p.z_sl, p.ED, es, te);
  if (p.y) ok = ok && aligned16(p.y) && (p.y_sl * es) % 16 == 0 && (p.y_sb * es) % 16 == 0;
  return ok && tma_encoder() != nullptr;
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" int mb200_sscan_chunk(void) { return kChunk; }

// Internal: the tensor-map forward on a prepared parameter block (used by the reverse carry pass).
// Returns 0 when launched, a negative code on failure, 1 when these tensors need the generic path.
int mb200_fwd_tma_try(const mb200::SscanFwdParams& p, int N, int dtype, cudaStream_t st) {
  const int es = dtype == MB200_F32 ? 4 : 2;
  if (!tma_path_ok(p, N, es)) return 1;
  return dtype == MB200_F32 ? tma_launch_t<float>(p, N, st) : tma_launch_t<__nv_bfloat16>(p, N, st);
}

// Reads (and clears) the device-side status word of the forward kernels: non-zero when a bounded
// wait inside a kernel gave up.  Synchronises the device.
int mb200_fwd_device_status() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_fwd_status, sizeof(int)) != cudaSuccess) return -1;
  if (v) cudaMemcpyToSymbol(g_fwd_status, &zero, sizeof(int));
  return v;
}

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
  p.delta_bias = delta_bias; p.h0 = h0; p.y = y; p.hT = hT; p.pT = nullptr; p.carries = carries;
  p.B = B; p.L = L; p.ED = ED;
  p.x_sb = x_sb; p.x_sl = x_sl; p.d_sb = d_sb; p.d_sl = d_sl; p.z_sb = z_sb; p.z_sl = z_sl;
  p.b_sb = b_sb; p.b_sl = b_sl; p.c_sb = c_sb; p.c_sl = c_sl; p.y_sb = y_sb; p.y_sl = y_sl;
  p.flags = flags;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = dtype == MB200_F32 ? 4 : 2;
  if (tma_path_ok(p, N, es)) {
    const int rc = dtype == MB200_F32 ? tma_launch_t<float>(p, N, st) : tma_launch_t<__nv_bfloat16>(p, N, st);
    if (rc <= 0) return rc;                        // launched (0) or failed hard (< 0)
  }
  if (flags & MB200_REVERSE) return MB200_EUNSUPPORTED;   // the reverse direction exists on the tensor-map path only
  const int kv = dtype == MB200_F32 ? 4 : 8;
  bool vec = ED % kv == 0 && aligned16(x) && aligned16(delta) && aligned16(z) && aligned16(y) &&
             aligned16(Bm) && aligned16(Cm);
  for (int64_t s : {x_sb, x_sl, d_sb, d_sl, y_sb, y_sl, b_sb, b_sl, c_sb, c_sl}) vec = vec && s % kv == 0;
  if (z) vec = vec && z_sb % kv == 0 && z_sl % kv == 0;
  return dtype == MB200_F32 ? generic_launch_t<float>(p, N, vec, st)
                            : generic_launch_t<__nv_bfloat16>(p, N, vec, st);
}

// Forward carry pass of a split sequence: the state a span reaches from a zero state, and the span's decay
// product, in one pass over x, delta, B (no y, no C, no saved states).
extern "C" int mb200_sscan_fwd_carry(const void* x, const void* delta, const float* A, const void* Bm,
                                     const float* delta_bias, float* h_out, float* p_out,
                                     int64_t B, int64_t L, int64_t ED, int N,
                                     int64_t x_sb, int64_t x_sl, int64_t d_sb, int64_t d_sl,
                                     int64_t b_sb, int64_t b_sl, int dtype, int flags, void* stream) {
  if (B < 0 || L < 0 || ED < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (N != 8 && N != 16 && N != 32 && N != 64) return MB200_ENSTATE;
  if (B == 0 || ED == 0) return MB200_OK;
  if (!h_out || !p_out || !A) return MB200_EINVAL;
  if ((flags & MB200_DELTA_SOFTPLUS) && !delta_bias) return MB200_EINVAL;
  if (flags & MB200_REVERSE) return MB200_EUNSUPPORTED;
  if (!aligned16(h_out) || !aligned16(p_out)) return MB200_EALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (L > 0 && (!x || !delta || !Bm)) return MB200_EINVAL;
  if (L > 0) {
    SscanFwdParams p;
    p.x = x; p.delta = delta; p.z = nullptr; p.A = A; p.Bm = Bm; p.Cm = Bm; p.D = nullptr;
    p.delta_bias = delta_bias; p.h0 = nullptr; p.y = nullptr; p.hT = h_out; p.pT = p_out; p.carries = nullptr;
    p.B = B; p.L = L; p.ED = ED;
    p.x_sb = x_sb; p.x_sl = x_sl; p.d_sb = d_sb; p.d_sl = d_sl; p.z_sb = 0; p.z_sl = 0;
    p.b_sb = b_sb; p.b_sl = b_sl; p.c_sb = b_sb; p.c_sl = b_sl; p.y_sb = 0; p.y_sl = 0;
    p.flags = flags & (MB200_DELTA_SOFTPLUS | MB200_GENERAL_DECAY);
    const int rc = mb200_fwd_tma_try(p, N, dtype, st);
    if (rc <= 0) return rc;                        // launched (0) or failed hard (< 0)
  }
  // tensors the tensor-map path cannot take (or an empty span): the two pieces as separate launches
  int rc = mb200_sscan_fwd(x, delta, nullptr, A, Bm, Bm, nullptr, delta_bias, nullptr, nullptr, h_out, nullptr, B, L, ED,
                           N, x_sb, x_sl, d_sb, d_sl, 0, 0, b_sb, b_sl, b_sb, b_sl, 0, 0, dtype,
                           flags & (MB200_DELTA_SOFTPLUS | MB200_GENERAL_DECAY), stream);
  if (rc != MB200_OK) return rc;
  return mb200_decay_prod(delta, A, delta_bias, p_out, B, L, ED, N, d_sb, d_sl, dtype, flags & MB200_DELTA_SOFTPLUS,
                          stream);
}
