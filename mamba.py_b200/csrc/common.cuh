// Shared device helpers for the selective-scan kernels (sm_100a).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include "mamba_b200.h"

namespace mb200 {

constexpr float kLog2e = 1.4426950408889634f;

// ---- element <-> float conversion -------------------------------------------------
template <typename T> struct Elem;
template <> struct Elem<float> {
  static constexpr int kVec = 4;                       // elements per 16-byte vector
  __device__ static float to_f(float v) { return v; }
  __device__ static float from_f(float v) { return v; }
};
template <> struct Elem<__nv_bfloat16> {
  static constexpr int kVec = 8;
  __device__ static float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
  __device__ static __nv_bfloat16 from_f(float v) { return __float2bfloat16_rn(v); }
};

// A 16-byte vector of T, loaded / stored with one 128-bit access.
template <typename T> struct alignas(16) Vec16 {
  T v[Elem<T>::kVec];
};

template <typename T>
__device__ __forceinline__ Vec16<T> ldg16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  return r;
}
// streaming variants: data touched exactly once should not displace reusable lines
template <typename T>
__device__ __forceinline__ Vec16<T> ldcs16(const T* p) {
  Vec16<T> r;
  *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  return r;
}
template <typename T>
__device__ __forceinline__ void stcs16(T* p, const Vec16<T>& r) {
  __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
}

__host__ __device__ __forceinline__ int64_t min64(int64_t a, int64_t b) { return a < b ? a : b; }

// ---- math ---------------------------------------------------------------------------
__device__ __forceinline__ float ex2f(float x) {       // 2^x on the MUFU pipe
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ float softplusf(float x) {   // torch semantics: threshold 20
  return x > 20.f ? x : log1pf(__expf(x));
}
__device__ __forceinline__ float sigmoidf(float x) { return 1.f / (1.f + __expf(-x)); }
// Cheaper forms for the streaming kernels: approximate reciprocal / logarithm, with a short
// series where 1 + e^x would lose the small term to rounding.  Relative error below 1e-5.
__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.f, 1.f + __expf(-x)); }
__device__ __forceinline__ float softplus_fast(float x) {
  if (x > 20.f) return x;
  const float e = __expf(x);
  return e < 1e-2f ? e * (1.f - e * (0.5f - e * (1.f / 3.f))) : __logf(1.f + e);
}

// Two-lane versions of softplus_fast and x*sigmoid_fast(x) on the packed f32x2 instructions (the MUFU
// calls stay scalar): the per-element warps of the fused kernels are bound by instruction issue.
__device__ __forceinline__ float2 softplus_fast2(float2 x) {
  const float2 m = __fmul2_rn(x, make_float2(1.4426950408889634f, 1.4426950408889634f));
  const float2 e = make_float2(ex2f(m.x), ex2f(m.y));
  // e*(1 - e*(1/2 - e/3)) where 1 + e would lose the small term, log(1 + e) elsewhere
  const float2 third = make_float2(-1.f / 3.f, -1.f / 3.f), half = make_float2(0.5f, 0.5f), one = make_float2(1.f, 1.f);
  const float2 nh = make_float2(-1.f, -1.f);
  const float2 inner = __ffma2_rn(e, third, half);                       // 1/2 - e/3
  const float2 poly = __fmul2_rn(e, __ffma2_rn(__fmul2_rn(e, inner), nh, one));
  const float2 s = __fadd2_rn(e, one);
  const float ln2 = 0.6931471805599453f;
  const float2 lg = make_float2(__log2f(s.x) * ln2, __log2f(s.y) * ln2);
  float2 r;
  r.x = x.x > 20.f ? x.x : (e.x < 1e-2f ? poly.x : lg.x);
  r.y = x.y > 20.f ? x.y : (e.y < 1e-2f ? poly.y : lg.y);
  return r;
}
__device__ __forceinline__ float2 sigmoid_fast2(float2 x) {
  const float2 m = __fmul2_rn(x, make_float2(-1.4426950408889634f, -1.4426950408889634f));
  const float2 d = __fadd2_rn(make_float2(ex2f(m.x), ex2f(m.y)), make_float2(1.f, 1.f));
  return make_float2(__fdividef(1.f, d.x), __fdividef(1.f, d.y));
}

// ---- packed float2 arithmetic (one issue slot for two lanes of FMA work) ------------
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
  float2 d;
  asm("{.reg .b64 ra, rb, rc, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mov.b64 rc, {%6, %7};\n\t"
      "fma.rn.f32x2 rd, ra, rb, rc;\n\t"
      "mov.b64 {%0, %1}, rd;}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y));
  return d;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
  float2 d;
  asm("{.reg .b64 ra, rb, rd;\n\t"
      "mov.b64 ra, {%2, %3};\n\t"
      "mov.b64 rb, {%4, %5};\n\t"
      "mul.rn.f32x2 rd, ra, rb;\n\t"
      "mov.b64 {%0, %1}, rd;}"
      : "=f"(d.x), "=f"(d.y)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y));
  return d;
}

// ---- CTA-local mbarriers with bounded waits --------------------------------------------
// Producer and consumer warps of one CTA hand tiles to each other through these.  A wait
// that does not complete within kSpinLimit polls gives up and reports it; nothing spins
// without a limit.
#ifndef MB200_POLL_NS
#define MB200_POLL_NS 100
#endif
constexpr int kSpinLimit = 1 << 22;          // polls at least 100 ns apart: gives up after roughly a second
enum { MB200_DEV_OK = 0, MB200_DEV_WAIT_TIMEOUT = 1 };

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint64_t* bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
  asm volatile("{\n\t.reg .b64 st;\n\tmbarrier.arrive.shared::cta.b64 st, [%0];\n\t}" ::"r"(smem_u32(bar))
               : "memory");
}
// true when the phase with the given parity has completed; false after kSpinLimit polls.
// A pending poll is followed by a short sleep: a waiting warp must not spend issue slots and
// shared-memory bandwidth (the poll is a shared-memory access) that the working warps need.
__device__ __forceinline__ bool mbar_poll(uint32_t addr, int parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(addr), "r"(parity)
      : "memory");
  return ok != 0;
}
// Non-blocking test of a phase.  Issued ahead of the work that does not need the answer, it takes
// the barrier's round trip through the shared-memory pipe off the critical path; mbar_wait follows
// only when the answer was "not yet".
__device__ __forceinline__ bool mbar_test(uint64_t* bar, int parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok)
      : "r"(smem_u32(bar)), "r"(parity)
      : "memory");
  return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, int parity) {
  const uint32_t addr = smem_u32(bar);
  if (mbar_poll(addr, parity)) return true;
  for (int i = 0; i < kSpinLimit; ++i) {
    if (MB200_POLL_NS > 0) __nanosleep(MB200_POLL_NS);
    if (mbar_poll(addr, parity)) return true;
  }
  return false;
}

// ---- host-side helpers ----------------------------------------------------------------
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

inline int check_launch() {
  return cudaGetLastError() == cudaSuccess ? MB200_OK : MB200_ELAUNCH;
}

}  // namespace mb200
