// Register-staged tile movement between global and shared memory.
//
// A tile is ROWS timesteps by COLS channels of element type T.  The CTA's kThreadsPerCta
// threads each own a fixed set of KV-element vectors of the tile (KV = 16 bytes worth of
// elements on the aligned path, 1 on the fallback path), so a tile is fetched with
// 128-bit coalesced loads into registers while the previous tile is being computed on,
// and committed to shared memory afterwards.
#pragma once
#include "common.cuh"

namespace mb200 {

constexpr int kThreadsPerCta = 128;

template <typename T, int KV> struct TVec {
  T v[KV];
};

template <typename T, int KV>
__device__ __forceinline__ TVec<T, KV> tvec_zero() {
  TVec<T, KV> r;
#pragma unroll
  for (int i = 0; i < KV; ++i) r.v[i] = Elem<T>::from_f(0.f);
  return r;
}

template <typename T, int KV>
__device__ __forceinline__ TVec<T, KV> tvec_load(const T* p) {
  TVec<T, KV> r;
  if constexpr (KV == 1) {
    r.v[0] = __ldg(p);
  } else {
    static_assert(sizeof(T) * KV == 16, "aligned path moves 16 bytes");
    *reinterpret_cast<uint4*>(&r) = __ldg(reinterpret_cast<const uint4*>(p));
  }
  return r;
}

template <typename T, int KV>
__device__ __forceinline__ void tvec_store(T* p, const TVec<T, KV>& r) {
  if constexpr (KV == 1) {
    *p = r.v[0];
  } else {
    *reinterpret_cast<uint4*>(p) = *reinterpret_cast<const uint4*>(&r);
  }
}

// Static description of how a ROWS x COLS tile is split over NT cooperating threads
// (tid is the thread's index among those NT threads).
template <int ROWS, int COLS, int KV, int NT = kThreadsPerCta> struct TileMap {
  static_assert(COLS % KV == 0, "tile width must hold whole vectors");
  static constexpr int kVecPerRow = COLS / KV;
  static constexpr int kVecs = ROWS * kVecPerRow;
  static constexpr int kPerThread = (kVecs + NT - 1) / NT;
  __device__ static __forceinline__ bool owns(int i, int tid) {
    return tid + i * NT < kVecs;
  }
  __device__ static __forceinline__ int row(int i, int tid) {
    return (tid + i * NT) / kVecPerRow;
  }
  __device__ static __forceinline__ int col(int i, int tid) {
    return ((tid + i * NT) % kVecPerRow) * KV;
  }
};

// Registers of one thread's share of a tile.
template <typename T, int ROWS, int COLS, int KV, int NT = kThreadsPerCta> struct TileRegs {
  using Map = TileMap<ROWS, COLS, KV, NT>;
  TVec<T, KV> r[Map::kPerThread];

  // base points at (row 0, col 0) of the tile; rows >= rows_ok or cols >= cols_ok read as 0.
  __device__ __forceinline__ void load(const T* base, int64_t row_stride, int rows_ok,
                                       int cols_ok, int tid) {
#pragma unroll
    for (int i = 0; i < Map::kPerThread; ++i) {
      const int rr = Map::row(i, tid), cc = Map::col(i, tid);
      if (Map::owns(i, tid) && rr < rows_ok && cc < cols_ok)
        r[i] = tvec_load<T, KV>(base + rr * row_stride + cc);
      else
        r[i] = tvec_zero<T, KV>();
    }
  }
  __device__ __forceinline__ void store(T* base, int64_t row_stride, int rows_ok, int cols_ok,
                                        int tid) const {
#pragma unroll
    for (int i = 0; i < Map::kPerThread; ++i) {
      const int rr = Map::row(i, tid), cc = Map::col(i, tid);
      if (Map::owns(i, tid) && rr < rows_ok && cc < cols_ok)
        tvec_store<T, KV>(base + rr * row_stride + cc, r[i]);
    }
  }
};

}  // namespace mb200
