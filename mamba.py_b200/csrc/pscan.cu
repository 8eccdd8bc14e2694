// PScan operator on (B, L, D, N) tensors: H[t] = A[t]*H[t-1] + X[t] along L, and its backward.
//
// Mapping.  The D*N recurrences of one batch row are independent and contiguous in memory,
// so a thread owns one 16-byte vector of channels and walks L serially, keeping the state in
// registers: every input element is read once and every output element written once, with
// fully coalesced 128-bit accesses (a warp covers 512 contiguous bytes of a (b, t) slab).
// The loads of a block of kUnroll timesteps do not depend on the recurrence and are issued
// together, which is what keeps enough bytes in flight to cover HBM latency.
//
// When B*D*N alone cannot fill the GPU, L is cut into segments handled by different CTAs:
// a first pass reduces every segment to (prod A, state reached from zero), a tiny fold
// turns those into the state entering each segment, and the main pass starts from it.  That
// costs one extra read of the inputs and is only chosen when the single pass would leave
// most SMs idle.
#include <initializer_list>
#include "common.cuh"

namespace mb200 {
namespace {

constexpr int kUnroll = 8;
constexpr int kThreads = 128;

struct PscanDims {
  int64_t L, CH;          // sequence length, channels per batch row (D*N)
  int64_t seg_len;        // timesteps per segment
  int nseg;
};

template <typename T, int V> struct Chan {             // V channels of one timestep
  T v[V];
};
template <typename T, int V>
__device__ __forceinline__ Chan<T, V> load_chan(const T* p) {
  Chan<T, V> r;
  if constexpr (V == 1) {
    r.v[0] = *p;
  } else {
    static_assert(sizeof(T) * V == 16, "vector path is 16 bytes wide");
    *reinterpret_cast<uint4*>(&r) = __ldcs(reinterpret_cast<const uint4*>(p));
  }
  return r;
}
template <typename T, int V>
__device__ __forceinline__ void store_chan(T* p, const Chan<T, V>& r) {
  if constexpr (V == 1) {
    *p = r.v[0];
  } else {
    __stcs(reinterpret_cast<uint4*>(p), *reinterpret_cast<const uint4*>(&r));
  }
}

// ------------------------------------------------------------------ forward, main pass
// state_in: (B, nseg, CH) float32 or NULL (zero).  hT: (B, CH) or NULL.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
pscan_fwd_kernel(const T* __restrict__ A, const T* __restrict__ X, T* __restrict__ H,
                 PscanDims d, int64_t a_sb, int64_t a_sl, int64_t x_sb, int64_t x_sl,
                 int64_t h_sb, int64_t h_sl, const float* __restrict__ state_in,
                 float* __restrict__ hT) {
  const int64_t c = (int64_t(blockIdx.x) * kThreads + threadIdx.x) * V;
  if (c >= d.CH) return;
  const int64_t b = blockIdx.y, s = blockIdx.z;
  const int64_t t0 = s * d.seg_len;
  const int64_t t1 = min(d.L, t0 + d.seg_len);
  float h[V];
#pragma unroll
  for (int i = 0; i < V; ++i) h[i] = 0.f;
  if (state_in) {
    const float* p = state_in + (b * d.nseg + s) * d.CH + c;
#pragma unroll
    for (int i = 0; i < V; ++i) h[i] = p[i];
  }
  const T* a = A + b * a_sb + t0 * a_sl + c;
  const T* x = X + b * x_sb + t0 * x_sl + c;
  T* o = H + b * h_sb + t0 * h_sl + c;
  int64_t t = t0;
  for (; t + kUnroll <= t1; t += kUnroll) {
    Chan<T, V> av[kUnroll], xv[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      av[u] = load_chan<T, V>(a + u * a_sl);
      xv[u] = load_chan<T, V>(x + u * x_sl);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      Chan<T, V> ov;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        h[i] = fmaf(Elem<T>::to_f(av[u].v[i]), h[i], Elem<T>::to_f(xv[u].v[i]));
        ov.v[i] = Elem<T>::from_f(h[i]);
      }
      store_chan<T, V>(o + u * h_sl, ov);
    }
    a += kUnroll * a_sl; x += kUnroll * x_sl; o += kUnroll * h_sl;
  }
  for (; t < t1; ++t) {
    Chan<T, V> av = load_chan<T, V>(a), xv = load_chan<T, V>(x), ov;
#pragma unroll
    for (int i = 0; i < V; ++i) {
      h[i] = fmaf(Elem<T>::to_f(av.v[i]), h[i], Elem<T>::to_f(xv.v[i]));
      ov.v[i] = Elem<T>::from_f(h[i]);
    }
    store_chan<T, V>(o, ov);
    a += a_sl; x += x_sl; o += h_sl;
  }
  if (hT && s == d.nseg - 1) {
#pragma unroll
    for (int i = 0; i < V; ++i) hT[b * d.CH + c + i] = h[i];
  }
}

// ------------------------------------------------------------ segment aggregates (fwd)
// wsP/wsS: (B, nseg, CH): product of A over the segment / state reached from zero.
template <typename T, int V>
__global__ void __launch_bounds__(kThreads)
pscan_fwd_agg_kernel(const T* __restrict__ A, const T* __restrict__ X, PscanDims d,
                     int64_t a_sb, int64_t a_sl, int64_t x_sb, int64_t x_sl,
                     float* __restrict__ wsP, float* __restrict__ wsS) {
  const int64_t c = (int64_t(blockIdx.x) * kThreads + threadIdx.x) * V;
  if (c >= d.CH) return;
  const int64_t b = blockIdx.y, s = blockIdx.z;
  const int64_t t0 = s * d.seg_len;
  const int64_t t1 = min(d.L, t0 + d.seg_len);
  float h[V], P[V];
#pragma unroll
  for (int i = 0; i < V; ++i) { h[i] = 0.f; P[i] = 1.f; }
  const T* a = A + b * a_sb + t0 * a_sl + c;
  const T* x = X + b * x_sb + t0 * x_sl + c;
  int64_t t = t0;
  for (; t + kUnroll <= t1; t += kUnroll) {
    Chan<T, V> av[kUnroll], xv[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      av[u] = load_chan<T, V>(a + u * a_sl);
      xv[u] = load_chan<T, V>(x + u * x_sl);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u)
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float af = Elem<T>::to_f(av[u].v[i]);
        h[i] = fmaf(af, h[i], Elem<T>::to_f(xv[u].v[i]));
        P[i] *= af;
      }
    a += kUnroll * a_sl; x += kUnroll * x_sl;
  }
  for (; t < t1; ++t) {
    Chan<T, V> av = load_chan<T, V>(a), xv = load_chan<T, V>(x);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float af = Elem<T>::to_f(av.v[i]);
      h[i] = fmaf(af, h[i], Elem<T>::to_f(xv.v[i]));
      P[i] *= af;
    }
    a += a_sl; x += x_sl;
  }
  const int64_t w = (b * d.nseg + s) * d.CH + c;
#pragma unroll
  for (int i = 0; i < V; ++i) { wsP[w + i] = P[i]; wsS[w + i] = h[i]; }
}

// Fold over segments, in place: wsS[b, s, c] <- the state ENTERING segment s.
// reverse: segments are folded from the last to the first (carry arriving from the right).
__global__ void pscan_fold_kernel(const float* __restrict__ wsP, float* __restrict__ wsS,
                                  const float* __restrict__ start, int64_t CH, int nseg,
                                  int reverse) {
  const int64_t c = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (c >= CH) return;
  const int64_t b = blockIdx.y;
  float cur = start ? start[b * CH + c] : 0.f;
  for (int i = 0; i < nseg; ++i) {
    const int s = reverse ? nseg - 1 - i : i;
    const int64_t w = (b * nseg + s) * CH + c;
    const float P = wsP[w], S = wsS[w];
    wsS[w] = cur;
    cur = fmaf(P, cur, S);
  }
}

// ----------------------------------------------------------------- backward, main pass
// carry_in: (B, nseg, CH) = A[t1]*G[t1] arriving at the right end of each segment, or NULL.
// Walks t from t1-1 down to t0:  G[t] = gH[t] + carry;  gA[t] = H[t-1]*G[t];  carry = A[t]*G[t].
template <typename T, int V, bool kAggOnly>
__global__ void __launch_bounds__(kThreads)
pscan_bwd_kernel(const T* __restrict__ A, const T* __restrict__ H, const T* __restrict__ GH,
                 T* __restrict__ GA, T* __restrict__ GX, PscanDims d,
                 int64_t a_sb, int64_t a_sl, int64_t h_sb, int64_t h_sl,
                 int64_t g_sb, int64_t g_sl, int64_t ga_sb, int64_t ga_sl,
                 int64_t gx_sb, int64_t gx_sl, const float* __restrict__ carry_in,
                 const float* __restrict__ h0, float* __restrict__ wsP, float* __restrict__ wsS) {
  const int64_t c = (int64_t(blockIdx.x) * kThreads + threadIdx.x) * V;
  if (c >= d.CH) return;
  const int64_t b = blockIdx.y, s = blockIdx.z;
  const int64_t t0 = s * d.seg_len;
  const int64_t t1 = min(d.L, t0 + d.seg_len);
  float cy[V], P[V];
#pragma unroll
  for (int i = 0; i < V; ++i) { cy[i] = 0.f; P[i] = 1.f; }
  if (!kAggOnly && carry_in) {
    const float* p = carry_in + (b * d.nseg + s) * d.CH + c;
#pragma unroll
    for (int i = 0; i < V; ++i) cy[i] = p[i];
  }
  const T* a = A + b * a_sb + c;
  const T* hh = H + b * h_sb + c;
  const T* g = GH + b * g_sb + c;
  T* ga = GA + b * ga_sb + c;
  T* gx = GX + b * gx_sb + c;
  int64_t t = t1 - 1;
  // blocks of kUnroll timesteps whose H[t-1] all exist (t - kUnroll + 1 >= 1)
  for (; t - kUnroll + 1 >= t0 && t - kUnroll + 1 >= 1; t -= kUnroll) {
    Chan<T, V> av[kUnroll], gv[kUnroll], hv[kUnroll];
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      av[u] = load_chan<T, V>(a + (t - u) * a_sl);
      gv[u] = load_chan<T, V>(g + (t - u) * g_sl);
      if (!kAggOnly) hv[u] = load_chan<T, V>(hh + (t - u - 1) * h_sl);
    }
#pragma unroll
    for (int u = 0; u < kUnroll; ++u) {
      Chan<T, V> oa, ox;
#pragma unroll
      for (int i = 0; i < V; ++i) {
        const float G = Elem<T>::to_f(gv[u].v[i]) + cy[i];
        const float af = Elem<T>::to_f(av[u].v[i]);
        cy[i] = af * G;
        if (kAggOnly) {
          P[i] *= af;
        } else {
          ox.v[i] = Elem<T>::from_f(G);
          oa.v[i] = Elem<T>::from_f(Elem<T>::to_f(hv[u].v[i]) * G);
        }
      }
      if (!kAggOnly) {
        store_chan<T, V>(gx + (t - u) * gx_sl, ox);
        store_chan<T, V>(ga + (t - u) * ga_sl, oa);
      }
    }
  }
  for (; t >= t0; --t) {
    Chan<T, V> av = load_chan<T, V>(a + t * a_sl), gv = load_chan<T, V>(g + t * g_sl), hv, oa, ox;
    if (!kAggOnly && t >= 1) hv = load_chan<T, V>(hh + (t - 1) * h_sl);
#pragma unroll
    for (int i = 0; i < V; ++i) {
      const float G = Elem<T>::to_f(gv.v[i]) + cy[i];
      const float af = Elem<T>::to_f(av.v[i]);
      cy[i] = af * G;
      if (kAggOnly) {
        P[i] *= af;
      } else {
        float hp;
        if (t >= 1) hp = Elem<T>::to_f(hv.v[i]);
        else hp = h0 ? h0[b * d.CH + c + i] : 0.f;
        ox.v[i] = Elem<T>::from_f(G);
        oa.v[i] = Elem<T>::from_f(hp * G);
      }
    }
    if (!kAggOnly) {
      store_chan<T, V>(gx + t * gx_sl, ox);
      store_chan<T, V>(ga + t * ga_sl, oa);
    }
  }
  if (kAggOnly) {
    const int64_t w = (b * d.nseg + s) * d.CH + c;
#pragma unroll
    for (int i = 0; i < V; ++i) { wsP[w + i] = P[i]; wsS[w + i] = cy[i]; }
  }
}

int pick_segments(int64_t B, int64_t L, int64_t CH) {
  int dev = 0, sms = 148;
  cudaGetDevice(&dev);
  cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t threads = B * ((CH + 3) / 4);
  if (threads >= int64_t(sms) * 256 || L < 128) return 1;
  int64_t want = (int64_t(sms) * 512 + threads - 1) / threads;
  int64_t cap = L / 64;
  int64_t s = want < cap ? want : cap;
  return s < 1 ? 1 : int(s);
}

template <typename T>
bool vec_ok(int64_t CH, std::initializer_list<const void*> ptrs,
            std::initializer_list<int64_t> strides) {
  constexpr int V = Elem<T>::kVec;
  if (CH % V) return false;
  for (const void* p : ptrs) if (p && !aligned16(p)) return false;
  for (int64_t s : strides) if (s % V) return false;
  return true;
}

template <typename T>
int fwd_impl(const void* A_, const void* X_, void* H_, int64_t B, int64_t L, int64_t CH,
             int64_t a_sb, int64_t a_sl, int64_t x_sb, int64_t x_sl, int64_t h_sb, int64_t h_sl,
             const float* h0, float* hT, float* ws, int nseg, cudaStream_t st) {
  const T* A = static_cast<const T*>(A_);
  const T* X = static_cast<const T*>(X_);
  T* H = static_cast<T*>(H_);
  PscanDims d{L, CH, (L + nseg - 1) / nseg, nseg};
  float* wsP = ws;
  float* wsS = ws ? ws + B * nseg * CH : nullptr;
  const bool vec = vec_ok<T>(CH, {A_, X_, H_}, {a_sb, a_sl, x_sb, x_sl, h_sb, h_sl});
  constexpr int V = Elem<T>::kVec;
  const int v = vec ? V : 1;
  dim3 grid(unsigned((CH + int64_t(v) * kThreads - 1) / (int64_t(v) * kThreads)), unsigned(B),
            unsigned(nseg));
  const float* state_in = h0;
  if (nseg > 1) {
    if (vec) pscan_fwd_agg_kernel<T, V><<<grid, kThreads, 0, st>>>(A, X, d, a_sb, a_sl, x_sb, x_sl, wsP, wsS);
    else pscan_fwd_agg_kernel<T, 1><<<grid, kThreads, 0, st>>>(A, X, d, a_sb, a_sl, x_sb, x_sl, wsP, wsS);
    dim3 fg(unsigned((CH + 255) / 256), unsigned(B));
    pscan_fold_kernel<<<fg, 256, 0, st>>>(wsP, wsS, h0, CH, nseg, 0);
    state_in = wsS;
  }
  if (vec) pscan_fwd_kernel<T, V><<<grid, kThreads, 0, st>>>(A, X, H, d, a_sb, a_sl, x_sb, x_sl, h_sb, h_sl, state_in, hT);
  else pscan_fwd_kernel<T, 1><<<grid, kThreads, 0, st>>>(A, X, H, d, a_sb, a_sl, x_sb, x_sl, h_sb, h_sl, state_in, hT);
  return check_launch();
}

template <typename T>
int bwd_impl(const void* A_, const void* H_, const void* G_, void* GA_, void* GX_,
             int64_t B, int64_t L, int64_t CH,
             int64_t a_sb, int64_t a_sl, int64_t h_sb, int64_t h_sl, int64_t g_sb, int64_t g_sl,
             int64_t ga_sb, int64_t ga_sl, int64_t gx_sb, int64_t gx_sl,
             const float* h0, float* ws, int nseg, cudaStream_t st) {
  const T* A = static_cast<const T*>(A_);
  const T* H = static_cast<const T*>(H_);
  const T* G = static_cast<const T*>(G_);
  T* GA = static_cast<T*>(GA_);
  T* GX = static_cast<T*>(GX_);
  PscanDims d{L, CH, (L + nseg - 1) / nseg, nseg};
  float* wsP = ws;
  float* wsS = ws ? ws + B * nseg * CH : nullptr;
  const bool vec = vec_ok<T>(CH, {A_, H_, G_, GA_, GX_},
                             {a_sb, a_sl, h_sb, h_sl, g_sb, g_sl, ga_sb, ga_sl, gx_sb, gx_sl});
  constexpr int V = Elem<T>::kVec;
  const int v = vec ? V : 1;
  dim3 grid(unsigned((CH + int64_t(v) * kThreads - 1) / (int64_t(v) * kThreads)), unsigned(B),
            unsigned(nseg));
  const float* carry_in = nullptr;
#define MB200_BWD_LAUNCH(VV, AGG)                                                              \
  pscan_bwd_kernel<T, VV, AGG><<<grid, kThreads, 0, st>>>(A, H, G, GA, GX, d, a_sb, a_sl, h_sb, \
      h_sl, g_sb, g_sl, ga_sb, ga_sl, gx_sb, gx_sl, carry_in, h0, wsP, wsS)
  if (nseg > 1) {
    if (vec) MB200_BWD_LAUNCH(V, true); else MB200_BWD_LAUNCH(1, true);
    dim3 fg(unsigned((CH + 255) / 256), unsigned(B));
    pscan_fold_kernel<<<fg, 256, 0, st>>>(wsP, wsS, nullptr, CH, nseg, 1);
    carry_in = wsS;
  }
  if (vec) MB200_BWD_LAUNCH(V, false); else MB200_BWD_LAUNCH(1, false);
#undef MB200_BWD_LAUNCH
  return check_launch();
}

}  // namespace
}  // namespace mb200

using namespace mb200;

extern "C" int mb200_pscan_segments(int64_t B, int64_t L, int64_t DN) {
  if (B <= 0 || L <= 0 || DN <= 0) return 1;
  return pick_segments(B, L, DN);
}

extern "C" int mb200_pscan_fwd(const void* A, const void* X, void* H, int64_t B, int64_t L,
                               int64_t DN, int64_t a_sb, int64_t a_sl, int64_t x_sb, int64_t x_sl,
                               int64_t h_sb, int64_t h_sl, const float* h0, float* hT,
                               float* ws, int nseg, int dtype, void* stream) {
  if (B < 0 || L < 0 || DN < 0 || nseg < 1) return MB200_EINVAL;
  if (B == 0 || L == 0 || DN == 0) return MB200_OK;
  if (!A || !X || !H || (nseg > 1 && !ws)) return MB200_EINVAL;
  if (B > 65535 || nseg > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MB200_F32)
    return fwd_impl<float>(A, X, H, B, L, DN, a_sb, a_sl, x_sb, x_sl, h_sb, h_sl, h0, hT, ws, nseg, st);
  if (dtype == MB200_BF16)
    return fwd_impl<__nv_bfloat16>(A, X, H, B, L, DN, a_sb, a_sl, x_sb, x_sl, h_sb, h_sl, h0, hT, ws, nseg, st);
  return MB200_EDTYPE;
}

extern "C" int mb200_pscan_bwd(const void* A, const void* H, const void* gradH, void* gradA,
                               void* gradX, int64_t B, int64_t L, int64_t DN,
                               int64_t a_sb, int64_t a_sl, int64_t h_sb, int64_t h_sl,
                               int64_t g_sb, int64_t g_sl, int64_t ga_sb, int64_t ga_sl,
                               int64_t gx_sb, int64_t gx_sl, const float* h0,
                               float* ws, int nseg, int dtype, void* stream) {
  if (B < 0 || L < 0 || DN < 0 || nseg < 1) return MB200_EINVAL;
  if (B == 0 || L == 0 || DN == 0) return MB200_OK;
  if (!A || !H || !gradH || !gradA || !gradX || (nseg > 1 && !ws)) return MB200_EINVAL;
  if (B > 65535 || nseg > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MB200_F32)
    return bwd_impl<float>(A, H, gradH, gradA, gradX, B, L, DN, a_sb, a_sl, h_sb, h_sl, g_sb, g_sl,
                           ga_sb, ga_sl, gx_sb, gx_sl, h0, ws, nseg, st);
  if (dtype == MB200_BF16)
    return bwd_impl<__nv_bfloat16>(A, H, gradH, gradA, gradX, B, L, DN, a_sb, a_sl, h_sb, h_sl,
                                   g_sb, g_sl, ga_sb, ga_sl, gx_sb, gx_sl, h0, ws, nseg, st);
  return MB200_EDTYPE;
}

// ---------------------------------------------------------------------------------------------
// Allocation-free variant of the forward.  The segmented forward needs scratch (the per-segment
// aggregates).  Callers that cannot obtain device memory at call time get that scratch from a
// fixed array that lives in the library image instead: every GPU that loads the library holds
// kStaticWsFloats * 4 bytes (8 MiB) for it until the process exits.
//
// In host code `g_static_ws` is only a stand-in symbol, not a device address; the address a
// kernel can use is looked up once per device with cudaGetSymbolAddress while that device is
// current, and cached.
namespace mb200 {
namespace {
constexpr int64_t kStaticWsFloats = int64_t(1) << 21;
static __device__ __align__(256) float g_static_ws[kStaticWsFloats];

constexpr int kMaxDevices = 64;
float* g_static_ws_addr[kMaxDevices] = {};

// Returns the device address of g_static_ws on the current device, or nullptr on failure.
float* static_ws_for_current_device() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return nullptr;
  float* p = __atomic_load_n(&g_static_ws_addr[dev], __ATOMIC_ACQUIRE);
  if (p) return p;
  void* addr = nullptr;
  if (cudaGetSymbolAddress(&addr, g_static_ws) != cudaSuccess || !addr) {
    (void)cudaGetLastError();
    return nullptr;
  }
  // two threads racing here look up the same address; either store is fine
  __atomic_store_n(&g_static_ws_addr[dev], static_cast<float*>(addr), __ATOMIC_RELEASE);
  return static_cast<float*>(addr);
}
}  // namespace
}  // namespace mb200

extern "C" int64_t mb200_pscan_noalloc_max_ws_floats(void) { return kStaticWsFloats; }

extern "C" int mb200_pscan_fwd_noalloc(const void* A, const void* X, void* H, int64_t B, int64_t L,
                                       int64_t DN, int64_t a_sb, int64_t a_sl, int64_t x_sb,
                                       int64_t x_sl, int64_t h_sb, int64_t h_sl, const float* h0,
                                       float* hT, int nseg, int dtype, void* stream) {
  if (B < 0 || L < 0 || DN < 0 || nseg < 0) return MB200_EINVAL;
  if (B == 0 || L == 0 || DN == 0) return MB200_OK;
  if (!A || !X || !H) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (nseg == 0) nseg = pick_segments(B, L, DN);
  if (B > 65535 || nseg > 65535) return MB200_ETOOBIG;
  float* ws = nullptr;
  if (nseg > 1) {
    // 2 * B * nseg * DN floats of aggregates must fit the fixed array
    if (B * int64_t(nseg) > kStaticWsFloats / 2 / DN) return MB200_ETOOBIG;
    ws = static_ws_for_current_device();
    if (!ws) return MB200_ESETUP;
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dtype == MB200_F32)
    return fwd_impl<float>(A, X, H, B, L, DN, a_sb, a_sl, x_sb, x_sl, h_sb, h_sl, h0, hT, ws, nseg, st);
  return fwd_impl<__nv_bfloat16>(A, X, H, B, L, DN, a_sb, a_sl, x_sb, x_sl, h_sb, h_sl, h0, hT, ws, nseg, st);
}
