// Single-token decode kernels: the SSM state update of MambaBlock.ssm_step and the
// conv-window update of MambaBlock.step.  Both are pure streaming work: the (B, ED, N)
// float32 state is read once and written once per layer-step, which is what bounds them.
//
// Mapping for the state update: N/4 lanes share a channel, each lane moves one float4 of the
// state (so a warp reads 512 contiguous bytes of h), computes its four decays and partial
// C-contraction, and the lanes of a channel combine with warp shuffles.
#include "common.cuh"
#include "sscan.cuh"

namespace mb200 {
namespace {

constexpr int kStepThreads = 256;

// States per lane.  The work per (batch row, channel) - softplus, the gate, index arithmetic - is repeated
// by every lane of the channel, and the kernel is bound as much by instruction issue as by memory, so
// a lane takes MB200_STEP_SPL consecutive states (N / SPL lanes share a channel).
#ifndef MB200_STEP_SPL
#define MB200_STEP_SPL 8
#endif

template <typename T, int N, bool kVecBC>
__global__ void __launch_bounds__(kStepThreads)
ssm_step_kernel(const T* __restrict__ x, const T* __restrict__ delta, const T* __restrict__ z,
                const float* __restrict__ A, const T* __restrict__ Bm, const T* __restrict__ Cm,
                const float* __restrict__ D, const float* __restrict__ delta_bias,
                const float* __restrict__ h_in, float* __restrict__ h_out, T* __restrict__ y,
                int64_t ED, int64_t x_sb, int64_t d_sb, int64_t z_sb, int64_t b_sb,
                int64_t c_sb, int64_t y_sb, int flags) {
  constexpr int kSPL = MB200_STEP_SPL < N ? MB200_STEP_SPL : N;   // states per lane
  constexpr int kV = kSPL / 4;                                    // float4 per lane
  constexpr int kLPE = N / kSPL;                                  // lanes per channel
  constexpr int kEPB = kStepThreads / kLPE;                       // channels per CTA
  const int tid = threadIdx.x;
  const int q = tid % kLPE;
  const int64_t e = int64_t(blockIdx.x) * kEPB + tid / kLPE;
  const int64_t b = blockIdx.y;
  const bool ok = e < ED;
  float yv = 0.f, xv = 0.f;
  if (ok) {
    // the state is the only large stream: get it moving first, everything else is small
    float4 hv[kV];
    const float4* hp = reinterpret_cast<const float4*>(h_in + (b * ED + e) * N + kSPL * q);
#pragma unroll
    for (int v = 0; v < kV; ++v) hv[v] = h_in ? __ldcs(hp + v) : make_float4(0.f, 0.f, 0.f, 0.f);
    float4 Av[kV];
#pragma unroll
    for (int v = 0; v < kV; ++v) Av[v] = *reinterpret_cast<const float4*>(A + e * N + kSPL * q + 4 * v);
    float b4[kSPL], c4[kSPL];
    if constexpr (kVecBC) {
#pragma unroll
      for (int v = 0; v < kV; ++v) {
        const Vec4<T> bv = *reinterpret_cast<const Vec4<T>*>(Bm + b * b_sb + kSPL * q + 4 * v);
        const Vec4<T> cv = *reinterpret_cast<const Vec4<T>*>(Cm + b * c_sb + kSPL * q + 4 * v);
#pragma unroll
        for (int j = 0; j < 4; ++j) { b4[4 * v + j] = Elem<T>::to_f(bv.v[j]); c4[4 * v + j] = Elem<T>::to_f(cv.v[j]); }
      }
    } else {
#pragma unroll
      for (int j = 0; j < kSPL; ++j) {
        b4[j] = Elem<T>::to_f(Bm[b * b_sb + kSPL * q + j]);
        c4[j] = Elem<T>::to_f(Cm[b * c_sb + kSPL * q + j]);
      }
    }
    xv = Elem<T>::to_f(x[b * x_sb + e]);
    float dv = Elem<T>::to_f(delta[b * d_sb + e]);
    if (flags & MB200_DELTA_SOFTPLUS) dv = softplus_fast(dv + delta_bias[e]);
    const float dxs = dv * xv, d2s = dv * kLog2e;
    const float2 dx = make_float2(dxs, dxs), d2 = make_float2(d2s, d2s);
    float2 y2 = make_float2(0.f, 0.f);
    float4* op = reinterpret_cast<float4*>(h_out + (b * ED + e) * N + kSPL * q);
#pragma unroll
    for (int v = 0; v < kV; ++v) {
      // packed f32x2 arithmetic: two states per instruction (the decays stay scalar ex2)
      const float2 e01 = __fmul2_rn(d2, make_float2(Av[v].x, Av[v].y)), e23 = __fmul2_rn(d2, make_float2(Av[v].z, Av[v].w));
      const float2 a01 = make_float2(ex2f(e01.x), ex2f(e01.y)), a23 = make_float2(ex2f(e23.x), ex2f(e23.y));
      const float2 h01 = __ffma2_rn(a01, make_float2(hv[v].x, hv[v].y), __fmul2_rn(dx, make_float2(b4[4 * v], b4[4 * v + 1])));
      const float2 h23 = __ffma2_rn(a23, make_float2(hv[v].z, hv[v].w), __fmul2_rn(dx, make_float2(b4[4 * v + 2], b4[4 * v + 3])));
      y2 = __ffma2_rn(h01, make_float2(c4[4 * v], c4[4 * v + 1]), y2);
      y2 = __ffma2_rn(h23, make_float2(c4[4 * v + 2], c4[4 * v + 3]), y2);
      __stcs(op + v, make_float4(h01.x, h01.y, h23.x, h23.y));
    }
    yv = y2.x + y2.y;
  }
#pragma unroll
  for (int s = kLPE / 2; s >= 1; s >>= 1) yv += __shfl_xor_sync(0xffffffffu, yv, s);
  if (ok && q == 0) {
    yv = fmaf(D ? D[e] : 0.f, xv, yv);
    if (z) {
      const float zv = Elem<T>::to_f(z[b * z_sb + e]);
      yv *= zv * sigmoid_fast(zv);
    }
    y[b * y_sb + e] = Elem<T>::from_f(yv);
  }
}

// xc = silu(sum_k w[e,k]*win[k] + bias[e]) with win = [conv_in[b,e,:], xin[b,e]]; conv_out = win[1:].
template <typename T>
__global__ void conv_step_kernel(const T* __restrict__ xin, const T* __restrict__ conv_in,
                                 const float* __restrict__ w, const float* __restrict__ bias,
                                 T* __restrict__ xc, T* __restrict__ conv_out,
                                 int64_t ED, int K, int64_t x_sb) {
  const int64_t e = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t b = blockIdx.y;
  if (e >= ED) return;
  const T* ci = conv_in + (b * ED + e) * (K - 1);
  T* co = conv_out + (b * ED + e) * (K - 1);
  const float xn = Elem<T>::to_f(xin[b * x_sb + e]);
  float acc = bias ? bias[e] : 0.f;
  float win[8];
  for (int k = 0; k < K - 1; ++k) win[k] = Elem<T>::to_f(ci[k]);
  win[K - 1] = xn;
  for (int k = 0; k < K; ++k) acc = fmaf(w[e * K + k], win[k], acc);
  for (int k = 0; k < K - 1; ++k) co[k] = Elem<T>::from_f(win[k + 1]);
  xc[b * ED + e] = Elem<T>::from_f(acc * sigmoidf(acc));
}

// Same for the common d_conv = 4: a thread owns 4 neighbouring channels, so the 3-wide windows of
// those channels (12 contiguous elements) and the new inputs move as 8- or 16-byte vectors.
template <typename T>
__global__ void __launch_bounds__(256)
conv_step_k4_kernel(const T* __restrict__ xin, const T* __restrict__ conv_in, const float* __restrict__ w,
                    const float* __restrict__ bias, T* __restrict__ xc, T* __restrict__ conv_out,
                    int64_t ED, int64_t x_sb) {
  const int64_t e = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  const int64_t b = blockIdx.y;
  if (e >= ED) return;
  const Vec4<T>* ci = reinterpret_cast<const Vec4<T>*>(conv_in + (b * ED + e) * 3);
  Vec4<T>* co = reinterpret_cast<Vec4<T>*>(conv_out + (b * ED + e) * 3);
  const Vec4<T> w0 = ci[0], w1 = ci[1], w2 = ci[2];            // 12 window values of 4 channels
  const Vec4<T> xn = *reinterpret_cast<const Vec4<T>*>(xin + b * x_sb + e);
  T win[12] = {w0.v[0], w0.v[1], w0.v[2], w0.v[3], w1.v[0], w1.v[1], w1.v[2], w1.v[3],
               w2.v[0], w2.v[1], w2.v[2], w2.v[3]};
  T out[12];
  Vec4<T> xo;
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    const float4 wf = *reinterpret_cast<const float4*>(w + (e + c) * 4);
    float acc = bias ? bias[e + c] : 0.f;
    acc = fmaf(wf.x, Elem<T>::to_f(win[3 * c]), acc);
    acc = fmaf(wf.y, Elem<T>::to_f(win[3 * c + 1]), acc);
    acc = fmaf(wf.z, Elem<T>::to_f(win[3 * c + 2]), acc);
    acc = fmaf(wf.w, Elem<T>::to_f(xn.v[c]), acc);
    out[3 * c] = win[3 * c + 1];
    out[3 * c + 1] = win[3 * c + 2];
    out[3 * c + 2] = xn.v[c];
    xo.v[c] = Elem<T>::from_f(acc * sigmoid_fast(acc));
  }
  Vec4<T> o0, o1, o2;
#pragma unroll
  for (int k = 0; k < 4; ++k) { o0.v[k] = out[k]; o1.v[k] = out[4 + k]; o2.v[k] = out[8 + k]; }
  co[0] = o0; co[1] = o1; co[2] = o2;
  *reinterpret_cast<Vec4<T>*>(xc + b * ED + e) = xo;
}

// Fold of all-gathered shard carries (see mamba_b200.h).
__global__ void carry_fold_kernel(const float* __restrict__ P, const float* __restrict__ S,
                                  float* __restrict__ out, int64_t R, int64_t M, int rank,
                                  int reverse) {
  const int64_t m = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  if (m >= M) return;
  float cur = 0.f;
  if (!reverse) {
    for (int64_t r = 0; r < rank; ++r) cur = fmaf(P[r * M + m], cur, S[r * M + m]);
  } else {
    for (int64_t r = R - 1; r > rank; --r) cur = fmaf(P[r * M + m], cur, S[r * M + m]);
  }
  out[m] = cur;
}

// States entering pieces first .. first+num-1 of sequences cut into R pieces, in one launch.
// P, S: (batch, R, M); init: (batch, M) or null; out: (batch, num, M).
__global__ void carry_fold_range_kernel(const float* __restrict__ P, const float* __restrict__ S,
                                        const float* __restrict__ init, float* __restrict__ out, int R,
                                        int64_t M, int first, int num, int reverse) {
  const int64_t m = int64_t(blockIdx.x) * blockDim.x + threadIdx.x;
  const int64_t bb = blockIdx.y;
  if (m >= M) return;
  P += bb * R * M; S += bb * R * M; out += bb * num * M;
  float cur = init ? init[bb * M + m] : 0.f;
  if (!reverse) {
    for (int r = 0; r < first + num; ++r) {
      if (r >= first) out[int64_t(r - first) * M + m] = cur;
      if (r + 1 < first + num) cur = fmaf(P[int64_t(r) * M + m], cur, S[int64_t(r) * M + m]);
    }
  } else {
    for (int r = R - 1; r >= first; --r) {
      if (r < first + num) out[int64_t(r - first) * M + m] = cur;
      if (r > first) cur = fmaf(P[int64_t(r) * M + m], cur, S[int64_t(r) * M + m]);
    }
  }
}

// P[b,e,n] = exp(A[e,n] * sum_t delta[b,t,e]); a CTA column-sums a strip of 32 channels.
template <typename T>
__global__ void decay_prod_kernel(const T* __restrict__ delta, const float* __restrict__ A,
                                  const float* __restrict__ delta_bias, float* __restrict__ P,
                                  int64_t L, int64_t ED, int N, int64_t d_sb, int64_t d_sl,
                                  int flags) {
  __shared__ float part[8][33];
  const int lx = threadIdx.x, ly = threadIdx.y;              // 32 x 8
  const int64_t e = int64_t(blockIdx.x) * 32 + lx;
  const int64_t b = blockIdx.y;
  // Kahan-compensated column sum: L can be 10^5 and the sum feeds an exponent
  float s = 0.f, comp = 0.f;
  if (e < ED) {
    const float bias = (flags & MB200_DELTA_SOFTPLUS) ? delta_bias[e] : 0.f;
    for (int64_t t = ly; t < L; t += 8) {
      float dv = Elem<T>::to_f(delta[b * d_sb + t * d_sl + e]);
      if (flags & MB200_DELTA_SOFTPLUS) dv = softplusf(dv + bias);
      const float yk = dv - comp;
      const float tk = s + yk;
      comp = (tk - s) - yk;
      s = tk;
    }
  }
  part[ly][lx] = s;
  __syncthreads();
  if (ly == 0 && e < ED) {
    float tot = 0.f;
    for (int k = 0; k < 8; ++k) tot += part[k][lx];
    for (int n = 0; n < N; ++n) P[(b * ED + e) * N + n] = ex2f(tot * A[e * N + n] * kLog2e);
  }
}

}  // namespace
}  // namespace mb200

using namespace mb200;

template <typename T>
static int ssm_step_t(const void* x, const void* delta, const void* z, const float* A,
                      const void* Bm, const void* Cm, const float* D, const float* delta_bias,
                      const float* h_in, float* h_out, void* y, int64_t B, int64_t ED, int N,
                      int64_t x_sb, int64_t d_sb, int64_t z_sb, int64_t b_sb, int64_t c_sb,
                      int64_t y_sb, int flags, cudaStream_t st) {
  const bool vec_bc = (reinterpret_cast<uintptr_t>(Bm) % (4 * sizeof(T)) == 0) &&
                      (reinterpret_cast<uintptr_t>(Cm) % (4 * sizeof(T)) == 0) && b_sb % 4 == 0 && c_sb % 4 == 0;
#define MB200_STEP(NN)                                                                          \
  {                                                                                             \
    constexpr int epb = kStepThreads / (NN / (MB200_STEP_SPL < NN ? MB200_STEP_SPL : NN));      \
    dim3 grid(unsigned((ED + epb - 1) / epb), unsigned(B));                                     \
    if (vec_bc)                                                                                 \
      ssm_step_kernel<T, NN, true><<<grid, kStepThreads, 0, st>>>(                              \
          (const T*)x, (const T*)delta, (const T*)z, A, (const T*)Bm, (const T*)Cm, D, delta_bias, \
          h_in, h_out, (T*)y, ED, x_sb, d_sb, z_sb, b_sb, c_sb, y_sb, flags);                   \
    else                                                                                        \
      ssm_step_kernel<T, NN, false><<<grid, kStepThreads, 0, st>>>(                             \
          (const T*)x, (const T*)delta, (const T*)z, A, (const T*)Bm, (const T*)Cm, D, delta_bias, \
          h_in, h_out, (T*)y, ED, x_sb, d_sb, z_sb, b_sb, c_sb, y_sb, flags);                   \
    return check_launch();                                                                      \
  }
  switch (N) {
    case 8: MB200_STEP(8)
    case 16: MB200_STEP(16)
    case 32: MB200_STEP(32)
    case 64: MB200_STEP(64)
    default: return MB200_ENSTATE;
  }
#undef MB200_STEP
}

extern "C" int mb200_ssm_step(const void* x, const void* delta, const void* z, const float* A,
                              const void* Bm, const void* Cm, const float* D,
                              const float* delta_bias, const float* h_in, float* h_out, void* y,
                              int64_t B, int64_t ED, int N, int64_t x_sb, int64_t d_sb,
                              int64_t z_sb, int64_t b_sb, int64_t c_sb, int64_t y_sb, int dtype,
                              int flags, void* stream) {
  if (B < 0 || ED < 0) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (N != 8 && N != 16 && N != 32 && N != 64) return MB200_ENSTATE;
  if (B == 0 || ED == 0) return MB200_OK;
  if (!x || !delta || !A || !Bm || !Cm || !h_out || !y) return MB200_EINVAL;
  if ((flags & MB200_DELTA_SOFTPLUS) && !delta_bias) return MB200_EINVAL;
  if (B > 65535) return MB200_ETOOBIG;
  if (!aligned16(h_in) || !aligned16(h_out) || !aligned16(A)) return MB200_EALIGN;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  return dtype == MB200_F32
             ? ssm_step_t<float>(x, delta, z, A, Bm, Cm, D, delta_bias, h_in, h_out, y, B, ED, N,
                                 x_sb, d_sb, z_sb, b_sb, c_sb, y_sb, flags, st)
             : ssm_step_t<__nv_bfloat16>(x, delta, z, A, Bm, Cm, D, delta_bias, h_in, h_out, y, B,
                                         ED, N, x_sb, d_sb, z_sb, b_sb, c_sb, y_sb, flags, st);
}

extern "C" int mb200_conv_step(const void* xin, const void* conv_in, const float* w,
                               const float* bias, void* xc, void* conv_out, int64_t B, int64_t ED,
                               int K, int64_t x_sb, int dtype, void* stream) {
  if (B < 0 || ED < 0 || K < 1) return MB200_EINVAL;
  if (K > 8) return MB200_ETOOBIG;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (B == 0 || ED == 0) return MB200_OK;
  if (!xin || !w || !xc || (K > 1 && (!conv_in || !conv_out))) return MB200_EINVAL;
  if (B > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int es = dtype == MB200_F32 ? 4 : 2;
  if (K == 4 && ED % 4 == 0 && aligned16(xin) && aligned16(conv_in) && aligned16(conv_out) && aligned16(xc) &&
      aligned16(w) && (x_sb * es) % 16 == 0) {
    dim3 g4(unsigned((ED / 4 + 255) / 256), unsigned(B));
    if (dtype == MB200_F32)
      conv_step_k4_kernel<float><<<g4, 256, 0, st>>>((const float*)xin, (const float*)conv_in, w, bias,
                                                     (float*)xc, (float*)conv_out, ED, x_sb);
    else
      conv_step_k4_kernel<__nv_bfloat16><<<g4, 256, 0, st>>>(
          (const __nv_bfloat16*)xin, (const __nv_bfloat16*)conv_in, w, bias, (__nv_bfloat16*)xc,
          (__nv_bfloat16*)conv_out, ED, x_sb);
    return check_launch();
  }
  dim3 grid(unsigned((ED + 255) / 256), unsigned(B));
  if (dtype == MB200_F32)
    conv_step_kernel<float><<<grid, 256, 0, st>>>((const float*)xin, (const float*)conv_in, w, bias,
                                                  (float*)xc, (float*)conv_out, ED, K, x_sb);
  else
    conv_step_kernel<__nv_bfloat16><<<grid, 256, 0, st>>>(
        (const __nv_bfloat16*)xin, (const __nv_bfloat16*)conv_in, w, bias, (__nv_bfloat16*)xc,
        (__nv_bfloat16*)conv_out, ED, K, x_sb);
  return check_launch();
}

extern "C" int mb200_carry_fold(const float* P, const float* S, float* out, int64_t R, int64_t M,
                                int rank, int reverse, void* stream) {
  if (R < 1 || M < 0 || rank < 0 || rank >= R) return MB200_EINVAL;
  if (M == 0) return MB200_OK;
  if (!P || !S || !out) return MB200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  carry_fold_kernel<<<unsigned((M + 255) / 256), 256, 0, st>>>(P, S, out, R, M, rank, reverse);
  return check_launch();
}

extern "C" int mb200_carry_fold_range(const float* P, const float* S, const float* init, float* out, int64_t batch,
                                      int64_t R, int64_t M, int first, int num, int reverse, void* stream) {
  if (batch < 0 || batch > 65535 || R < 1 || R > (1 << 20) || M < 0 || first < 0 || num < 1 || first + num > R)
    return MB200_EINVAL;
  if (M == 0 || batch == 0) return MB200_OK;
  if (!P || !S || !out) return MB200_EINVAL;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(unsigned((M + 255) / 256), unsigned(batch));
  carry_fold_range_kernel<<<grid, 256, 0, st>>>(P, S, init, out, int(R), M, first, num, reverse);
  return check_launch();
}

extern "C" int mb200_decay_prod(const void* delta, const float* A, const float* delta_bias,
                                float* P, int64_t B, int64_t L, int64_t ED, int N, int64_t d_sb,
                                int64_t d_sl, int dtype, int flags, void* stream) {
  if (B < 0 || L < 0 || ED < 0 || N < 1) return MB200_EINVAL;
  if (dtype != MB200_F32 && dtype != MB200_BF16) return MB200_EDTYPE;
  if (B == 0 || ED == 0) return MB200_OK;
  if (!A || !P || (L > 0 && !delta)) return MB200_EINVAL;
  if ((flags & MB200_DELTA_SOFTPLUS) && !delta_bias) return MB200_EINVAL;
  if (B > 65535) return MB200_ETOOBIG;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  dim3 grid(unsigned((ED + 31) / 32), unsigned(B)), block(32, 8);
  if (dtype == MB200_F32)
    decay_prod_kernel<float><<<grid, block, 0, st>>>((const float*)delta, A, delta_bias, P, L, ED, N,
                                                     d_sb, d_sl, flags);
  else
    decay_prod_kernel<__nv_bfloat16><<<grid, block, 0, st>>>((const __nv_bfloat16*)delta, A,
                                                             delta_bias, P, L, ED, N, d_sb, d_sl, flags);
  return check_launch();
}

extern "C" const char* mb200_strerror(int code) {
  switch (code) {
    case MB200_OK: return "ok";
    case MB200_EINVAL: return "invalid argument (shape, size or missing pointer)";
    case MB200_EDTYPE: return "unsupported dtype code";
    case MB200_ENSTATE: return "d_state must be 8, 16, 32 or 64";
    case MB200_EALIGN: return "a float32 state/carry pointer is not 16-byte aligned";
    case MB200_ELAUNCH: return "CUDA kernel launch failed";
    case MB200_ETOOBIG: return "size exceeds a limit of this entry point";
    case MB200_ESETUP: return "per-device set-up failed";
    case MB200_EUNSUPPORTED: return "option not available for these tensors";
    default: return "unknown error";
  }
}

extern "C" int mb200_version(void) { return 100; }

// ---- self-test of the bounded-wait mechanism -------------------------------------------------
// One warp waits on a CTA-local mbarrier that nothing ever arrives at, with the same poll-and-sleep
// loop the fused kernels use but a caller-chosen limit; when the polls run out it records
// MB200_DEV_WAIT_TIMEOUT in a status word and returns.  Nothing faults and nothing spins without a
// limit: this is how a test can see the give-up path without a broken kernel.
namespace mb200 {
namespace {
__device__ int g_selftest_status = MB200_DEV_OK;

__global__ void wait_timeout_selftest_kernel(int polls) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncwarp();
  const uint32_t addr = smem_u32(&bar);
  bool done = mbar_poll(addr, 0);
  for (int i = 0; i < polls && !done; ++i) {
    __nanosleep(100);
    done = mbar_poll(addr, 0);
  }
  if (!done && threadIdx.x == 0) atomicExch(&g_selftest_status, MB200_DEV_WAIT_TIMEOUT);
}
}  // namespace
}  // namespace mb200

extern "C" int mb200_selftest_wait_timeout(int polls, void* stream) {
  if (polls < 1 || polls > (1 << 20)) return MB200_EINVAL;       // at most ~0.1 s of polling
  wait_timeout_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(polls);
  return check_launch();
}

extern "C" int mb200_device_status(void) {
  const int f = mb200_fwd_device_status(), b = mb200_bwd_device_status();
  int s = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&s, g_selftest_status, sizeof(int)) != cudaSuccess) return -1;
  if (s) cudaMemcpyToSymbol(g_selftest_status, &zero, sizeof(int));
  return (f < 0 || b < 0) ? -1 : (f | b | s);
}
