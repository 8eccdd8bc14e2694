/* C ABI of libmamba_b200.so: the selective-scan path of mamba.py as sm_100a CUDA kernels.
 *
 * The reference project is pure Python; its "interface" for this path is a handful of
 * Python callables.  Each entry point below names the reference callable it replaces
 * (path inside the reference project : lines).  The Python host layer of this repository
 * binds these symbols with ctypes and mirrors the reference's call signatures on top.
 *
 * Conventions
 *   - Every pointer is a DEVICE pointer on the current CUDA device unless said otherwise.
 *   - The caller owns every buffer (inputs, outputs, workspaces); nothing here allocates
 *     or frees device memory, and nothing synchronises the device.
 *   - `stream` is a cudaStream_t passed as void* (NULL = the legacy default stream).
 *   - Strides are in ELEMENTS.  The innermost dimension is always unit-stride.
 *   - dtype codes: MB200_F32 = 0, MB200_BF16 = 1 for the activation tensors; the scan
 *     state, A, D and all carries are always float32.
 *   - Return value: 0 on success, a negative MB200_E* code otherwise (mb200_strerror()).
 *     Nothing traps or aborts the device.
 */
#ifndef MAMBA_B200_H
#define MAMBA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { MB200_F32 = 0, MB200_BF16 = 1 };

enum {
  MB200_OK = 0,
  MB200_EINVAL = -1,      /* bad shape / null pointer / negative size            */
  MB200_EDTYPE = -2,      /* unknown dtype code                                   */
  MB200_ENSTATE = -3,     /* d_state N not one of the compiled sizes (8,16,32,64) */
  MB200_EALIGN = -4,      /* a float32 state/carry pointer is not 16-byte aligned */
  MB200_ELAUNCH = -5,     /* the CUDA runtime refused the launch                  */
  MB200_ETOOBIG = -6,     /* size beyond a documented limit of the entry point    */
  MB200_ESETUP = -7,      /* per-device set-up of the library failed              */
  MB200_EUNSUPPORTED = -8 /* the option is not available for these tensors (see the entry point) */
};

/* Flags of mb200_sscan_fwd / mb200_sscan_bwd. */
enum {
  MB200_DELTA_SOFTPLUS = 1, /* delta = softplus(delta_raw + delta_bias[e]) is applied inside;
                               without it `delta` is taken as already discretised           */
  MB200_GENERAL_DECAY = 4,  /* evaluate every decay exp(delta*A[e,n]) with its own ex2.  Without this
                               flag the kernels notice (per warp, on the device) when the rows of A they
                               own follow the S4D-real structure A[e,n] = (n+1)*A[e,0] to within 2^-20
                               relative (the reference's initialisation, mambapy/mamba.py:168-169) and
                               then form the four decays of a state quad from two ex2 and three
                               multiplies; any other A takes the general path on its own.            */
  MB200_REVERSE = 2         /* scan from t = L-1 down to 0 (h[t] = a[t] h[t+1] + ...): what the
                               reference's bidirectional model gets by flipping the sequence,
                               scanning and flipping back (mambapy/vim.py:228-261).  h0 is then the
                               state entering t = L-1, hT the one leaving t = 0, and entry c of
                               `carries` the state entering time chunk c from the right.  Served
                               only by the tensor-map path (16-byte aligned bases and strides;
                               backward: d_state 16); otherwise MB200_EUNSUPPORTED is returned
                               and the caller flips the tensors itself.                     */
};

const char* mb200_strerror(int code);
int mb200_version(void);

/* Device-side status of the kernels launched so far on the current device: 0, or 1 when a
 * bounded wait between the producer and consumer warps of the fused scan gave up (the launch's
 * outputs are then invalid).  Reads and clears the word; SYNCHRONISES the device, so it is for
 * tests and diagnostics, not for the hot path.  Returns -1 if the word cannot be read. */
int mb200_device_status(void);

/* Self-test of that mechanism (no counterpart in the reference): launches one warp that waits, with
 * the kernels' own poll-and-sleep loop but only `polls` (1 .. 2^20) polls, on a barrier nothing
 * arrives at; it then records the give-up in the status word and returns normally.  After a
 * synchronisation mb200_device_status() reports 1.  Nothing faults, traps or spins unbounded. */
int mb200_selftest_wait_timeout(int polls, void* stream);

/* Number of timesteps between two saved scan states ("chunk carries").  The carries
 * tensor of the fused scan has shape (B, ceil(L / chunk), ED, N), float32. */
int mb200_sscan_chunk(void);

/* Number of L-segments the PScan kernels should be launched with for this problem size
 * (1 = single pass).  With nseg > 1 the caller passes a float32 workspace `ws` of
 * 2 * B * nseg * D*N elements to mb200_pscan_fwd / mb200_pscan_bwd. */
int mb200_pscan_segments(int64_t B, int64_t L, int64_t DN);

/* ---- PScan.apply forward: H[t] = A[t]*H[t-1] + X[t], H[-1] = 0, along L.
 * Replaces mambapy/pscan.py:151-186 (PScan.forward) without padding L to a power of two
 * and without touching the inputs.
 * A, X, H: (B, L, D, N) with the (D, N) block dense; strides (sb, sl) per tensor.
 * h0 (optional, may be NULL): (B, D*N) float32 incoming state; hT (optional): outgoing state. */
int mb200_pscan_fwd(const void* A, const void* X, void* H,
                    int64_t B, int64_t L, int64_t DN,
                    int64_t a_sb, int64_t a_sl, int64_t x_sb, int64_t x_sl,
                    int64_t h_sb, int64_t h_sl,
                    const float* h0, float* hT, float* ws, int nseg, int dtype, void* stream);

/* ---- PScan forward for callers that must not allocate.  This entry point has no counterpart
 * in the reference; it exists for hosts of this library that cannot hand it a workspace: an
 * inference server whose device memory is one arena carved up at start-up, a control loop that
 * cannot afford the device-wide synchronisation cudaMalloc/cudaFree imply, or a foreign runtime
 * that reaches this library through the C ABI and has no allocator of its own to call.
 *
 * Same arithmetic and arguments as mb200_pscan_fwd, minus `ws`: when the launch is segmented
 * (nseg > 1) the per-segment aggregates go to a fixed 8 MiB array inside the library image
 * (mb200_pscan_noalloc_max_ws_floats() floats; every GPU that loads the library keeps it until
 * the process ends).  nseg == 0 lets the library choose as mb200_pscan_segments would.
 *   - Limit: 2 * B * nseg * DN floats must fit the array, otherwise MB200_ETOOBIG is returned and
 *     nothing is launched.  nseg == 1 needs no scratch and has no such limit.
 *   - The function, and everything it calls, performs no cudaMalloc / cudaFree and calls no
 *     allocating library routine; inputs and outputs are the caller's.
 *   - The first call on each device looks up the array's device address (cudaGetSymbolAddress
 *     with that device current; MB200_ESETUP if it fails).  Make that first call before starting
 *     any stream capture on the device.
 *   - All calls on a device share the one array, and it keeps whatever the previous call left.
 *     Each call overwrites the part it uses before reading it, so nothing needs clearing, but two
 *     calls that overlap on the GPU (different streams, or different host threads) race: keep
 *     calls of this entry point ordered on one stream per device. */
int64_t mb200_pscan_noalloc_max_ws_floats(void);
int mb200_pscan_fwd_noalloc(const void* A, const void* X, void* H,
                            int64_t B, int64_t L, int64_t DN,
                            int64_t a_sb, int64_t a_sl, int64_t x_sb, int64_t x_sl,
                            int64_t h_sb, int64_t h_sl,
                            const float* h0, float* hT, int nseg, int dtype, void* stream);

/* ---- PScan.apply backward.  Replaces mambapy/pscan.py:188-224 (PScan.backward):
 * gradX[t] = gradH[t] + A[t+1]*gradX[t+1];  gradA[t] = H[t-1]*gradX[t], gradA[0] = 0
 * (or h0*gradX[0] when an incoming state h0 is given).
 * A, H, gradH in; gradA, gradX out; all (B, L, D, N) with dense (D, N) blocks. */
int mb200_pscan_bwd(const void* A, const void* H, const void* gradH,
                    void* gradA, void* gradX,
                    int64_t B, int64_t L, int64_t DN,
                    int64_t a_sb, int64_t a_sl, int64_t h_sb, int64_t h_sl,
                    int64_t g_sb, int64_t g_sl, int64_t ga_sb, int64_t ga_sl,
                    int64_t gx_sb, int64_t gx_sl,
                    const float* h0, float* ws, int nseg, int dtype, void* stream);

/* ---- Fused selective scan, forward.
 * Replaces mambapy/mamba.py:274-295 (MambaBlock.selective_scan), :297-327
 * (selective_scan_seq) and, when z != NULL, the gate of MambaBlock.forward (:229-231);
 * with MB200_DELTA_SOFTPLUS also the softplus(delta + dt_bias) of MambaBlock.ssm (:264-265).
 *   y[b,t,e] = ( sum_n C[b,t,n]*h[b,t,e,n] + D[e]*x[b,t,e] ) * silu(z[b,t,e])
 *   h[b,t,e,n] = exp(delta[b,t,e]*A[e,n]) * h[b,t-1,e,n] + delta[b,t,e]*Bm[b,t,n]*x[b,t,e]
 * x, delta, z, y: (B, L, ED) activations, strides (sb, sl) each.  Bm, Cm: (B, L, N).
 * A: (ED, N) float32 dense.  D: (ED) float32 or NULL (treated as 0).
 * h0 / hT: optional (B, ED, N) float32 incoming / outgoing state.
 * carries: optional (B, ceil(L/chunk), ED, N) float32; entry c receives the state that
 *          enters timestep c*chunk.  Needed by mb200_sscan_bwd. */
int mb200_sscan_fwd(const void* x, const void* delta, const void* z,
                    const float* A, const void* Bm, const void* Cm, const float* D,
                    const float* delta_bias, const float* h0,
                    void* y, float* hT, float* carries,
                    int64_t B, int64_t L, int64_t ED, int N,
                    int64_t x_sb, int64_t x_sl, int64_t d_sb, int64_t d_sl,
                    int64_t z_sb, int64_t z_sl, int64_t b_sb, int64_t b_sl,
                    int64_t c_sb, int64_t c_sl, int64_t y_sb, int64_t y_sl,
                    int dtype, int flags, void* stream);

/* ---- Fused selective scan, backward (the autograd the reference gets from PyTorch for
 * mambapy/mamba.py:274-295 + :229-231 together with mambapy/pscan.py:188-224).
 * Recomputes h chunk by chunk from `carries`, runs the reverse scan, and writes
 *   dx, ddelta, dz : (B, L, ED) in the activation dtype (dz only when z != NULL)
 *   dB, dC         : (B, L, N)  float32, ACCUMULATED into (caller zero-fills)
 *   dA (ED, N), dD (ED), ddelta_bias (ED): float32, ACCUMULATED into (caller zero-fills)
 * g_in (optional): (B, ED, N) float32, a[t_L]*g[t_L] arriving from the sequence that follows
 *                  (sequence-sharded use); g_out (optional): the same quantity leaving t = 0.
 * dh0 is g_out; dy is the gradient w.r.t. y. */
int mb200_sscan_bwd(const void* x, const void* delta, const void* z,
                    const float* A, const void* Bm, const void* Cm, const float* D,
                    const float* delta_bias, const void* dy, const float* carries,
                    const float* g_in,
                    void* dx, void* ddelta, void* dz,
                    float* dB, float* dC, float* dA, float* dD, float* ddelta_bias,
                    float* g_out,
                    int64_t B, int64_t L, int64_t ED, int N,
                    int64_t x_sb, int64_t x_sl, int64_t d_sb, int64_t d_sl,
                    int64_t z_sb, int64_t z_sl, int64_t b_sb, int64_t b_sl,
                    int64_t c_sb, int64_t c_sl, int64_t dy_sb, int64_t dy_sl,
                    int64_t dx_sb, int64_t dx_sl, int64_t dd_sb, int64_t dd_sl,
                    int64_t dz_sb, int64_t dz_sl,
                    int dtype, int flags, void* stream);

/* ---- Reverse carry pass of the sequence-sharded backward (no reference counterpart; the
 * reference is single-device).  For one shard of the sequence it returns, in g_out (B, ED, N)
 * float32, the gradient carry a[0]*g[0] that leaves the shard's first timestep when NO carry
 * enters its last one:  gc <- exp(delta[t]*A) * (dy[t]*silu(z[t])*C[t] + gc),  t = L-1 .. 0.
 * Reads delta, z (optional), dy, Cm once; needs no hidden states. */
int mb200_sscan_bwd_carry(const void* delta, const void* z, const void* dy, const void* Cm,
                          const float* A, const float* delta_bias, float* g_out,
                          int64_t B, int64_t L, int64_t ED, int N,
                          int64_t d_sb, int64_t d_sl, int64_t z_sb, int64_t z_sl,
                          int64_t dy_sb, int64_t dy_sl, int64_t c_sb, int64_t c_sl,
                          int dtype, int flags, void* stream);

/* ---- Fused decode step.  Replaces the arithmetic of mambapy/mamba.py:398-412
 * (MambaBlock.ssm_step after the projections) and the gate of MambaBlock.step (:373-375):
 *   h'[b,e,n] = exp(delta*A[e,n]) * h[b,e,n] + delta*Bm[b,n]*x[b,e]
 *   y[b,e]    = ( sum_n h'[b,e,n]*Cm[b,n] + D[e]*x[b,e] ) * silu(z[b,e])
 *   x     : (B, ED) activations, the post-conv, post-SiLU x (see mb200_conv_step).
 *   delta : (B, ED) activations; MB200_DELTA_SOFTPLUS applies softplus(delta + delta_bias).
 *   Bm, Cm: (B, N) activations.  z: (B, ED) or NULL (no gate).  D: (ED) or NULL.
 *   h_in  : (B, ED, N) float32 or NULL (= 0, the reference's h = None first step).
 *   h_out : (B, ED, N) float32 (may alias h_in).  y: (B, ED).  Row strides *_sb in elements. */
int mb200_ssm_step(const void* x, const void* delta, const void* z,
                   const float* A, const void* Bm, const void* Cm, const float* D,
                   const float* delta_bias, const float* h_in, float* h_out, void* y,
                   int64_t B, int64_t ED, int N,
                   int64_t x_sb, int64_t d_sb, int64_t z_sb, int64_t b_sb, int64_t c_sb,
                   int64_t y_sb, int dtype, int flags, void* stream);

/* ---- Conv-window step of MambaBlock.step (mambapy/mamba.py:366-369 and :379):
 *   xc[b,e]        = silu( sum_k w[e,k]*win[b,e,k] + bias[e] ),  win = [conv_in[b,e,:], xin[b,e]]
 *   conv_out[b,e,:] = win[b,e,1:]
 * xin: (B, ED) activations (row stride x_sb); conv_in/conv_out: (B, ED, K-1) dense, same
 * dtype; w: (ED, K) float32 dense; bias: (ED) float32 or NULL; xc: (B, ED) dense.  K <= 8. */
int mb200_conv_step(const void* xin, const void* conv_in, const float* w, const float* bias,
                    void* xc, void* conv_out,
                    int64_t B, int64_t ED, int K, int64_t x_sb, int dtype, void* stream);

/* ---- Depthwise causal conv1d + SiLU in the (B, L, ED) layout, d_conv = 4 (K must be 4, else
 * MB200_ETOOBIG).  Replaces the transpose / nn.Conv1d(padding=3) / slice / transpose / F.silu sequence
 * of MambaBlock.forward (mambapy/mamba.py:217-221):
 *   y[b,t,e] = silu( bias[e] + sum_k w[e,k] * x[b, t-3+k, e] ),  x[b, t<0, e] = 0.
 * x, y: (B, L, ED) activations with strides (sb, sl); w: (ED, 4) float32 dense; bias: (ED) or NULL. */
int mb200_conv1d_silu_fwd(const void* x, const float* w, const float* bias, void* y,
                          int64_t B, int64_t L, int64_t ED, int K,
                          int64_t x_sb, int64_t x_sl, int64_t y_sb, int64_t y_sl,
                          int dtype, void* stream);

/* Backward of mb200_conv1d_silu_fwd (what autograd derives for mambapy/mamba.py:217-221).
 * dy in; dx out (activation dtype); dw (ED, 4) and dbias (ED, may be NULL) float32, ACCUMULATED into
 * (caller zero-fills).  The pre-activation is recomputed from x. */
int mb200_conv1d_silu_bwd(const void* x, const float* w, const float* bias, const void* dy,
                          void* dx, float* dw, float* dbias,
                          int64_t B, int64_t L, int64_t ED, int K,
                          int64_t x_sb, int64_t x_sl, int64_t dy_sb, int64_t dy_sl,
                          int64_t dx_sb, int64_t dx_sl, int dtype, void* stream);

/* ---- Sequence-sharded scan: fold the per-shard carries after they were all-gathered.
 * No reference counterpart (the reference is single-device); the single-device answer on
 * the concatenated sequence is what it must reproduce.
 *   P, S : (R, M) float32 — per shard r the decay product over the shard and the state the
 *          shard reaches from a zero start, M = B*ED*N.
 *   reverse == 0: out[m] = state entering shard `rank`  = fold of shards 0..rank-1 in order
 *                 (h <- P_q*h + S_q), starting from 0.
 *   reverse == 1: out[m] = gradient carry entering shard `rank` from the right = fold of
 *                 shards R-1..rank+1 (g <- S_q + P_q*g), starting from 0. */
int mb200_carry_fold(const float* P, const float* S, float* out,
                     int64_t R, int64_t M, int rank, int reverse, void* stream);

/* The same fold for a RANGE of pieces, and for `batch` independent sequences, in one launch (no reference
 * counterpart).  P, S: (batch, R, M); init: (batch, M) or NULL; out: (batch, num, M).  out[bb][i - first] is
 * the state entering piece i of sequence bb (reverse == 0: fold of pieces 0..i-1 in order, starting from
 * init[bb] or from 0) or the gradient carry entering piece i from the right (reverse == 1: fold of pieces
 * R-1..i+1, starting from init[bb] or 0), for i = first .. first+num-1.  Used when a device cuts its span
 * into several pieces that are scanned side by side as extra batch rows. */
int mb200_carry_fold_range(const float* P, const float* S, const float* init, float* out, int64_t batch,
                           int64_t R, int64_t M, int first, int num, int reverse, void* stream);

/* ---- Forward carry pass of a split sequence (no reference counterpart): for every batch row, the state
 * h_out (B, ED, N) the span reaches from a ZERO state and the span's decay product
 * p_out[b,e,n] = exp(A[e,n] * sum_t delta[b,t,e]), from one pass over x, delta, Bm (same layouts and
 * softplus option as mb200_sscan_fwd; no y, no C, no saved states).  Together with mb200_carry_fold[_range]
 * these give the state entering every piece.  MB200_REVERSE is not served here. */
int mb200_sscan_fwd_carry(const void* x, const void* delta, const float* A, const void* Bm,
                          const float* delta_bias, float* h_out, float* p_out,
                          int64_t B, int64_t L, int64_t ED, int N,
                          int64_t x_sb, int64_t x_sl, int64_t d_sb, int64_t d_sl,
                          int64_t b_sb, int64_t b_sl, int dtype, int flags, void* stream);

/* ---- Decay product of a shard: P[b,e,n] = exp(A[e,n] * sum_t delta[b,t,e]) (with the same
 * softplus option as the scan).  Used with mb200_carry_fold by the sequence-sharded scan. */
int mb200_decay_prod(const void* delta, const float* A, const float* delta_bias, float* P,
                     int64_t B, int64_t L, int64_t ED, int N,
                     int64_t d_sb, int64_t d_sl, int dtype, int flags, void* stream);

/* ---- RMSNorm over the last dimension (mambapy/mamba.py:416-433, used in front of every block at
 * mambapy/mamba.py:111 and for the optional inner normalisation of delta, B, C):
 *   y[r, d] = x[r, d] * rsqrt(mean_d x[r, :]^2 + eps) * weight[d]      (weight NULL = no gain, the muP case)
 * x, y: `rows` rows of D activations, last dimension unit-stride, row strides in elements; arithmetic is
 * float32.  rstd (rows) float32, optional: the per-row rsqrt, which mb200_rmsnorm_bwd needs. */
int mb200_rmsnorm_fwd(const void* x, const float* weight, void* y, float* rstd, int64_t rows, int64_t D,
                      int64_t x_rs, int64_t y_rs, float eps, int dtype, void* stream);

/* Backward of mb200_rmsnorm_fwd (what autograd derives for mambapy/mamba.py:427-433).
 * dx out (activation dtype); dweight (D) float32 or NULL, ACCUMULATED into (caller zero-fills);
 * D <= 12288 when dweight is given (MB200_ETOOBIG otherwise). */
int mb200_rmsnorm_bwd(const void* x, const float* weight, const float* rstd, const void* dy, void* dx,
                      float* dweight, int64_t rows, int64_t D, int64_t x_rs, int64_t dy_rs, int64_t dx_rs,
                      int dtype, void* stream);

/* ---- Residual add fused with the RMSNorm that follows it.  A stack of blocks computes
 * x_{l+1} = mixer(norm(x_l)) + x_l (ResidualBlock.forward, mambapy/mamba.py:106-112, looped by
 * Mamba.forward, mambapy/mamba.py:77-85); the add of layer l and the norm of layer l+1 become one pass:
 *   s = x + res_in (res_in NULL: s = x);   res_out = s;   y = s * rsqrt(mean(s^2) + eps) * weight.
 * x: the previous mixer's output; res_in / res_out: the residual stream; y: the next mixer's input.  Each of
 * the three has its own element type (under autocast the mixer works in bfloat16 while the residual stream
 * stays float32); served triples (x, res, y): fff, ffb, bff, bfb, bbb (MB200_EUNSUPPORTED otherwise).
 * Row strides in elements; rstd (rows) float32, optional, is what mb200_add_rmsnorm_bwd needs. */
int mb200_add_rmsnorm_fwd(const void* x, const void* res_in, const float* weight, void* res_out, void* y,
                          float* rstd, int64_t rows, int64_t D, int64_t x_rs, int64_t ri_rs, int64_t ro_rs,
                          int64_t y_rs, float eps, int dtype_x, int dtype_res, int dtype_y, void* stream);

/* Backward of mb200_add_rmsnorm_fwd: ds = d(loss)/d s = RMSNorm backward of dy at s, plus dres (the gradient
 * that reaches res_out from later layers; NULL = none).  ds has the residual stream's type and is the gradient
 * of BOTH x and res_in.  dweight (D) float32 or NULL, accumulated into; D <= 12288 when it is given. */
int mb200_add_rmsnorm_bwd(const void* s, const float* weight, const float* rstd, const void* dy,
                          const void* dres, void* ds, float* dweight, int64_t rows, int64_t D,
                          int64_t s_rs, int64_t dy_rs, int64_t dr_rs, int64_t ds_rs, int dtype_res,
                          int dtype_y, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* MAMBA_B200_H */
