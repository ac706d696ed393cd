// Two recurrent mixers whose state per request has a fixed size, float32 throughout.
//
//   lightning_recurrence   linear attention with a fixed decay per head:
//                              S <- decay_h S + k v^T,  o = S^T q        S: [dim x vdim] per head
//                          q, k, v are the silu of float32 projection columns.
//   scan_conv              short causal convolution per channel with bias, then silu (inputs before the portion come
//                          from the request's state)
//   selective_scan         per channel c and state n:  S[c, n] <- exp(dt_c A[c, n]) S[c, n] + dt_c x_c B_n,
//                              y_c = sum_n S[c, n] C_n + D_c x_c,  out_c = y_c silu(z_c),  dt = softplus(raw + bias),
//                              A = -exp(A_log)
//
// A step holds portions of several requests (qo_indptr, state_slots); a portion of one token is a decode step.  Every
// sum runs in an order fixed by the sizes alone, so a position's result does not depend on how the request was cut
// or on what else is in the step.
#include "common.cuh"
#include <math.h>
using namespace bspec;

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }
// S <- exp(x) S + b as S + ((exp(x) - 1) S + b).  A state with a long memory has exp(x) within 1e-4 of 1, where a
// float32 factor keeps only three digits of what matters, 1 - exp(x); taken a thousand times that shows in the sum.
// exp(x) - 1 keeps all its digits, and the state moves by the small difference.
// Near zero exp(x) - 1 is the series up to x^4 / 24 (the next term is below 1e-8 of the sum for |x| < 1/32); further
// out 2^(x log2 e) - 1, whose difference from 1 is large enough to keep its digits.
__device__ __forceinline__ float exp_minus_one(float x) {
  const float series = __fmul_rn(x, __fmaf_rn(x, __fmaf_rn(x, __fmaf_rn(x, 1.f / 24.f, 1.f / 6.f), 0.5f), 1.f));
  const float direct = exp2f(__fmul_rn(x, 1.4426950408889634f)) - 1.f;
  return fabsf(x) < 0.03125f ? series : direct;
}
__device__ __forceinline__ float scan_update(float s, float x, float b) {
  return __fadd_rn(s, __fmaf_rn(exp_minus_one(x), s, b));
}

// ---------------------------------------------------------------- lightning attention
// Block: COLS value columns of one head of one request, L lanes per column (8, 16 or 32: more lanes mean more warps
// per SM to hide the chain's latencies, and fewer rows per lane); lane r of a column keeps rows
// 4 L g + 4 r + e (e < 4, g < NR / 4) of that column of S in registers, so that a lane reads its four rows of q and k
// from shared memory in one 16-byte load.  Tokens are staged TT at a time in shared memory: the raw projection
// columns of the next TT tokens are fetched into registers while the recurrence runs over the current ones, so the
// memory latency is paid once per kernel and not once per batch of tokens.  The recurrence takes four tokens per
// pass (sixteen independent chains of four dependent multiply-adds); a token's sums run in the same order in the
// four-token pass and in the single-token tail, so a position's result does not depend on where a portion ends.
// State of a request: [H][vdim][dim] float32 at state + slot * state_stride.
constexpr int LT_COLS = 16;
constexpr int LT_TT = 16;

template <int NR, int L>
__global__ void __launch_bounds__(LT_COLS * L)
lightning_recurrence_kernel(const float* __restrict__ proj, long long ld, int q_off, int k_off, int v_off,
                            const float* __restrict__ decay, float* __restrict__ state, long long state_stride,
                            const int* __restrict__ qo_indptr, const int* __restrict__ state_slots,
                            float* __restrict__ out, int H, int dim, int vdim) {
  bspec::pdl_prologue_late(65);
  constexpr int LT_THREADS = LT_COLS * L;
  constexpr int DM = L * NR;                                // rows of S this instance holds (dim <= DM)
  constexpr int VR = (LT_TT * LT_COLS + LT_THREADS - 1) / LT_THREADS;          // staged v values per thread
  static_assert(NR % 4 == 0 && (L == 8 || L == 16 || L == 32) && LT_TT * DM == NR * LT_THREADS, "lanes and rows");
  __shared__ __align__(16) float qs[LT_TT][DM];
  __shared__ __align__(16) float ks[LT_TT][DM];
  __shared__ float vs[LT_TT][LT_COLS];
  const int e = blockIdx.z, h = blockIdx.y;
  const int col = threadIdx.x / L, r = threadIdx.x % L;
  const int j = blockIdx.x * LT_COLS + col;                 // value column of the head
  const bool live = j < vdim;
  const int t0 = qo_indptr[e], nt = qo_indptr[e + 1] - t0;
  const float d = decay[h];
  float* sp = state + (size_t)state_slots[e] * state_stride + ((size_t)h * vdim + (live ? j : 0)) * dim;
  float qn[NR], kn[NR], vn[VR];
  // the raw columns of tokens base .. base + TT - 1 (zeros beyond the portion, the head's rows and the columns)
  auto fetch = [&](int base) {
    const int cnt = min(LT_TT, nt - base);
#pragma unroll
    for (int u = 0; u < NR; ++u) {
      const int x = threadIdx.x + LT_THREADS * u;
      const int tt = x / DM, i = x % DM;                     // tt is the same for a whole warp (DM >= 32)
      if (tt >= cnt) break;
      const bool ok = i < dim;
      const float* row = proj + (size_t)(t0 + base + tt) * ld + (size_t)h * dim + (ok ? i : 0);
      qn[u] = ok ? row[q_off] : 0.f;
      kn[u] = ok ? row[k_off] : 0.f;
    }
#pragma unroll
    for (int u = 0; u < VR; ++u) {
      const int x = threadIdx.x + LT_THREADS * u;
      const int tt = x / LT_COLS, c = x % LT_COLS;
      const int jj = blockIdx.x * LT_COLS + c;
      const bool ok = x < LT_TT * LT_COLS && tt < cnt && jj < vdim;
      vn[u] = ok ? proj[(size_t)(t0 + base + tt) * ld + v_off + (size_t)h * vdim + jj] : 0.f;
    }
  };
  if (nt > 0) fetch(0);
  float s[NR];
  const bool vec = (dim & 3) == 0 && (reinterpret_cast<uintptr_t>(sp) & 15) == 0;
  if (vec) {
#pragma unroll
    for (int g = 0; g < NR / 4; ++g) {
      const int i = 4 * L * g + 4 * r;
      const float4 v4 = (live && i < dim) ? *reinterpret_cast<const float4*>(sp + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      s[4 * g] = v4.x, s[4 * g + 1] = v4.y, s[4 * g + 2] = v4.z, s[4 * g + 3] = v4.w;
    }
  } else {
#pragma unroll
    for (int m = 0; m < NR; ++m) {
      const int i = 4 * L * (m >> 2) + 4 * r + (m & 3);
      s[m] = (live && i < dim) ? sp[i] : 0.f;
    }
  }
  for (int base = 0; base < nt; base += LT_TT) {
    const int cnt = min(LT_TT, nt - base);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < NR; ++u) {                           // rows of tokens beyond cnt are never read
      const int x = threadIdx.x + LT_THREADS * u;
      if (x / DM >= cnt) break;
      qs[x / DM][x % DM] = silu_f(qn[u]);                    // silu(0) = 0: rows beyond dim
      ks[x / DM][x % DM] = silu_f(kn[u]);
    }
#pragma unroll
    for (int u = 0; u < VR; ++u) {
      const int x = threadIdx.x + LT_THREADS * u;
      if (x < LT_TT * LT_COLS && x / LT_COLS < cnt) vs[x / LT_COLS][x % LT_COLS] = silu_f(vn[u]);
    }
    __syncthreads();
    if (base + LT_TT < nt) fetch(base + LT_TT);
    float* orow = out + (size_t)(t0 + base) * H * vdim + (size_t)h * vdim + j;
    int tt = 0;
    for (; tt + 4 <= cnt; tt += 4) {
      float acc[4] = {0.f, 0.f, 0.f, 0.f}, vj[4];
#pragma unroll
      for (int a = 0; a < 4; ++a) vj[a] = vs[tt + a][col];
#pragma unroll
      for (int g = 0; g < NR / 4; ++g) {
        float4 k4[4], q4[4];
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          k4[a] = *reinterpret_cast<const float4*>(&ks[tt + a][4 * L * g + 4 * r]);
          q4[a] = *reinterpret_cast<const float4*>(&qs[tt + a][4 * L * g + 4 * r]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a) {
          const float kk[4] = {k4[a].x, k4[a].y, k4[a].z, k4[a].w}, qq[4] = {q4[a].x, q4[a].y, q4[a].z, q4[a].w};
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            s[4 * g + c] = __fmaf_rn(d, s[4 * g + c], __fmul_rn(kk[c], vj[a]));
            acc[a] = __fmaf_rn(s[4 * g + c], qq[c], acc[a]);
          }
        }
      }
#pragma unroll
      for (int o = 1; o < L; o <<= 1)
#pragma unroll
        for (int a = 0; a < 4; ++a) acc[a] += __shfl_xor_sync(0xffffffffu, acc[a], o);
      const float mine = r == 0 ? acc[0] : (r == 1 ? acc[1] : (r == 2 ? acc[2] : acc[3]));
      if (live && r < 4) orow[(size_t)(tt + r) * H * vdim] = mine;
    }
    for (; tt < cnt; ++tt) {
      const float vj = vs[tt][col];
      float acc = 0.f;
#pragma unroll
      for (int g = 0; g < NR / 4; ++g) {
        const float4 k4 = *reinterpret_cast<const float4*>(&ks[tt][4 * L * g + 4 * r]);
        const float4 q4 = *reinterpret_cast<const float4*>(&qs[tt][4 * L * g + 4 * r]);
        const float kk[4] = {k4.x, k4.y, k4.z, k4.w}, qq[4] = {q4.x, q4.y, q4.z, q4.w};
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          s[4 * g + c] = __fmaf_rn(d, s[4 * g + c], __fmul_rn(kk[c], vj));
          acc = __fmaf_rn(s[4 * g + c], qq[c], acc);
        }
      }
#pragma unroll
      for (int o = 1; o < L; o <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
      if (live && r == 0) orow[(size_t)tt * H * vdim] = acc;
    }
  }
  bspec::pdl_launch_dependents();
  if (live && vec) {
#pragma unroll
    for (int g = 0; g < NR / 4; ++g) {
      const int i = 4 * L * g + 4 * r;
      if (i < dim) *reinterpret_cast<float4*>(sp + i) = make_float4(s[4 * g], s[4 * g + 1], s[4 * g + 2], s[4 * g + 3]);
    }
  } else if (live) {
#pragma unroll
    for (int m = 0; m < NR; ++m) {
      const int i = 4 * L * (m >> 2) + 4 * r + (m & 3);
      if (i < dim) sp[i] = s[m];
    }
  }
}

// ---------------------------------------------------------------- selective scan
// xz [n, ld]: columns [x: inner | z: inner] of the in-projection.  State of a request at state + slot * stride:
// [N][inner] float32 (the scan's S, state index major), then at tail_off [(taps-1)][inner] the last inputs of the
// convolution, oldest first.  a2t [N][inner] float32: A[c, n] = -exp(A_log[c, n]), made once from the weights.

// xc[t, c] = silu(bias[c] + sum_j conv[c, j] * x[t - (taps-1) + j, c]); one thread per (token, channel).
template <typename T>
__global__ void __launch_bounds__(256)
scan_conv_kernel(const float* __restrict__ xz, long long ld, const void* __restrict__ conv, const void* __restrict__ bias,
                 int w_dtype, const float* __restrict__ state, long long state_stride, long long tail_off,
                 const int* __restrict__ qo_indptr, const int* __restrict__ tok_entry,
                 const int* __restrict__ state_slots, float* __restrict__ xc, T* __restrict__ xc_run, int inner,
                 int taps) {
  bspec::pdl_prologue(66);
  const int t = blockIdx.x;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= inner) return;
  const int e = tok_entry[t];
  const int i = t - qo_indptr[e];
  const float* tail = state + (size_t)state_slots[e] * state_stride + tail_off;
  float y = load_as_f32(bias, w_dtype, c);
  for (int j = 0; j < taps; ++j) {                           // oldest input first
    const int rel = i - (taps - 1 - j);
    const float x = rel >= 0 ? xz[(size_t)(t - (taps - 1 - j)) * ld + c] : tail[(size_t)(rel + taps - 1) * inner + c];
    y += load_as_f32(conv, w_dtype, (size_t)c * taps + j) * x;
  }
  const float v = silu_f(y);
  xc[(size_t)t * inner + c] = v;
  if (xc_run != nullptr) xc_run[(size_t)t * inner + c] = from_f32<T>(v);
}

constexpr int SC_THREADS = 128;
constexpr int SC_TT = 8;
constexpr int SC_MAX_N = 256;

// LN lanes per channel; lane l keeps states l, l + LN, ... (NPL of them) of its channel in registers.  Tokens go
// SC_TT at a time: the next batch's B and C rows and the channel's own x, dt and z are fetched into registers while
// the recurrence runs over the current batch, and softplus and silu are taken once per batch outside the chain, so
// what is left per token is one exponential and two multiply-adds per state.  Every token's arithmetic is the same
// wherever it falls in a batch, so a position's result does not depend on where a portion was cut.
template <typename T, int NPL, int LN>
__global__ void __launch_bounds__(SC_THREADS)
selective_scan_kernel(const float* __restrict__ xz, long long ld, const float* __restrict__ xc,
                      const float* __restrict__ dt_raw, const float* __restrict__ bc, long long ld_bc,
                      const float* __restrict__ a2t, const void* __restrict__ dvec, const void* __restrict__ dt_bias,
                      int w_dtype, float* __restrict__ state, long long state_stride, long long tail_off,
                      const int* __restrict__ qo_indptr, const int* __restrict__ state_slots, T* __restrict__ out,
                      long long out_stride, float out_scale, int inner, int N, int taps) {
  bspec::pdl_prologue_late(67);
  constexpr int NS = NPL * LN;                               // states this instance covers (N <= NS)
  constexpr int BCR = SC_TT * 2 * NS / SC_THREADS;           // staged B and C values per thread and batch
  static_assert(SC_TT * 2 * NS % SC_THREADS == 0, "the staged rows divide among the threads");
  __shared__ __align__(16) float bcs[SC_TT][2 * NS];         // [B: NS | C: NS] of a token, zeros beyond N
  const int e = blockIdx.y;
  const int lane = threadIdx.x % LN;
  const int c = blockIdx.x * (SC_THREADS / LN) + threadIdx.x / LN;
  const bool live = c < inner;
  const int cc = live ? c : 0;
  const int t0 = qo_indptr[e], nt = qo_indptr[e + 1] - t0;
  float* sp = state + (size_t)state_slots[e] * state_stride;
  float xn[SC_TT], dn[SC_TT], zn[SC_TT], bn[BCR];
  auto fetch = [&](int base) {
    const int cnt = min(SC_TT, nt - base);
#pragma unroll
    for (int tt = 0; tt < SC_TT; ++tt) {
      if (tt >= cnt) break;
      const size_t t = (size_t)(t0 + base + tt);
      xn[tt] = xc[t * inner + cc];
      dn[tt] = dt_raw[t * inner + cc];
      zn[tt] = xz[t * ld + inner + cc];
    }
#pragma unroll
    for (int u = 0; u < BCR; ++u) {
      const int x = threadIdx.x + SC_THREADS * u;
      const int tt = x / (2 * NS), k = x % (2 * NS);
      const int n = k % NS;
      const bool ok = tt < cnt && n < N;
      bn[u] = ok ? bc[(size_t)(t0 + base + tt) * ld_bc + (k < NS ? n : N + n)] : 0.f;
    }
  };
  if (nt > 0) fetch(0);
  float s[NPL], a2[NPL];
#pragma unroll
  for (int m = 0; m < NPL; ++m) {
    const int n = lane + LN * m;
    const bool has = live && n < N;
    s[m] = has ? sp[(size_t)n * inner + cc] : 0.f;
    a2[m] = has ? a2t[(size_t)n * inner + cc] : 0.f;
  }
  const float dskip = load_as_f32(dvec, w_dtype, cc), dtb = load_as_f32(dt_bias, w_dtype, cc);
  for (int base = 0; base < nt; base += SC_TT) {
    const int cnt = min(SC_TT, nt - base);
    float xv[SC_TT], dv[SC_TT], gv[SC_TT];
    __syncthreads();
#pragma unroll
    for (int u = 0; u < BCR; ++u) {
      const int x = threadIdx.x + SC_THREADS * u;
      bcs[x / (2 * NS)][x % (2 * NS)] = bn[u];
    }
#pragma unroll
    for (int tt = 0; tt < SC_TT; ++tt) {
      if (tt >= cnt) break;
      xv[tt] = xn[tt];
      dv[tt] = softplus_f(dn[tt] + dtb);
      gv[tt] = silu_f(zn[tt]) * out_scale;
    }
    __syncthreads();
    if (base + SC_TT < nt) fetch(base + SC_TT);
    // one token; the same arithmetic in a whole batch (unrolled without branches, so that the tokens' independent
    // work interleaves) and in a last, partial one
    auto token = [&](int tt, float xt, float dt, float gt) {
      const float dx = dt * xt;
      float y = 0.f;
      if constexpr (LN == 1 && NPL % 4 == 0) {
#pragma unroll
        for (int g = 0; g < NPL / 4; ++g) {
          const float4 b4 = *reinterpret_cast<const float4*>(&bcs[tt][4 * g]);
          const float4 c4 = *reinterpret_cast<const float4*>(&bcs[tt][NS + 4 * g]);
          const float bb[4] = {b4.x, b4.y, b4.z, b4.w}, cv[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            s[4 * g + q] = scan_update(s[4 * g + q], __fmul_rn(dt, a2[4 * g + q]), __fmul_rn(dx, bb[q]));
            y = __fmaf_rn(s[4 * g + q], cv[q], y);
          }
        }
      } else {
#pragma unroll
        for (int m = 0; m < NPL; ++m) {
          const int n = lane + LN * m;                       // states beyond N: a2 = 0, B = C = 0, s stays 0
          s[m] = scan_update(s[m], __fmul_rn(dt, a2[m]), __fmul_rn(dx, bcs[tt][n]));
          y = __fmaf_rn(s[m], bcs[tt][NS + n], y);
        }
      }
#pragma unroll
      for (int o = 1; o < LN; o <<= 1) y += __shfl_xor_sync(0xffffffffu, y, o);
      if (live && lane == 0)
        out[(size_t)(t0 + base + tt) * out_stride + cc] = from_f32<T>(__fmul_rn(__fmaf_rn(dskip, xt, y), gt));
    };
    if (cnt == SC_TT) {
#pragma unroll
      for (int tt = 0; tt < SC_TT; ++tt) token(tt, xv[tt], dv[tt], gv[tt]);
    } else {
#pragma unroll
      for (int tt = 0; tt < SC_TT; ++tt)
        if (tt < cnt) token(tt, xv[tt], dv[tt], gv[tt]);
    }
  }
  bspec::pdl_launch_dependents();
  if (!live) return;
#pragma unroll
  for (int m = 0; m < NPL; ++m) {
    const int n = lane + LN * m;
    if (n < N) sp[(size_t)n * inner + cc] = s[m];
  }
  if (lane == 0) {
    // the convolution's last taps-1 inputs, oldest first: rows of this portion, and before them what the state held
    float* tail = sp + tail_off;
    for (int u = 0; u < taps - 1; ++u) {
      const int rel = nt - (taps - 1) + u;
      tail[(size_t)u * inner + cc] = rel >= 0 ? xz[(size_t)(t0 + rel) * ld + cc] : tail[(size_t)(u + nt) * inner + cc];
    }
  }
}
}  // namespace

BSPEC_API int bspec_lightning_recurrence(const float* proj, long long ld, int q_off, int k_off, int v_off,
                                         const float* decay, float* state, long long state_stride,
                                         const int* qo_indptr, const int* state_slots, float* out, int n_entries, int H,
                                         int dim, int vdim, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (dim <= 0 || dim > 256 || vdim <= 0 || H <= 0 || H > 65535 || n_entries > 65535)
    return (int)cudaErrorInvalidValue;
  const dim3 grid((vdim + LT_COLS - 1) / LT_COLS, H, n_entries);
  // few blocks (a lone prompt): 32 lanes per column, so that an SM holds 16 warps of its one block; many blocks
  // (a decode batch): 8 lanes with more rows each, and the SMs fill with blocks
  const bool few = (long long)grid.x * grid.y * grid.z < 4 * 148;
#define LL(NR, L)                                                                                                  \
  BSPEC_LAUNCH_SERIALIZED((lightning_recurrence_kernel<NR, L>), grid, LT_COLS * L, 0, stream, proj, ld, q_off,     \
                          k_off, v_off, decay, state, state_stride, qo_indptr, state_slots, out, H, dim, vdim)
  if (dim <= 32) LL(4, 8);
  else if (dim <= 64) { if (few) LL(4, 16); else LL(8, 8); }
  else if (dim <= 128) { if (few) LL(4, 32); else LL(16, 8); }
  else { if (few) LL(8, 32); else LL(32, 8); }
#undef LL
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_scan_conv(const float* xz, long long ld, const void* conv, const void* bias, int w_dtype,
                              const float* state, long long state_stride, long long tail_off, const int* qo_indptr,
                              const int* tok_entry, const int* state_slots, float* xc, void* xc_run, int run_dtype,
                              int n, int inner, int taps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (inner <= 0 || taps < 1) return (int)cudaErrorInvalidValue;
  const int threads = inner >= 256 ? 256 : ((inner + 31) / 32) * 32;
  const dim3 grid(n, (inner + threads - 1) / threads);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  if (run_dtype == BSPEC_F32)
    BSPEC_LAUNCH((scan_conv_kernel<float>), grid, threads, 0, stream, xz, ld, conv, bias, w_dtype, state, state_stride,
                 tail_off, qo_indptr, tok_entry, state_slots, xc, (float*)nullptr, inner, taps);
  else
    BSPEC_LAUNCH((scan_conv_kernel<__nv_bfloat16>), grid, threads, 0, stream, xz, ld, conv, bias, w_dtype, state,
                 state_stride, tail_off, qo_indptr, tok_entry, state_slots, xc, (__nv_bfloat16*)xc_run, inner, taps);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_selective_scan(const float* xz, long long ld, const float* xc, const float* dt_raw, const float* bc,
                                   long long ld_bc, const float* a2t, const void* dvec, const void* dt_bias,
                                   int w_dtype, float* state, long long state_stride, long long tail_off,
                                   const int* qo_indptr, const int* state_slots, void* out, int out_dtype,
                                   long long out_stride, float out_scale, int n_entries, int inner, int N, int taps,
                                   cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (inner <= 0 || N <= 0 || N > SC_MAX_N || taps < 1 || n_entries > 65535) return (int)cudaErrorInvalidValue;
  // few channels x requests: more lanes per channel, so that a lone prompt's chain is shorter and more SMs take part
  const bool few = (long long)((inner + SC_THREADS - 1) / SC_THREADS) * n_entries < 148;
#define LS(T, NPL, LN)                                                                                               \
  BSPEC_LAUNCH_SERIALIZED((selective_scan_kernel<T, NPL, LN>),                                                       \
                          dim3((inner + SC_THREADS / LN - 1) / (SC_THREADS / LN), n_entries), SC_THREADS, 0, stream, \
                          xz, ld, xc, dt_raw, bc, ld_bc, a2t, dvec, dt_bias, w_dtype, state, state_stride, tail_off, \
                          qo_indptr, state_slots, (T*)out, out_stride, out_scale, inner, N, taps)
#define LSN(T)                                                                                                       \
  do {                                                                                                               \
    if (few) {                                                                                                       \
      if (N <= 16) LS(T, 4, 4); else if (N <= 32) LS(T, 8, 4); else if (N <= 64) LS(T, 8, 8);                        \
      else if (N <= 128) LS(T, 16, 8); else LS(T, 32, 8);                                                            \
    } else {                                                                                                         \
      if (N <= 16) LS(T, 16, 1); else if (N <= 32) LS(T, 32, 1); else if (N <= 64) LS(T, 32, 2);                     \
      else if (N <= 128) LS(T, 32, 4); else LS(T, 32, 8);                                                            \
    }                                                                                                                \
  } while (0)
  if (out_dtype == BSPEC_F32) LSN(float); else LSN(__nv_bfloat16);
#undef LSN
#undef LS
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_state_mixers)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_state_mixers)
