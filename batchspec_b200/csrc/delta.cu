// Gated delta rule mixer: a recurrent layer whose per-request state is one [key dim x value dim] matrix per head
// plus the last inputs of its short convolutions.  Per head and token, all in float32:
//
//     S <- g S;   u = beta (v - S^T k);   S <- S + k u^T;   o = S^T q
//
// Three kernels, one after the other on the stream:
//   delta_prepare     per (token, head): causal short convolution + silu of the q, k, v channels (the inputs before the
//                     portion come from the request's state), unit length of every q and k head (q also times a
//                     scale), beta = sigmoid(b), g = exp(-exp(A_log) softplus(a + dt_bias))
//   delta_recurrence  per (request, head, 32 or 8 value columns): the token loop over the portion with the state in
//                     registers (a column of S is spread over four lanes), state read at the start and written at
//                     the end; the request's blocks also move the convolutions' inputs on
//   gated_rmsnorm     per (token, head): o / rms(o) * w * silu(gate)
//
// The order of every sum depends on the sizes alone, not on how a request was cut into portions or on what else is
// in the step.
#include "common.cuh"
#include <cuda_pipeline.h>
#include <math.h>
using namespace bspec;

namespace {

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 30.f ? x : log1pf(expf(x)); }

// proj [n, ld] float32, columns [q: Gk*dim | k: Gk*dim | v: H*vdim | ... | b: H at b_off | a: H at a_off].
// conv [C, taps] (C = 2*Gk*dim + H*vdim).  State row of a request: [H*vdim*dim matrix | (taps-1) x C inputs, oldest
// first]; a column of the matrix holds dim numbers padded to a multiple of 4.  mix [n, C] and gates [n, 2H] (beta, then g) are float32.
constexpr int DP_WARPS = 4;
constexpr int MAX_DIM = 256;       // largest key size (a head's q or k)

// One warp per head: q heads, then k heads (dim channels each, made unit length), then v heads (vdim channels).
__global__ void __launch_bounds__(DP_WARPS * 32)
delta_prepare_kernel(const float* __restrict__ proj, int ld, int b_off, int a_off, const void* __restrict__ conv,
                     const void* __restrict__ a_log, const void* __restrict__ dt_bias, int w_dtype,
                     const float* __restrict__ state, long long state_stride, long long tail_off,
                     const int* __restrict__ qo_indptr, const int* __restrict__ tok_entry,
                     const int* __restrict__ state_slots, float* __restrict__ mix, float* __restrict__ gates, int H,
                     int Gk, int dim, int vdim, int taps, float q_scale, float unit_eps) {
  bspec::pdl_prologue(60);
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (blockIdx.y == 0) {
    for (int h = threadIdx.x; h < H; h += blockDim.x) {
      const float b = proj[(size_t)t * ld + b_off + h], a = proj[(size_t)t * ld + a_off + h];
      gates[(size_t)t * 2 * H + h] = 1.f / (1.f + expf(-b));
      const float rate = expf(load_as_f32(a_log, w_dtype, h)) * softplus_f(a + load_as_f32(dt_bias, w_dtype, h));
      gates[(size_t)t * 2 * H + H + h] = expf(-rate);
    }
  }
  const int slot = blockIdx.y * DP_WARPS + warp;
  if (slot >= 2 * Gk + H) return;
  const int e = tok_entry[t];
  const int i = t - qo_indptr[e];                  // index of the token in its portion
  const int C = 2 * Gk * dim + H * vdim;
  const float* tail = state + (size_t)state_slots[e] * state_stride + tail_off;
  const bool is_v = slot >= 2 * Gk;
  const int width = is_v ? vdim : dim;
  const int c0 = is_v ? 2 * Gk * dim + (slot - 2 * Gk) * vdim : slot * dim;
  float* row = mix + (size_t)t * C;
  auto convolved = [&](int c) {                    // silu of the causal convolution of channel c, oldest input first
    float y = 0.f;
    for (int j = taps - 1; j >= 0; --j) {
      const int rel = i - j;
      const float x = rel >= 0 ? proj[(size_t)(t - j) * ld + c] : tail[(size_t)(rel + taps - 1) * C + c];
      y += load_as_f32(conv, w_dtype, (size_t)c * taps + (taps - 1 - j)) * x;
    }
    return silu_f(y);
  };
  if (is_v) {
    for (int d = lane; d < width; d += 32) row[c0 + d] = convolved(c0 + d);
    return;
  }
  float y[8];                                      // dim <= 256
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int d = lane + 32 * k;
    y[k] = d < width ? convolved(c0 + d) : 0.f;
    ss += y[k] * y[k];
  }
  ss = warp_sum(ss);
  const float r = (slot < Gk ? q_scale : 1.f) / sqrtf(ss + unit_eps);
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int d = lane + 32 * k;
    if (d < width) row[c0 + d] = y[k] * r;
  }
}

// LANES: lanes that share one column of S; R: floats of the column that one lane holds (a multiple of 4, dim <=
// LANES R); COLS: value columns of a block.  Lane r holds rows 4 LANES c + 4 r + {0..3} for c < R / 4, so that the
// lanes of a column read contiguous bytes of state at a time.  Many short columns per block (LANES 4, COLS 32) when
// the step has enough (request, head) pairs to fill the device; else (one long prompt) a column is spread over 16
// lanes and a block holds 8 columns, which makes four times as many warps with dependent chains a quarter as long.  Per token both read-outs are taken from the state before the write,
//     a = S^T k,  b = S^T q,  u = beta (v - g a),  o = g b + u (k . q),  S <- g S + k u^T,
// which is the rule above with o = (g S + k u^T)^T q multiplied out: one pass over the registers for the three sums
// (reduced over the column's lanes together), one for the update.  The 16-lane form takes two tokens per pass.  The next tile of tokens is copied into the
// other half of the staging buffers while the current one is worked on.
template <int R, int COLS, int LANES>
__global__ void __launch_bounds__(COLS * LANES)
delta_recurrence_kernel(const float* __restrict__ mix, const float* __restrict__ gates, const float* __restrict__ proj,
                        int ld, float* __restrict__ state, long long state_stride, long long tail_off,
                        const int* __restrict__ qo_indptr, const int* __restrict__ state_slots,
                        float* __restrict__ out, int H, int Gk, int dim, int vdim, int taps) {
  bspec::pdl_prologue_late(61);
  constexpr int NT = COLS * LANES, DP = LANES * R;
  constexpr int TILE = DP > 128 ? 8 : 16;          // tokens whose q, k, v, beta, g are staged in shared memory at a time
  const int dimp = (dim + 3) & ~3;                 // a column of S is kept padded to whole float4s; the pad stays 0
  __shared__ __align__(16) float qs[2][TILE][DP];
  __shared__ __align__(16) float ks[2][TILE][DP];
  __shared__ float vs[2][TILE][COLS];
  __shared__ float bg[2][TILE][2];
  __shared__ float sc[TILE / 2][4];                // products between the two tokens of every pair of the tile
  const int e = blockIdx.z, h = blockIdx.y;
  const int q_begin = qo_indptr[e], n = qo_indptr[e + 1] - q_begin;
  const int C = 2 * Gk * dim + H * vdim;
  float* srow = state + (size_t)state_slots[e] * state_stride;
  if (n <= 0) return;
  if (taps > 1) {
    // the convolutions' inputs: slot s holds the input at index n + s - (taps - 1) of this portion, or what an
    // older slot held; ascending s, so that a slot is read before it is overwritten.  The request's blocks share
    // the channels (a thread moves all slots of its channel), so that no block is the step's long pole.
    float* tail = srow + tail_off;
    const int share = blockIdx.y * gridDim.x + blockIdx.x, shares = gridDim.y * gridDim.x;
    for (int c = share * NT + threadIdx.x; c < C; c += shares * NT)
      for (int s = 0; s < taps - 1; ++s) {
        const int rel = n + s - (taps - 1);
        tail[(size_t)s * C + c] = rel >= 0 ? proj[(size_t)(q_begin + rel) * ld + c] : tail[(size_t)(s + n) * C + c];
      }
  }
  const int col = threadIdx.x / LANES, r = threadIdx.x % LANES;
  const int j = blockIdx.x * COLS + col;
  const bool live = j < vdim;
  const int kh = h / (H / Gk);
  // the pad of a row is never copied into: zero it once in both halves
  for (int w = threadIdx.x; w < 2 * TILE * (DP - dim); w += NT) {
    const int bt = w / (DP - dim), d = dim + w % (DP - dim);
    qs[bt / TILE][bt % TILE][d] = 0.f;
    ks[bt / TILE][bt % TILE][d] = 0.f;
  }
  auto stage = [&](int t0, int buf) {              // asynchronous copies of tokens t0 .. t0 + TILE - 1 of the portion
    const int nt = min(TILE, n - t0);
    if (((dim | C) & 3) == 0) {                    // rows of q and k start on 16-byte boundaries
      for (int tt = threadIdx.x >> 5; tt < nt; tt += NT / 32) {        // a warp per token: equal work for all warps
        const float* row = mix + (size_t)(q_begin + t0 + tt) * C;
        for (int d = 4 * (threadIdx.x & 31); d < dim; d += 128) {
          __pipeline_memcpy_async(&qs[buf][tt][d], row + kh * dim + d, 16);
          __pipeline_memcpy_async(&ks[buf][tt][d], row + (Gk + kh) * dim + d, 16);
        }
      }
    } else {
      for (int w = threadIdx.x; w < nt * dim; w += NT) {
        const int tt = w / dim, d = w - tt * dim;
        const float* row = mix + (size_t)(q_begin + t0 + tt) * C;
        __pipeline_memcpy_async(&qs[buf][tt][d], row + kh * dim + d, 4);
        __pipeline_memcpy_async(&ks[buf][tt][d], row + (Gk + kh) * dim + d, 4);
      }
    }
    for (int w = threadIdx.x; w < nt * COLS; w += NT) {
      const int tt = w / COLS, cc = w - tt * COLS;
      const int jj = blockIdx.x * COLS + cc;
      if (jj < vdim)
        __pipeline_memcpy_async(&vs[buf][tt][cc], mix + (size_t)(q_begin + t0 + tt) * C + 2 * Gk * dim + h * vdim + jj, 4);
    }
    if (threadIdx.x < nt * 2) {
      const int tt = threadIdx.x >> 1, which = threadIdx.x & 1;
      __pipeline_memcpy_async(&bg[buf][tt][which], gates + (size_t)(q_begin + t0 + tt) * 2 * H + which * H + h, 4);
    }
    __pipeline_commit();
  };
  stage(0, 0);
  float s[R];
  float* sp = srow + ((size_t)h * vdim + (live ? j : 0)) * dimp;
#pragma unroll
  for (int c = 0; c < R / 4; ++c) {
    const int row = 4 * LANES * c + 4 * r;
    float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
    if (live && row < dimp) v = *reinterpret_cast<const float4*>(sp + row);
    s[4 * c] = v.x; s[4 * c + 1] = v.y; s[4 * c + 2] = v.z; s[4 * c + 3] = v.w;
  }
  int buf = 0;
  for (int t0 = 0; t0 < n; t0 += TILE, buf ^= 1) {
    const int nt = min(TILE, n - t0);
    __pipeline_wait_prior(0);
    __syncthreads();                                // the tile is there, and every thread is done with the other half
    if (t0 + TILE < n) stage(t0 + TILE, buf ^ 1);
    // one token: both read-outs from the state before the write, then the write
    auto one_token = [&](int tt, const float4* kr, const float4* qr) {
      const float beta = bg[buf][tt][0], g = bg[buf][tt][1], vj = vs[buf][tt][col];
      float a0 = 0.f, a1 = 0.f, b0 = 0.f, b1 = 0.f, kq = 0.f;
#pragma unroll
      for (int c = 0; c < R / 4; ++c) {
        const float4 k4 = kr[c], q4 = qr[c];
        a0 += s[4 * c] * k4.x; a1 += s[4 * c + 1] * k4.y; a0 += s[4 * c + 2] * k4.z; a1 += s[4 * c + 3] * k4.w;
        b0 += s[4 * c] * q4.x; b1 += s[4 * c + 1] * q4.y; b0 += s[4 * c + 2] * q4.z; b1 += s[4 * c + 3] * q4.w;
        kq += k4.x * q4.x; kq += k4.y * q4.y; kq += k4.z * q4.z; kq += k4.w * q4.w;
      }
      float a = a0 + a1, b = b0 + b1;
#pragma unroll
      for (int o = 1; o < LANES; o <<= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, o);
        b += __shfl_xor_sync(0xffffffffu, b, o);
        kq += __shfl_xor_sync(0xffffffffu, kq, o);
      }
      const float u = beta * (vj - g * a);
      if (live && r == 0) out[(size_t)(q_begin + t0 + tt) * H * vdim + h * vdim + j] = g * b + u * kq;
#pragma unroll
      for (int c = 0; c < R / 4; ++c) {
        const float4 k4 = kr[c];
        s[4 * c] = fmaf(k4.x, u, g * s[4 * c]);
        s[4 * c + 1] = fmaf(k4.y, u, g * s[4 * c + 1]);
        s[4 * c + 2] = fmaf(k4.z, u, g * s[4 * c + 2]);
        s[4 * c + 3] = fmaf(k4.w, u, g * s[4 * c + 3]);
      }
    };
    auto fetch = [&](int tt, float4* kd, float4* qd) {
#pragma unroll
      for (int c = 0; c < R / 4; ++c) {
        const int row = 4 * LANES * c + 4 * r;      // rows beyond dim hold zeros in the state and in the staging
        kd[c] = *reinterpret_cast<const float4*>(&ks[buf][tt][row]);
        qd[c] = *reinterpret_cast<const float4*>(&qs[buf][tt][row]);
      }
    };
    if constexpr (LANES == 16) {
      // The long chain of one prompt: two tokens per pass.  With a = S^T k and b = S^T q of BOTH tokens taken from
      // the state before either write, and the tokens' mutual products (the same for every column, formed once
      // per tile below),
      //   u1 = beta1 (v1 - g1 a1)                    o1 = g1 b1 + u1 (k1.q1)
      //   u2 = beta2 (v2 - g2 (g1 a2 + u1 (k1.k2)))  o2 = g2 (g1 b2 + u1 (k1.q2)) + u2 (k2.q2)
      //   S <- g1 g2 S + g2 u1 k1 + u2 k2,
      // which is the rule applied twice, multiplied out: one round of reductions and one pass over the registers
      // for two tokens.
      {
        const int pr = min((int)(threadIdx.x >> 4), TILE / 2 - 1), sub = threadIdx.x & 15;
        const float *k1 = ks[buf][2 * pr], *q1 = qs[buf][2 * pr], *k2 = ks[buf][2 * pr + 1], *q2 = qs[buf][2 * pr + 1];
        float x0 = 0.f, x1 = 0.f, x2 = 0.f, x3 = 0.f;
        for (int d = sub; d < dimp; d += 16) {
          x0 += k1[d] * q1[d]; x1 += k1[d] * k2[d]; x2 += k1[d] * q2[d]; x3 += k2[d] * q2[d];
        }
#pragma unroll
        for (int o = 1; o < 16; o <<= 1) {
          x0 += __shfl_xor_sync(0xffffffffu, x0, o); x1 += __shfl_xor_sync(0xffffffffu, x1, o);
          x2 += __shfl_xor_sync(0xffffffffu, x2, o); x3 += __shfl_xor_sync(0xffffffffu, x3, o);
        }
        if (sub == 0 && (int)(threadIdx.x >> 4) < TILE / 2 && 2 * pr + 1 < nt) {
          sc[pr][0] = x0; sc[pr][1] = x1; sc[pr][2] = x2; sc[pr][3] = x3;
        }
      }
      __syncthreads();
      const int np = nt >> 1;
      float4 k1n[R / 4], q1n[R / 4], k2n[R / 4], q2n[R / 4];
      if (np > 0) { fetch(0, k1n, q1n); fetch(1, k2n, q2n); }
      for (int pp = 0; pp < np; ++pp) {
        float4 k1[R / 4], q1[R / 4], k2[R / 4], q2[R / 4];
#pragma unroll
        for (int c = 0; c < R / 4; ++c) { k1[c] = k1n[c]; q1[c] = q1n[c]; k2[c] = k2n[c]; q2[c] = q2n[c]; }
        const int t1 = 2 * pp, t2 = 2 * pp + 1;
        const float beta1 = bg[buf][t1][0], g1 = bg[buf][t1][1], v1 = vs[buf][t1][col];
        const float beta2 = bg[buf][t2][0], g2 = bg[buf][t2][1], v2 = vs[buf][t2][col];
        const float kq11 = sc[pp][0], kk12 = sc[pp][1], kq12 = sc[pp][2], kq22 = sc[pp][3];
        float a1 = 0.f, b1 = 0.f, a2 = 0.f, b2 = 0.f;
#pragma unroll
        for (int c = 0; c < R / 4; ++c) {
          a1 += s[4 * c] * k1[c].x; a1 += s[4 * c + 1] * k1[c].y; a1 += s[4 * c + 2] * k1[c].z; a1 += s[4 * c + 3] * k1[c].w;
          b1 += s[4 * c] * q1[c].x; b1 += s[4 * c + 1] * q1[c].y; b1 += s[4 * c + 2] * q1[c].z; b1 += s[4 * c + 3] * q1[c].w;
          a2 += s[4 * c] * k2[c].x; a2 += s[4 * c + 1] * k2[c].y; a2 += s[4 * c + 2] * k2[c].z; a2 += s[4 * c + 3] * k2[c].w;
          b2 += s[4 * c] * q2[c].x; b2 += s[4 * c + 1] * q2[c].y; b2 += s[4 * c + 2] * q2[c].z; b2 += s[4 * c + 3] * q2[c].w;
        }
        if (pp + 1 < np) { fetch(2 * pp + 2, k1n, q1n); fetch(2 * pp + 3, k2n, q2n); }
#pragma unroll
        for (int o = 1; o < LANES; o <<= 1) {
          a1 += __shfl_xor_sync(0xffffffffu, a1, o); b1 += __shfl_xor_sync(0xffffffffu, b1, o);
          a2 += __shfl_xor_sync(0xffffffffu, a2, o); b2 += __shfl_xor_sync(0xffffffffu, b2, o);
        }
        const float u1 = beta1 * (v1 - g1 * a1);
        const float u2 = beta2 * (v2 - g2 * (g1 * a2 + u1 * kk12));
        if (live && r == 0) {
          float* op = out + (size_t)(q_begin + t0 + t1) * H * vdim + h * vdim + j;
          op[0] = g1 * b1 + u1 * kq11;
          op[(size_t)H * vdim] = g2 * (g1 * b2 + u1 * kq12) + u2 * kq22;
        }
        const float c0 = g1 * g2, c1 = g2 * u1;
#pragma unroll
        for (int c = 0; c < R / 4; ++c) {
          s[4 * c] = fmaf(k2[c].x, u2, fmaf(k1[c].x, c1, c0 * s[4 * c]));
          s[4 * c + 1] = fmaf(k2[c].y, u2, fmaf(k1[c].y, c1, c0 * s[4 * c + 1]));
          s[4 * c + 2] = fmaf(k2[c].z, u2, fmaf(k1[c].z, c1, c0 * s[4 * c + 2]));
          s[4 * c + 3] = fmaf(k2[c].w, u2, fmaf(k1[c].w, c1, c0 * s[4 * c + 3]));
        }
      }
      if (nt & 1) {                                 // the portion's last token
        float4 kr[R / 4], qr[R / 4];
        fetch(nt - 1, kr, qr);
        one_token(nt - 1, kr, qr);
      }
    } else {
      for (int tt = 0; tt < nt; ++tt) {
        float4 kr[R / 4], qr[R / 4];
        fetch(tt, kr, qr);
        one_token(tt, kr, qr);
      }
    }
  }
  bspec::pdl_launch_dependents();
  if (live) {
#pragma unroll
    for (int c = 0; c < R / 4; ++c) {
      const int row = 4 * LANES * c + 4 * r;
      if (row < dimp) *reinterpret_cast<float4*>(sp + row) = make_float4(s[4 * c], s[4 * c + 1], s[4 * c + 2], s[4 * c + 3]);
    }
  }
}

// out[t, h*V + j] = o[t, h, j] / sqrt(mean_j o^2 + eps) * w[j] * act(gate[t, h*V + j]), act = silu (gate_kind 0) or
// sigmoid (1); one warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(128)
gated_rmsnorm_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long gate_stride,
                     const void* __restrict__ w, int w_dtype, T* __restrict__ out, int n, int H, int V, float eps,
                     int gate_kind) {
  bspec::pdl_prologue(62);
  const int item = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= n * H) return;
  const int t = item / H, h = item - t * H;
  const float* x = o + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int j = lane; j < V; j += 32) ss += x[j] * x[j];
  ss = warp_sum(ss);
  const float r = 1.f / sqrtf(ss / (float)V + eps);
  const float* gp = gate + (size_t)t * gate_stride + (size_t)h * V;
  T* op = out + ((size_t)t * H + h) * V;
  for (int j = lane; j < V; j += 32) op[j] = from_f32<T>(x[j] * r * load_as_f32(w, w_dtype, j) * (gate_kind == 1 ? 1.f / (1.f + expf(-gp[j])) : silu_f(gp[j])));
}

// The same for wide groups (all heads normed together: V in the thousands), where a warp per group would leave a
// decode step on a handful of warps: a block of 256 threads per (token, group), the sum of squares joined through
// shared memory in a fixed order.
template <typename T>
__global__ void __launch_bounds__(256)
gated_rmsnorm_wide_kernel(const float* __restrict__ o, const float* __restrict__ gate, long long gate_stride,
                          const void* __restrict__ w, int w_dtype, T* __restrict__ out, int H, int V, float eps,
                          int gate_kind) {
  bspec::pdl_prologue(62);
  __shared__ float part[8];
  const int item = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = item / H, h = item - t * H;
  const float* x = o + ((size_t)t * H + h) * V;
  float ss = 0.f;
  for (int j = threadIdx.x; j < V; j += 256) ss += x[j] * x[j];
  ss = warp_sum(ss);
  if (lane == 0) part[warp] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += part[i];
  const float r = 1.f / sqrtf(tot / (float)V + eps);
  const float* gp = gate + (size_t)t * gate_stride + (size_t)h * V;
  T* op = out + ((size_t)t * H + h) * V;
  for (int j = threadIdx.x; j < V; j += 256)
    op[j] = from_f32<T>(x[j] * r * load_as_f32(w, w_dtype, j) * (gate_kind == 1 ? 1.f / (1.f + expf(-gp[j])) : silu_f(gp[j])));
}
}  // namespace

BSPEC_API int bspec_delta_prepare(const float* proj, int n, int ld, int b_off, int a_off, const void* conv,
                                  const void* a_log, const void* dt_bias, int w_dtype, const float* state,
                                  long long state_stride, long long tail_off, const int* qo_indptr,
                                  const int* tok_entry, const int* state_slots, float* mix, float* gates, int H, int Gk,
                                  int dim, int vdim, int taps, float q_scale, float unit_eps, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (H <= 0 || Gk <= 0 || H % Gk != 0 || taps < 1) return (int)cudaErrorInvalidValue;
  if (dim > 256) return (int)cudaErrorInvalidValue;
  const dim3 grid(n, (2 * Gk + H + DP_WARPS - 1) / DP_WARPS);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  BSPEC_LAUNCH(delta_prepare_kernel, grid, DP_WARPS * 32, 0, stream, proj, ld, b_off, a_off, conv, a_log, dt_bias, w_dtype,
               state, state_stride, tail_off, qo_indptr, tok_entry, state_slots, mix, gates, H, Gk, dim, vdim, taps,
               q_scale, unit_eps);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_delta_recurrence(const float* mix, const float* gates, const float* proj, int ld, float* state,
                                     long long state_stride, long long tail_off, const int* qo_indptr,
                                     const int* state_slots, float* out, int n_entries, int H, int Gk, int dim,
                                     int vdim, int taps, cudaStream_t stream) {
  if (n_entries <= 0) return 0;
  if (dim <= 0 || dim > MAX_DIM || H % Gk != 0 || n_entries > 65535 || H > 65535)
    return (int)cudaErrorInvalidValue;
  // 32 value columns of 4 lanes per block; 8 columns of 16 lanes when that would leave most of the device idle
  const bool narrow = (long long)((vdim + 31) / 32) * H * n_entries < 2ll * bspec::sm_count();
  const int cols = narrow ? 8 : 32;
  const dim3 grid((vdim + cols - 1) / cols, H, n_entries);
#define LR(R4, R16)                                                                                                \
  do {                                                                                                             \
    if (narrow)                                                                                                    \
      BSPEC_LAUNCH_SERIALIZED((delta_recurrence_kernel<R16, 8, 16>), grid, 8 * 16, 0, stream, mix, gates, proj, ld, state, \
                   state_stride, tail_off, qo_indptr, state_slots, out, H, Gk, dim, vdim, taps);                   \
    else                                                                                                           \
      BSPEC_LAUNCH_SERIALIZED((delta_recurrence_kernel<R4, 32, 4>), grid, 32 * 4, 0, stream, mix, gates, proj, ld, state,     \
                   state_stride, tail_off, qo_indptr, state_slots, out, H, Gk, dim, vdim, taps);                   \
  } while (0)
  if (dim <= 32) LR(8, 4); else if (dim <= 64) LR(16, 4); else if (dim <= 128) LR(32, 8); else LR(64, 16);
#undef LR
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_gated_rmsnorm(const float* o, const float* gate, long long gate_stride, const void* w, int w_dtype,
                                  void* out, int out_dtype, int n, int H, int V, float eps, int gate_kind,
                                  cudaStream_t stream) {
  if (n <= 0) return 0;
  if (V >= 512) {                                            // the choice rests on the group's size alone
    if (out_dtype == BSPEC_F32)
      BSPEC_LAUNCH((gated_rmsnorm_wide_kernel<float>), n * H, 256, 0, stream, o, gate, gate_stride, w, w_dtype,
                   (float*)out, H, V, eps, gate_kind);
    else
      BSPEC_LAUNCH((gated_rmsnorm_wide_kernel<__nv_bfloat16>), n * H, 256, 0, stream, o, gate, gate_stride, w, w_dtype,
                   (__nv_bfloat16*)out, H, V, eps, gate_kind);
    return BSPEC_LAUNCH_CHECK();
  }
  const int blocks = (n * H + 3) / 4;
  if (out_dtype == BSPEC_F32)
    BSPEC_LAUNCH((gated_rmsnorm_kernel<float>), blocks, 128, 0, stream, o, gate, gate_stride, w, w_dtype, (float*)out, n, H, V, eps, gate_kind);
  else
    BSPEC_LAUNCH((gated_rmsnorm_kernel<__nv_bfloat16>), blocks, 128, 0, stream, o, gate, gate_stride, w, w_dtype,
                 (__nv_bfloat16*)out, n, H, V, eps, gate_kind);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_delta)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_delta)
