// Routed feed-forward (mixture of experts): the router, the plan that sorts (token, choice) slots by expert, a
// grouped matrix product over the sorted rows, and the weighted sum that brings the rows back to their tokens.
//
//   route     per token: z = Wr h in float32, s = sigmoid(z), choice = s + correction; the experts come in equal
//             groups of neighbours, a group's score is the sum of its two largest choices, only the best `keep`
//             groups stay (the others count as minus infinity); the `top` largest choices are taken, ties to the
//             lower index; weights = s of the chosen * scale (no renormalisation).  With `softmax_top` instead:
//             choice = z + bias (the `correction` tensor), the `top` largest are taken, and the weights are the
//             softmax over the chosen logits alone
//   plan      one block: counts per expert, a stable counting sort of the n*top slots by expert (row r of the
//             sorted order holds slot perm[r]; inv[slot] = r), and the list of row tiles (expert, first row, rows)
//   grouped   C[r, :] = act(A[src(r), :] . W[expert(r)]^T) over the tiles of the plan; every output element is one
//             thread's sum over k in ascending order, so a row's result does not depend on where it was sorted to
//             (act: GELU on the outputs, or none; the operand A may be gated instead: its rows are [gate | up] and
//             silu(gate) * up is formed while they are staged, which is how gated experts run their down projection)
//   combine   out[t, :] = sum_k weight[t, k] * Y[inv[t*top + k], :], k ascending, float32
//
// Nothing here reads a count on the host: grids are sized by upper bounds and surplus blocks leave at once, so the
// kernels can be captured in a graph.
#include "common.cuh"
#include <math.h>
using namespace bspec;

namespace {

constexpr int ROUTE_THREADS = 128;
constexpr int MAX_EXPERTS = 1024;

template <typename T>
__global__ void __launch_bounds__(ROUTE_THREADS)
moe_route_kernel(const T* __restrict__ h, int d, const T* __restrict__ wr, const void* __restrict__ corr,
                 int corr_dtype, int E, int G, int keep, int top, float scale, int* __restrict__ ids,
                 float* __restrict__ wts, const float* __restrict__ logits, int softmax_top) {
  bspec::pdl_prologue(50);
  extern __shared__ float sm[];
  float* hs = sm;                 // [d]
  float* sc = hs + d;             // [E] sigmoid scores
  float* ch = sc + E;             // [E] choice scores (masked in place)
  const int t = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  if (logits != nullptr) {            // the logits were formed by a matrix product (many tokens)
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
      const float z = logits[(size_t)t * E + e], b = corr != nullptr ? load_as_f32(corr, corr_dtype, e) : 0.f;
      const float s = softmax_top ? z + b : 1.f / (1.f + expf(-z));
      sc[e] = s;
      ch[e] = softmax_top ? s : s + b;
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) hs[i] = to_f32(h[(size_t)t * d + i]);
    __syncthreads();
    for (int e = warp; e < E; e += ROUTE_THREADS / 32) {
      const T* w = wr + (size_t)e * d;
      float z = 0.f;
      for (int i = lane; i < d; i += 32) z += hs[i] * to_f32(w[i]);
      z = warp_sum(z);
      if (lane == 0) {
        const float b = corr != nullptr ? load_as_f32(corr, corr_dtype, e) : 0.f;
        const float s = softmax_top ? z + b : 1.f / (1.f + expf(-z));
        sc[e] = s;
        ch[e] = softmax_top ? s : s + b;
      }
    }
  }
  __syncthreads();
  if (warp != 0) return;
  // The choice is made by warp 0: every lane scans its share of the candidates, a shuffle tree finds the best
  // (the larger value, the lower index among equals), lane 0 marks it as taken (NaN).
  auto best_of = [&](const float* v, int n) -> int {
    float bv = 0.f;
    int bi = 0x7fffffff;
    for (int i = lane; i < n; i += 32) {
      const float x = v[i];
      if (!isnan(x) && (bi == 0x7fffffff || x > bv)) { bv = x; bi = i; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (oi != 0x7fffffff && (bi == 0x7fffffff || ov > bv || (ov == bv && oi < bi))) { bv = ov; bi = oi; }
    }
    return bi;
  };
  if (G > 1 && keep < G) {
    const int per = E / G;
    for (int g = lane; g < G; g += 32) {          // group scores into the start of hs (no longer needed)
      float a = -INFINITY, b = -INFINITY;         // the two largest
      for (int j = 0; j < per; ++j) {
        const float v = ch[g * per + j];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      hs[g] = per > 1 ? a + b : a;
    }
    __syncwarp();
    for (int k = 0; k < keep; ++k) {
      const int best = best_of(hs, G);
      if (lane == 0 && best != 0x7fffffff) hs[best] = NAN;      // NaN marks a kept group
      __syncwarp();
    }
    for (int i = lane; i < E; i += 32)
      if (!isnan(hs[i / per])) ch[i] = -INFINITY;
    __syncwarp();
  }
  for (int k = 0; k < top; ++k) {
    int best = best_of(ch, E);
    if (best == 0x7fffffff) best = 0;
    if (lane == 0) {
      ids[(size_t)t * top + k] = best;
      wts[(size_t)t * top + k] = sc[best] * scale;
      ch[best] = NAN;                             // taken
    }
    __syncwarp();
  }
  if (softmax_top && lane == 0) {                 // the weights: softmax over the chosen logits alone
    float* w = wts + (size_t)t * top;
    float mx = -INFINITY, sum = 0.f;
    for (int k = 0; k < top; ++k) mx = fmaxf(mx, sc[ids[(size_t)t * top + k]]);
    for (int k = 0; k < top; ++k) sum += expf(sc[ids[(size_t)t * top + k]] - mx);
    for (int k = 0; k < top; ++k) w[k] = expf(sc[ids[(size_t)t * top + k]] - mx) / sum * scale;
  }
}

// One block of 1024 threads.  tiles: int [max_tiles][3] = {expert, first sorted row, rows}; n_tiles_out: int [1].
__global__ void __launch_bounds__(1024)
moe_plan_kernel(const int* __restrict__ ids, int slots, int E, int BM, int* __restrict__ perm, int* __restrict__ inv,
                int* __restrict__ offsets, int* __restrict__ tiles, int* __restrict__ n_tiles_out, int max_tiles) {
  bspec::pdl_prologue(51);
  __shared__ int cnt[MAX_EXPERTS + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
  for (int e = warp; e < E; e += nwarps) {
    int c = 0;
    for (int s0 = 0; s0 < slots; s0 += 32) {
      const int s = s0 + lane;
      c += __popc(__ballot_sync(0xffffffffu, s < slots && ids[s] == e));
    }
    if (lane == 0) cnt[e] = c;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0, nt = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cnt[e];
      cnt[e] = run;
      offsets[e] = run;
      for (int r = 0; r < c && nt < max_tiles; r += BM) {
        tiles[3 * nt] = e;
        tiles[3 * nt + 1] = run + r;
        tiles[3 * nt + 2] = min(BM, c - r);
        ++nt;
      }
      run += c;
    }
    cnt[E] = run;
    offsets[E] = run;
    *n_tiles_out = nt;
  }
  __syncthreads();
  for (int e = warp; e < E; e += nwarps) {
    int at = cnt[e];
    for (int s0 = 0; s0 < slots; s0 += 32) {
      const int s = s0 + lane;
      const bool mine = s < slots && ids[s] == e;
      const unsigned mask = __ballot_sync(0xffffffffu, mine);
      if (mine) {
        const int r = at + __popc(mask & ((1u << lane) - 1u));
        perm[r] = s;
        inv[s] = r;
      }
      at += __popc(mask);
    }
  }
}

// The same plan for many rows, in three kernels over all SMs.  Rows of one expert are placed in the order in which
// their warps reach the expert's counter, so the placement (not any value: a row's result does not depend on where
// it lies) may differ from run to run.
__global__ void __launch_bounds__(256)
moe_rank_kernel(const int* __restrict__ ids, int slots, int* __restrict__ counts, int* __restrict__ rank) {
  bspec::pdl_prologue(57);
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  const bool live = s < slots;
  const int e = live ? ids[s] : -1;
  const unsigned same = __match_any_sync(0xffffffffu, e);
  const int lane = threadIdx.x & 31;
  const int leader = __ffs(same) - 1;
  int base = 0;
  if (live && lane == leader) base = atomicAdd(&counts[e], __popc(same));
  base = __shfl_sync(0xffffffffu, base, leader);
  if (live) rank[s] = base + __popc(same & ((1u << lane) - 1u));
}

__global__ void moe_offsets_kernel(const int* __restrict__ counts, int E, int BM, int* __restrict__ offsets,
                                   int* __restrict__ tiles, int* __restrict__ n_tiles_out, int max_tiles) {
  bspec::pdl_prologue(58);
  __shared__ int cnt[MAX_EXPERTS];
  for (int e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = counts[e];      // one round trip for all counts
  __syncthreads();
  if (threadIdx.x != 0) return;
  int run = 0, nt = 0;
  for (int e = 0; e < E; ++e) {
    const int c = cnt[e];
    offsets[e] = run;
    for (int r = 0; r < c && nt < max_tiles; r += BM) {
      tiles[3 * nt] = e;
      tiles[3 * nt + 1] = run + r;
      tiles[3 * nt + 2] = min(BM, c - r);
      ++nt;
    }
    run += c;
  }
  offsets[E] = run;
  *n_tiles_out = nt;
}

__global__ void __launch_bounds__(256)
moe_place_kernel(const int* __restrict__ ids, const int* __restrict__ rank, const int* __restrict__ offsets, int slots,
                 int* __restrict__ perm, int* __restrict__ inv) {
  bspec::pdl_prologue(59);
  const int s = blockIdx.x * blockDim.x + threadIdx.x;
  if (s >= slots) return;
  const int r = offsets[ids[s]] + rank[s];
  perm[r] = s;
  inv[s] = r;
}

__device__ __forceinline__ float gelu_erf(float v) { return 0.5f * v * (1.f + erff(v * 0.70710678118654752440f)); }

// A gated operand (``gated_a`` in the kernels below): the rows of A are [gate | up], 2 K numbers, and the product's
// operand is silu(gate) * up, formed while a tile's rows are staged and rounded to A's type, as a kernel of its own
// between the two products would have left it.
__device__ __forceinline__ float silu_gate(float g, float u) { return __fdividef(g, 1.f + __expf(-g)) * u; }
__device__ __forceinline__ uint4 silu_gate8(const uint4& gv, const uint4& uv) {
  const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&gv);
  const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
  uint4 ov;
  __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
  for (int j = 0; j < 4; ++j)
    o2[j] = __floats2bfloat162_rn(silu_gate(__low2float(g2[j]), __low2float(u2[j])),
                                  silu_gate(__high2float(g2[j]), __high2float(u2[j])));
  return ov;
}

// A [*, K] rows; row r of the sorted order reads A[perm[r] / top] when perm is given (the up projection), else
// A[r] (the down projection).  W [E, N, K].  C [slots, N].  Thread tiles of TM x 4, 16 x 16 threads.
template <typename T, typename TO, int BM, bool GELU>
__global__ void __launch_bounds__(256)
moe_grouped_kernel(const T* __restrict__ A, const int* __restrict__ perm, int top, const T* __restrict__ W,
                   TO* __restrict__ C, int N, int K, const int* __restrict__ tiles, const int* __restrict__ n_tiles,
                   int gated_a) {
  bspec::pdl_prologue(52);
  constexpr int BN = 64, BK = 16, TM = BM / 16, TN = 4;
  if ((int)blockIdx.y >= *n_tiles) return;
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ int src[BM];
  const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int tid = threadIdx.x, tx = tid % 16, ty = tid / 16;
  const int n0 = blockIdx.x * BN;
  if (tid < BM) src[tid] = tid < rows ? (perm != nullptr ? perm[row0 + tid] / top : row0 + tid) : -1;
  __syncthreads();
  const T* We = W + (size_t)e * N * K;
  float acc[TM][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
  for (int k0 = 0; k0 < K; k0 += BK) {
    for (int idx = tid; idx < BM * BK; idx += 256) {
      const int r = idx / BK, k = k0 + idx % BK;
      float a = 0.f;
      if (src[r] >= 0 && k < K) {
        if (gated_a) {
          const T* row = A + (size_t)src[r] * 2 * K;
          a = to_f32(from_f32<T>(silu_gate(to_f32(row[k]), to_f32(row[K + k]))));
        } else {
          a = to_f32(A[(size_t)src[r] * K + k]);
        }
      }
      As[idx % BK][r] = a;
    }
    for (int idx = tid; idx < BN * BK; idx += 256) {
      const int r = idx / BK, k = k0 + idx % BK;
      Ws[idx % BK][r] = (n0 + r < N && k < K) ? to_f32(We[(size_t)(n0 + r) * K + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BK; ++k) {
      float a[TM], b[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[k][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) b[j] = Ws[k][tx * TN + j];
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = ty * TM + i;
    if (r >= rows) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n < N) C[(size_t)(row0 + r) * N + n] = from_f32<TO>(GELU ? gelu_erf(acc[i][j]) : acc[i][j]);
    }
  }
}

// The same product for tiles of at most 8 rows (decode-sized steps: a handful of rows per expert), bfloat16, bound
// by the read of the experts' weights.  The tile's rows wait in shared memory; every warp owns 8 output columns,
// 4 at a time; its lanes stride over K in 16-byte pieces of the weight rows (four loads in flight per lane) and a
// shuffle tree adds the lanes' sums.  A value depends on its row and column alone.
__device__ __forceinline__ float dot8(const uint4& w, const uint4& a, float acc) {
  const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&w);
  const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 x = __bfloat1622float2(w2[i]), y = __bfloat1622float2(a2[i]);
    acc = fmaf(x.x, y.x, acc);
    acc = fmaf(x.y, y.y, acc);
  }
  return acc;
}

template <typename TO, bool GELU>
__global__ void __launch_bounds__(256)
moe_skinny_kernel(const __nv_bfloat16* __restrict__ A, const int* __restrict__ perm, int top,
                  const __nv_bfloat16* __restrict__ W, TO* __restrict__ C, int N, int K, const int* __restrict__ tiles,
                  const int* __restrict__ n_tiles, int gated_a) {
  bspec::pdl_prologue(55);
  constexpr int RMAX = 8;
  if ((int)blockIdx.y >= *n_tiles) return;
  extern __shared__ uint4 As4[];                  // [rows][K / 8]
  const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K8 = K / 8;
  for (int idx = tid; idx < rows * K8; idx += 256) {
    const int r = idx / K8, c = idx - r * K8;
    const int src = perm != nullptr ? perm[row0 + r] / top : row0 + r;
    if (gated_a) {
      const uint4* row = reinterpret_cast<const uint4*>(A + (size_t)src * 2 * K);
      As4[idx] = silu_gate8(row[c], row[K8 + c]);
    } else {
      As4[idx] = reinterpret_cast<const uint4*>(A + (size_t)src * K)[c];
    }
  }
  __syncthreads();
  const __nv_bfloat16* We = W + (size_t)e * N * K;
  const int n_base = blockIdx.x * 64 + warp * 8;
#pragma unroll 1
  for (int g = 0; g < 2; ++g) {
    const int n0 = n_base + 4 * g;
    if (n0 >= N) break;
    const uint4* wrow[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) wrow[j] = reinterpret_cast<const uint4*>(We + (size_t)min(n0 + j, N - 1) * K);
    float acc[4][RMAX];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < RMAX; ++r) acc[j][r] = 0.f;
    for (int c = lane; c < K8; c += 32) {
      uint4 w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) w[j] = __ldg(wrow[j] + c);
#pragma unroll
      for (int r = 0; r < RMAX; ++r)
        if (r < rows) {
          const uint4 a = As4[r * K8 + c];
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[j][r] = dot8(w[j], a, acc[j][r]);
        }
    }
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int r = 0; r < RMAX; ++r)
        if (r < rows) {
          const float v = warp_sum(acc[j][r]);
          if (lane == 0 && n0 + j < N) C[(size_t)(row0 + r) * N + n0 + j] = from_f32<TO>(GELU ? gelu_erf(v) : v);
        }
  }
}

// The same on the tensor cores (mma.sync m16n8k16, float32 accumulation) for K a multiple of 32: the WEIGHT rows
// take the 16 rows of the product and the tile's (at most 16) token rows its 8 columns, twice.  A lane fetches 16
// contiguous bytes of two weight rows straight from global memory (no staging: every weight is used once) and 16
// bytes of a token row from shared memory; both sides number the 32 k of a step in the same permuted order
// (lane l % 4 holds k = 8 (l % 4) .. + 7), which a sum over k does not notice.  Eight loads are in flight per lane.
__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename TO, bool GELU, int RT>          // RT: token rows a tile may hold, 8 or 16
__global__ void __launch_bounds__(256)
moe_skinny_mma_kernel(const __nv_bfloat16* __restrict__ A, const int* __restrict__ perm, int top,
                      const __nv_bfloat16* __restrict__ W, TO* __restrict__ C, int N, int K,
                      const int* __restrict__ tiles, const int* __restrict__ n_tiles, int gated_a) {
  bspec::pdl_prologue(56);
  if ((int)blockIdx.y >= *n_tiles) return;
  extern __shared__ uint4 Xs[];                   // [RT][K / 8 + 1]: token rows (rows past the tile are zero)
  const int e = tiles[3 * blockIdx.y], row0 = tiles[3 * blockIdx.y + 1], rows = tiles[3 * blockIdx.y + 2];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int K8 = K / 8, XS = K8 + 1;              // the odd stride spreads the rows over the banks
  for (int idx = tid; idx < RT * K8; idx += 256) {
    const int r = idx / K8, c = idx - r * K8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) {
      const int src = perm != nullptr ? perm[row0 + r] / top : row0 + r;
      if (gated_a) {
        const uint4* row = reinterpret_cast<const uint4*>(A + (size_t)src * 2 * K);
        v = silu_gate8(row[c], row[K8 + c]);
      } else {
        v = reinterpret_cast<const uint4*>(A + (size_t)src * K)[c];
      }
    }
    Xs[r * XS + c] = v;
  }
  __syncthreads();
  const int n0 = blockIdx.x * 128 + warp * 16;    // this warp's 16 weight rows
  if (n0 >= N) return;
  const int g = lane >> 2, q = lane & 3;
  const __nv_bfloat16* We = W + (size_t)e * N * K;
  const uint4* w_lo = reinterpret_cast<const uint4*>(We + (size_t)min(n0 + g, N - 1) * K) + q;
  const uint4* w_hi = reinterpret_cast<const uint4*>(We + (size_t)min(n0 + g + 8, N - 1) * K) + q;
  const uint4* x_lo = Xs + g * XS + q;            // token row g, and g + 8 for the second half
  const uint4* x_hi = Xs + (RT == 16 ? g + 8 : g) * XS + q;
  const bool two = RT == 16 && rows > 8;
  float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
  const int steps = K / 32;
  int s = 0;
  for (; s + 3 < steps; s += 4) {
    uint4 a[4], b[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      a[u] = __ldg(w_lo + 4 * (s + u));
      b[u] = __ldg(w_hi + 4 * (s + u));
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const uint4 x = x_lo[4 * (s + u)];
      mma_bf16_16816(acc0, a[u].x, b[u].x, a[u].y, b[u].y, x.x, x.y);
      mma_bf16_16816(acc0, a[u].z, b[u].z, a[u].w, b[u].w, x.z, x.w);
      if (two) {
        const uint4 y = x_hi[4 * (s + u)];
        mma_bf16_16816(acc1, a[u].x, b[u].x, a[u].y, b[u].y, y.x, y.y);
        mma_bf16_16816(acc1, a[u].z, b[u].z, a[u].w, b[u].w, y.z, y.w);
      }
    }
  }
  for (; s < steps; ++s) {
    const uint4 a = __ldg(w_lo + 4 * s), b = __ldg(w_hi + 4 * s), x = x_lo[4 * s];
    mma_bf16_16816(acc0, a.x, b.x, a.y, b.y, x.x, x.y);
    mma_bf16_16816(acc0, a.z, b.z, a.w, b.w, x.z, x.w);
    if (two) {
      const uint4 y = x_hi[4 * s];
      mma_bf16_16816(acc1, a.x, b.x, a.y, b.y, y.x, y.y);
      mma_bf16_16816(acc1, a.z, b.z, a.w, b.w, y.z, y.w);
    }
  }
  // acc[0], acc[1]: weight row n0 + g, tokens 2 q and 2 q + 1;  acc[2], acc[3]: weight row n0 + g + 8
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const float* acc = half == 0 ? acc0 : acc1;
    if (half == 1 && !two) break;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int tok = 8 * half + 2 * q + (i & 1), n = n0 + g + 8 * (i >> 1);
      if (tok < rows && n < N) C[(size_t)(row0 + tok) * N + n] = from_f32<TO>(GELU ? gelu_erf(acc[i]) : acc[i]);
    }
  }
}

// sorted[r, :] = h[perm[r] / top, :]   (16-byte pieces when the rows allow it)
template <typename T>
__global__ void moe_gather_kernel(const T* __restrict__ h, const int* __restrict__ perm, int top, T* __restrict__ out,
                                  int d, int vec) {
  bspec::pdl_prologue(53);
  const size_t src = (size_t)(perm[blockIdx.x] / top) * d, dst = (size_t)blockIdx.x * d;
  if (vec) {
    const int n16 = d * (int)sizeof(T) / 16;
    const uint4* a = reinterpret_cast<const uint4*>(h + src);
    uint4* b = reinterpret_cast<uint4*>(out + dst);
    for (int i = threadIdx.x; i < n16; i += blockDim.x) b[i] = a[i];
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) out[dst + i] = h[src + i];
  }
}

template <typename TY, typename TO>
__global__ void moe_combine_kernel(const TY* __restrict__ y, const int* __restrict__ inv, const float* __restrict__ wts,
                                   int top, TO* __restrict__ out, int d) {
  bspec::pdl_prologue(54);
  const int t = blockIdx.x;
  for (int i = 2 * threadIdx.x; i < d; i += 2 * blockDim.x) {
    float a0 = 0.f, a1 = 0.f;
    const bool pair = i + 1 < d && (d % 2) == 0;
    for (int k = 0; k < top; ++k) {
      const float w = wts[(size_t)t * top + k];
      const TY* row = y + (size_t)inv[(size_t)t * top + k] * d + i;
      a0 += w * to_f32(row[0]);
      if (i + 1 < d) a1 += w * to_f32(row[1]);
    }
    out[(size_t)t * d + i] = from_f32<TO>(a0);
    if (i + 1 < d) out[(size_t)t * d + i + 1] = from_f32<TO>(a1);
    (void)pair;
  }
}

}  // namespace

BSPEC_API int bspec_moe_route(const void* h, int dtype, int n, int d, const void* wr, const void* corr, int corr_dtype,
                              int E, int G, int keep, int top, float scale, int* ids, float* wts,
                              const float* logits, int softmax_top, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (E <= 0 || E > MAX_EXPERTS || top <= 0 || top > E || G <= 0 || E % G || keep <= 0 || keep > G ||
      (long long)keep * (E / G) < top)
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)((d > 1024 ? d : 1024) + 2 * E + 8) * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  if (dtype == BSPEC_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BSPEC_LAUNCH((moe_route_kernel<float>), n, ROUTE_THREADS, smem, stream, (const float*)h, d, (const float*)wr, corr,
                 corr_dtype, E, G, keep, top, scale, ids, wts, logits, softmax_top);
  } else {
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_route_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    BSPEC_LAUNCH((moe_route_kernel<__nv_bfloat16>), n, ROUTE_THREADS, smem, stream, (const __nv_bfloat16*)h, d,
                 (const __nv_bfloat16*)wr, corr, corr_dtype, E, G, keep, top, scale, ids, wts, logits, softmax_top);
  }
  return BSPEC_LAUNCH_CHECK();
}

// counts [E] and rank [slots]: scratch of the many-rows path (may be null: the one-block kernel then runs).
BSPEC_API int bspec_moe_plan(const int* ids, int slots, int E, int BM, int* perm, int* inv, int* offsets, int* tiles,
                             int* n_tiles, int max_tiles, int* counts, int* rank, cudaStream_t stream) {
  if (slots <= 0) return 0;
  if (E <= 0 || E > MAX_EXPERTS || (BM != 8 && BM != 16 && BM != 64)) return (int)cudaErrorInvalidValue;
  if (slots <= 2048 || counts == nullptr || rank == nullptr) {
    BSPEC_LAUNCH((moe_plan_kernel), 1, 1024, 0, stream, ids, slots, E, BM, perm, inv, offsets, tiles, n_tiles, max_tiles);
    return BSPEC_LAUNCH_CHECK();
  }
  cudaError_t err = cudaMemsetAsync(counts, 0, (size_t)E * sizeof(int), stream);
  if (err != cudaSuccess) return (int)err;
  const int blocks = (slots + 255) / 256;
  BSPEC_LAUNCH((moe_rank_kernel), blocks, 256, 0, stream, ids, slots, counts, rank);
  BSPEC_LAUNCH((moe_offsets_kernel), 1, 256, 0, stream, (const int*)counts, E, BM, offsets, tiles, n_tiles, max_tiles);
  BSPEC_LAUNCH((moe_place_kernel), blocks, 256, 0, stream, ids, (const int*)rank, (const int*)offsets, slots, perm, inv);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_moe_grouped(const void* A, const int* perm, int top, const void* W, void* C, int dtype,
                                int out_dtype, int N, int K, const int* tiles, const int* n_tiles, int max_tiles,
                                int BM, int act, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  const int gelu = act == 1, gated_a = act == 2;       // act: 0 none, 1 GELU on the outputs, 2 a gated operand A
  dim3 grid((N + 63) / 64, max_tiles);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
#define LK(T, TO, B, G) BSPEC_LAUNCH((moe_grouped_kernel<T, TO, B, G>), grid, 256, 0, stream, (const T*)A, perm, top, \
                                     (const T*)W, (TO*)C, N, K, tiles, n_tiles, gated_a)
#define LB(T, TO) do { if (BM == 64) { if (gelu) LK(T, TO, 64, true); else LK(T, TO, 64, false); }                  \
                       else { if (gelu) LK(T, TO, 16, true); else LK(T, TO, 16, false); } } while (0)
  if (dtype == BSPEC_F32) LB(float, float);
  else if (out_dtype == BSPEC_F32) LB(__nv_bfloat16, float);
  else LB(__nv_bfloat16, __nv_bfloat16);
#undef LB
#undef LK
  return BSPEC_LAUNCH_CHECK();
}

// Tiles of at most 8 rows (a plan made with BM = 8), bfloat16 operands, K a multiple of 8.
BSPEC_API int bspec_moe_skinny(const void* A, const int* perm, int top, const void* W, void* C, int out_dtype, int N,
                               int K, const int* tiles, const int* n_tiles, int max_tiles, int act,
                               cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  const int gelu = act == 1, gated_a = act == 2;
  if (K % 8 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return (int)cudaErrorInvalidValue;
  dim3 grid((N + 63) / 64, max_tiles);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  const size_t smem = (size_t)8 * K * 2;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
#define LS(TO, G)                                                                                                   \
  do {                                                                                                              \
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_skinny_kernel<TO, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    BSPEC_LAUNCH((moe_skinny_kernel<TO, G>), grid, 256, smem, stream, (const __nv_bfloat16*)A, perm, top,           \
                 (const __nv_bfloat16*)W, (TO*)C, N, K, tiles, n_tiles, gated_a);                                   \
  } while (0)
  if (out_dtype == BSPEC_F32) { if (gelu) LS(float, true); else LS(float, false); }
  else { if (gelu) LS(__nv_bfloat16, true); else LS(__nv_bfloat16, false); }
#undef LS
  return BSPEC_LAUNCH_CHECK();
}

// Tiles of at most `rows_per_tile` rows (8 or 16: a plan made with that BM), bfloat16 operands, K a multiple of 32.
BSPEC_API int bspec_moe_skinny_mma(const void* A, const int* perm, int top, const void* W, void* C, int out_dtype,
                                   int N, int K, const int* tiles, const int* n_tiles, int max_tiles, int act,
                                   int rows_per_tile, cudaStream_t stream) {
  if (max_tiles <= 0 || N <= 0) return 0;
  const int gelu = act == 1, gated_a = act == 2;
  if (K % 32 != 0 || (reinterpret_cast<uintptr_t>(A) & 15) || (reinterpret_cast<uintptr_t>(W) & 15))
    return (int)cudaErrorInvalidValue;
  dim3 grid((N + 127) / 128, max_tiles);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  if (rows_per_tile != 8 && rows_per_tile != 16) return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)rows_per_tile * (K / 8 + 1) * 16;
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
#define LS(TO, G, RT)                                                                                               \
  do {                                                                                                              \
    if (smem > 48 * 1024) cudaFuncSetAttribute(moe_skinny_mma_kernel<TO, G, RT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    BSPEC_LAUNCH((moe_skinny_mma_kernel<TO, G, RT>), grid, 256, smem, stream, (const __nv_bfloat16*)A, perm, top,   \
                 (const __nv_bfloat16*)W, (TO*)C, N, K, tiles, n_tiles, gated_a);                                   \
  } while (0)
#define LR(TO, G) do { if (rows_per_tile == 16) LS(TO, G, 16); else LS(TO, G, 8); } while (0)
  if (out_dtype == BSPEC_F32) { if (gelu) LR(float, true); else LR(float, false); }
  else { if (gelu) LR(__nv_bfloat16, true); else LR(__nv_bfloat16, false); }
#undef LR
#undef LS
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_moe_gather(const void* h, int dtype, const int* perm, int top, void* out, int slots, int d,
                               cudaStream_t stream) {
  if (slots <= 0) return 0;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((moe_gather_kernel<float>), slots, 128, 0, stream, (const float*)h, perm, top, (float*)out, d,
                 (int)(d % 4 == 0 && !(reinterpret_cast<uintptr_t>(h) & 15) && !(reinterpret_cast<uintptr_t>(out) & 15)));
  else
    BSPEC_LAUNCH((moe_gather_kernel<__nv_bfloat16>), slots, 128, 0, stream, (const __nv_bfloat16*)h, perm, top,
                 (__nv_bfloat16*)out, d,
                 (int)(d % 8 == 0 && !(reinterpret_cast<uintptr_t>(h) & 15) && !(reinterpret_cast<uintptr_t>(out) & 15)));
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_moe_combine(const void* y, int y_dtype, const int* inv, const float* wts, int top, void* out,
                                int out_dtype, int n, int d, cudaStream_t stream) {
  if (n <= 0) return 0;
  const int threads = d >= 1024 ? 256 : 128;
#define LC(TY, TO) BSPEC_LAUNCH((moe_combine_kernel<TY, TO>), n, threads, 0, stream, (const TY*)y, inv, wts, top, (TO*)out, d)
  if (y_dtype == BSPEC_F32 && out_dtype == BSPEC_F32) LC(float, float);
  else if (y_dtype == BSPEC_F32) LC(float, __nv_bfloat16);
  else if (out_dtype == BSPEC_F32) LC(__nv_bfloat16, float);
  else LC(__nv_bfloat16, __nv_bfloat16);
#undef LC
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_moe)
