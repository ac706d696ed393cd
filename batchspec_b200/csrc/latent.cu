// Latent attention: every token stores ONE cache entry [c | kr], c the normalised key/value latent (R numbers)
// and kr a rotated key part shared by all heads (P numbers).  Attention runs in the latent space: a head's query
// is [ql | qr], ql its unrotated query already multiplied by the head's key up-projection (R numbers) and qr its
// rotated part (P numbers); score(i, j) = scale * ([ql | qr] . entry_j), causal softmax, and the head's output
// is sum_j p_j c_j (R numbers), which the caller multiplies by the head's value up-projection.  All heads read the
// same entries.  ``window`` > 0: a query sees its own entry and the window - 1 before it; ``sink``: a logit per head
// that only enlarges the softmax's denominator (nothing is attended through it; ``scale`` does not touch it).
//
// Kernels here:
//   latent_prepare      per token: RMS norm of the query latent, RMS norm of the key/value latent, rotation of kr
//                       (adjacent pairs, magnitude on cosine and sine), entry written to its cache page
//   latent_attn_generic any sizes, float32 or bfloat16 storage, float32 arithmetic, one warp per (token, head)
//   gate_heads          out[t, h*V + j] = v[h, t, j] * sigmoid(gate[t, h])
//
// Cache layout of a layer: [pages][page_size][R + P].
#include "common.cuh"
#include <math.h>
#include <stdint.h>
using namespace bspec;

namespace {

__device__ __forceinline__ void sincos_at(int pos, const float* __restrict__ inv_freq, int half, int j, float* s,
                                          float* c) {
  // the frequency as two floats whose sum is its float64 value; the product and its reduction in float64
  const double f = (double)inv_freq[j] + (double)inv_freq[half + j];
  double a = (double)pos * f;
  a -= 6.283185307179586476925286766559 * rint(a * 0.15915494309189533576888376337251);
  sincosf((float)a, s, c);
}

// down: float32 [n, ld]; columns [q_off, q_off + Rq) the query latent, [kv_off, kv_off + R) the key/value latent,
// [kv_off + R, kv_off + R + P) the key part to rotate.
template <typename T>
__global__ void __launch_bounds__(128)
latent_prepare_kernel(const float* __restrict__ down, int ld, int q_off, int Rq, int kv_off, int R, int P,
                      const void* __restrict__ wq, const void* __restrict__ wkv, int w_dtype, float eps,
                      const float* __restrict__ inv_freq, float magnitude, const int* __restrict__ positions,
                      const int* __restrict__ tok_entry, const int* __restrict__ kv_indptr,
                      const int* __restrict__ kv_indices, T* __restrict__ cq, T* __restrict__ cache, int page_size,
                      int write_kv, long long n_pages) {
  bspec::pdl_prologue(40);
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const float* row = down + (size_t)t * ld;
  if (Rq > 0) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < Rq; i += blockDim.x) ss += row[q_off + i] * row[q_off + i];
    const float r = rsqrtf(block_sum(ss, scratch) / (float)Rq + eps);
    for (int i = threadIdx.x; i < Rq; i += blockDim.x)
      cq[(size_t)t * Rq + i] = from_f32<T>(row[q_off + i] * r * load_as_f32(wq, w_dtype, i));
  }
  if (!write_kv) return;
  const int pos = positions[t];
  const int e = tok_entry[t];
  T* dst = nullptr;
  if (bspec::in_range(pos / page_size, kv_indptr[e + 1] - kv_indptr[e], 109)) {
    const int page = kv_indices[kv_indptr[e] + pos / page_size];
    if (bspec::in_range(page, n_pages, 110)) dst = cache + ((size_t)page * page_size + pos % page_size) * (R + P);
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < R; i += blockDim.x) ss += row[kv_off + i] * row[kv_off + i];
  const float r = rsqrtf(block_sum(ss, scratch) / (float)R + eps);
  if (dst == nullptr) return;
  for (int i = threadIdx.x; i < R; i += blockDim.x)
    dst[i] = from_f32<T>(row[kv_off + i] * r * load_as_f32(wkv, w_dtype, i));
  const int half = P / 2;
  for (int j = threadIdx.x; j < half; j += blockDim.x) {
    float s, c;
    sincos_at(pos, inv_freq, half, j, &s, &c);
    s *= magnitude;
    c *= magnitude;
    const float u = row[kv_off + R + 2 * j], v = row[kv_off + R + 2 * j + 1];
    dst[R + 2 * j] = from_f32<T>(u * c - v * s);
    dst[R + 2 * j + 1] = from_f32<T>(v * c + u * s);
  }
}

constexpr int GW = 4;   // warps (query tokens) per block of the generic kernel

// One warp per (query token, head).  Keys in chunks of 32 that start at multiples of 32 of the key index, so the
// order of every sum depends on the query's position alone.  ``split``: the CTA's z index takes the chunks
// z, z + n_splits, ... and leaves (m, l, unnormalised sum) in the scratch when n_splits > 1.
template <typename T, int ND>
__global__ void __launch_bounds__(GW * 32)
latent_attn_generic_kernel(const T* __restrict__ ql, long long ql_row, long long ql_head, const T* __restrict__ qr,
                           long long qr_row, long long qr_head, T* __restrict__ out, long long o_row, long long o_head,
                           const T* __restrict__ cache, const int* __restrict__ qo_indptr,
                           const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                           const int* __restrict__ kv_indices, int H, int R, int P, int page_size, float scale,
                           long long n_pages, int window, const float* __restrict__ sink) {
  bspec::pdl_prologue(41);
  extern __shared__ float qs_all[];
  const int D = R + P;
  const int e = blockIdx.y, h = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float* qs = qs_all + (size_t)warp * D;
  const int q_begin = qo_indptr[e], q_len = qo_indptr[e + 1] - q_begin;
  const int qi = blockIdx.x * GW + warp;
  if (qi >= q_len) return;
  const int t = q_begin + qi;
  for (int d = lane; d < R; d += 32) qs[d] = to_f32(ql[(size_t)t * ql_row + (size_t)h * ql_head + d]);
  for (int d = lane; d < P; d += 32) qs[R + d] = to_f32(qr[(size_t)t * qr_row + (size_t)h * qr_head + d]);
  __syncwarp();
  const int hi = positions[t];
  const int* table = kv_indices + kv_indptr[e];
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  // a window keeps the keys hi - window + 1 .. hi; pages before it may have been given back and are never touched
  const int lo = window > 0 ? max(0, hi - window + 1) : 0;
  for (int kb = lo & ~31; kb <= hi; kb += 32) {
    const int key = kb + lane;
    bool valid = key <= hi && key >= lo;
    long long koff = 0;
    float s = -INFINITY;
    if (valid && !bspec::in_range(table[key / page_size], n_pages, 111)) valid = false;
    if (valid) {
      koff = ((long long)table[key / page_size] * page_size + key % page_size) * D;
      const T* kp = cache + koff;
      float dot = 0.f;
      for (int d = 0; d < D; ++d) dot += qs[d] * to_f32(kp[d]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
    const int nk = min(32, hi - kb + 1);
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const long long off = __shfl_sync(0xffffffffu, koff, kk);
      if (pk != 0.f) {
        const T* vp = cache + off;
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const int d = lane + 32 * i;
          if (d < R) acc[i] += pk * to_f32(vp[d]);
        }
      }
    }
    m = m_new;
  }
  if (sink != nullptr) {                          // a logit per head that joins the denominator only
    const float sk = sink[h];
    const float m_new = fmaxf(m, sk);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
  }
  const float inv = 1.f / l;
  T* op = out + (size_t)t * o_row + (size_t)h * o_head;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < R) op[d] = from_f32<T>(acc[i] * inv);
  }
}

// v [H, n, V] (head stride, row stride given), gate float32 rows of stride ld (column h of a row is head h's
// logit) -> out [n, H * V]
template <typename T>
__global__ void gate_heads_kernel(const T* __restrict__ v, long long v_head, long long v_row,
                                  const float* __restrict__ gate, int ld, T* __restrict__ out, int H, int V) {
  bspec::pdl_prologue(42);
  const int t = blockIdx.x;
  for (int i = threadIdx.x; i < H * V; i += blockDim.x) {
    const int h = i / V, j = i - h * V;
    const float g = 1.f / (1.f + expf(-gate[(size_t)t * ld + h]));
    out[(size_t)t * H * V + i] = from_f32<T>(to_f32(v[(size_t)h * v_head + (size_t)t * v_row + j]) * g);
  }
}

// The same for bfloat16 with eight numbers (16 bytes) per thread: V, both strides of v and every address multiples
// of 8 numbers; a thread's eight numbers lie in one head, so it forms that head's sigmoid once.  Grid-stride over
// all (token, piece) pairs.
__global__ void gate_heads_bf16x8_kernel(const __nv_bfloat16* __restrict__ v, long long v_head, long long v_row,
                                         const float* __restrict__ gate, int ld, __nv_bfloat16* __restrict__ out,
                                         int H, int V, long long total) {
  bspec::pdl_prologue(42);
  const int per_row = H * V / 8, per_head = V / 8;
  for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
       idx += (long long)gridDim.x * blockDim.x) {
    const long long t = idx / per_row;
    const int piece = (int)(idx - t * per_row);
    const int h = piece / per_head, j = (piece - h * per_head) * 8;
    const float g = 1.f / (1.f + expf(-gate[t * ld + h]));
    uint4 x = *reinterpret_cast<const uint4*>(v + (size_t)h * v_head + (size_t)t * v_row + j);
    __nv_bfloat162* p = reinterpret_cast<__nv_bfloat162*>(&x);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const float2 f = __bfloat1622float2(p[k]);
      p[k] = __floats2bfloat162_rn(f.x * g, f.y * g);
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * H * V + (size_t)piece * 8) = x;
  }
}

}  // namespace

BSPEC_API int bspec_latent_prepare(const float* down, int n, int ld, int q_off, int Rq, int kv_off, int R, int P,
                                   const void* wq, const void* wkv, int w_dtype, float eps, const float* inv_freq,
                                   float magnitude, const int* positions, const int* tok_entry, const int* kv_indptr,
                                   const int* kv_indices, void* cq, void* cache, int dtype, int page_size,
                                   int write_kv, long long n_pages, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (P % 2) return (int)cudaErrorInvalidValue;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((latent_prepare_kernel<float>), n, 128, 0, stream, down, ld, q_off, Rq, kv_off, R, P, wq, wkv, w_dtype,
                 eps, inv_freq, magnitude, positions, tok_entry, kv_indptr, kv_indices, (float*)cq, (float*)cache,
                 page_size, write_kv, n_pages);
  else
    BSPEC_LAUNCH((latent_prepare_kernel<__nv_bfloat16>), n, 128, 0, stream, down, ld, q_off, Rq, kv_off, R, P, wq, wkv,
                 w_dtype, eps, inv_freq, magnitude, positions, tok_entry, kv_indptr, kv_indices, (__nv_bfloat16*)cq,
                 (__nv_bfloat16*)cache, page_size, write_kv, n_pages);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_latent_attention_generic(const void* ql, long long ql_row, long long ql_head, const void* qr,
                                             long long qr_row, long long qr_head, void* out, long long o_row,
                                             long long o_head, const void* cache, int dtype, const int* qo_indptr,
                                             const int* positions, const int* kv_indptr, const int* kv_indices,
                                             int n_entries, int max_q_len, int H, int R, int P, int page_size,
                                             float scale, long long n_pages, int window, const float* sink,
                                             cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (R <= 0 || R > 1024 || P < 0) return (int)cudaErrorInvalidValue;
  dim3 grid((max_q_len + GW - 1) / GW, n_entries, H);
  if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidConfiguration;
  const size_t smem = (size_t)GW * (R + P) * sizeof(float);
  if (smem > 48 * 1024) return (int)cudaErrorInvalidValue;
#define LG(T, ND) BSPEC_LAUNCH((latent_attn_generic_kernel<T, ND>), grid, GW * 32, smem, stream, (const T*)ql, ql_row, \
                               ql_head, (const T*)qr, qr_row, qr_head, (T*)out, o_row, o_head, (const T*)cache,       \
                               qo_indptr, positions, kv_indptr, kv_indices, H, R, P, page_size, scale, n_pages,   \
                               window, sink)
  const int nd = (R + 31) / 32;
  if (dtype == BSPEC_F32) {
    if (nd <= 4) LG(float, 4); else if (nd <= 8) LG(float, 8); else if (nd <= 16) LG(float, 16); else LG(float, 32);
  } else {
    if (nd <= 4) LG(__nv_bfloat16, 4); else if (nd <= 8) LG(__nv_bfloat16, 8);
    else if (nd <= 16) LG(__nv_bfloat16, 16); else LG(__nv_bfloat16, 32);
  }
#undef LG
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_gate_heads(const void* v, long long v_head, long long v_row, const float* gate, int ld, void* out,
                               int dtype, int n, int H, int V, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (dtype != BSPEC_F32 && V % 8 == 0 && v_head % 8 == 0 && v_row % 8 == 0 &&
      !((reinterpret_cast<uintptr_t>(v) | reinterpret_cast<uintptr_t>(out)) & 15)) {
    const long long total = (long long)n * (H * V / 8);
    const long long want = (total + 255) / 256, cap = (long long)bspec::sm_count() * 16;
    BSPEC_LAUNCH((gate_heads_bf16x8_kernel), (int)(want > cap ? cap : want), 256, 0, stream, (const __nv_bfloat16*)v,
                 v_head, v_row, gate, ld, (__nv_bfloat16*)out, H, V, total);
    return BSPEC_LAUNCH_CHECK();
  }
  const int threads = H * V >= 1024 ? 256 : 128;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((gate_heads_kernel<float>), n, threads, 0, stream, (const float*)v, v_head, v_row, gate, ld, (float*)out, H, V);
  else
    BSPEC_LAUNCH((gate_heads_kernel<__nv_bfloat16>), n, threads, 0, stream, (const __nv_bfloat16*)v, v_head, v_row, gate,
                 ld, (__nv_bfloat16*)out, H, V);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_latent)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_latent)
