// Paged causal attention, generic path: any head_dim that is a multiple of 16 up
// to 256, any number of heads and groups, any page size, float32 or bfloat16
// storage, float32 arithmetic throughout.  One warp per (query token, query
// head); a block holds WARPS consecutive query tokens of one request and one
// head.  Keys are visited in chunks of 32 that start at multiples of 32 of the
// key index, so the order of every sum depends only on the query's own position,
// not on how the request was cut into steps or on what else is in the batch.
//
// Cache layer layout: [pages][k: [Hkv][page_size][hd] | v: [Hkv][page_size][vd]] (vd = hd unless values have a size
// of their own).
//
// Masks: causal; ``window`` > 0 keeps the last ``window`` keys; ``chunk`` > 0 keeps the keys of the query's own
// chunk, floor(key / chunk) == floor(query / chunk), chunks counted from position 0 of the request.  ``sink``: one
// float32 per query head: exp(sink) is added to the softmax denominator, nothing to the numerator.  ``softcap`` c > 0:
// a score s (after the scale) becomes c tanh(s / c).  ``v_is_k``: the values are the keys; a page then holds
// [Hkv][page_size][hd] only.  ``gate`` (float32 rows [Hq*vd] of stride gate_stride, or null): the output is multiplied
// element by element by sigmoid(gate); ``out_scale`` multiplies it too; output rows have stride out_stride.
#include "common.cuh"
#include <math.h>
using namespace bspec;

namespace {
constexpr int WARPS = 4;
constexpr int MAX_HD = 256;

template <typename T>
__global__ void __launch_bounds__(WARPS * 32)
attn_generic_kernel(const T* __restrict__ q, long long q_row_stride, T* __restrict__ out,
                    const T* __restrict__ cache, const int* __restrict__ qo_indptr,
                    const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                    const int* __restrict__ kv_indices, int Hq, int Hkv, int hd, int page_size, float scale,
                    int window, long long n_pages, int vd, int chunk, const float* __restrict__ sink,
                    float softcap, int v_is_k, const float* __restrict__ gate, long long gate_stride,
                    long long out_stride, float out_scale, int gate_per_head) {
  bspec::pdl_prologue(7);
  __shared__ float qs[WARPS][MAX_HD];
  const int e = blockIdx.y, h = blockIdx.z;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int q_begin = qo_indptr[e], q_len = qo_indptr[e + 1] - q_begin;
  const int qi = blockIdx.x * WARPS + warp;
  if (blockIdx.x * WARPS >= q_len) return;   // whole block beyond this request's tokens
  const bool active = qi < q_len;
  const int t = q_begin + (active ? qi : 0);
  const int kvh = h / (Hq / Hkv);
  if (active) {
    const T* qp = q + (size_t)t * q_row_stride + (size_t)h * hd;
    for (int d = lane; d < hd; d += 32) qs[warp][d] = to_f32(qp[d]);
  }
  __syncwarp();
  if (!active) return;
  const int pos = positions[t];
  const int hi = pos;                                   // last visible key (inclusive)
  int lo = window > 0 ? max(0, pos - window + 1) : 0;
  if (chunk > 0) lo = max(lo, (pos / chunk) * chunk);
  const int* table = kv_indices + kv_indptr[e];
  const size_t k_elems = (size_t)Hkv * page_size * hd;          // the keys of a page; its values follow them
  const size_t page_elems = k_elems + (v_is_k ? (size_t)0 : (size_t)Hkv * page_size * vd);
  const size_t head_off = (size_t)kvh * page_size * hd;
  constexpr int ND = MAX_HD / 32;
  float acc[ND];
#pragma unroll
  for (int i = 0; i < ND; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;
  for (int kb = (lo / 32) * 32; kb <= hi; kb += 32) {
    const int key = kb + lane;
    bool valid = key >= lo && key <= hi;
    long long koff = 0, voff = 0;
    float s = -INFINITY;
    if (valid && !bspec::in_range(table[key / page_size], n_pages, 107)) valid = false;
    if (valid) {
      const int page = table[key / page_size];
      koff = (long long)((size_t)page * page_elems + head_off + (size_t)(key % page_size) * hd);
      voff = v_is_k ? koff
                    : (long long)((size_t)page * page_elems + k_elems + ((size_t)kvh * page_size + (size_t)(key % page_size)) * vd);
      const T* kp = cache + koff;
      float dot = 0.f;
      for (int d = 0; d < hd; ++d) dot += qs[warp][d] * to_f32(kp[d]);
      s = dot * scale;
      if (softcap > 0.f) s = softcap * tanhf(s / softcap);
    }
    const float m_new = fmaxf(m, warp_max(s));        // finite: the chunk holds at least one valid key
    const float p = valid ? expf(s - m_new) : 0.f;
    const float corr = expf(m - m_new);               // m = -inf on the first chunk -> 0
    l = l * corr + warp_sum(p);
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
    const int nk = min(32, hi - kb + 1);
    for (int kk = 0; kk < nk; ++kk) {
      const float pk = __shfl_sync(0xffffffffu, p, kk);
      const long long off = __shfl_sync(0xffffffffu, voff, kk);
      if (pk != 0.f) {
        const T* vp = cache + off;
#pragma unroll
        for (int i = 0; i < ND; ++i) {
          const int d = lane + 32 * i;
          if (d < vd) acc[i] += pk * to_f32(vp[d]);
        }
      }
    }
    m = m_new;
  }
  if (sink != nullptr) {                                // one more term of the denominator only
    const float sk = sink[h];
    const float m_new = fmaxf(m, sk);
    const float corr = expf(m - m_new);
    l = l * corr + expf(sk - m_new);
#pragma unroll
    for (int i = 0; i < ND; ++i) acc[i] *= corr;
  }
  const float inv = 1.f / l;
  T* op = out + (size_t)t * out_stride + (size_t)h * vd;
  // one gate logit per output number, or (gate_per_head) one per head: row [Hq] instead of [Hq * vd]
  const float* gp = gate != nullptr ? gate + (size_t)t * gate_stride + (size_t)h * (gate_per_head ? 1 : vd) : nullptr;
#pragma unroll
  for (int i = 0; i < ND; ++i) {
    const int d = lane + 32 * i;
    if (d < vd) {
      float o = acc[i] * inv;
      if (gp != nullptr) o = o / (1.f + expf(-gp[gate_per_head ? 0 : d]));
      op[d] = from_f32<T>(o * out_scale);
    }
  }
}
}  // namespace

// q: rows of row stride q_row_stride (elements), heads packed [Hq][hd] at the row start.
// out: [n, Hq*vd].  max_q_len: the longest request portion in the step (sizes the grid).
static int launch_attention_generic(const void* q, long long q_row_stride, void* out, const void* cache, int dtype,
                                    const int* qo_indptr, const int* positions, const int* kv_indptr,
                                    const int* kv_indices, int n_entries, int max_q_len, int Hq, int Hkv, int hd,
                                    int page_size, float scale, int window, long long n_pages, int vd, int chunk,
                                    const float* sink, float softcap, int v_is_k, const float* gate,
                                    long long gate_stride, long long out_stride, float out_scale, int gate_per_head,
                                    cudaStream_t stream) {
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (v_is_k && vd != hd) return (int)cudaErrorInvalidValue;
  if (hd > MAX_HD || hd <= 0 || vd > MAX_HD || vd <= 0 || Hq % Hkv != 0) return (int)cudaErrorInvalidValue;
  dim3 grid((max_q_len + WARPS - 1) / WARPS, n_entries, Hq);
  if (grid.y > 65535 || grid.z > 65535) return (int)cudaErrorInvalidConfiguration;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((attn_generic_kernel<float>), grid, WARPS * 32, 0, stream, 
        (const float*)q, q_row_stride, (float*)out, (const float*)cache, qo_indptr, positions, kv_indptr, kv_indices,
        Hq, Hkv, hd, page_size, scale, window, n_pages, vd, chunk, sink, softcap, v_is_k, gate, gate_stride, out_stride,
        out_scale, gate_per_head);
  else
    BSPEC_LAUNCH((attn_generic_kernel<__nv_bfloat16>), grid, WARPS * 32, 0, stream, 
        (const __nv_bfloat16*)q, q_row_stride, (__nv_bfloat16*)out, (const __nv_bfloat16*)cache, qo_indptr, positions,
        kv_indptr, kv_indices, Hq, Hkv, hd, page_size, scale, window, n_pages, vd, chunk, sink, softcap, v_is_k, gate,
        gate_stride, out_stride, out_scale, gate_per_head);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_attention_generic(const void* q, long long q_row_stride, void* out, const void* cache, int dtype,
                                      const int* qo_indptr, const int* positions, const int* kv_indptr,
                                      const int* kv_indices, int n_entries, int max_q_len, int Hq, int Hkv, int hd,
                                      int page_size, float scale, int window, long long n_pages,
                                      cudaStream_t stream) {
  return launch_attention_generic(q, q_row_stride, out, cache, dtype, qo_indptr, positions, kv_indptr, kv_indices,
                                  n_entries, max_q_len, Hq, Hkv, hd, page_size, scale, window, n_pages, hd, 0, nullptr,
                                  0.f, 0, nullptr, 0, (long long)Hq * hd, 1.f, 0, stream);
}

// The same with values of their own size ``vd``, a chunk mask (0: none), a sink per query head (null: none), a soft
// cap on the scores (0: none), values that are the keys, a sigmoid gate on the output (per number, or per head), an output scale and stride.
BSPEC_API int bspec_attention_masked(const void* q, long long q_row_stride, void* out, const void* cache, int dtype,
                                     const int* qo_indptr, const int* positions, const int* kv_indptr,
                                     const int* kv_indices, int n_entries, int max_q_len, int Hq, int Hkv, int hd,
                                     int vd, int page_size, float scale, int window, int chunk, const float* sink,
                                     long long n_pages, float softcap, int v_is_k, const float* gate,
                                     long long gate_stride, long long out_stride, float out_scale,
                                     int gate_per_head, cudaStream_t stream) {
  return launch_attention_generic(q, q_row_stride, out, cache, dtype, qo_indptr, positions, kv_indptr, kv_indices,
                                  n_entries, max_q_len, Hq, Hkv, hd, page_size, scale, window, n_pages, vd, chunk, sink,
                                  softcap, v_is_k, gate, gate_stride, out_stride, out_scale, gate_per_head, stream);
}

// ---------------------------------------------------------------- q/k/v preparation
// From the float32 rows of the fused projection [q: Hq*hd | k: Hkv*hd | v: Hkv*vd]: add the bias (if any), rotate the
// first ``rot`` numbers of every q and k head (pair (i, i + rot/2), or (2i, 2i+1) with ``interleaved``; cosine and
// sine times ``magnitude``), divide every q and k head by its root mean square (``norm_eps`` > 0; none otherwise; times ``q_norm_w`` / ``k_norm_w``,
// a weight per number of a head, when given; before the rotation with ``norm_first``),
// all in float32; then write q to ``q_out`` [n, Hq*hd] and k and v into the cache page of the token's position.
// Rows of the input have stride ``ld`` (they may hold more columns).  vd == 0: there are no values (they are the
// keys); a page then holds keys only.  One warp per head.
namespace {
constexpr int PREP_WARPS = 8;

__device__ __forceinline__ void prep_sincos(int pos, const float* __restrict__ inv_freq, int half, int j, float* s,
                                            float* c) {
  const double f = (double)inv_freq[j] + (double)inv_freq[half + j];
  double a = (double)pos * f;
  a -= 6.283185307179586476925286766559 * rint(a * 0.15915494309189533576888376337251);
  sincosf((float)a, s, c);
}

__device__ __forceinline__ void prep_store4(float* p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
__device__ __forceinline__ void prep_store4(__nv_bfloat16* p, float a, float b, float c, float d) {
  const __nv_bfloat162 lo = __floats2bfloat162_rn(a, b), hi = __floats2bfloat162_rn(c, d);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&lo);
  v.y = *reinterpret_cast<const uint32_t*>(&hi);
  *reinterpret_cast<uint2*>(p) = v;
}

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32)
qkv_prepare_kernel(const float* __restrict__ qkv, long long ld, int Hq, int Hkv, int hd, int vd, const void* __restrict__ bias,
                   int bias_dtype, const float* __restrict__ inv_freq, int rot, int interleaved, float magnitude,
                   float norm_eps, const int* __restrict__ positions, const int* __restrict__ tok_entry,
                   const int* __restrict__ kv_indptr, const int* __restrict__ kv_indices, T* __restrict__ q_out,
                   T* __restrict__ cache, int page_size, int write_kv, long long n_pages,
                   const void* __restrict__ q_norm_w, const void* __restrict__ k_norm_w, int norm_w_dtype,
                   int norm_first) {
  bspec::pdl_prologue(19);
  __shared__ __align__(16) float xs[PREP_WARPS][MAX_HD];
  __shared__ float cs[MAX_HD];                                // [rot/2] cosines, then [rot/2] sines, of this token
  const int t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = blockIdx.y * PREP_WARPS + warp;            // q heads, then k heads, then v heads
  const int pos = positions[t];
  const bool has = slot < Hq + Hkv + (vd > 0 ? Hkv : 0);
  const bool is_v = slot >= Hq + Hkv;
  const int width = is_v ? vd : hd;
  const int col0 = is_v ? (Hq + Hkv) * hd + (slot - Hq - Hkv) * vd : slot * hd;
  const float* src = qkv + (size_t)t * ld + (has ? col0 : 0);
  float* x = xs[warp];
  const bool vec = ((hd | vd | (int)ld) & 3) == 0;           // every head starts on a 16-byte boundary: four numbers per lane
  // the head's numbers are asked for first, so that their way from memory runs under the angles' arithmetic
  float4 v0 = make_float4(0.f, 0.f, 0.f, 0.f), v1 = v0;
  if (has && vec) {
    if (4 * lane < width) v0 = *reinterpret_cast<const float4*>(src + 4 * lane);
    if (4 * lane + 128 < width) v1 = *reinterpret_cast<const float4*>(src + 4 * lane + 128);
  }
  if (blockIdx.y * PREP_WARPS < Hq + Hkv) {                   // the block holds a q or k head: the angles once for all
    const int half = rot / 2;
    for (int j = threadIdx.x; j < half; j += blockDim.x) {
      float sn, c;
      prep_sincos(pos, inv_freq, half, j, &sn, &c);
      cs[j] = c * magnitude;
      cs[half + j] = sn * magnitude;
    }
  }
  __syncthreads();
  if (!has) return;
  if (vec) {
#pragma unroll
    for (int part = 0; part < 2; ++part) {
      const int d = 4 * lane + 128 * part;
      if (d < width) {
        float4 v = part ? v1 : v0;
        if (bias != nullptr) {
          v.x += load_as_f32(bias, bias_dtype, (size_t)col0 + d);
          v.y += load_as_f32(bias, bias_dtype, (size_t)col0 + d + 1);
          v.z += load_as_f32(bias, bias_dtype, (size_t)col0 + d + 2);
          v.w += load_as_f32(bias, bias_dtype, (size_t)col0 + d + 3);
        }
        *reinterpret_cast<float4*>(x + d) = v;
      }
    }
  } else {
    for (int d = lane; d < width; d += 32)
      x[d] = src[d] + (bias != nullptr ? load_as_f32(bias, bias_dtype, (size_t)col0 + d) : 0.f);
  }
  __syncwarp();
  if (!is_v) {
    // every q and k head divided by its root mean square, times a weight per number when one is given (the same
    // for all heads); before the rotation (norm_first) or after it
    const void* nw = slot < Hq ? q_norm_w : k_norm_w;
    auto normalise = [&]() {
      float ss = 0.f;
      for (int d = lane; d < hd; d += 32) ss += x[d] * x[d];
      ss = warp_sum(ss);
      const float r = 1.f / sqrtf(ss / (float)hd + norm_eps);
      for (int d = lane; d < hd; d += 32) x[d] = x[d] * r * (nw != nullptr ? load_as_f32(nw, norm_w_dtype, d) : 1.f);
      __syncwarp();
    };
    if (norm_eps > 0.f && norm_first) normalise();
    const int half = rot / 2;
    for (int j = lane; j < half; j += 32) {
      const float c = cs[j], sn = cs[half + j];
      const int a = interleaved ? 2 * j : j, b = interleaved ? 2 * j + 1 : j + half;
      const float u = x[a], v = x[b];
      x[a] = u * c - v * sn;
      x[b] = v * c + u * sn;
    }
    __syncwarp();
    if (norm_eps > 0.f && !norm_first) normalise();
  }
  const float r = 1.f;
  T* dst = nullptr;
  if (slot < Hq) {
    dst = q_out + ((size_t)t * Hq + slot) * hd;
  } else if (write_kv) {
    const int e = tok_entry[t];
    if (bspec::in_range(pos / page_size, kv_indptr[e + 1] - kv_indptr[e], 113)) {
      const int page = kv_indices[kv_indptr[e] + pos / page_size];
      if (bspec::in_range(page, n_pages, 114)) {
        const size_t k_elems = (size_t)Hkv * page_size * hd;
        const size_t page_elems = k_elems + (size_t)Hkv * page_size * vd;
        const int row = pos % page_size;
        dst = cache + (size_t)page * page_elems +
              (is_v ? k_elems + ((size_t)(slot - Hq - Hkv) * page_size + row) * vd
                    : ((size_t)(slot - Hq) * page_size + row) * hd);
      }
    }
  }
  if (dst != nullptr) {
    if (vec) {
      for (int d = 4 * lane; d < width; d += 128) {
        const float4 v = *reinterpret_cast<const float4*>(x + d);
        prep_store4(dst + d, v.x * r, v.y * r, v.z * r, v.w * r);
      }
    } else {
      for (int d = lane; d < width; d += 32) dst[d] = from_f32<T>(x[d] * r);
    }
  }
}
}  // namespace

BSPEC_API int bspec_qkv_prepare(const float* qkv, long long ld, int n, int Hq, int Hkv, int hd, int vd, const void* bias,
                                int bias_dtype, const float* inv_freq, int rot, int interleaved, float magnitude,
                                float norm_eps, const int* positions, const int* tok_entry, const int* kv_indptr,
                                const int* kv_indices, void* q_out, void* cache, int dtype, int page_size, int write_kv,
                                long long n_pages, const void* q_norm_w, const void* k_norm_w, int norm_w_dtype,
                                int norm_first, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (hd <= 0 || hd > MAX_HD || vd < 0 || vd > MAX_HD || ld < (long long)(Hq + Hkv) * hd + (long long)Hkv * vd || rot < 0 || rot > hd || rot % 2 != 0 ||
      (rot > 0 && inv_freq == nullptr))
    return (int)cudaErrorInvalidValue;
  const dim3 grid(n, (Hq + 2 * Hkv + PREP_WARPS - 1) / PREP_WARPS);
  if (grid.y > 65535) return (int)cudaErrorInvalidConfiguration;
  if (dtype == BSPEC_F32)
    BSPEC_LAUNCH((qkv_prepare_kernel<float>), grid, PREP_WARPS * 32, 0, stream, qkv, ld, Hq, Hkv, hd, vd, bias, bias_dtype,
                 inv_freq, rot, interleaved, magnitude, norm_eps, positions, tok_entry, kv_indptr, kv_indices,
                 (float*)q_out, (float*)cache, page_size, write_kv, n_pages, q_norm_w, k_norm_w, norm_w_dtype, norm_first);
  else
    BSPEC_LAUNCH((qkv_prepare_kernel<__nv_bfloat16>), grid, PREP_WARPS * 32, 0, stream, qkv, ld, Hq, Hkv, hd, vd, bias,
                 bias_dtype, inv_freq, rot, interleaved, magnitude, norm_eps, positions, tok_entry, kv_indptr,
                 kv_indices, (__nv_bfloat16*)q_out, (__nv_bfloat16*)cache, page_size, write_kv, n_pages, q_norm_w, k_norm_w,
                 norm_w_dtype, norm_first);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_attention_generic)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_attention_generic)
