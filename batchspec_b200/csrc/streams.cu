// A residual stream kept as several copies ("streams") per token that learned coefficients mix:
// x [n, S, d] float32.  A sublayer reads u = sum_s read[s] x_s, and its result y joins all streams at once,
//   x_t <- sum_s mix[s, t] x_s + write[t] * (vec * y),   vec a factor per column (or none),
// with ``mixw`` = [mix: S x S, indexed (from, to) | write: S] as one float32 table.
//
// Kernels:
//   stream_expand   x[t, s, :] = src[t, :] for every s
//   stream_norm     the pending sublayer result joins the streams (if one is given), then the next sublayer's
//                   input is read and RMS-normalised: out = u / sqrt(mean(u^2) + eps) * w, one rounding
//                   (the counterpart of add + RMSNorm for one stream; without ``read`` it only updates; with
//                   ``expand`` it fills the streams from one row per token first, as a step's first norm does)
//   stream_gather   out[i, :] = sum_t x'_t of row rows[i], x' the streams after the pending result has joined
//                   (nothing is written back): the rows that go to the final norm and the head
// All arithmetic is float32; sums over the streams run in the order of the stream index.
#include "common.cuh"
using namespace bspec;

namespace {

constexpr int MAX_STREAMS = 16;

__global__ void stream_expand_kernel(const float* __restrict__ src, float* __restrict__ x, int S, int d) {
  bspec::pdl_prologue(70);
  const size_t t = blockIdx.x;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float v = src[t * d + i];
    for (int s = 0; s < S; ++s) x[(t * S + s) * d + i] = v;
  }
}

template <typename T> __device__ __forceinline__ void load4(const T* p, float (&f)[4]);
template <> __device__ __forceinline__ void load4<float>(const float* p, float (&f)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
}
template <> __device__ __forceinline__ void load4<__nv_bfloat16>(const __nv_bfloat16* p, float (&f)[4]) {
  const uint2 v = *reinterpret_cast<const uint2*>(p);
  const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&v.x), b = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
  f[0] = __low2float(a); f[1] = __high2float(a); f[2] = __low2float(b); f[3] = __high2float(b);
}
template <typename T> __device__ __forceinline__ void store4(T* p, const float (&f)[4]);
template <> __device__ __forceinline__ void store4<float>(float* p, const float (&f)[4]) {
  *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* p, const float (&f)[4]) {
  const __nv_bfloat162 a = __floats2bfloat162_rn(f[0], f[1]), b = __floats2bfloat162_rn(f[2], f[3]);
  uint2 v;
  v.x = *reinterpret_cast<const uint32_t*>(&a);
  v.y = *reinterpret_cast<const uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = v;
}

// The new streams of one column: old[] in, fresh[] out.  SC > 0: the number of streams is known at compile time.
template <int SC>
__device__ __forceinline__ void join_column(const float* old, float y, const float* mixw, int S, float* fresh) {
#pragma unroll
  for (int t = 0; t < (SC > 0 ? SC : S); ++t) {
    float acc = 0.f;
#pragma unroll
    for (int s = 0; s < (SC > 0 ? SC : S); ++s) acc += mixw[s * S + t] * old[s];
    fresh[t] = acc + mixw[S * S + t] * y;
  }
}

// One block per token.  u is kept in shared memory between the sum of squares and the scaling.  SC: the number of
// streams when it is 1, 2, 3, 4 or 8 (loops unrolled, a column's streams in registers), 0: any number up to 16.
// VEC: four columns per thread and pass (d a multiple of 4).
template <typename TD, typename TO, int SC, bool VEC>
__global__ void stream_norm_kernel(float* __restrict__ x, const TD* __restrict__ pending,
                                   const float* __restrict__ vec, const float* __restrict__ mixw,
                                   const float* __restrict__ read, const void* __restrict__ weight, int w_dtype,
                                   TO* __restrict__ out, int S_rt, int d, float eps,
                                   const float* __restrict__ expand) {
  bspec::pdl_prologue(71);
  constexpr int SMAX = SC > 0 ? SC : MAX_STREAMS;
  constexpr int W = VEC ? 4 : 1;
  const int S = SC > 0 ? SC : S_rt;
  extern __shared__ float u_row[];                // [d]
  __shared__ float coef[MAX_STREAMS * MAX_STREAMS + 2 * MAX_STREAMS];
  __shared__ float scratch[32];
  const size_t t = blockIdx.x;
  if (pending != nullptr)
    for (int i = threadIdx.x; i < S * S + S; i += blockDim.x) coef[i] = mixw[i];
  if (read != nullptr)
    for (int i = threadIdx.x; i < S; i += blockDim.x) coef[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS + i] = read[i];
  __syncthreads();
  const float* rd = coef + MAX_STREAMS * MAX_STREAMS + MAX_STREAMS;
  float* xt = x + t * S * d;
  float ss = 0.f;
  for (int i = W * threadIdx.x; i < d; i += W * blockDim.x) {
    float cur[W][SMAX];
    // ``expand``: the streams do not exist yet; every one starts as this row [n, d] (the embedding) and is written
    float4 first = make_float4(0.f, 0.f, 0.f, 0.f);
    if (expand != nullptr) {
      if (VEC) first = *reinterpret_cast<const float4*>(expand + t * d + i);
      else first.x = expand[t * d + i];
    }
#pragma unroll
    for (int s = 0; s < SMAX; ++s) {
      if (s < S) {
        if (VEC) {
          const float4 v = expand != nullptr ? first : *reinterpret_cast<const float4*>(xt + (size_t)s * d + i);
          cur[0][s] = v.x; cur[W > 1 ? 1 : 0][s] = v.y; cur[W > 1 ? 2 : 0][s] = v.z; cur[W > 1 ? 3 : 0][s] = v.w;
        } else {
          cur[0][s] = expand != nullptr ? first.x : xt[(size_t)s * d + i];
        }
      }
    }
    if (pending != nullptr) {
      float yv[W], vv[W];
      if (VEC) {
        load4<TD>(pending + t * d + i, *reinterpret_cast<float(*)[4]>(yv));
        if (vec != nullptr) load4<float>(vec + i, *reinterpret_cast<float(*)[4]>(vv));
      } else {
        yv[0] = to_f32(pending[t * d + i]);
        if (vec != nullptr) vv[0] = vec[i];
      }
#pragma unroll
      for (int c = 0; c < W; ++c) {
        const float y = yv[c] * (vec != nullptr ? vv[c] : 1.f);
        float fresh[SMAX];
        join_column<SC>(cur[c], y, coef, S, fresh);
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < S) cur[c][s] = fresh[s];
      }
    }
    if (pending != nullptr || expand != nullptr) {
#pragma unroll
      for (int s = 0; s < SMAX; ++s) {
        if (s < S) {
          if (VEC)
            *reinterpret_cast<float4*>(xt + (size_t)s * d + i) =
                make_float4(cur[0][s], cur[W > 1 ? 1 : 0][s], cur[W > 1 ? 2 : 0][s], cur[W > 1 ? 3 : 0][s]);
          else
            xt[(size_t)s * d + i] = cur[0][s];
        }
      }
    }
    if (read != nullptr) {
#pragma unroll
      for (int c = 0; c < W; ++c) {
        float u = 0.f;
#pragma unroll
        for (int s = 0; s < SMAX; ++s)
          if (s < S) u += rd[s] * cur[c][s];
        u_row[i + c] = u;
        ss += u * u;
      }
    }
  }
  if (read == nullptr) return;
  const float r = 1.f / sqrtf(block_sum(ss, scratch) / (float)d + eps);
  if (VEC) {                                      // a thread scales the columns it formed itself
    for (int i = W * threadIdx.x; i < d; i += W * blockDim.x) {
      float y[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) y[c] = u_row[i + c] * r * load_as_f32(weight, w_dtype, i + c);
      store4<TO>(out + t * d + i, y);
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x)
      out[t * d + i] = from_f32<TO>(u_row[i] * r * load_as_f32(weight, w_dtype, i));
  }
}

template <typename TD>
__global__ void stream_gather_kernel(const float* __restrict__ x, const TD* __restrict__ pending,
                                     const float* __restrict__ vec, const float* __restrict__ mixw,
                                     const int* __restrict__ rows, float* __restrict__ out, int S, int d, int n_src) {
  bspec::pdl_prologue(72);
  __shared__ float coef[MAX_STREAMS * MAX_STREAMS + MAX_STREAMS];
  if (!bspec::in_range(rows[blockIdx.x], n_src, 102)) return;
  if (pending != nullptr)
    for (int i = threadIdx.x; i < S * S + S; i += blockDim.x) coef[i] = mixw[i];
  __syncthreads();
  const size_t t = rows[blockIdx.x];
  const float* xt = x + t * S * d;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    float cur[MAX_STREAMS];
    for (int s = 0; s < S; ++s) cur[s] = xt[(size_t)s * d + i];
    if (pending != nullptr) {
      const float y = to_f32(pending[t * d + i]) * (vec != nullptr ? vec[i] : 1.f);
      float fresh[MAX_STREAMS];
      join_column<0>(cur, y, coef, S, fresh);
      for (int s = 0; s < S; ++s) cur[s] = fresh[s];
    }
    float sum = 0.f;
    for (int s = 0; s < S; ++s) sum += cur[s];
    out[(size_t)blockIdx.x * d + i] = sum;
  }
}

}  // namespace

BSPEC_API int bspec_stream_expand(const float* src, float* x, int n, int S, int d, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (S <= 0 || S > MAX_STREAMS) return (int)cudaErrorInvalidValue;
  BSPEC_LAUNCH((stream_expand_kernel), n, d >= 1024 ? 256 : 128, 0, stream, src, x, S, d);
  return BSPEC_LAUNCH_CHECK();
}

// pending null: nothing joins.  read null: the streams are only updated (weight and out unused).  expand (float32
// [n, d]) given: x is not read; every stream starts as that row and is written (the first norm of a step).
BSPEC_API int bspec_stream_norm(float* x, const void* pending, int pending_dtype, const float* vec, const float* mixw,
                                const float* read, const void* weight, int w_dtype, void* out, int out_dtype, int n,
                                int S, int d, float eps, const float* expand, cudaStream_t stream) {
  if (n <= 0) return 0;
  if (S <= 0 || S > MAX_STREAMS || (pending != nullptr && mixw == nullptr) || (read != nullptr && (!weight || !out)))
    return (int)cudaErrorInvalidValue;
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
  const bool v4 = d % 4 == 0;
  const int cols = v4 ? d / 4 : d;
  // at most 256 threads: with a column's streams in registers, several smaller blocks share an SM and cover each
  // other's barrier between the two passes
  const int threads = cols >= 256 ? 256 : 128;
#define LN3(TD, TO, SC, V)                                                                                          \
  do {                                                                                                              \
    if (smem > 48 * 1024)                                                                                           \
      cudaFuncSetAttribute(stream_norm_kernel<TD, TO, SC, V>, cudaFuncAttributeMaxDynamicSharedMemorySize,          \
                           (int)smem);                                                                              \
    BSPEC_LAUNCH((stream_norm_kernel<TD, TO, SC, V>), n, threads, smem, stream, x, (const TD*)pending, vec, mixw,   \
                 read, weight, w_dtype, (TO*)out, S, d, eps, expand); \
  } while (0)
#define LN2(TD, TO, SC) do { if (v4) LN3(TD, TO, SC, true); else LN3(TD, TO, SC, false); } while (0)
#define LN(TD, TO)                                                                                                  \
  do {                                                                                                              \
    switch (S) {                                                                                                    \
      case 1: LN2(TD, TO, 1); break;                                                                                \
      case 2: LN2(TD, TO, 2); break;                                                                                \
      case 3: LN2(TD, TO, 3); break;                                                                                \
      case 4: LN2(TD, TO, 4); break;                                                                                \
      case 8: LN2(TD, TO, 8); break;                                                                                \
      default: LN3(TD, TO, 0, false); break;                                                                        \
    }                                                                                                               \
  } while (0)
  if (pending_dtype == BSPEC_F32 && out_dtype == BSPEC_F32) LN(float, float);
  else if (pending_dtype == BSPEC_BF16 && out_dtype == BSPEC_BF16) LN(__nv_bfloat16, __nv_bfloat16);
  else if (pending_dtype == BSPEC_F32 && out_dtype == BSPEC_BF16) LN(float, __nv_bfloat16);
  else LN(__nv_bfloat16, float);
#undef LN3
#undef LN2
#undef LN
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_API int bspec_stream_gather(const float* x, const void* pending, int pending_dtype, const float* vec,
                                  const float* mixw, const int* rows, float* out, int n_out, int S, int d, int n_src,
                                  cudaStream_t stream) {
  if (n_out <= 0) return 0;
  if (S <= 0 || S > MAX_STREAMS || (pending != nullptr && mixw == nullptr)) return (int)cudaErrorInvalidValue;
  if (pending_dtype == BSPEC_F32)
    BSPEC_LAUNCH((stream_gather_kernel<float>), n_out, 256, 0, stream, x, (const float*)pending, vec, mixw, rows, out,
                 S, d, n_src);
  else
    BSPEC_LAUNCH((stream_gather_kernel<__nv_bfloat16>), n_out, 256, 0, stream, x, (const __nv_bfloat16*)pending, vec,
                 mixw, rows, out, S, d, n_src);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_streams)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_streams)
