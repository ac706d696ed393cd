// Latent attention in bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulation), prompt portions and
// decoded tokens alike.  All heads of a request read the same cache entries [c | kr] (R + P numbers), so the rows
// of a tile are (token, head) pairs: row = token * H + head, 16 * RG rows per CTA (RG row groups of 16: 64 rows for
// prompt portions, 16 or 32 for decoded tokens of models with up to 16 or 32 heads), and one pass over the request's
// entries serves every head.  A CTA is RG x CH warps: warp (rg, ch) owns 16 rows, 32 / CH keys of every score tile
// and R / CH columns of the output.  Per tile of 32 entries:
//
//   S = Q K^T over all R + P numbers (the entry is the key), scaled, causal mask, to shared memory in float32;
//   online softmax in float32, four threads per row; the weights are left as TWO bfloat16 numbers, the rounded
//   weight and the rounding's remainder, so that the product with the values carries them to 2^-17;
//   O += P_hi V + P_lo V with V the first R numbers of the same tile.
// The warps of a row group meet at a barrier of their own between these phases (the row groups drift apart, so
// one's softmax runs under another's products); the whole CTA meets once per tile, when the next tile has landed.
//
// Entries arrive by cp.async; the block-table lookup of a tile is made one tile before its copies.  A CTA holds
// two tiles of entries (the next one arrives under the current one's products: the 64-row tiles) or one (32-row
// tiles of prompt portions and the 16- and 32-row tiles of decoded tokens: two to four CTAs then share an SM and
// cover each other's loads, which measured faster).  With n_splits > 1 (decode: few rows, many entries) CTA z takes
// the z-th share of the key tiles and leaves (max, sum, unnormalised output) for the join kernel, which adds the
// shares in their order.  How the tiles are cut into shares follows from the request's length, read on the device.
#include "common.cuh"
#include <math.h>
#include <stdlib.h>
using namespace bspec;

namespace {

constexpr int BN = 32;

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
// ldmatrix on 32-bit shared-space addresses (formed once per kernel, advanced by byte offsets)
__device__ __forceinline__ uint32_t smem_addr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];\n"
               : "=r"(r[0]), "=r"(r[1]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], uint32_t a) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__host__ __device__ inline size_t smem_bytes(int D, int BM, int stages = 2) {
  const int DP = D + 8;
  return (size_t)(BM + stages * BN) * DP * 2 + (size_t)BM * (BN + 8) * 4 + 2 * (size_t)BM * (BN + 8) * 2 + 3 * BM * 4;
}

// RG row groups x CH column groups of warps; NT: n-tiles (of 8 columns) of the output one warp may own,
// R / (8 CH) <= NT.
// ST: tiles of entries in shared memory: 2 (the next one arrives under the current one's products) or 1 (two CTAs
// share an SM instead and cover each other's loads).
template <int RG, int CH, int NT, int ST = 2>
__global__ void __launch_bounds__(32 * RG * CH)
latent_attn_mma_kernel(const __nv_bfloat16* __restrict__ ql, long long ql_row, long long ql_head,
                       const __nv_bfloat16* __restrict__ qr, long long qr_row, long long qr_head,
                       __nv_bfloat16* __restrict__ out, long long o_row, long long o_head,
                       const __nv_bfloat16* __restrict__ cache, const int* __restrict__ qo_indptr,
                       const int* __restrict__ positions, const int* __restrict__ kv_indptr,
                       const int* __restrict__ kv_indices, int H, int R, int P, int page_size, float scale,
                       int n_splits, float* __restrict__ o_part, float* __restrict__ ml_part, long long n_pages,
                       const float* __restrict__ inv_freq, float magnitude, int window,
                       const float* __restrict__ sink) {
  constexpr int BM = 16 * RG;
  constexpr int KW = BN / CH;                     // keys of a score tile per warp: 16 or 8
  constexpr int TPR = 2 * CH, KPT = BN / TPR;     // softmax: threads per row, keys per thread
  bspec::pdl_prologue(43);
  extern __shared__ __align__(16) unsigned char smem_raw[];
  const int D = R + P, DP = D + 8;
  constexpr int PP = BN + 8, SP = BN + 8;
  __nv_bfloat16* Qs = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* Ks = Qs + (size_t)BM * DP;
  float* Ss = reinterpret_cast<float*>(Ks + (size_t)ST * BN * DP);
  __nv_bfloat16* Ph = reinterpret_cast<__nv_bfloat16*>(Ss + (size_t)BM * SP);
  __nv_bfloat16* Pl = Ph + (size_t)BM * PP;
  float* row_m = reinterpret_cast<float*>(Pl + (size_t)BM * PP);
  float* row_l = row_m + BM;
  float* row_c = row_l + BM;

  const int e = blockIdx.y, split = blockIdx.z;
  const int q_begin = qo_indptr[e], q_len = qo_indptr[e + 1] - q_begin;
  const long long rows_total = (long long)q_len * H;
  const long long row0 = (long long)blockIdx.x * BM;
  if (row0 >= rows_total) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = warp % RG, ch = warp / RG;
  const int pos0 = positions[q_begin];
  const int last_tok = (int)min((long long)q_len - 1, (row0 + BM - 1) / H);
  const int max_pos = pos0 + last_tok;
  // with a window the CTA's first row sees nothing before min_key: the tiles start there, and entries before it
  // (their pages may have been given back) are never looked up
  const int min_key = window > 0 ? max(0, pos0 + (int)(row0 / H) - window + 1) : 0;
  const int tile0 = min_key / BN;
  const int n_tiles = max_pos / BN + 1;
  const int per = (n_tiles - tile0 + n_splits - 1) / n_splits;
  const int t_begin = tile0 + split * per, t_end = min(n_tiles, t_begin + per);
  const int* table = kv_indices + kv_indptr[e];

  // ---- queries: row r holds [ql | qr] of (token, head) = divmod(row0 + r, H); rows past the portion are zero.
  // With a frequency table the rotated part arrives unrotated and is rotated here (adjacent pairs, the angle in
  // float64 from the two-float frequencies, cosine and sine times the magnitude), then rounded as a separate
  // rotation kernel would have left it.
  for (int r = warp; r < BM; r += RG * CH) {      // a warp per row: its token and head are found once
    const long long row = row0 + r;
    const bool live = row < rows_total;
    const int tq = live ? (int)((unsigned)row / (unsigned)H) : 0;          // rows_total fits 32 bits (checked at launch)
    const int h = live ? (int)((unsigned)row - (unsigned)tq * (unsigned)H) : 0;
    const long long t = q_begin + tq;
    const __nv_bfloat16* src_l = ql + t * ql_row + h * ql_head;
    const __nv_bfloat16* src_r = qr + t * qr_row + h * qr_head;
    __nv_bfloat16* dst = Qs + (size_t)r * DP;
    for (int d = 2 * lane; d < R; d += 64) {
      const float u = live ? __bfloat162float(src_l[d]) : 0.f, v = live ? __bfloat162float(src_l[d + 1]) : 0.f;
      *reinterpret_cast<__nv_bfloat162*>(dst + d) = __floats2bfloat162_rn(u, v);
    }
    const int pos = live ? positions[t] : 0;
    for (int d = 2 * lane; d < P; d += 64) {
      float u = live ? __bfloat162float(src_r[d]) : 0.f, v = live ? __bfloat162float(src_r[d + 1]) : 0.f;
      if (inv_freq != nullptr && live) {
        const int j = d / 2, half = P / 2;
        const double f = (double)inv_freq[j] + (double)inv_freq[half + j];
        double ang = (double)pos * f;
        ang -= 6.283185307179586476925286766559 * rint(ang * 0.15915494309189533576888376337251);
        float sn, cs;
        sincosf((float)ang, &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float ru = u * cs - v * sn, rv = v * cs + u * sn;
        u = ru;
        v = rv;
      }
      *reinterpret_cast<__nv_bfloat162*>(dst + R + d) = __floats2bfloat162_rn(u, v);
    }
  }
  if (tid < BM) {
    row_m[tid] = -INFINITY;
    row_l[tid] = 0.f;
  }

  // A tile's entries are dealt to the warps, one entry at a time; the lanes copy its 16-byte pieces.  The page
  // of an entry is looked up once per entry (a shift when the page size is a power of two).
  const int chunks = D / 8;                       // 16-byte pieces of an entry
  const int ps_shift = (page_size & (page_size - 1)) == 0 ? 31 - __clz(page_size) : -1;
  // Lane j of a warp looks up the page of the warp's j-th entry of a tile; the lookup for a tile is made one
  // tile ahead of its copies, so that its latency passes under the products in between.
  constexpr int NW = RG * CH, KPW = BN / NW;      // warps; entries of a tile per warp
  auto lookup = [&](int tile) -> long long {      // element offset of the lane's entry in the cache, -1: none
    long long off = -1;
    if (lane < KPW && tile < t_end) {
      const int key = tile * BN + warp + lane * NW;
      if (key <= max_pos && key >= min_key) {
        const int slot = ps_shift >= 0 ? key >> ps_shift : key / page_size;
        const int page = table[slot];
        if (bspec::in_range(page, n_pages, 112)) off = ((long long)page * page_size + (key - slot * page_size)) * D;
      }
    }
    return off;
  };
  auto load_tile = [&](int buf, long long mine) {
    __nv_bfloat16* dst = Ks + (size_t)buf * BN * DP;
#pragma unroll
    for (int j = 0; j < KPW; ++j) {
      const long long off = __shfl_sync(0xffffffffu, mine, j);
      const bool valid = off >= 0;
      const __nv_bfloat16* src = cache + (valid ? off : 0);
      __nv_bfloat16* d = dst + (size_t)(warp + j * NW) * DP;
      for (int part = lane; part < chunks; part += 32) cp_async16(d + part * 8, src + (valid ? part * 8 : 0), valid);
    }
  };
  auto group_barrier = [&]() {
    if (RG == 1) __syncthreads();
    else asm volatile("bar.sync %0, %1;" ::"r"(1 + rg), "r"(32 * CH) : "memory");
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  const int ntw = R / (8 * CH);                   // n-tiles this warp owns
  const int col0 = ch * (R / CH);                 // its first output column
  const int mat = lane >> 3, r8 = lane & 7;
  const int qrow = lane >> 2, qcol = 2 * (lane & 3);
  // this thread's softmax row: the row group's 32 CH threads, TPR per row
  const int tg = ch * 32 + lane;
  const int srow = 16 * rg + tg / TPR, spart = tg % TPR;
  // this lane's ldmatrix addresses (shared space, bytes): its row of the query fragments, of a key tile's score
  // fragments, of the weight fragments, and of the value fragments (transposed loads)
  const uint32_t qa_s = smem_addr(Qs + (size_t)(16 * rg + 8 * (mat & 1) + r8) * DP + 8 * (mat >> 1));
  const uint32_t kb_s = KW == 16 ? smem_addr(Ks + (size_t)(KW * ch + 8 * (mat >> 1) + r8) * DP + 8 * (mat & 1))
                                 : smem_addr(Ks + (size_t)(KW * ch + r8) * DP + 8 * (mat & 1));
  const uint32_t ph_s = smem_addr(Ph + (size_t)(16 * rg + 8 * (mat & 1) + r8) * PP + 8 * (mat >> 1));
  const uint32_t pl_s = smem_addr(Pl + (size_t)(16 * rg + 8 * (mat & 1) + r8) * PP + 8 * (mat >> 1));
  const uint32_t vt_s = smem_addr(Ks + (size_t)(8 * (mat & 1) + r8) * DP + col0 + 8 * (mat >> 1));
  // the last key each of this thread's two score rows may see (-1: the row is past the portion)
  int row_pos[2], row_lo[2];
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const long long row = row0 + 16 * rg + qrow + 8 * half;
    row_pos[half] = row < rows_total ? pos0 + (int)(row / H) : -1;
    row_lo[half] = window > 0 ? row_pos[half] - window + 1 : 0;         // the first key the row sees
  }

  long long ahead = lookup(t_begin);
  if (t_begin < t_end) load_tile(0, ahead);
  cp_async_commit();
  ahead = lookup(t_begin + 1);
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buf = ST == 2 ? (tile - t_begin) & 1 : 0;
    cp_async_wait<0>();
    __syncthreads();                              // the tile is here, and everybody is done with the tile before
    if (ST == 2) {
      if (tile + 1 < t_end) load_tile(buf ^ 1, ahead);
      cp_async_commit();
      ahead = lookup(tile + 2);
    }
    // ---- S: this warp's 16 rows x KW keys, two accumulator sets over alternating k steps
    {
      constexpr int NS = KW / 8;
      float s[4][NS][4];
#pragma unroll
      for (int x = 0; x < 4; ++x)
#pragma unroll
        for (int y = 0; y < NS; ++y) s[x][y][0] = s[x][y][1] = s[x][y][2] = s[x][y][3] = 0.f;
      const uint32_t kb = kb_s + (uint32_t)buf * (uint32_t)(BN * DP * 2);
      const int nks = D / 16;
      // The asm statements keep their order, so the loop is pipelined by hand: the fragments of k step i + 1 are
      // fetched before the products of step i are issued (two sets of fragment registers, four accumulator chains).
      uint32_t fa[2][4], fb[2][4];
      auto fetch = [&](int slot, uint32_t off) {                 // off: bytes along the row, 32 per k step
        ldsm_x4(fa[slot], qa_s + off);
        if (KW == 16) {
          ldsm_x4(fb[slot], kb + off);
        } else {
          uint32_t t[2];
          ldsm_x2(t, kb + off);
          fb[slot][0] = t[0];
          fb[slot][1] = t[1];
        }
      };
      auto mul = [&](float (&acc)[NS][4], int slot) {
        mma_bf16(acc[0], fa[slot], fb[slot][0], fb[slot][1]);
        if (KW == 16) mma_bf16(acc[NS - 1], fa[slot], fb[slot][2], fb[slot][3]);
      };
      fetch(0, 0u);
      int ks = 0;
      for (; ks + 4 <= nks; ks += 4) {
        fetch(1, 32u * (ks + 1));
        mul(s[0], 0);
        fetch(0, 32u * (ks + 2));
        mul(s[1], 1);
        fetch(1, 32u * (ks + 3));
        mul(s[2], 0);
        if (ks + 4 < nks) fetch(0, 32u * (ks + 4));
        mul(s[3], 1);
      }
      for (; ks < nks; ++ks) {
        mul(s[0], 0);
        if (ks + 1 < nks) fetch(0, 32u * (ks + 1));
      }
#pragma unroll
      for (int y = 0; y < NS; ++y)
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          s[0][y][x] += s[1][y][x];
          s[2][y][x] += s[3][y][x];
        }
#pragma unroll
      for (int nt = 0; nt < NS; ++nt)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int r = 16 * rg + qrow + 8 * half;
          const int c = KW * ch + 8 * nt + qcol;
          const int key = tile * BN + c;
          float2 v;
          v.x = (key <= row_pos[half] && key >= row_lo[half])
                    ? (s[0][nt][2 * half] + s[2][nt][2 * half]) * scale : -INFINITY;
          v.y = (key + 1 <= row_pos[half] && key + 1 >= row_lo[half])
                    ? (s[0][nt][2 * half + 1] + s[2][nt][2 * half + 1]) * scale : -INFINITY;
          *reinterpret_cast<float2*>(Ss + r * SP + c) = v;
        }
    }
    group_barrier();
    // ---- softmax: TPR threads per row, KPT keys each
    {
      float v[KPT];
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < KPT; j += 4) {
        const float4 x = *reinterpret_cast<const float4*>(Ss + srow * SP + KPT * spart + j);
        v[j] = x.x; v[j + 1] = x.y; v[j + 2] = x.z; v[j + 3] = x.w;
      }
#pragma unroll
      for (int j = 0; j < KPT; ++j) mx = fmaxf(mx, v[j]);
#pragma unroll
      for (int x = 1; x < TPR; x <<= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, x));
      const float m_old = row_m[srow], l_old = row_l[srow];
      const float m_new = fmaxf(m_old, mx);
      float sum = 0.f;
      __align__(16) __nv_bfloat16 hi[KPT], lo[KPT];
#pragma unroll
      for (int j = 0; j < KPT; ++j) {
        const float p = m_new == -INFINITY ? 0.f : __expf(v[j] - m_new);
        sum += p;
        hi[j] = __float2bfloat16_rn(p);
        lo[j] = __float2bfloat16_rn(p - __bfloat162float(hi[j]));
      }
      if (KPT == 8) {
        *reinterpret_cast<uint4*>(Ph + srow * PP + KPT * spart) = *reinterpret_cast<const uint4*>(hi);
        *reinterpret_cast<uint4*>(Pl + srow * PP + KPT * spart) = *reinterpret_cast<const uint4*>(lo);
      } else {
        *reinterpret_cast<uint2*>(Ph + srow * PP + KPT * spart) = *reinterpret_cast<const uint2*>(hi);
        *reinterpret_cast<uint2*>(Pl + srow * PP + KPT * spart) = *reinterpret_cast<const uint2*>(lo);
      }
#pragma unroll
      for (int x = 1; x < TPR; x <<= 1) sum += __shfl_xor_sync(0xffffffffu, sum, x);
      if (spart == 0) {
        const float corr = m_new == -INFINITY ? 1.f : __expf(m_old - m_new);
        row_m[srow] = m_new;
        row_l[srow] = l_old * corr + sum;
        row_c[srow] = corr;
      }
    }
    group_barrier();
    // ---- O = O * corr + P V over this warp's columns
    {
      const float c_lo = row_c[16 * rg + qrow], c_hi = row_c[16 * rg + qrow + 8];
      if (!__all_sync(0xffffffffu, c_lo == 1.f && c_hi == 1.f)) {      // some row's maximum moved
#pragma unroll
        for (int i = 0; i < NT; ++i) {
          o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
        }
      }
      const uint32_t vt = vt_s + (uint32_t)buf * (uint32_t)(BN * DP * 2);
#pragma unroll
      for (int kk = 0; kk < BN / 16; ++kk) {
        uint32_t ah[4], al[4];
        ldsm_x4(ah, ph_s + 32 * kk);
        ldsm_x4(al, pl_s + 32 * kk);
        const uint32_t vk = vt + (uint32_t)kk * (uint32_t)(16 * DP * 2);
        uint32_t vb[2][4];                         // the value fragments, fetched one pair of tiles ahead
        ldsm_x4_trans(vb[0], vk);
#pragma unroll
        for (int nd = 0; nd < NT; nd += 2) {
          if (nd < ntw) {
            const int cur = (nd >> 1) & 1;
            if (nd + 2 < ntw) ldsm_x4_trans(vb[cur ^ 1], vk + 16 * (nd + 2));
            mma_bf16(o[nd], ah, vb[cur][0], vb[cur][1]);
            if (nd + 1 < ntw) mma_bf16(o[nd + 1], ah, vb[cur][2], vb[cur][3]);
            mma_bf16(o[nd], al, vb[cur][0], vb[cur][1]);
            if (nd + 1 < ntw) mma_bf16(o[nd + 1], al, vb[cur][2], vb[cur][3]);
          }
        }
      }
    }
    if (ST == 1) {                                // the one buffer is free once every warp has left the tile
      __syncthreads();
      if (tile + 1 < t_end) load_tile(0, ahead);
      cp_async_commit();
      ahead = lookup(tile + 2);
    }
  }
  cp_async_wait<0>();
  __syncthreads();          // row_m / row_l of the init (no tiles) or of the last tile, for every warp
  // The sink: a logit per head whose exponential joins the denominator.  The first share takes it, as one more
  // (valueless) key: its maximum, sum and output are rescaled the way a tile rescales them.
  if (sink != nullptr && split == 0) {
    if (tid < BM) {
      const long long row = row0 + tid;
      float corr = 1.f;
      if (row < rows_total) {
        const float sk = sink[(int)(row % H)];
        const float m_old = row_m[tid], m_new = fmaxf(m_old, sk);
        corr = m_old == -INFINITY ? 0.f : __expf(m_old - m_new);
        row_m[tid] = m_new;
        row_l[tid] = row_l[tid] * corr + __expf(sk - m_new);
      }
      row_c[tid] = corr;
    }
    __syncthreads();
    const float c_lo = row_c[16 * rg + qrow], c_hi = row_c[16 * rg + qrow + 8];
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      o[i][0] *= c_lo; o[i][1] *= c_lo; o[i][2] *= c_hi; o[i][3] *= c_hi;
    }
  }

  // ---- results
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = 16 * rg + qrow + 8 * half;
    const long long row = row0 + r;
    if (row >= rows_total) continue;
    const long long t = q_begin + row / H;
    const int h = (int)(row % H);
    if (n_splits == 1) {
      const float inv = 1.f / row_l[r];
      __nv_bfloat16* op = out + t * o_row + h * o_head;
#pragma unroll
      for (int nd = 0; nd < NT; ++nd)
        if (nd < ntw) {
          const int c = col0 + 8 * nd + qcol;
          *reinterpret_cast<__nv_bfloat162*>(op + c) =
              __floats2bfloat162_rn(o[nd][2 * half] * inv, o[nd][2 * half + 1] * inv);
        }
    } else {
      const size_t slot = ((size_t)t * H + h) * n_splits + split;
      float* op = o_part + slot * R;
#pragma unroll
      for (int nd = 0; nd < NT; ++nd)
        if (nd < ntw) {
          const int c = col0 + 8 * nd + qcol;
          *reinterpret_cast<float2*>(op + c) = make_float2(o[nd][2 * half], o[nd][2 * half + 1]);
        }
      if (ch == 0 && (lane & 3) == 0) {
        ml_part[2 * slot] = row_m[r];
        ml_part[2 * slot + 1] = row_l[r];
      }
    }
  }
}

// out[row, :] = sum_s w_s O_s / sum_s w_s l_s with w_s = exp(m_s - max m), s ascending.  One block per (token, head):
// the shares' weights are formed once (in parallel, into shared memory), then every thread adds its columns.
__global__ void latent_attn_join_kernel(const float* __restrict__ o_part, const float* __restrict__ ml_part,
                                        __nv_bfloat16* __restrict__ out, long long o_row, long long o_head, int H,
                                        int R, int n_splits) {
  bspec::pdl_prologue(44);
  __shared__ float w[64];
  __shared__ float inv_l;
  const size_t row = blockIdx.x;
  const long long t = row / H;
  const int h = (int)(row % H);
  if (threadIdx.x < 32) {
    const int lane = threadIdx.x;
    float m0 = lane < n_splits ? ml_part[2 * (row * n_splits + lane)] : -INFINITY;
    float m1 = lane + 32 < n_splits ? ml_part[2 * (row * n_splits + lane + 32)] : -INFINITY;
    const float M = warp_max(fmaxf(m0, m1));
    const float w0 = m0 == -INFINITY ? 0.f : expf(m0 - M), w1 = m1 == -INFINITY ? 0.f : expf(m1 - M);
    w[lane] = w0;
    w[lane + 32] = w1;
    __syncwarp();
    if (lane == 0) {                 // the sum in the order of the shares
      float L = 0.f;
      for (int s = 0; s < n_splits; ++s)
        if (w[s] != 0.f) L += w[s] * ml_part[2 * (row * n_splits + s) + 1];
      inv_l = 1.f / L;
    }
  }
  __syncthreads();
  const float inv = inv_l;
  for (int c = threadIdx.x; c < R; c += blockDim.x) {
    float acc = 0.f;
#pragma unroll 4
    for (int s = 0; s < n_splits; ++s) {
      const float x = o_part[(row * n_splits + s) * R + c];
      if (w[s] != 0.f) acc += w[s] * x;
    }
    out[t * o_row + h * o_head + c] = __float2bfloat16_rn(acc * inv);
  }
}

}  // namespace

// 1 if the tensor-core kernel takes these sizes (ranks and rotated part multiples of 16, latent at most 512,
// the tile fits shared memory), else 0.
BSPEC_API int bspec_latent_attention_mma_supported(int R, int P) {
  return (R > 0 && R % 16 == 0 && P >= 16 && P % 16 == 0 && R <= 512 && smem_bytes(R + P, 64) <= 220 * 1024) ? 1 : 0;
}

// How prompt portions are tiled: 2 (default) = 32 rows, 8 warps, one tile of entries, two CTAs per SM, when those
// fit (else as 0); 0 = 64 rows, 16 warps, two tiles of entries in flight; 1 = 64 rows, 8 warps.  Measured on a
// 4,096-token prompt with 16 / 32 heads, latent 512 + 64: 127 / 134, 118 / 126 and 110 / 116 TFLOP/s.  The
// environment variable is a tuning switch.
static int prompt_mode() {
  static const int mode = [] {
    const char* e = getenv("BSPEC_LATENT_PROMPT");
    return e != nullptr ? atoi(e) : 2;
  }();
  return mode;
}
// Decoded tokens (16- and 32-row tiles): 1 (default) = one tile of entries per CTA, so that four CTAs share an SM;
// 2 = two tiles in flight per CTA, two CTAs per SM.
static int decode_stages() {
  static const int st = [] {
    const char* e = getenv("BSPEC_LATENT_DECODE_STAGES");
    return e != nullptr && atoi(e) == 2 ? 2 : 1;
  }();
  return st;
}
BSPEC_API int bspec_latent_attention_mma_smem(int rows, int R, int P, int prompt) {
  return (int)smem_bytes(R + P, rows, (rows == 64 || (rows < 64 && !prompt && decode_stages() == 2)) ? 2 : 1);
}
static bool two_small_ctas(int R, int P) {
  return prompt_mode() == 2 && R % 32 == 0 && smem_bytes(R + P, 32, 1) <= 112 * 1024;
}

// Rows per CTA for a step whose longest portion has max_q_len tokens: 16 or 32 when every request's (token, head)
// rows fit (decoded tokens of models with few heads; needs a latent that is a multiple of 32), else 64.
BSPEC_API int bspec_latent_attention_mma_rows(int max_q_len, int H, int R, int P) {
  const long long rows = (long long)max_q_len * H;
  if (R % 32 == 0 && rows <= 16) return 16;
  if (R % 32 == 0 && rows <= 32) return 32;
  return two_small_ctas(R, P) ? 32 : 64;
}

BSPEC_API int bspec_latent_attention_mma(const void* ql, long long ql_row, long long ql_head, const void* qr,
                                         long long qr_row, long long qr_head, void* out, long long o_row,
                                         long long o_head, const void* cache, const int* qo_indptr,
                                         const int* positions, const int* kv_indptr, const int* kv_indices,
                                         int n_entries, int n_tokens, int max_q_len, int H, int R, int P,
                                         int page_size, float scale, int n_splits, float* o_part, float* ml_part,
                                         long long n_pages, const float* inv_freq, float magnitude, int window,
                                         const float* sink, cudaStream_t stream) {
  const bool wide = prompt_mode() != 1;
  if (n_entries <= 0 || max_q_len <= 0) return 0;
  if (!bspec_latent_attention_mma_supported(R, P) || n_splits < 1 || (n_splits > 1 && (!o_part || !ml_part)))
    return (int)cudaErrorInvalidValue;
  const int BM = bspec_latent_attention_mma_rows(max_q_len, H, R, P);
  const bool small_pair = BM == 32 && (long long)max_q_len * H > 32;     // prompt portions on 32-row tiles, one buffer
  const long long row_tiles = ((long long)max_q_len * H + BM - 1) / BM;
  if ((long long)max_q_len * H > 2147483647ll || n_entries > 65535 || n_splits > 64) return (int)cudaErrorInvalidConfiguration;
  dim3 grid((unsigned)row_tiles, n_entries, n_splits);
  const bool one_stage = small_pair || (BM < 64 && decode_stages() == 1);
  const size_t smem = smem_bytes(R + P, BM, one_stage ? 1 : 2);
#define LM(RG, CH, N)                                                                                                \
  do {                                                                                                               \
    cudaFuncSetAttribute(latent_attn_mma_kernel<RG, CH, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    BSPEC_LAUNCH((latent_attn_mma_kernel<RG, CH, N>), grid, 32 * RG * CH, smem, stream, (const __nv_bfloat16*)ql,    \
                 ql_row, ql_head, (const __nv_bfloat16*)qr, qr_row, qr_head, (__nv_bfloat16*)out, o_row, o_head,     \
                 (const __nv_bfloat16*)cache, qo_indptr, positions, kv_indptr, kv_indices, H, R, P, page_size,       \
                 scale, n_splits, o_part, ml_part, n_pages, inv_freq, magnitude, window, sink); \
  } while (0)
#define LM1(RG, CH, N)                                                                                               \
  do {                                                                                                               \
    cudaFuncSetAttribute(latent_attn_mma_kernel<RG, CH, N, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    BSPEC_LAUNCH((latent_attn_mma_kernel<RG, CH, N, 1>), grid, 32 * RG * CH, smem, stream, (const __nv_bfloat16*)ql, \
                 ql_row, ql_head, (const __nv_bfloat16*)qr, qr_row, qr_head, (__nv_bfloat16*)out, o_row, o_head,     \
                 (const __nv_bfloat16*)cache, qo_indptr, positions, kv_indptr, kv_indices, H, R, P, page_size,       \
                 scale, n_splits, o_part, ml_part, n_pages, inv_freq, magnitude, window, sink); \
  } while (0)
  if (small_pair) {
    const int ntw = R / 32;
    if (ntw <= 4) LM1(2, 4, 4); else if (ntw <= 8) LM1(2, 4, 8); else LM1(2, 4, 16);
  } else if (BM == 64 && R % 32 == 0 && wide) {
    // sixteen warps: twice the warps to hide the latencies of the same tile (a warp owns a quarter of the columns)
    const int ntw = R / 32;
    if (ntw <= 4) LM(4, 4, 4); else if (ntw <= 8) LM(4, 4, 8); else LM(4, 4, 16);
  } else if (BM == 64) {
    const int ntw = R / 16;
    if (ntw <= 8) LM(4, 2, 8); else if (ntw <= 16) LM(4, 2, 16); else LM(4, 2, 32);
  } else if (one_stage) {
    const int ntw = R / 32;
    if (BM == 16) { if (ntw <= 4) LM1(1, 4, 4); else if (ntw <= 8) LM1(1, 4, 8); else LM1(1, 4, 16); }
    else { if (ntw <= 4) LM1(2, 4, 4); else if (ntw <= 8) LM1(2, 4, 8); else LM1(2, 4, 16); }
  } else {
    const int ntw = R / 32;
    if (BM == 16) { if (ntw <= 4) LM(1, 4, 4); else if (ntw <= 8) LM(1, 4, 8); else LM(1, 4, 16); }
    else { if (ntw <= 4) LM(2, 4, 4); else if (ntw <= 8) LM(2, 4, 8); else LM(2, 4, 16); }
  }
#undef LM1
#undef LM
  int err = BSPEC_LAUNCH_CHECK();
  if (err != 0 || n_splits == 1) return err;
  BSPEC_LAUNCH((latent_attn_join_kernel), (unsigned)((long long)n_tokens * H), R >= 256 ? 128 : 64, 0, stream, o_part,
               ml_part, (__nv_bfloat16*)out, o_row, o_head, H, R, n_splits);
  return BSPEC_LAUNCH_CHECK();
}

BSPEC_DEFINE_TRACE_SETTER(bspec_trace_set_latent_mma)
BSPEC_DEFINE_BOUNDS_REPORT(bspec_bounds_report_latent_mma)
