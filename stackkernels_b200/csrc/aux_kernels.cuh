// The two steps that sit immediately before attention in every caller, as plain bandwidth-bound kernels:
// rotary position embedding with a start position, and the in-place append of new K/V rows to a KV cache.
#pragma once
#include "common.cuh"

namespace skb {
namespace aux {

// ------------------------------------------------------------------------------------------------
// RoPE.  x, out: (B, S, H, D) (the reference's layout); cos, sin: (max_seq, D) tables of type TT.
// Forward  (src/stackkernels/_reference/torch/rope.py:41-59):  out = x*cos + rotate_half(x)*sin,
//          rotate_half(x) = cat(-x[half:], x[:half]), position = start_pos + s, arithmetic in fp32.
// Backward (src/stackkernels/torch/embedding.py:46-64):        dx  = dy*cos - rotate_half(dy)*sin.
// With out_bhsd the result is written as (B, H, S, D), the layout the attention kernels take, which
// saves the transpose + contiguous copy callers otherwise make.
// x is contiguous, so its rows (one head of one position, D elements) are numbered b*S*H + s*H + h.  A CTA rotates
// kRopeRows(D) consecutive rows -- 256 threads, each owning VE consecutive columns of the first half and their
// partners in the second half of two rows -- whatever H is: one position's 64 heads at D = 128, eight positions
// when H = 8.  The cos/sin rows of the positions it touches are staged in dynamic shared memory as fp32
// (2*D floats per position).  The kernel is pure streaming, so what matters is bytes in flight: a thread issues the
// loads of both rows (64 bytes) before the tables are staged, and the tables are re-read from shared memory per row
// rather than held in registers, which leaves room for five resident CTAs per SM.
// ------------------------------------------------------------------------------------------------
// rows per CTA: two passes of the rows that 256 threads cover with one 16-byte vector pair each
inline int rope_rows_per_cta(int D, int ve) { return 2 * (256 / (D / 2 / ve)); }
// positions a CTA can touch (its rows may start in the middle of a position)
inline int rope_positions_per_cta(int D, int ve, int H) { return (rope_rows_per_cta(D, ve) - 1) / H + 2; }

// MODE 3: a CTA's rows are exactly one position; 0: they lie within one position (H is a multiple of the rows per
// CTA); 1: they are pos_per_cta whole positions; 2: any other head count (needs a 64-bit division).  A CTA lives for a couple of
// memory round trips, so a few hundred clocks of index arithmetic show in the bandwidth (measured: 5.4 against
// 5.8 TB/s with the three cases behind run-time branches), hence the specialisation.
template <typename T, typename TT, int MODE>
__global__ void __launch_bounds__(256, 5)
rope_kernel(const T* __restrict__ x, const TT* __restrict__ cos_t, const TT* __restrict__ sin_t, T* __restrict__ out,
            int S, int H, int D, int start_pos, int backward, int out_bhsd, long long n_rows, int pos_per_cta,
            int cta_per_pos) {
  constexpr int VE = Vec16<T>::N;
  extern __shared__ __align__(16) float s_table[];                 // per staged position: cos row [0, D), sin row [D, 2D)
  const int half = D / 2;
  const int vph = half / VE;                         // vectors per half row (<= 256)
  const int tid = threadIdx.x;
  const int rstep = 256 / vph;                       // rows covered per pass
  const int c = (tid % vph) * VE;
  const bool active = tid / vph < rstep;             // threads beyond a whole number of rows per pass only stage
  // B*S fits 32 bits (checked by the launcher); only the row number itself needs 64
  const long long row0 = (long long)blockIdx.x * (2 * rstep);
  const int n_here = (int)min((long long)(2 * rstep), n_rows - row0);   // rows of this CTA
  const int lr0 = tid / vph;                         // this thread's rows: lr0 and lr0 + rstep of the CTA's rows

  uint4 r1[2], r2[2];                                // raw vectors of two rows: first-half and second-half columns
  if (active) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int lr = lr0 + u * rstep;
      if (lr < n_here) {
        const T* xr = x + (size_t)(row0 + lr) * D;
        r1[u] = __ldg(reinterpret_cast<const uint4*>(xr + c));
        r2[u] = __ldg(reinterpret_cast<const uint4*>(xr + half + c));
      }
    }
  }
  // First position (b*S + s) this CTA touches and the head of its first row.  The launcher passes the exact
  // ratio when a CTA's rows are a whole number of positions (pos_per_cta) or a position is a whole number of CTAs
  // (cta_per_pos); only other head counts need the 64-bit division.
  int p0, h_off, n_pos;
  if constexpr (MODE == 3) {
    p0 = (int)blockIdx.x;
    h_off = 0;
    n_pos = 1;
  } else if constexpr (MODE == 0) {
    p0 = (int)(blockIdx.x / (unsigned)cta_per_pos);
    h_off = ((int)blockIdx.x - p0 * cta_per_pos) * 2 * rstep;
    n_pos = 1;
  } else if constexpr (MODE == 1) {
    p0 = (int)blockIdx.x * pos_per_cta;
    h_off = 0;
    n_pos = (n_here - 1) / H + 1;
  } else {
    p0 = (int)(row0 / H);
    h_off = (int)(row0 - (long long)p0 * H);
    n_pos = (h_off + n_here - 1) / H + 1;
  }
  if (n_pos == 1) {
    const size_t trow = (size_t)(start_pos + p0 % S) * D;
    for (int col = tid; col < D; col += 256) {
      s_table[col] = to_f(cos_t[trow + col]);
      s_table[D + col] = to_f(sin_t[trow + col]);
    }
  } else {
    for (int i = tid; i < n_pos * D; i += 256) {
      const int lp = i / D, col = i - lp * D;
      const size_t trow = (size_t)(start_pos + (p0 + lp) % S) * D;
      s_table[lp * 2 * D + col] = to_f(cos_t[trow + col]);
      s_table[lp * 2 * D + D + col] = to_f(sin_t[trow + col]);
    }
  }
  __syncthreads();
  if (!active) return;
  const float sg = backward ? -1.f : 1.f;            // forward: +rot*sin ; backward: -rot*sin
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int lr = lr0 + u * rstep;
    if (lr >= n_here) break;
    asm volatile("" ::: "memory");   // re-read the table per row instead of holding 4*VE values across both
    const int lp = (MODE == 0 || MODE == 3) ? 0 : (h_off + lr) / H;   // staged position of this row
    const float* tab = s_table + lp * 2 * D;
    float x1[VE], x2[VE];
    unpack_vec16<T>(r1[u], x1);
    unpack_vec16<T>(r2[u], x2);
    T o1[VE], o2[VE];
#pragma unroll
    for (int e0 = 0; e0 < VE; e0 += 4) {
      // 16-byte shared-memory reads: c, half and D are multiples of 4 floats (scalar reads made the kernel wait
      // on the shared-memory instruction queue)
      const float4 c1 = *reinterpret_cast<const float4*>(tab + c + e0);
      const float4 c2 = *reinterpret_cast<const float4*>(tab + half + c + e0);
      const float4 s1 = *reinterpret_cast<const float4*>(tab + D + c + e0);
      const float4 s2 = *reinterpret_cast<const float4*>(tab + D + half + c + e0);
      const float c1v[4] = {c1.x, c1.y, c1.z, c1.w}, c2v[4] = {c2.x, c2.y, c2.z, c2.w};
      const float s1v[4] = {s1.x, s1.y, s1.z, s1.w}, s2v[4] = {s2.x, s2.y, s2.z, s2.w};
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const int e = e0 + i;
        // rot[:half] = -x2, rot[half:] = x1
        o1[e] = from_f<T>(x1[e] * c1v[i] + sg * (-x2[e]) * s1v[i]);
        o2[e] = from_f<T>(x2[e] * c2v[i] + sg * x1[e] * s2v[i]);
      }
    }
    size_t orow = (size_t)(row0 + lr);
    if (out_bhsd) {
      const int h = h_off + lr - lp * H, bs = p0 + lp;
      const int b = bs / S, sp = bs - b * S;
      orow = ((size_t)b * H + h) * S + sp;
    }
    *reinterpret_cast<uint4*>(out + orow * D + c) = *reinterpret_cast<const uint4*>(o1);
    *reinterpret_cast<uint4*>(out + orow * D + half + c) = *reinterpret_cast<const uint4*>(o2);
  }
}

// ------------------------------------------------------------------------------------------------
// KV-cache append: cache[b, h, len_b + t, :] = new[b, h, t, :] for t < T, for K and V together, where
// len_b = cache_seqlens[b] (or `fixed_len` when the pointer is NULL).  Rows that would fall beyond the
// capacity are dropped.  The reference only reserves this op (src/stackkernels/_core/cache/kv_update.py);
// it is what produces the cache_seqlens that flash_decode consumes.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
kv_append_kernel(const T* __restrict__ k_new, const T* __restrict__ v_new, T* __restrict__ k_cache,
                 T* __restrict__ v_cache, const int32_t* __restrict__ seqlens, int fixed_len, int Hkv, int T_new,
                 int Scap, int D, size_t n_vec) {
  constexpr int VE = Vec16<T>::N;
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_vec) return;
  const int vpr = D / VE;
  const int c = (int)(i % vpr) * VE;
  const size_t row = i / vpr;                        // (b*Hkv + h)*T_new + t
  const int t = (int)(row % T_new);
  const size_t bh = row / T_new;
  const size_t b = bh / Hkv;
  const int len = seqlens ? min(max(seqlens[b], 0), Scap) : fixed_len;
  const int dst = len + t;
  if (dst >= Scap) return;
  const size_t src_off = row * D + c, dst_off = (bh * Scap + dst) * D + c;
  *reinterpret_cast<uint4*>(k_cache + dst_off) = __ldg(reinterpret_cast<const uint4*>(k_new + src_off));
  *reinterpret_cast<uint4*>(v_cache + dst_off) = __ldg(reinterpret_cast<const uint4*>(v_new + src_off));
}

// cache_seqlens[b] = min(cache_seqlens[b] + T_new, Scap), run after the append on the same stream
__global__ void kv_advance_kernel(int32_t* __restrict__ seqlens, int B, int T_new, int Scap) {
  const int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) seqlens[b] = min(max(seqlens[b], 0) + T_new, Scap);
}

}  // namespace aux
}  // namespace skb
