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
// Grid (batch * positions, rounds): a CTA stages its position's cos/sin row in shared memory as fp32 (2*D floats of
// dynamic shared memory) and rotates 2 * (256 / vectors per half row) heads of that position; a thread owns VE
// consecutive columns of the first half (and their partners in the second half) of two heads.  The kernel is pure
// streaming, so what matters is bytes in flight: a thread issues the loads of both heads (64 bytes) before the table
// is staged, and keeping the table out of registers leaves room for more resident CTAs per SM.
// ------------------------------------------------------------------------------------------------
template <typename T, typename TT>
__global__ void __launch_bounds__(256, 4)
rope_kernel(const T* __restrict__ x, const TT* __restrict__ cos_t, const TT* __restrict__ sin_t, T* __restrict__ out,
            int S, int H, int D, int start_pos, int backward, int out_bhsd) {
  constexpr int VE = Vec16<T>::N;
  extern __shared__ float s_table[];                 // cos row [0, D), sin row [D, 2D)
  const int half = D / 2;
  const int vph = half / VE;                         // vectors per half row (<= 256)
  const int tid = threadIdx.x;
  const int hstep = 256 / vph;                       // heads covered per pass
  const int c = (tid % vph) * VE;
  const int h0 = tid / vph;
  const bool active = h0 < hstep;                    // threads beyond a whole number of heads per pass only stage
  const size_t bs = blockIdx.x;                      // b*S + s
  const int s = (int)(bs % S);
  const size_t b = bs / S;

  uint4 r1[2], r2[2];                                // raw vectors of two heads: first-half and second-half columns
  auto load_round = [&](int hb) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int h = hb + u * hstep;
      if (h < H) {
        const T* xr = x + (bs * H + h) * D;
        r1[u] = __ldg(reinterpret_cast<const uint4*>(xr + c));
        r2[u] = __ldg(reinterpret_cast<const uint4*>(xr + half + c));
      }
    }
  };
  const float sg = backward ? -1.f : 1.f;            // forward: +rot*sin ; backward: -rot*sin
  auto rotate_round = [&](int hb) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int h = hb + u * hstep;
      if (h >= H) break;
      float x1[VE], x2[VE];
      unpack_vec16<T>(r1[u], x1);
      unpack_vec16<T>(r2[u], x2);
      T o1[VE], o2[VE];
#pragma unroll
      for (int e = 0; e < VE; ++e) {
        const float c1 = s_table[c + e], c2 = s_table[half + c + e];
        const float s1 = s_table[D + c + e], s2 = s_table[D + half + c + e];
        // rot[:half] = -x2, rot[half:] = x1
        o1[e] = from_f<T>(x1[e] * c1 + sg * (-x2[e]) * s1);
        o2[e] = from_f<T>(x2[e] * c2 + sg * x1[e] * s2);
      }
      const size_t orow = out_bhsd ? ((b * H + h) * S + s) : (bs * H + h);
      *reinterpret_cast<uint4*>(out + orow * D + c) = *reinterpret_cast<const uint4*>(o1);
      *reinterpret_cast<uint4*>(out + orow * D + half + c) = *reinterpret_cast<const uint4*>(o2);
    }
  };

  const int hb = h0 + (int)blockIdx.y * 2 * hstep;   // grid.y = rounds of 2*hstep heads
  if (active) load_round(hb);
  const size_t trow = (size_t)(start_pos + s) * D;
  for (int i = tid; i < D; i += 256) {
    s_table[i] = to_f(cos_t[trow + i]);
    s_table[D + i] = to_f(sin_t[trow + i]);
  }
  __syncthreads();
  if (active) rotate_round(hb);
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
