// Prefill forward, second generation: both GEMMs of the inner loop take their A operand from tensor
// memory.  16-bit inputs, head dim 128.
//
// Measured on B200, a tcgen05 MMA whose A and B both come from shared memory is limited by operand
// fetch (about 64 bytes per clock per SM), so S = Q K^T with Q in shared memory runs at half the
// tensor-pipe rate.  Here one CTA owns 128 query rows and keeps Q in TMEM for the whole kernel
// (row i in lane i, two 16-bit values per column: the A-operand layout), so QK^T reads only K from
// shared memory, like P V reads only V.
//
//   warp 0      TMA producer: K and V tiles through a 3-stage ring (3-D maps, 128-byte swizzle, no multicast)
//   warp 1      MMA issuer (one lane): S[j+1] = Q K_{j+1}^T is queued before O += P_j V_j, so the
//               tensor core computes the next scores while the softmax warps work on the current ones
//   warp 2      TMEM allocation / release
//   warps 4-11  softmax: two threads per query row (warpgroup h takes columns [64h, 64h+64) of every
//               score tile); the halves exchange their row maxima through shared memory
// TMEM columns: S[0] [0,128)  S[1] [128,256)  O [256,384)  Q [384,448).  P (16-bit) overwrites the first
// 32 columns of each half of S[buf] and feeds the PV MMA from TMEM.
// Softmax arithmetic is that of fwd_kernel in fwd_sm100.cuh (fp32 statistics, exp2 with folded scale,
// half of the exponentials on the FMA pipe, lazy rescale with threshold 8, LSE stored for backward);
// the algorithm follows _flash_fwd_kernel (src/stackkernels/_core/attention/flash_fwd.py:15-179).
#pragma once
#include "fwd_sm100.cuh"

namespace skb {
namespace sm100 {

constexpr int kF2Threads = 384;
constexpr int kF2Stages = 3;
constexpr int kF2Tile = 2 * kBoxBytes;     // 128 x 128 16-bit tile = 32 KB

enum F2Bar {
  F2_K_FULL = 0,     // +stage
  F2_K_EMPTY = 3,    // +stage
  F2_V_FULL = 6,     // +stage
  F2_V_EMPTY = 9,    // +stage
  F2_Q_READY = 12,   // softmax -> MMA: Q stored to TMEM (256)
  F2_S_FULL = 13,    // +buf  MMA -> softmax
  F2_P_FULL = 15,    // +buf  softmax -> MMA (256)
  F2_O_READY = 17,   // MMA -> softmax: PV of tile j finished (one phase per tile)
  F2_DRAIN = 18,
  F2_PAIR = 19,      // +quadrant: the two warps that share 32 query rows exchange row statistics (64)
  F2_NUM = 23
};

// shared memory: K/V ring, row-max exchange [2 bufs][2 halves][128 rows], row-sum exchange [2 halves][128], barriers
constexpr int kF2SmemBytes = 1024 + kF2Stages * 2 * kF2Tile + 2 * 2 * 128 * 4 + 2 * 128 * 4 + 256;

template <typename T>
__global__ void __launch_bounds__(kF2Threads, 1)
fwd2_kernel(const T* __restrict__ q, const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
            T* __restrict__ o, float* __restrict__ lse, int Hq, int Hkv, int Sq, int Sk, int causal, float scale_log2) {
  constexpr int HD = 128;
  constexpr uint32_t IDESC_QK = ptx::idesc_f16(Fmt<T>::v, 128, 128, 0, 0);
  constexpr uint32_t IDESC_PV = ptx::idesc_f16(Fmt<T>::v, 128, 128, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - ptx::smem_u32(smem_raw));
  auto sK = [&](int st) -> uint32_t { return sbase + (uint32_t)st * 2u * kF2Tile; };
  auto sV = [&](int st) -> uint32_t { return sbase + (uint32_t)st * 2u * kF2Tile + kF2Tile; };
  float* s_mx = reinterpret_cast<float*>(gbase + kF2Stages * 2 * kF2Tile);        // [buf][half][row]
  float* s_sum = s_mx + 2 * 2 * 128;                                              // [half][row]
  const uint32_t sBar = sbase + kF2Stages * 2 * kF2Tile + 2 * 2 * 128 * 4 + 2 * 128 * 4;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gbase + (sBar - sbase) + F2_NUM * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(gbase + (sBar - sbase) + F2_NUM * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sBar + 8u * (uint32_t)i; };

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int qt = (int)gridDim.x - 1 - (int)blockIdx.x;      // heaviest (latest) causal tiles first
  const int hq = blockIdx.y, b = blockIdx.z;
  const int bhq = b * Hq + hq;
  const int hkv = hq / (Hq / Hkv);
  const int row0 = qt * 128;
  const int shift = Sk - Sq;
  int lim = Sk;
  if (causal) lim = min(Sk, row0 + 128 + shift);
  const int nt = lim > 0 ? cdiv(lim, 128) : 0;               // KV tiles this query tile attends to

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int i = 0; i < F2_NUM; ++i)
      ptx::mbar_init(bar(i), (i == F2_Q_READY || i == F2_P_FULL || i == F2_P_FULL + 1) ? 256u
                             : (i >= F2_PAIR && i < F2_PAIR + 4) ? 64u : 1u);
    ptx::fence_mbar_init();
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(s_tmem)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, *s_tmem, 0);
  const uint32_t tO = tmem + 256, tQ = tmem + 384;
  auto tS = [&](int buf) -> uint32_t { return tmem + 128u * (uint32_t)buf; };

  if (warp < 4) {
    ptx::setmaxnreg_dec<56>();
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------------ TMA producer
      ptx::prefetch_tmap(&tm_k);
      ptx::prefetch_tmap(&tm_v);
      bool ok = true;
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j % kF2Stages;
        const uint32_t ph = (uint32_t)((j / kF2Stages) & 1) ^ 1u;
        ok = ptx::mbar_wait(bar(F2_K_EMPTY + st), ph, s_abort);
        if (!ok) break;
        ptx::mbar_expect_tx(bar(F2_K_FULL + st), kF2Tile);
        for (int h = 0; h < 2; ++h) ptx::tma_load_4d(sK(st) + h * kBoxBytes, &tm_k, h * 64, j * 128, hkv, b, bar(F2_K_FULL + st));
        ok = ptx::mbar_wait(bar(F2_V_EMPTY + st), ph, s_abort);
        if (!ok) break;
        ptx::mbar_expect_tx(bar(F2_V_FULL + st), kF2Tile);
        for (int h = 0; h < 2; ++h) ptx::tma_load_4d(sV(st) + h * kBoxBytes, &tm_v, h * 64, j * 128, hkv, b, bar(F2_V_FULL + st));
      }
      if (!ok) atomicCAS(&g_dev_status, 0u, (10u << 16));
    } else if (warp == 1) {
      // ------------------------------------------------------------------ MMA issuer (whole warp, one lane issues)
      const bool leader = ptx::elect_one();
      bool ok = true;
      auto issue_qk = [&](int j) {      // S[j & 1] = Q K_j^T, Q from TMEM (8 columns per k-step)
        const uint32_t k = sK(j % kF2Stages);
        if (leader)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ts(tS(j & 1), tQ + kk * 8, ptx::desc_sw128_kmajor(k + (kk >> 2) * kBoxBytes + (kk & 3) * 32), IDESC_QK, kk > 0);
        if (leader) ptx::mma_commit(bar(F2_S_FULL + (j & 1)));
        if (leader) ptx::mma_commit(bar(F2_K_EMPTY + j % kF2Stages));
      };
      if (nt > 0) {
        ok = ptx::mbar_wait_warp(bar(F2_Q_READY), 0, s_abort) && ptx::mbar_wait_warp(bar(F2_K_FULL), 0, s_abort);
        if (ok) { ptx::tc_fence_after(); issue_qk(0); }
      }
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j % kF2Stages, buf = j & 1;
        if (j + 1 < nt) {
          // S[buf^1] last held P of tile j-1, consumed by the PV issued in the previous iteration
          ok = ptx::mbar_wait_warp(bar(F2_K_FULL + (j + 1) % kF2Stages), (uint32_t)((j + 1) / kF2Stages) & 1u, s_abort);
          if (!ok) break;
          ptx::tc_fence_after();
          issue_qk(j + 1);
        }
        ok = ptx::mbar_wait_warp(bar(F2_V_FULL + st), (uint32_t)(j / kF2Stages) & 1u, s_abort) &&
             ptx::mbar_wait_warp(bar(F2_P_FULL + buf), (uint32_t)(j >> 1) & 1u, s_abort);
        if (!ok) break;
        ptx::tc_fence_after();
        // O += P_j V_j : P columns of half h sit at S[buf] + 64h + [0,32)
        if (leader)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ts(tO, tS(buf) + (kk >> 2) * 64 + (kk & 3) * 8, ptx::desc_sw128_mnmajor(sV(st) + kk * 2048, kBoxBytes),
                      IDESC_PV, (j > 0) || (kk > 0));
        if (leader) ptx::mma_commit(bar(F2_V_EMPTY + st));
        if (leader) ptx::mma_commit(bar(F2_O_READY));
      }
      if (leader) ptx::mma_commit(bar(F2_DRAIN));
      if (!ptx::mbar_wait_warp(bar(F2_DRAIN), 0, s_abort)) ok = false;
      if (!ok && leader) atomicCAS(&g_dev_status, 0u, (11u << 16));
    }
  } else {
    ptx::setmaxnreg_inc<224>();
    // -------------------------------------------------------------------- softmax: 2 threads per query row
    const int h = (warp - 4) >> 2;                 // column half of every score tile
    const int wq = warp & 3;
    const int r = wq * 32 + lane;                  // query row within the tile = TMEM lane
    const int grow = row0 + r;
    const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
    const int lim_col = causal ? min(Sk - 1, grow + shift) : Sk - 1;   // last visible key of this row
    bool ok = true;
    uint32_t pair_ph = 0;                          // phase of this quadrant's exchange barrier
    // Bounded rendezvous of the two warps that share these 32 rows (shared-memory writes made before
    // it are visible to the partner after it).
    auto pair_sync = [&]() -> bool {
      ptx::mbar_arrive(bar(F2_PAIR + wq));
      bool w = ptx::mbar_wait(bar(F2_PAIR + wq), pair_ph, s_abort);
      pair_ph ^= 1u;
      return __all_sync(0xffffffffu, w);
    };

    // ---- Q -> TMEM: this thread's 64 elements (128 bytes) of row r go to 32 columns of lane r
    if (nt > 0) {
      uint32_t qr[32];
      if (grow < Sq) {
        const uint4* src = reinterpret_cast<const uint4*>(q + ((size_t)bhq * Sq + grow) * HD + 64 * h);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const uint4 v = __ldg(src + i);
          qr[4 * i] = v.x; qr[4 * i + 1] = v.y; qr[4 * i + 2] = v.z; qr[4 * i + 3] = v.w;
        }
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) qr[i] = 0u;
      }
      ptx::tmem_st32(tQ + t_lane + 32 * h, qr);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(F2_Q_READY));
    }

    float m = -INFINITY, l = 0.f;                  // m: shared by both halves of the row; l: this half's partial sum
    for (int j = 0; j < nt; ++j) {
      const int buf = j & 1;
      ok = ptx::mbar_wait(bar(F2_S_FULL + buf), (uint32_t)(j >> 1) & 1u, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      if (wq == 0 && lane == 0) SKB_TR(1 + h, j, 0);
      ptx::tc_fence_after();
      uint32_t sr[64];
      ptx::tmem_ld32(tS(buf) + t_lane + 64 * h, sr);
      ptx::tmem_ld32(tS(buf) + t_lane + 64 * h + 32, sr + 32);
      ptx::tmem_wait_ld();

      const int c0 = j * 128 + 64 * h;             // key index of this thread's first column
      if (__any_sync(0xffffffffu, c0 + 63 > lim_col)) {
#pragma unroll
        for (int c = 0; c < 64; ++c)
          if (c0 + c > lim_col) sr[c] = 0xff800000u;  // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {
        mx0 = ptx::max3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
        mx1 = ptx::max3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
        mx2 = ptx::max3(mx2, __uint_as_float(sr[c + 4]), __uint_as_float(sr[c + 5]));
        mx3 = ptx::max3(mx3, __uint_as_float(sr[c + 6]), __uint_as_float(sr[c + 7]));
      }
      const float lmax = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3));
      // exchange with the thread that holds the other half of this row (same quadrant, other warpgroup)
      s_mx[(buf * 2 + h) * 128 + r] = lmax;
      ok = pair_sync();
      if (!ok) break;
      const float mx = fmaxf(lmax, s_mx[(buf * 2 + (h ^ 1)) * 128 + r]) * scale_log2;
      const bool grow_m = mx > m + 8.f;            // same decision in both halves; false when both are -inf
      float alpha = 1.f;
      if (grow_m) {
        alpha = ptx::ex2(m - mx);                  // m = -inf -> 0
        m = mx;
        l *= alpha;
      }
      const float mref = (m == -INFINITY) ? 0.f : m;
      if (wq == 0 && lane == 0) SKB_TR(1 + h, j, 1);
      const uint64_t sc2 = ptx::f2_pack(scale_log2, scale_log2), nm2 = ptx::f2_pack(-mref, -mref);
      uint64_t sumA = ptx::f2_pack(0.f, 0.f), sumB = sumA;
#pragma unroll
      for (int c = 0; c < 64; c += 8) {      // of every eight exponentials, six on the MUFU unit, two on the FMA pipe
        float x[8], pe[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2)
          ptx::f2_unpack(ptx::f2_fma(ptx::f2_pack(__uint_as_float(sr[c + e]), __uint_as_float(sr[c + e + 1])), sc2, nm2),
                         x[e], x[e + 1]);
#pragma unroll
        for (int e = 0; e < 6; ++e) pe[e] = ptx::ex2(x[e]);
        ptx::exp2_poly2(x[6], x[7], pe[6], pe[7]);
        sumA = ptx::f2_add(sumA, ptx::f2_add(ptx::f2_pack(pe[0], pe[1]), ptx::f2_pack(pe[2], pe[3])));
        sumB = ptx::f2_add(sumB, ptx::f2_add(ptx::f2_pack(pe[4], pe[5]), ptx::f2_pack(pe[6], pe[7])));
#pragma unroll
        for (int e = 0; e < 8; e += 2) sr[(c + e) >> 1] = pack2(pe[e], pe[e + 1], T());
      }
      {
        float a0, a1, b0, b1;
        ptx::f2_unpack(sumA, a0, a1);
        ptx::f2_unpack(sumB, b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
      if (wq == 0 && lane == 0) SKB_TR(1 + h, j, 2);
      ptx::tmem_st32(tS(buf) + t_lane + 64 * h, sr);
      if (j > 0 && __any_sync(0xffffffffu, grow_m)) {
        // O must be quiescent: wait for the PV of tile j-1, then rescale this thread's 64 columns
        ok = ptx::mbar_wait(bar(F2_O_READY), (uint32_t)(j - 1) & 1u, s_abort);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          uint32_t orr[32];
          ptx::tmem_ld32(tO + t_lane + 64 * h + c * 32, orr);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          ptx::tmem_st32(tO + t_lane + 64 * h + c * 32, orr);
        }
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(F2_P_FULL + buf));
      if (wq == 0 && lane == 0) SKB_TR(1 + h, j, 3);
    }

    // ------------------------------------------------------------------ epilogue
    if (ok && nt > 0) {
      ok = ptx::mbar_wait(bar(F2_O_READY), (uint32_t)(nt - 1) & 1u, s_abort);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok) {
      ptx::tc_fence_after();
      // total row sum = this half + the other half
      s_sum[h * 128 + r] = l;
      ok = pair_sync();
      l = s_sum[r] + s_sum[128 + r];
      const bool seen = (m != -INFINITY) && l > 0.f;    // false: no visible key in the whole row
      const float inv = seen ? 1.f / l : 0.f;
      T* orow = o + ((size_t)bhq * Sq + (size_t)min(grow, Sq - 1)) * HD + 64 * h;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t orr[32];
        if (nt > 0) {
          ptx::tmem_ld32(tO + t_lane + 64 * h + c * 32, orr);
          ptx::tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = 0u;
        }
        if (grow < Sq) {
#pragma unroll
          for (int i = 0; i < 32; i += 8) {
            uint4 wv;
            wv.x = pack2(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv, T());
            wv.y = pack2(__uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv, T());
            wv.z = pack2(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv, T());
            wv.w = pack2(__uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv, T());
            *reinterpret_cast<uint4*>(orow + c * 32 + i) = wv;
          }
        }
      }
      if (h == 0 && grow < Sq) lse[(size_t)bhq * Sq + grow] = seen ? (m + log2f(l)) * kLn2 : -INFINITY;
    } else if (lane == 0) {
      atomicCAS(&g_dev_status, 0u, (12u << 16) | (unsigned)warp);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 2) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

}  // namespace sm100
}  // namespace skb
