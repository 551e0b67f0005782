// Split-KV decode on tcgen05 tensor cores for wide GQA/MQA groups (16-bit, head dim 128, group <= 128).
//
// With G query heads per KV head the decode step needs G FLOP per KV byte; at G = 64 that is more than
// warp-level mma.sync and its ldmatrix traffic sustain (decode_group.cuh becomes compute bound), so this
// kernel puts the group's heads on the M dimension of 128-row tcgen05 MMAs (rows >= G are don't-care):
//   S[buf] = Q K_j^T  (Q and K from shared memory)      O += P_j V_j  (P from TMEM, V from shared memory)
// One CTA = (split, kv head, batch).  Warp 0 streams 128-row K/V tiles with TMA through a 3-stage ring,
// warp 1 owns TMEM and issues the MMAs (S of the next tile is queued before PV of the current one: S is
// double buffered), warps 4-7 run the same fp32 online softmax as the prefill kernel, one head per thread.
// V rows past the sequence end are zeroed in shared memory before PV (stale cache rows may hold NaNs).
// Partials (unnormalised O, max, sum) use the layout of decode_combine_kernel.
// TMEM columns: S[0] [0,128) S[1] [128,256) O [256,384).
#pragma once
#include "fwd_sm100.cuh"

namespace skb {
namespace dtc {

using sm100::Fmt;
using sm100::kBoxBytes;
using sm100::pack2;

constexpr int kThreads = 256;
constexpr int kStages = 3;
constexpr int kTile = 2 * kBoxBytes;     // 128 x 128 16-bit tile = 32 KB

enum Bar {
  Q_FULL = 0,
  K_FULL = 1,     // +stage
  K_EMPTY = 4,    // +stage
  V_FULL = 7,     // +stage
  V_EMPTY = 10,   // +stage
  S_FULL = 13,    // +buf
  P_FULL = 15,    // +buf (128)
  O_READY = 17,
  DRAIN = 18,
  NUM = 19
};
constexpr int kSmemBytes = 1024 + (1 + 2 * kStages) * kTile + 256;

template <typename T>
__global__ void __launch_bounds__(kThreads, 1)
decode_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
              const __grid_constant__ CUtensorMap tm_v, const int32_t* __restrict__ seqlens,
              float* __restrict__ part_o, float2* __restrict__ part_ml, int Hq, int Hkv, int Scap, int D, int nsplit,
              float scale_log2) {
  // D <= 128 (a multiple of 8) is the head dimension in memory; the bulk copies zero columns [D, 128).
  constexpr uint32_t IDESC_QK = ptx::idesc_f16(Fmt<T>::v, 128, 128, 0, 0);
  constexpr uint32_t IDESC_PV = ptx::idesc_f16(Fmt<T>::v, 128, 128, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - ptx::smem_u32(smem_raw));
  const uint32_t sQ = sbase;
  auto sK = [&](int st) -> uint32_t { return sbase + kTile + (uint32_t)st * 2u * kTile; };
  auto sV = [&](int st) -> uint32_t { return sbase + 2 * kTile + (uint32_t)st * 2u * kTile; };
  const uint32_t sBar = sbase + (1 + 2 * kStages) * kTile;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gbase + (sBar - sbase) + NUM * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(gbase + (sBar - sbase) + NUM * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sBar + 8u * (uint32_t)i; };

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int split = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int len = seqlens ? min(max(seqlens[b], 0), Scap) : Scap;
  const int chunk = cdiv(cdiv(len, nsplit), 128) * 128;
  const int start = split * chunk;
  const int end = min(len, start + chunk);
  const int nt = end > start ? cdiv(end - start, 128) : 0;

  if (threadIdx.x == 0) {
    *s_abort = 0;
    for (int i = 0; i < NUM; ++i) ptx::mbar_init(bar(i), (i == P_FULL || i == P_FULL + 1) ? 128u : 1u);
    ptx::fence_mbar_init();
  }
  if (warp == 1) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(s_tmem)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = __shfl_sync(0xffffffffu, *s_tmem, 0);
  const uint32_t tO = tmem + 256;
  auto tS = [&](int buf) -> uint32_t { return tmem + 128u * (uint32_t)buf; };

  if (warp == 0) {
    if (lane == 0 && nt > 0) {
      // ------------------------------------------------------------------ TMA producer
      ptx::prefetch_tmap(&tm_q); ptx::prefetch_tmap(&tm_k); ptx::prefetch_tmap(&tm_v);
      ptx::mbar_expect_tx(bar(Q_FULL), kTile);
      // rows = query heads of this group (q viewed as {D, Hq, B}); rows >= G are other heads or zero fill
      for (int h = 0; h < 2; ++h) ptx::tma_load_3d(sQ + h * kBoxBytes, &tm_q, h * 64, hkv * G, b, bar(Q_FULL));
      bool ok = true;
      for (int j = 0; j < nt && ok; ++j) {
        const int st = j % kStages;
        const uint32_t ph = (uint32_t)((j / kStages) & 1) ^ 1u;
        const int row = start + j * 128;
        ok = ptx::mbar_wait(bar(K_EMPTY + st), ph, s_abort);
        if (!ok) break;
        ptx::mbar_expect_tx(bar(K_FULL + st), kTile);
        for (int h = 0; h < 2; ++h) ptx::tma_load_4d(sK(st) + h * kBoxBytes, &tm_k, h * 64, row, hkv, b, bar(K_FULL + st));
        ok = ptx::mbar_wait(bar(V_EMPTY + st), ph, s_abort);
        if (!ok) break;
        ptx::mbar_expect_tx(bar(V_FULL + st), kTile);
        for (int h = 0; h < 2; ++h) ptx::tma_load_4d(sV(st) + h * kBoxBytes, &tm_v, h * 64, row, hkv, b, bar(V_FULL + st));
      }
      if (!ok) atomicCAS(&g_dev_status, 0u, (13u << 16));
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer (whole warp, one lane issues)
    const bool leader = ptx::elect_one();
    bool ok = true;
    auto issue_qk = [&](int j) {
      const uint32_t k = sK(j % kStages);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {
          const uint32_t off = (uint32_t)(kk >> 2) * kBoxBytes + (uint32_t)(kk & 3) * 32u;
          ptx::mma_ss(tS(j & 1), ptx::desc_sw128_kmajor(sQ + off), ptx::desc_sw128_kmajor(k + off), IDESC_QK, kk > 0);
        }
        ptx::mma_commit(bar(S_FULL + (j & 1)));
        ptx::mma_commit(bar(K_EMPTY + j % kStages));
      }
    };
    if (nt > 0) {
      ok = ptx::mbar_wait_warp(bar(Q_FULL), 0, s_abort) && ptx::mbar_wait_warp(bar(K_FULL), 0, s_abort);
      if (ok) { ptx::tc_fence_after(); issue_qk(0); }
    }
    for (int j = 0; j < nt && ok; ++j) {
      const int st = j % kStages, buf = j & 1;
      if (j + 1 < nt) {
        ok = ptx::mbar_wait_warp(bar(K_FULL + (j + 1) % kStages), (uint32_t)((j + 1) / kStages) & 1u, s_abort);
        if (!ok) break;
        ptx::tc_fence_after();
        issue_qk(j + 1);
      }
      ok = ptx::mbar_wait_warp(bar(V_FULL + st), (uint32_t)(j / kStages) & 1u, s_abort) &&
           ptx::mbar_wait_warp(bar(P_FULL + buf), (uint32_t)(j >> 1) & 1u, s_abort);
      if (!ok) break;
      ptx::tc_fence_after();
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ts(tO, tS(buf) + kk * 8, ptx::desc_sw128_mnmajor(sV(st) + kk * 2048, kBoxBytes), IDESC_PV, (j > 0) || (kk > 0));
        ptx::mma_commit(bar(V_EMPTY + st));
        ptx::mma_commit(bar(O_READY));
      }
    }
    if (leader) ptx::mma_commit(bar(DRAIN));
    if (!ptx::mbar_wait_warp(bar(DRAIN), 0, s_abort)) ok = false;
    if (!ok && leader) atomicCAS(&g_dev_status, 0u, (14u << 16));
  } else if (warp >= 4) {
    // -------------------------------------------------------------------- softmax: one query head per thread
    const int wq = warp & 3;
    const int r = wq * 32 + lane;                  // head within the group = TMEM lane
    const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      const int buf = j & 1, st = j % kStages;
      ok = ptx::mbar_wait_warp(bar(S_FULL + buf), (uint32_t)(j >> 1) & 1u, s_abort);
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t sr[128];
#pragma unroll
      for (int c = 0; c < 4; ++c) ptx::tmem_ld32(tS(buf) + t_lane + c * 32, sr + c * 32);
      ptx::tmem_wait_ld();
      const int valid = end - (start + j * 128);   // rows of this tile inside the sequence (>= 1)
      if (valid < 128) {
#pragma unroll
        for (int c = 0; c < 128; ++c)
          if (c >= valid) sr[c] = 0xff800000u;     // -inf
        // clear the V rows past the end (each thread clears whole rows r' = its lane index)
        ok = ptx::mbar_wait_warp(bar(V_FULL + st), (uint32_t)(j / kStages) & 1u, s_abort);
        if (!ok) break;
        if (r >= valid) {
          uint8_t* vrow = gbase + (sV(st) - sbase) + r * 128;
#pragma unroll
          for (int c = 0; c < 8; ++c) {
            *reinterpret_cast<uint4*>(vrow + c * 16) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4*>(vrow + kBoxBytes + c * 16) = make_uint4(0u, 0u, 0u, 0u);
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < 128; c += 8) {
        mx0 = ptx::max3(mx0, __uint_as_float(sr[c]), __uint_as_float(sr[c + 1]));
        mx1 = ptx::max3(mx1, __uint_as_float(sr[c + 2]), __uint_as_float(sr[c + 3]));
        mx2 = ptx::max3(mx2, __uint_as_float(sr[c + 4]), __uint_as_float(sr[c + 5]));
        mx3 = ptx::max3(mx3, __uint_as_float(sr[c + 6]), __uint_as_float(sr[c + 7]));
      }
      const float mx = fmaxf(fmaxf(mx0, mx1), fmaxf(mx2, mx3)) * scale_log2;
      const bool grow_m = mx > m + 8.f;
      float alpha = 1.f;
      if (grow_m) {
        alpha = ptx::ex2(m - mx);
        m = mx;
        l *= alpha;
      }
      const float mref = (m == -INFINITY) ? 0.f : m;
      const uint64_t sc2 = ptx::f2_pack(scale_log2, scale_log2), nm2 = ptx::f2_pack(-mref, -mref);
      uint64_t sumA = ptx::f2_pack(0.f, 0.f), sumB = sumA;
#pragma unroll
      for (int c = 0; c < 128; c += 8) {
        float x[8], pe[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2)
          ptx::f2_unpack(ptx::f2_fma(ptx::f2_pack(__uint_as_float(sr[c + e]), __uint_as_float(sr[c + e + 1])), sc2, nm2),
                         x[e], x[e + 1]);
#pragma unroll
        for (int e = 0; e < 6; ++e) pe[e] = ptx::ex2(x[e]);
        ptx::exp2_poly2(x[6], x[7], pe[6], pe[7]);
        if (valid < 128) {                         // polynomial exponentials of -inf are tiny, not zero
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (c + e >= valid) pe[e] = 0.f;
        }
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
      ptx::tmem_st32(tS(buf) + t_lane, sr);
      ptx::tmem_st32(tS(buf) + t_lane + 32, sr + 32);
      if (j > 0 && __any_sync(0xffffffffu, grow_m)) {
        ok = ptx::mbar_wait_warp(bar(O_READY), (uint32_t)(j - 1) & 1u, s_abort);   // PV of tile j-1 finished
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          uint32_t orr[32];
          ptx::tmem_ld32(tO + t_lane + c * 32, orr);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = __float_as_uint(__uint_as_float(orr[i]) * alpha);
          ptx::tmem_st32(tO + t_lane + c * 32, orr);
        }
      }
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(P_FULL + buf));
    }
    // ------------------------------------------------------------------ partial results for the combine kernel
    // DRAIN completes once, after every MMA of the CTA. O_READY cannot be used here: with S double-buffered
    // this warp may be two tiles ahead of the last finished PV product, and a parity wait on a barrier that is
    // two phases behind returns at once.
    if (ok) ok = ptx::mbar_wait_warp(bar(DRAIN), 0, s_abort);
    if (ok) {
      ptx::tc_fence_after();
      const size_t pbase = ((size_t)b * Hq + (size_t)hkv * G + min(r, G - 1)) * nsplit + split;
      const bool seen = (m != -INFINITY) && l > 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t orr[32];
        if (nt > 0) {
          ptx::tmem_ld32(tO + t_lane + c * 32, orr);
          ptx::tmem_wait_ld();
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) orr[i] = 0u;
        }
        if (r < G) {
#pragma unroll
          for (int i = 0; i < 32; i += 4)
            if (c * 32 + i < D)
              *reinterpret_cast<uint4*>(part_o + pbase * D + c * 32 + i) =
                seen ? make_uint4(orr[i], orr[i + 1], orr[i + 2], orr[i + 3]) : make_uint4(0u, 0u, 0u, 0u);
        }
      }
      if (r < G) part_ml[pbase] = seen ? make_float2(m, l) : make_float2(-INFINITY, 0.f);
    } else if (lane == 0) {
      atomicCAS(&g_dev_status, 0u, (15u << 16) | (unsigned)warp);
    }
  }

  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    ptx::tc_fence_after();
    ptx::tmem_dealloc(tmem, 512);
  }
}

}  // namespace dtc
}  // namespace skb
