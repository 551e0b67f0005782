// Attention backward on Blackwell tensor cores (tcgen05 + TMEM + TMA).  16-bit inputs, head dim 128.
//
// One CTA owns 128 KV rows of one (batch, kv head) and keeps dK and dV for them in tensor memory
// for the whole kernel; it loops over the query heads of its GQA group and over the 128-row query
// tiles that can see those keys, so dK/dV have a single writer and need no atomics -- the loop
// structure of _flash_bwd_dkv_kernel (src/stackkernels/_core/attention/flash_bwd.py:201-359 in the
// reference).  Unlike the reference, which recomputes S and dP in a second kernel to get dQ
// (flash_bwd.py:58-198, 7 tile GEMMs per tile pair), dQ is produced here from the same dS with
// 5 GEMMs per pair and added into an fp32 accumulator in global memory.
//
// Everything is computed transposed so that probabilities can feed the next MMA from TMEM:
//   (a) S^T  = K Q^T          [kv x q]   A = K (smem), B = Q (smem)            -> TMEM R_S
//   (b) dP^T = V dO^T         [kv x q]   A = V (smem), B = dO (smem)           -> TMEM R_P
//       P^T  = exp2(S^T * scale*log2e - LSE*log2e)          (16-bit, stored over R_S)
//   (c) dV  += P^T dO         [kv x d]   A = P^T (TMEM), B = dO (smem, MN-major)
//       dS^T = P^T o (dP^T - Delta)                         (16-bit, to shared memory)
//   (d) dK  += dS^T Q         [kv x d]   A = dS^T (smem), B = Q (smem, MN-major)
//   (e) dQ^T = K^T dS^T       [d x q]    A = K (smem, MN-major), B = dS^T (smem, MN-major) -> R_P
// TMEM columns: dK [0,128) dV [128,256) R_S [256,384) R_P [384,512).
//
// Warps: 0 TMA producer, 1 MMA issuer, 2 TMEM owner, 4-11 two compute warpgroups that split the
// 128 query columns of every tile (thread = one KV row = one TMEM lane, 64 columns).
// The issue order c(i) b(i) a(i+1) d(i) e(i) lets the tensor core run dV / the next S^T while the
// compute warps turn dP^T into dS^T, and d/e while they compute the next P^T and drain dQ^T.
#pragma once
#include "sm100_ptx.cuh"

namespace skb {
namespace sm100 {

constexpr int kBwdThreads = 384;
constexpr int kBwdTile = 128;
constexpr int kBwdBox = 128 * 128;                 // 128 rows x 64 16-bit columns
constexpr int kBwdTileBytes = 2 * kBwdBox;         // 128 x 128 16-bit tile
constexpr int kBwdQStage = kBwdTileBytes + 1024;   // Q tile + LSE*log2e row (512 B) + Delta row (512 B)

enum BwdBar {
  B_KV_FULL = 0,
  B_Q_FULL = 1,     // +stage
  B_Q_EMPTY = 3,    // +stage
  B_DO_FULL = 5,    // +stage
  B_DO_EMPTY = 7,   // +stage
  B_S_READY = 9,    // MMA -> compute
  B_P_READY = 10,   // compute -> MMA (256)
  B_DP_READY = 11,  // MMA -> compute
  B_DS_READY = 12,  // compute -> MMA (256)
  B_DQ_DONE = 13,   // MMA -> compute
  B_RP_FREE = 14,   // compute -> MMA (256)
  B_ACC_DONE = 15,
  B_NUM = 16
};

// shared memory: K, V, dS tiles, 2 Q stages, 2 dO stages, barriers
constexpr int kBwdSmemUsed = 3 * kBwdTileBytes + 2 * kBwdQStage + 2 * kBwdTileBytes + 256;
constexpr int kBwdSmemBytes = 232448;   // everything the SM offers one CTA; leaves alignment slack

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(dst), "l"(reinterpret_cast<uint64_t>(src)), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void red_add(float* addr, float v) {
  asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v) : "memory");
}

// Preprocess: delta = rowsum(dO o O) and lse2 = LSE*log2e, both padded to a multiple of 128 rows per
// (batch, head) so that the main kernel can fetch 128-row slices with aligned bulk copies.
// Padding rows and rows without any visible key get lse2 = +inf (their probabilities become 0).
template <typename T>
__global__ void __launch_bounds__(256)
bwd_prep_kernel(const T* __restrict__ dout, const T* __restrict__ o, const float* __restrict__ lse,
                float* __restrict__ delta, float* __restrict__ lse2, int Sq, int Sq_pad, int D, size_t bh_count) {
  constexpr int VE = Vec16<T>::N;
  const size_t prow = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (prow >= bh_count * Sq_pad) return;
  const size_t bh = prow / Sq_pad;
  const int r = (int)(prow % Sq_pad);
  if (r >= Sq) {
    if (lane == 0) { delta[prow] = 0.f; lse2[prow] = INFINITY; }
    return;
  }
  const size_t row = bh * Sq + r;
  float s = 0.f;
  for (int c = lane * VE; c < D; c += 32 * VE) {
    float a[VE], b2[VE];
    load_vec16<T>(dout + row * D + c, a);
    load_vec16<T>(o + row * D + c, b2);
#pragma unroll
    for (int i = 0; i < VE; ++i) s += a[i] * b2[i];
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
  if (lane == 0) {
    delta[prow] = s;
    const float l = lse[row];
    lse2[prow] = (l == -INFINITY) ? INFINITY : l * kLog2e;
  }
}

// Postprocess: dQ = T(scale * dQ_accumulator)
template <typename T>
__global__ void __launch_bounds__(256)
bwd_post_kernel(const float* __restrict__ acc, T* __restrict__ dq, float scale, size_t n4) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n4) return;
  const float4 v = reinterpret_cast<const float4*>(acc)[i];
  T out[4] = {from_f<T>(v.x * scale), from_f<T>(v.y * scale), from_f<T>(v.z * scale), from_f<T>(v.w * scale)};
  *reinterpret_cast<uint2*>(dq + i * 4) = *reinterpret_cast<uint2*>(out);
}

template <typename T>
__global__ void __launch_bounds__(kBwdThreads, 1)
bwd_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
           const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
           const float* __restrict__ lse2, const float* __restrict__ delta, float* __restrict__ dq_acc,
           T* __restrict__ dk, T* __restrict__ dv, int Hq, int Hkv, int Sq, int Sk, int Sq_pad, int causal,
           float scale, float scale_log2) {
  constexpr int HD = 128;
  constexpr uint32_t IDESC_KK = ptx::idesc_f16(Fmt<T>::v, 128, 128, 0, 0);   // A K-major,  B K-major
  constexpr uint32_t IDESC_KM = ptx::idesc_f16(Fmt<T>::v, 128, 128, 0, 1);   // A K-major,  B MN-major
  constexpr uint32_t IDESC_MM = ptx::idesc_f16(Fmt<T>::v, 128, 128, 1, 1);   // A MN-major, B MN-major

  extern __shared__ uint8_t smem_raw[];
  const uint32_t raw = ptx::smem_u32(smem_raw);
  const uint32_t sbase = (raw + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - raw);
  const uint32_t sK = sbase;
  const uint32_t sV = sK + kBwdTileBytes;
  const uint32_t sdS = sV + kBwdTileBytes;
  const uint32_t sQ0 = sdS + kBwdTileBytes;                 // 2 stages of kBwdQStage
  const uint32_t sdO0 = sQ0 + 2 * kBwdQStage;               // 2 stages of kBwdTileBytes
  const uint32_t sBar = sdO0 + 2 * kBwdTileBytes;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gbase + (sBar - sbase) + B_NUM * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(gbase + (sBar - sbase) + B_NUM * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sBar + 8u * (uint32_t)i; };
  auto sQ = [&](int st) -> uint32_t { return sQ0 + (uint32_t)st * kBwdQStage; };
  auto sdO = [&](int st) -> uint32_t { return sdO0 + (uint32_t)st * kBwdTileBytes; };

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int jt = blockIdx.x, hkv = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const int shift = Sk - Sq;
  const int kv0 = jt * kBwdTile;
  const int nq = cdiv(Sq, kBwdTile);
  int i_start = 0;
  if (causal) i_start = max(0, kv0 - shift) / kBwdTile;      // first query tile that sees key kv0
  const int per_head = max(0, nq - i_start);
  const int n_it = per_head * G;
  const bool fits = (sbase - raw) + (uint32_t)kBwdSmemUsed <= (uint32_t)kBwdSmemBytes;

  if (threadIdx.x == 0) {
    *s_abort = fits ? 0 : 1;
    for (int i = 0; i < B_NUM; ++i)
      ptx::mbar_init(bar(i), (i == B_P_READY || i == B_DS_READY || i == B_RP_FREE) ? 256u : 1u);
    ptx::fence_mbar_init();
    if (!fits) atomicCAS(&g_dev_status, 0u, (6u << 16));
  }
  if (warp == 2) {
    ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(s_tmem)), 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  const uint32_t tmem = *s_tmem;
  const uint32_t tDK = tmem, tDV = tmem + 128, tRS = tmem + 256, tRP = tmem + 384;
  const int n_run = fits ? n_it : 0;

  // iteration -> (query head, query tile)
  auto head_of = [&](int it) { return hkv * G + it / per_head; };
  auto tile_of = [&](int it) { return i_start + it % per_head; };

  if (warp < 4) {
    ptx::setmaxnreg_dec<56>();
    if (warp == 0 && lane == 0 && n_run > 0) {
      // ------------------------------------------------------------------ TMA producer
      ptx::prefetch_tmap(&tm_q); ptx::prefetch_tmap(&tm_k); ptx::prefetch_tmap(&tm_v); ptx::prefetch_tmap(&tm_do);
      ptx::mbar_expect_tx(bar(B_KV_FULL), 2 * kBwdTileBytes);
      for (int h = 0; h < 2; ++h) {
        ptx::tma_load_3d(sK + h * kBwdBox, &tm_k, h * 64, kv0, b * Hkv + hkv, bar(B_KV_FULL));
        ptx::tma_load_3d(sV + h * kBwdBox, &tm_v, h * 64, kv0, b * Hkv + hkv, bar(B_KV_FULL));
      }
      bool ok = true;
      for (int it = 0; it < n_run && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (uint32_t)((it >> 1) & 1) ^ 1u;
        const int bh = b * Hq + head_of(it), q0 = tile_of(it) * kBwdTile;
        ok = ptx::mbar_wait(bar(B_Q_EMPTY + st), ph, s_abort);
        if (!ok) break;
        ptx::mbar_expect_tx(bar(B_Q_FULL + st), kBwdQStage);
        for (int h = 0; h < 2; ++h) ptx::tma_load_3d(sQ(st) + h * kBwdBox, &tm_q, h * 64, q0, bh, bar(B_Q_FULL + st));
        bulk_load_1d(sQ(st) + kBwdTileBytes, lse2 + (size_t)bh * Sq_pad + q0, 512, bar(B_Q_FULL + st));
        bulk_load_1d(sQ(st) + kBwdTileBytes + 512, delta + (size_t)bh * Sq_pad + q0, 512, bar(B_Q_FULL + st));
        ok = ptx::mbar_wait(bar(B_DO_EMPTY + st), ph, s_abort);
        if (!ok) break;
        ptx::mbar_expect_tx(bar(B_DO_FULL + st), kBwdTileBytes);
        for (int h = 0; h < 2; ++h) ptx::tma_load_3d(sdO(st) + h * kBwdBox, &tm_do, h * 64, q0, bh, bar(B_DO_FULL + st));
      }
      if (!ok) atomicCAS(&g_dev_status, 0u, (7u << 16));
    } else if (warp == 1 && lane == 0 && n_run > 0) {
      // ------------------------------------------------------------------ MMA issuer
      bool ok = true;
      // k-step offsets: K-major operands step 32 bytes inside a 128-byte row and switch box after 4 steps;
      // MN-major operands step 16 rows (2048 bytes).
      auto koff = [](int kk) -> uint32_t { return (uint32_t)(kk >> 2) * kBwdBox + (uint32_t)(kk & 3) * 32u; };
      auto issue_a = [&](int st) {   // S^T = K Q^T
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(tRS, ptx::desc_sw128_kmajor(sK + koff(kk)), ptx::desc_sw128_kmajor(sQ(st) + koff(kk)), IDESC_KK, kk > 0);
      };
      ok = ptx::mbar_wait(bar(B_KV_FULL), 0, s_abort) && ptx::mbar_wait(bar(B_Q_FULL), 0, s_abort);
      if (ok) {
        ptx::tc_fence_after();
        issue_a(0);
        ptx::mma_commit(bar(B_S_READY));
      }
      for (int it = 0; it < n_run && ok; ++it) {
        const int st = it & 1;
        const uint32_t ph = (uint32_t)it & 1u;
        ok = ptx::mbar_wait(bar(B_DO_FULL + st), (uint32_t)(it >> 1) & 1u, s_abort) &&
             ptx::mbar_wait(bar(B_P_READY), ph, s_abort);
        if (!ok) break;
        ptx::tc_fence_after();
        // (c) dV += P^T dO : P^T columns of query half h sit at R_S + 64h + [0,32)
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ts(tDV, tRS + (kk >> 2) * 64 + (kk & 3) * 8, ptx::desc_sw128_mnmajor(sdO(st) + kk * 2048, kBwdBox),
                      IDESC_KM, (it > 0) || (kk > 0));
        if (it > 0) {
          ok = ptx::mbar_wait(bar(B_RP_FREE), (uint32_t)(it - 1) & 1u, s_abort);
          if (!ok) break;
          ptx::tc_fence_after();
        }
        // (b) dP^T = V dO^T
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(tRP, ptx::desc_sw128_kmajor(sV + koff(kk)), ptx::desc_sw128_kmajor(sdO(st) + koff(kk)), IDESC_KK, kk > 0);
        ptx::mma_commit(bar(B_DP_READY));
        ptx::mma_commit(bar(B_DO_EMPTY + st));
        if (it + 1 < n_run) {
          ok = ptx::mbar_wait(bar(B_Q_FULL + (st ^ 1)), (uint32_t)((it + 1) >> 1) & 1u, s_abort);
          if (!ok) break;
          ptx::tc_fence_after();
          issue_a(st ^ 1);
          ptx::mma_commit(bar(B_S_READY));
        }
        ok = ptx::mbar_wait(bar(B_DS_READY), ph, s_abort);
        if (!ok) break;
        ptx::tc_fence_after();
        // (d) dK += dS^T Q
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(tDK, ptx::desc_sw128_kmajor(sdS + koff(kk)), ptx::desc_sw128_mnmajor(sQ(st) + kk * 2048, kBwdBox),
                      IDESC_KM, (it > 0) || (kk > 0));
        // (e) dQ^T = K^T dS^T
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          ptx::mma_ss(tRP, ptx::desc_sw128_mnmajor(sK + kk * 2048, kBwdBox), ptx::desc_sw128_mnmajor(sdS + kk * 2048, kBwdBox),
                      IDESC_MM, kk > 0);
        ptx::mma_commit(bar(B_DQ_DONE));
        ptx::mma_commit(bar(B_Q_EMPTY + st));
      }
      ptx::mma_commit(bar(B_ACC_DONE));
      if (!ptx::mbar_wait(bar(B_ACC_DONE), 0, s_abort)) ok = false;   // drain before TMEM is released
      if (!ok) atomicCAS(&g_dev_status, 0u, (8u << 16));
    }
  } else {
    ptx::setmaxnreg_inc<224>();
    // -------------------------------------------------------------------- compute warpgroups
    const int h = (warp - 4) >> 2;                 // which 64 query columns of the tile
    const int wq = warp & 3;
    const int r = wq * 32 + lane;                  // TMEM lane: KV row in S^T / dP^T, d index in dQ^T
    const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
    const int kvidx = kv0 + r;
    float p[64];
    bool ok = true;

    // P^T for iteration `it`: exp2(S^T*scale*log2e - lse2[q]), masked, kept in p[] and stored to TMEM
    auto compute_p = [&](int it) -> bool {
      const int st = it & 1;
      bool w = ptx::mbar_wait(bar(B_Q_FULL + st), (uint32_t)(it >> 1) & 1u, s_abort) &&
               ptx::mbar_wait(bar(B_S_READY), (uint32_t)it & 1u, s_abort);
      w = __all_sync(0xffffffffu, w);
      if (!w) return false;
      ptx::tc_fence_after();
      const float* l2 = reinterpret_cast<const float*>(gbase + (sQ(st) - sbase) + kBwdTileBytes) + 64 * h;
      const int q0 = tile_of(it) * kBwdTile + 64 * h;
      // visible iff kvidx <= q + shift  <=>  column c >= kvidx - shift - q0
      const int cmin = causal ? kvidx - shift - q0 : -1;
      uint32_t pk[32];
#pragma unroll
      for (int c2 = 0; c2 < 2; ++c2) {
        uint32_t sr[32];
        ptx::tmem_ld32(tRS + t_lane + 64 * h + 32 * c2, sr);
        ptx::tmem_wait_ld();
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
          const float4 lv = *reinterpret_cast<const float4*>(l2 + 32 * c2 + c);
          const float le[4] = {lv.x, lv.y, lv.z, lv.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int cc = 32 * c2 + c + e;
            float v = ptx::ex2(fmaf(__uint_as_float(sr[c + e]), scale_log2, -le[e]));
            if (cc < cmin) v = 0.f;
            p[cc] = v;
          }
        }
#pragma unroll
        for (int c = 0; c < 32; c += 2) pk[16 * c2 + (c >> 1)] = pack2(p[32 * c2 + c], p[32 * c2 + c + 1], T());
      }
      ptx::tmem_st32(tRS + t_lane + 64 * h, pk);
      ptx::tmem_wait_st();
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(B_P_READY));
      return true;
    };

    if (n_run > 0) ok = compute_p(0);
    for (int it = 0; it < n_run && ok; ++it) {
      const int st = it & 1;
      const uint32_t ph = (uint32_t)it & 1u;
      // ---- dS^T = P^T o (dP^T - Delta) -> shared memory (rows = KV, 64 query columns per 128-byte row)
      ok = ptx::mbar_wait(bar(B_DP_READY), ph, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      {
        const float* dl = reinterpret_cast<const float*>(gbase + (sQ(st) - sbase) + kBwdTileBytes + 512) + 64 * h;
        uint8_t* ds_row = gbase + (sdS - sbase) + h * kBwdBox + r * 128;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t dr[32];
          ptx::tmem_ld32(tRP + t_lane + 64 * h + 32 * c2, dr);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; c += 8) {
            const float4 d0 = *reinterpret_cast<const float4*>(dl + 32 * c2 + c);
            const float4 d1 = *reinterpret_cast<const float4*>(dl + 32 * c2 + c + 4);
            const float de[8] = {d0.x, d0.y, d0.z, d0.w, d1.x, d1.y, d1.z, d1.w};
            float ds[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) ds[e] = p[32 * c2 + c + e] * (__uint_as_float(dr[c + e]) - de[e]);
            uint4 w;
            w.x = pack2(ds[0], ds[1], T()); w.y = pack2(ds[2], ds[3], T());
            w.z = pack2(ds[4], ds[5], T()); w.w = pack2(ds[6], ds[7], T());
            const int chunk = (32 * c2 + c) >> 3;
            *reinterpret_cast<uint4*>(ds_row + ((chunk ^ (r & 7)) << 4)) = w;
          }
        }
      }
      fence_async_smem();          // make the generic-proxy stores visible to the tensor core
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(B_DS_READY));
      // ---- next tile's P^T while the tensor core runs dK and dQ^T of this one
      if (it + 1 < n_run) {
        ok = compute_p(it + 1);
        if (!ok) break;
      }
      // ---- drain dQ^T (lane = d, columns = query rows) into the fp32 accumulator with coalesced reductions
      ok = ptx::mbar_wait(bar(B_DQ_DONE), ph, s_abort);
      ok = __all_sync(0xffffffffu, ok);
      if (!ok) break;
      ptx::tc_fence_after();
      {
        const int q0 = tile_of(it) * kBwdTile + 64 * h;
        float* dst = dq_acc + ((size_t)(b * Hq + head_of(it)) * Sq + q0) * HD + r;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t qr[32];
          ptx::tmem_ld32(tRP + t_lane + 64 * h + 32 * c2, qr);
          ptx::tmem_wait_ld();
#pragma unroll
          for (int c = 0; c < 32; ++c)
            if (q0 + 32 * c2 + c < Sq) red_add(dst + (size_t)(32 * c2 + c) * HD, __uint_as_float(qr[c]));
        }
      }
      ptx::tc_fence_before();
      ptx::mbar_arrive(bar(B_RP_FREE));
    }

    // ------------------------------------------------------------------ epilogue: dK, dV
    if (ok && n_run > 0) {
      ok = ptx::mbar_wait(bar(B_ACC_DONE), 0, s_abort);
      ok = __all_sync(0xffffffffu, ok);
    }
    if (ok && fits) {
      ptx::tc_fence_after();
      const size_t row = ((size_t)b * Hkv + hkv) * Sk + min(kvidx, Sk - 1);
#pragma unroll
      for (int which = 0; which < 2; ++which) {
        T* dst = (which == 0 ? dk : dv) + row * HD + 64 * h;
        const float mul = which == 0 ? scale : 1.f;
#pragma unroll
        for (int c2 = 0; c2 < 2; ++c2) {
          uint32_t ar[32];
          if (n_run > 0) {
            ptx::tmem_ld32((which == 0 ? tDK : tDV) + t_lane + 64 * h + 32 * c2, ar);
            ptx::tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) ar[i] = 0u;
          }
          if (kvidx < Sk) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              uint4 w;
              w.x = pack2(__uint_as_float(ar[i]) * mul, __uint_as_float(ar[i + 1]) * mul, T());
              w.y = pack2(__uint_as_float(ar[i + 2]) * mul, __uint_as_float(ar[i + 3]) * mul, T());
              w.z = pack2(__uint_as_float(ar[i + 4]) * mul, __uint_as_float(ar[i + 5]) * mul, T());
              w.w = pack2(__uint_as_float(ar[i + 6]) * mul, __uint_as_float(ar[i + 7]) * mul, T());
              *reinterpret_cast<uint4*>(dst + 32 * c2 + i) = w;
            }
          }
        }
      }
    } else if (lane == 0) {
      atomicCAS(&g_dev_status, 0u, (9u << 16) | (unsigned)warp);
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
