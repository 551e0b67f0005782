// One-tile attention on tcgen05 tensor cores: split-KV decode for wide GQA/MQA groups, and prefill forward for
// head dimensions the two-tile kernel of fwd_sm100.cuh has no tensor memory for (16-bit, tiles of 128 or 256
// columns), and for fp32 tensors, whose operands the tensor cores take as TF32 (tiles of 128 columns).
//
// Decode (PREFILL = false).  With G query heads per KV head the decode step needs G FLOP per KV byte; at G = 64
// that is more than warp-level mma.sync and its ldmatrix traffic sustain (decode_group.cuh becomes compute
// bound), so this kernel puts the group's heads on the M dimension of 128-row tcgen05 MMAs (rows >= G are
// don't-care).  One CTA = (split, kv head, batch); partials (unnormalised O, max, sum) use the layout of
// decode_combine_kernel.  V rows past the sequence end are zeroed in shared memory before PV (stale cache rows
// may hold NaNs).
// Prefill (PREFILL = true).  One CTA = 128 query rows of one (batch, q head); rows are query positions, the
// bottom-right causal mask limits each row to a prefix of the keys, O is normalised and stored with LSE.
//
// Both:  S[buf] = Q K_j^T  (Q and K from shared memory)      O += P_j V_j  (P from TMEM, V from shared memory)
// Warp 0 streams K/V tiles with TMA through a ring (HD = 128: 128-row tiles, 3 stages; HD = 256: 64-row tiles,
// 2 stages), warp 1 owns TMEM and issues the MMAs (S of the next tile is queued before PV of the current one:
// S is double buffered), warps 4-7 run the fp32 online softmax of the prefill kernel, one row per thread.
// TMEM columns: S[0] [0,128) S[1] [128,256) O [256, 256+HD).
#pragma once
#include "fwd_sm100.cuh"

namespace skb {
namespace dtc {

using sm100::Fmt;
using sm100::kBoxBytes;
using sm100::pack2;

constexpr int kThreads = 256;

// The tile shapes follow the bytes per row, HD * sizeof(T): 256 bytes (16-bit HD = 128, fp32 HD = 64): 128-row K/V
// tiles, 3 stages; 512 bytes (16-bit HD = 256, fp32 HD = 128): 64-row tiles, 2 stages.
template <typename T, int HD> struct Cfg {
  static constexpr int kRowBytes = HD * (int)sizeof(T);
  static_assert(kRowBytes == 256 || kRowBytes == 512, "tile rows are 256 or 512 bytes");
  static constexpr int kBoxes = kRowBytes / 128;                // 128-byte (swizzle-width) column boxes per row
  static constexpr int kBoxElems = 128 / (int)sizeof(T);        // elements per box row
  static constexpr int kKvRows = kRowBytes == 256 ? 128 : 64;   // KV rows per tile
  static constexpr int kStages = kRowBytes == 256 ? 3 : 2;
  static constexpr int kQBytes = 128 * kRowBytes;               // Q tile: 128 rows
  static constexpr int kKvBytes = kKvRows * kRowBytes;          // one K or V tile
  static constexpr int kKvBox = kKvRows * 128;                  // one 64-column box of a K/V tile
  static constexpr int kSmemBytes = 1024 + kQBytes + 2 * kStages * kKvBytes + 256;
};

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

// Arguments that differ between the two uses of the kernel.
struct DecodeArgs {            // PREFILL = false
  PagedKv pg;                  // block_table == nullptr: dense cache
  const int32_t* seqlens;      // (B,) or null
  float* part_o;               // (B, Hq, nsplit, D) fp32
  float2* part_ml;             // (B, Hq, nsplit) (max, sum), max in the log2 domain
  int nsplit;
};
template <typename T> struct PrefillArgs {   // PREFILL = true
  T* o;
  Strides o_str;
  float* lse;                  // (B, Hq, Sq); packed batch: (Hq, total_q)
  int Sq, causal;              // packed batch: Sq is only the grid's upper bound
  Varlen vl;                   // cu_q == nullptr: dense batch
};

// Sk: rows of the K/V tensors (decode: cache capacity).  D <= HD (a multiple of 8) is the head dimension in
// memory; the bulk copies zero columns [D, HD).
template <typename T, int HD, bool PREFILL>
__global__ void __launch_bounds__(kThreads, 1)
tile_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
            const __grid_constant__ CUtensorMap tm_v, const DecodeArgs dec, const PrefillArgs<T> pre, int Hq, int Hkv,
            int Sk, int D, float scale_log2) {
  using C = Cfg<T, HD>;
  constexpr bool TF32 = sizeof(T) == 4;         // fp32 operands go through the tensor cores as TF32
  constexpr int KSTEP = 32 / (int)sizeof(T);     // elements of the contraction per MMA instruction (32 bytes)
  constexpr int KV = C::kKvRows, STAGES = C::kStages;
  constexpr uint32_t IDESC_QK = ptx::idesc_f16(Fmt<T>::v, 128, KV, 0, 0);
  constexpr uint32_t IDESC_PV = ptx::idesc_f16(Fmt<T>::v, 128, HD, 0, 1);

  extern __shared__ uint8_t smem_raw[];
  const uint32_t sbase = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* gbase = smem_raw + (sbase - ptx::smem_u32(smem_raw));
  const uint32_t sQ = sbase;
  auto sK = [&](int st) -> uint32_t { return sbase + C::kQBytes + (uint32_t)st * 2u * C::kKvBytes; };
  auto sV = [&](int st) -> uint32_t { return sK(st) + C::kKvBytes; };
  const uint32_t sBar = sbase + C::kQBytes + 2 * STAGES * C::kKvBytes;
  volatile uint32_t* s_tmem = reinterpret_cast<volatile uint32_t*>(gbase + (sBar - sbase) + NUM * 8);
  volatile int* s_abort = reinterpret_cast<volatile int*>(gbase + (sBar - sbase) + NUM * 8 + 8);
  auto bar = [&](int i) -> uint32_t { return sBar + 8u * (uint32_t)i; };

  const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
  const int lane = threadIdx.x & 31;
  const int G = Hq / Hkv;
  const int b = blockIdx.z;
  // decode: the combine kernel behind this one is launched as a programmatic dependent; letting it be scheduled
  // right away costs nothing (its CTAs block on the grid dependency) and hides its launch latency
  if (!PREFILL) asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  // decode: blockIdx = (split, kv head, batch); prefill: (query tile, q head, batch), heaviest tiles first
  const int split = PREFILL ? 0 : blockIdx.x;
  const int hq = PREFILL ? blockIdx.y : 0;
  const int hkv = PREFILL ? hq / G : blockIdx.y;
  const int qtile = PREFILL ? (pre.causal ? gridDim.x - 1 - blockIdx.x : blockIdx.x) : 0;
  const int q0 = qtile * 128;
  // packed batch (prefill only): rows [qoff, qoff+Sq) of q/o and [koff, koff+Sk) of k/v, "batch" 0 of the maps
  int Sq = PREFILL ? pre.Sq : 1, qoff = 0, koff = 0, zb = b;
  if (PREFILL && pre.vl.cu_q != nullptr) {
    qoff = pre.vl.cu_q[b];
    Sq = pre.vl.cu_q[b + 1] - qoff;
    koff = pre.vl.cu_k[b];
    Sk = pre.vl.cu_k[b + 1] - koff;
    zb = 0;
  }
  const int shift = PREFILL ? Sk - Sq : 0;                     // bottom-right causal alignment
  int start, end, len = Sk;
  if (PREFILL) {
    start = 0;
    end = q0 < Sq ? (pre.causal ? max(0, min(Sk, q0 + 128 + shift)) : Sk) : 0;
  } else {
    len = dec.seqlens ? min(max(dec.seqlens[b], 0), Sk) : Sk;
    const int chunk = cdiv(cdiv(len, dec.nsplit), KV) * KV;
    start = split * chunk;
    end = min(len, start + chunk);
  }
  const int nt = end > start ? cdiv(end - start, KV) : 0;

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
    // -------------------------------------------------------------------- TMA producer
    const bool paged = !PREFILL && dec.pg.block_table != nullptr;
    if (lane == 0 && nt > 0) {
      ptx::prefetch_tmap(&tm_q); ptx::prefetch_tmap(&tm_k); ptx::prefetch_tmap(&tm_v);
      ptx::mbar_expect_tx(bar(Q_FULL), C::kQBytes);
      for (int h = 0; h < C::kBoxes; ++h) {
        if (PREFILL)   // rows = query positions of head hq (q as {D, Sq, Hq, B})
          ptx::tma_load_4d(sQ + h * kBoxBytes, &tm_q, h * C::kBoxElems, qoff + q0, hq, zb, bar(Q_FULL));
        else           // rows = query heads of this group (q as {D, Hq, B}); rows >= G: other heads or zero fill
          ptx::tma_load_3d(sQ + h * kBoxBytes, &tm_q, h * C::kBoxElems, hkv * G, b, bar(Q_FULL));
      }
    }
    if (!paged) {
      if (lane == 0 && nt > 0) {
        // dense K/V: one lane, one copy per 64-column box
        bool ok = true;
        for (int j = 0; j < nt && ok; ++j) {
          const int st = j % STAGES;
          const uint32_t ph = (uint32_t)((j / STAGES) & 1) ^ 1u;
          const int row = start + j * KV;
          ok = ptx::mbar_wait(bar(K_EMPTY + st), ph, s_abort);
          if (!ok) break;
          ptx::mbar_expect_tx(bar(K_FULL + st), C::kKvBytes);
          for (int h = 0; h < C::kBoxes; ++h)
            ptx::tma_load_4d(sK(st) + h * C::kKvBox, &tm_k, h * C::kBoxElems, koff + row, hkv, zb, bar(K_FULL + st));
          ok = ptx::mbar_wait(bar(V_EMPTY + st), ph, s_abort);
          if (!ok) break;
          ptx::mbar_expect_tx(bar(V_FULL + st), C::kKvBytes);
          for (int h = 0; h < C::kBoxes; ++h)
            ptx::tma_load_4d(sV(st) + h * C::kKvBox, &tm_v, h * C::kBoxElems, koff + row, hkv, zb, bar(V_FULL + st));
        }
        if (!ok) atomicCAS(&g_dev_status, 0u, (13u << 16));
      }
    } else if (nt > 0) {
      // paged K/V: the whole warp.  Lane i owns sub-tile i (sub_rows rows): it reads that sub-tile's page from the
      // block table and issues its copies, so the lookups and the copy issue run in parallel across lanes.
      // Sub-tiles that start past the end of the sequence re-read the last valid one (their scores are masked and
      // their V rows zeroed), so the table is never read past the sequence's own pages.
      const int sub_rows = dec.pg.sub_rows, nsub = KV / sub_rows;
      const int last_sub = (len - 1) / sub_rows * sub_rows;
      bool ok = true;
      for (int j = 0; j < nt; ++j) {
        const int st = j % STAGES;
        const uint32_t ph = (uint32_t)((j / STAGES) & 1) ^ 1u;
        int page = 0, prow = 0;
        if (lane < nsub) {
          const int lr = min(start + j * KV + lane * sub_rows, last_sub);
          page = dec.pg.block_table[(size_t)b * dec.pg.max_pages + lr / dec.pg.page_size];
          prow = lr % dec.pg.page_size;
        }
        ok = ptx::mbar_wait_warp(bar(K_EMPTY + st), ph, s_abort);
        if (!ok) break;
        if (lane == 0) ptx::mbar_expect_tx(bar(K_FULL + st), C::kKvBytes);
        __syncwarp();
        if (lane < nsub)
          for (int h = 0; h < C::kBoxes; ++h)
            ptx::tma_load_4d(sK(st) + h * C::kKvBox + lane * sub_rows * 128, &tm_k, h * C::kBoxElems, prow, hkv, page, bar(K_FULL + st));
        ok = ptx::mbar_wait_warp(bar(V_EMPTY + st), ph, s_abort);
        if (!ok) break;
        if (lane == 0) ptx::mbar_expect_tx(bar(V_FULL + st), C::kKvBytes);
        __syncwarp();
        if (lane < nsub)
          for (int h = 0; h < C::kBoxes; ++h)
            ptx::tma_load_4d(sV(st) + h * C::kKvBox + lane * sub_rows * 128, &tm_v, h * C::kBoxElems, prow, hkv, page, bar(V_FULL + st));
      }
      if (!ok && lane == 0) atomicCAS(&g_dev_status, 0u, (13u << 16));
    }
  } else if (warp == 1) {
    // -------------------------------------------------------------------- MMA issuer (whole warp, one lane issues)
    const bool leader = ptx::elect_one();
    bool ok = true;
    auto issue_qk = [&](int j) {
      const uint32_t k = sK(j % STAGES);
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < HD / KSTEP; ++kk) {   // K-major: 32 bytes per k-step, next 128-byte box after 4
          const uint32_t in_row = (uint32_t)(kk & 3) * 32u;
          const uint64_t da = ptx::desc_sw128_kmajor(sQ + (uint32_t)(kk >> 2) * kBoxBytes + in_row);
          const uint64_t db = ptx::desc_sw128_kmajor(k + (uint32_t)(kk >> 2) * C::kKvBox + in_row);
          if (TF32) ptx::mma_ss_tf32(tS(j & 1), da, db, IDESC_QK, kk > 0);
          else ptx::mma_ss(tS(j & 1), da, db, IDESC_QK, kk > 0);
        }
        ptx::mma_commit(bar(S_FULL + (j & 1)));
        ptx::mma_commit(bar(K_EMPTY + j % STAGES));
      }
    };
    if (nt > 0) {
      ok = ptx::mbar_wait_warp(bar(Q_FULL), 0, s_abort) && ptx::mbar_wait_warp(bar(K_FULL), 0, s_abort);
      if (ok) { ptx::tc_fence_after(); issue_qk(0); }
    }
    for (int j = 0; j < nt && ok; ++j) {
      const int st = j % STAGES, buf = j & 1;
      if (j + 1 < nt) {
        ok = ptx::mbar_wait_warp(bar(K_FULL + (j + 1) % STAGES), (uint32_t)((j + 1) / STAGES) & 1u, s_abort);
        if (!ok) break;
        ptx::tc_fence_after();
        issue_qk(j + 1);
      }
      ok = ptx::mbar_wait_warp(bar(V_FULL + st), (uint32_t)(j / STAGES) & 1u, s_abort) &&
           ptx::mbar_wait_warp(bar(P_FULL + buf), (uint32_t)(j >> 1) & 1u, s_abort);
      if (!ok) break;
      ptx::tc_fence_after();
      if (leader) {
#pragma unroll
        for (int kk = 0; kk < KV / KSTEP; ++kk) {   // MN-major V: KSTEP rows of 128 bytes per k-step, boxes kKvBox apart;
          // P: KSTEP values = 8 TMEM columns per k-step (two 16-bit values or one TF32 value per column)
          const uint64_t dv = TF32 ? ptx::desc_sw128_atom32_mnmajor(sV(st) + kk * KSTEP * 128, C::kKvBox)
                                   : ptx::desc_sw128_mnmajor(sV(st) + kk * KSTEP * 128, C::kKvBox);
          if (TF32) ptx::mma_ts_tf32(tO, tS(buf) + kk * 8, dv, IDESC_PV, (j > 0) || (kk > 0));
          else ptx::mma_ts(tO, tS(buf) + kk * 8, dv, IDESC_PV, (j > 0) || (kk > 0));
        }
        ptx::mma_commit(bar(V_EMPTY + st));
        ptx::mma_commit(bar(O_READY));
      }
    }
    if (leader) ptx::mma_commit(bar(DRAIN));
    if (!ptx::mbar_wait_warp(bar(DRAIN), 0, s_abort)) ok = false;
    if (!ok && leader) atomicCAS(&g_dev_status, 0u, (14u << 16));
  } else if (warp >= 4) {
    // -------------------------------------------------------------------- softmax: one row per thread
    const int wq = warp & 3;
    const int r = wq * 32 + lane;                  // row of the tile = TMEM lane (decode: head within the group)
    const uint32_t t_lane = (uint32_t)(wq * 32) << 16;
    // prefill: last key this row may see (bottom-right causal alignment); decode rows all see the whole tile
    const int row_limit = PREFILL ? (pre.causal ? min(Sk - 1, q0 + r + shift) : Sk - 1) : 0;
    float m = -INFINITY, l = 0.f;
    bool ok = true;
    for (int j = 0; j < nt; ++j) {
      const int buf = j & 1, st = j % STAGES;
      ok = ptx::mbar_wait_warp(bar(S_FULL + buf), (uint32_t)(j >> 1) & 1u, s_abort);
      if (!ok) break;
      ptx::tc_fence_after();
      uint32_t sr[KV];
#pragma unroll
      for (int c = 0; c < KV / 32; ++c) ptx::tmem_ld32(tS(buf) + t_lane + c * 32, sr + c * 32);
      ptx::tmem_wait_ld();
      // columns [0, valid) of this tile are visible to this row
      const int tile_rows = end - (start + j * KV);                       // rows of the tile inside the sequence
      const int valid = PREFILL ? max(0, min(KV, row_limit - j * KV + 1)) : min(KV, tile_rows);
      if (valid < KV) {
#pragma unroll
        for (int c = 0; c < KV; ++c)
          if (c >= valid) sr[c] = 0xff800000u;     // -inf
      }
      if (!PREFILL && tile_rows < KV) {
        // decode: clear the V rows past the end of the sequence -- stale cache rows may hold NaNs (a prefill tile
        // past the end of K/V is zero-filled by the bulk copy).  Thread r clears row r.
        ok = ptx::mbar_wait_warp(bar(V_FULL + st), (uint32_t)(j / STAGES) & 1u, s_abort);
        if (!ok) break;
        if (r >= tile_rows && r < KV) {
          uint8_t* vrow = gbase + (sV(st) - sbase) + r * 128;
#pragma unroll
          for (int h = 0; h < C::kBoxes; ++h)
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(vrow + h * C::kKvBox + c * 16) = make_uint4(0u, 0u, 0u, 0u);
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      }
      float mx0 = -INFINITY, mx1 = -INFINITY, mx2 = -INFINITY, mx3 = -INFINITY;
#pragma unroll
      for (int c = 0; c < KV; c += 8) {
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
      for (int c = 0; c < KV; c += 8) {
        float x[8], pe[8];
#pragma unroll
        for (int e = 0; e < 8; e += 2)
          ptx::f2_unpack(ptx::f2_fma(ptx::f2_pack(__uint_as_float(sr[c + e]), __uint_as_float(sr[c + e + 1])), sc2, nm2),
                         x[e], x[e + 1]);
#pragma unroll
        for (int e = 0; e < 6; ++e) pe[e] = ptx::ex2(x[e]);
        ptx::exp2_poly2(x[6], x[7], pe[6], pe[7]);
        if constexpr (TF32) {
          // round P to TF32 here (the MMA would truncate it) and sum the rounded values, so that numerator and
          // denominator of the softmax use the same probabilities and the truncation bias (-2^-11) disappears
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            uint32_t rbits;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(rbits) : "f"(pe[e]));
            pe[e] = __uint_as_float(rbits);
          }
        }
        if (valid < KV) {                          // polynomial exponentials of -inf are tiny, not zero
#pragma unroll
          for (int e = 0; e < 8; ++e)
            if (c + e >= valid) pe[e] = 0.f;
        }
        sumA = ptx::f2_add(sumA, ptx::f2_add(ptx::f2_pack(pe[0], pe[1]), ptx::f2_pack(pe[2], pe[3])));
        sumB = ptx::f2_add(sumB, ptx::f2_add(ptx::f2_pack(pe[4], pe[5]), ptx::f2_pack(pe[6], pe[7])));
#pragma unroll
        for (int e = 0; e < 8; e += 2) {
          if constexpr (TF32) {                    // P as fp32 bits, one value per TMEM column (used as TF32)
            sr[c + e] = __float_as_uint(pe[e]);
            sr[c + e + 1] = __float_as_uint(pe[e + 1]);
          } else {                                 // P as 16-bit pairs, two values per TMEM column
            sr[(c + e) >> 1] = pack2(pe[e], pe[e + 1], T());
          }
        }
      }
      {
        float a0, a1, b0, b1;
        ptx::f2_unpack(sumA, a0, a1);
        ptx::f2_unpack(sumB, b0, b1);
        l += (a0 + a1) + (b0 + b1);
      }
#pragma unroll
      for (int c = 0; c < (TF32 ? KV / 32 : KV / 64); ++c) ptx::tmem_st32(tS(buf) + t_lane + c * 32, sr + c * 32);
      if (j > 0 && __any_sync(0xffffffffu, grow_m)) {
        // PV of tile j-1 finished?  (S_FULL of tile j implies PV of tile j-2 finished, so the barrier is at most
        // one phase behind and the parity wait cannot return early.)
        ok = ptx::mbar_wait_warp(bar(O_READY), (uint32_t)(j - 1) & 1u, s_abort);
        if (!ok) break;
        ptx::tc_fence_after();
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
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
    // ------------------------------------------------------------------ results
    // DRAIN completes once, after every MMA of the CTA. O_READY cannot be used here: with S double-buffered
    // this warp may be two tiles ahead of the last finished PV product, and a parity wait on a barrier that is
    // two phases behind returns at once.
    if (ok) ok = ptx::mbar_wait_warp(bar(DRAIN), 0, s_abort);
    if (ok) {
      ptx::tc_fence_after();
      const bool seen = (m != -INFINITY) && l > 0.f;
      if (PREFILL) {
        const int grow = q0 + r;
        const float inv = seen ? 1.f / l : 0.f;
        T* orow = pre.o + pre.o_str.at(zb, hq, qoff + max(0, min(grow, Sq - 1)));
        const size_t lse_base = pre.vl.cu_q != nullptr ? (size_t)hq * pre.vl.total_q + qoff : ((size_t)b * Hq + hq) * Sq;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
          uint32_t orr[32];
          if (nt > 0) {
            ptx::tmem_ld32(tO + t_lane + c * 32, orr);
            ptx::tmem_wait_ld();
          } else {
#pragma unroll
            for (int i = 0; i < 32; ++i) orr[i] = 0u;
          }
          if (grow < Sq) {
#pragma unroll
            for (int i = 0; i < 32; i += 8) {
              if (c * 32 + i >= D) break;
              if constexpr (TF32) {
                *reinterpret_cast<float4*>(orow + c * 32 + i) =
                    make_float4(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv,
                                __uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv);
                if (c * 32 + i + 4 < D)
                  *reinterpret_cast<float4*>(orow + c * 32 + i + 4) =
                      make_float4(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv,
                                  __uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv);
              } else {
                uint4 w;
                w.x = pack2(__uint_as_float(orr[i]) * inv, __uint_as_float(orr[i + 1]) * inv, T());
                w.y = pack2(__uint_as_float(orr[i + 2]) * inv, __uint_as_float(orr[i + 3]) * inv, T());
                w.z = pack2(__uint_as_float(orr[i + 4]) * inv, __uint_as_float(orr[i + 5]) * inv, T());
                w.w = pack2(__uint_as_float(orr[i + 6]) * inv, __uint_as_float(orr[i + 7]) * inv, T());
                *reinterpret_cast<uint4*>(orow + c * 32 + i) = w;
              }
            }
          }
        }
        if (grow < Sq) pre.lse[lse_base + grow] = seen ? (m + log2f(l)) * kLn2 : -INFINITY;
      } else {
        // partial results for the combine kernel
        const size_t pbase = ((size_t)b * Hq + (size_t)hkv * G + min(r, G - 1)) * dec.nsplit + split;
#pragma unroll
        for (int c = 0; c < HD / 32; ++c) {
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
                *reinterpret_cast<uint4*>(dec.part_o + pbase * D + c * 32 + i) =
                    seen ? make_uint4(orr[i], orr[i + 1], orr[i + 2], orr[i + 3]) : make_uint4(0u, 0u, 0u, 0u);
          }
        }
        if (r < G) dec.part_ml[pbase] = seen ? make_float2(m, l) : make_float2(-INFINITY, 0.f);
      }
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
