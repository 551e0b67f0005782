// General attention kernels: fp32 CUDA-core arithmetic, any dtype, any head dim <= 256.
//
// These cover every shape the API accepts (head dims 64/80/96/128/256, ragged sequence
// lengths, S_q != S_k, fp32 inputs) and are the path for shapes the tcgen05 kernels do
// not take.  Tiles live in shared memory as fp32; 256 threads form a 16x16 grid and each
// thread owns a register micro-tile (rows ty*RI+i, columns tx+16*j), so the three GEMM
// forms below are bank-conflict free with a row pitch of DPAD+4 floats.
#pragma once
#include "common.cuh"

namespace skb {
namespace general {

constexpr int kThreads = 256;

// ---- shared-memory tile load: rows [r0, r0+R) of a (S, D) matrix -> fp32 [R][LD], zero filled ----
template <typename T, int DPAD>
__device__ __forceinline__ void load_tile(float* __restrict__ dst, const T* __restrict__ src, int r0, int R,
                                          int S, int D, int tid) {
  constexpr int VE = Vec16<T>::N;
  constexpr int LD = DPAD + 4;
  constexpr int CH = DPAD / VE;
  for (int idx = tid; idx < R * CH; idx += kThreads) {
    const int r = idx / CH, c = (idx % CH) * VE;
    float vals[VE];
    if (r0 + r < S && c < D) {
      load_vec16<T>(src + (size_t)(r0 + r) * D + c, vals);
    } else {
#pragma unroll
      for (int i = 0; i < VE; ++i) vals[i] = 0.f;
    }
#pragma unroll
    for (int i = 0; i < VE; i += 4)
      *reinterpret_cast<float4*>(dst + r * LD + c + i) = make_float4(vals[i], vals[i + 1], vals[i + 2], vals[i + 3]);
  }
}

// acc[i][j] += sum_k A[(ra+i)*lda + k] * B[(tx+16j)*ldb + k],  k in [0, K), K % 4 == 0
template <int RI, int CJ>
__device__ __forceinline__ void gemm_nt(float (&acc)[RI][CJ], const float* __restrict__ A, int lda, int ra,
                                        const float* __restrict__ B, int ldb, int tx, int K) {
  for (int k = 0; k < K; k += 4) {
    float4 a[RI], b[CJ];
#pragma unroll
    for (int i = 0; i < RI; ++i) a[i] = *reinterpret_cast<const float4*>(A + (ra + i) * lda + k);
#pragma unroll
    for (int j = 0; j < CJ; ++j) b[j] = *reinterpret_cast<const float4*>(B + (tx + 16 * j) * ldb + k);
#pragma unroll
    for (int i = 0; i < RI; ++i)
#pragma unroll
      for (int j = 0; j < CJ; ++j)
        acc[i][j] += a[i].x * b[j].x + a[i].y * b[j].y + a[i].z * b[j].z + a[i].w * b[j].w;
  }
}

// acc[i][j] += sum_k A[(ra+i)*lda + k] * B[k*ldb + tx+16j],  k in [0, K)
template <int RI, int CJ>
__device__ __forceinline__ void gemm_nn(float (&acc)[RI][CJ], const float* __restrict__ A, int lda, int ra,
                                        const float* __restrict__ B, int ldb, int tx, int K) {
#pragma unroll 4
  for (int k = 0; k < K; ++k) {
    float a[RI], b[CJ];
#pragma unroll
    for (int i = 0; i < RI; ++i) a[i] = A[(ra + i) * lda + k];
#pragma unroll
    for (int j = 0; j < CJ; ++j) b[j] = B[k * ldb + tx + 16 * j];
#pragma unroll
    for (int i = 0; i < RI; ++i)
#pragma unroll
      for (int j = 0; j < CJ; ++j) acc[i][j] += a[i] * b[j];
  }
}

// acc[i][j] += sum_k A[k*lda + ra+i] * B[k*ldb + tx+16j],  k in [0, K)   (RI == 4, ra % 4 == 0)
template <int CJ>
__device__ __forceinline__ void gemm_tn(float (&acc)[4][CJ], const float* __restrict__ A, int lda, int ra,
                                        const float* __restrict__ B, int ldb, int tx, int K) {
#pragma unroll 2
  for (int k = 0; k < K; ++k) {
    const float4 a4 = *reinterpret_cast<const float4*>(A + k * lda + ra);
    const float a[4] = {a4.x, a4.y, a4.z, a4.w};
    float b[CJ];
#pragma unroll
    for (int j = 0; j < CJ; ++j) b[j] = B[k * ldb + tx + 16 * j];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < CJ; ++j) acc[i][j] += a[i] * b[j];
  }
}

__device__ __forceinline__ float half_warp_max(float x) {
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}
__device__ __forceinline__ float half_warp_sum(float x) {
#pragma unroll
  for (int o = 8; o >= 1; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}

template <int DPAD, int BM, int BN> constexpr size_t fwd_smem_bytes() {
  return sizeof(float) * ((size_t)(BM + 2 * BN) * (DPAD + 4) + (size_t)BM * (BN + 4));
}

// ------------------------------------------------------------------------------------------------
// Forward: one CTA per (BM query rows, q head, batch); online softmax over BN-row KV tiles.
// ------------------------------------------------------------------------------------------------
template <typename T, int DPAD, int BM, int BN>
__global__ void __launch_bounds__(kThreads)
fwd_kernel(const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v, T* __restrict__ o,
           float* __restrict__ lse, int Hq, int Hkv, int Sq, int Sk, int D, int causal, float scale_log2) {
  constexpr int LD = DPAD + 4, LDP = BN + 4, RI = BM / 16, CJ = BN / 16, CD = DPAD / 16;
  extern __shared__ __align__(16) float smem[];
  float* sQ = smem;
  float* sK = sQ + BM * LD;
  float* sV = sK + BN * LD;
  float* sP = sV + BN * LD;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * BM, hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (Hq / Hkv);
  const T* qb = q + ((size_t)b * Hq + hq) * Sq * D;
  const T* kb = k + ((size_t)b * Hkv + hkv) * Sk * D;
  const T* vb = v + ((size_t)b * Hkv + hkv) * Sk * D;
  const int shift = Sk - Sq;
  const int Kd = (D + 3) & ~3;

  load_tile<T, DPAD>(sQ, qb, m0, BM, Sq, D, tid);

  float m_i[RI], l_i[RI], acc[RI][CD];
#pragma unroll
  for (int i = 0; i < RI; ++i) {
    m_i[i] = -INFINITY; l_i[i] = 0.f;
#pragma unroll
    for (int j = 0; j < CD; ++j) acc[i][j] = 0.f;
  }
  int n_end = Sk;
  if (causal) n_end = min(Sk, max(0, m0 + BM + shift));

  for (int n0 = 0; n0 < n_end; n0 += BN) {
    __syncthreads();  // previous tile's sK/sV/sP fully consumed (also covers the sQ load)
    load_tile<T, DPAD>(sK, kb, n0, BN, Sk, D, tid);
    load_tile<T, DPAD>(sV, vb, n0, BN, Sk, D, tid);
    __syncthreads();

    float s[RI][CJ];
#pragma unroll
    for (int i = 0; i < RI; ++i)
#pragma unroll
      for (int j = 0; j < CJ; ++j) s[i][j] = 0.f;
    gemm_nt<RI, CJ>(s, sQ, LD, ty * RI, sK, LD, tx, Kd);

#pragma unroll
    for (int i = 0; i < RI; ++i) {
      const int row = m0 + ty * RI + i;
      float mx = -INFINITY;
#pragma unroll
      for (int j = 0; j < CJ; ++j) {
        const int col = n0 + tx + 16 * j;
        const bool ok = col < Sk && (!causal || col <= row + shift);
        s[i][j] = ok ? s[i][j] * scale_log2 : -INFINITY;
        mx = fmaxf(mx, s[i][j]);
      }
      mx = half_warp_max(mx);
      const float m_new = fmaxf(m_i[i], mx);
      const float m_safe = (m_new == -INFINITY) ? 0.f : m_new;
      const float alpha = exp2f(m_i[i] - m_safe);
      float rs = 0.f;
#pragma unroll
      for (int j = 0; j < CJ; ++j) {
        const float p = exp2f(s[i][j] - m_safe);
        rs += p;
        sP[(ty * RI + i) * LDP + tx + 16 * j] = p;
      }
      rs = half_warp_sum(rs);
      l_i[i] = l_i[i] * alpha + rs;
      m_i[i] = m_new;
#pragma unroll
      for (int j = 0; j < CD; ++j) acc[i][j] *= alpha;
    }
    __syncthreads();
    gemm_nn<RI, CD>(acc, sP, LDP, ty * RI, sV, LD, tx, BN);
  }

#pragma unroll
  for (int i = 0; i < RI; ++i) {
    const int row = m0 + ty * RI + i;
    if (row >= Sq) continue;
    const float inv = l_i[i] > 0.f ? 1.f / l_i[i] : 0.f;
    T* orow = o + (((size_t)b * Hq + hq) * Sq + row) * D;
#pragma unroll
    for (int j = 0; j < CD; ++j) {
      const int c = tx + 16 * j;
      if (c < D) orow[c] = from_f<T>(acc[i][j] * inv);
    }
    if (tx == 0)
      lse[((size_t)b * Hq + hq) * Sq + row] = l_i[i] > 0.f ? (m_i[i] + log2f(l_i[i])) * kLn2 : -INFINITY;
  }
}

// ------------------------------------------------------------------------------------------------
// Backward preprocess: delta[b,h,i] = sum_d dO * O  (fp32).  One warp per row.
// ------------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256)
bwd_delta_kernel(const T* __restrict__ dout, const T* __restrict__ o, float* __restrict__ delta, size_t rows, int D) {
  constexpr int VE = Vec16<T>::N;
  const size_t row = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= rows) return;
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
  if (lane == 0) delta[row] = s;
}

template <int DPAD, int BM, int BN> constexpr size_t bwd_smem_bytes() {
  return sizeof(float) * ((size_t)(2 * BM + 2 * BN) * (DPAD + 4) + (size_t)2 * BM * (BN + 4));
}

// ------------------------------------------------------------------------------------------------
// Backward dQ: one CTA per (BM query rows, q head, batch), loops over KV tiles.
//   P = exp(S*scale - LSE), dP = dO V^T, dS = P*(dP - delta)*scale, dQ = sum dS K
// ------------------------------------------------------------------------------------------------
template <typename T, int DPAD, int BM, int BN>
__global__ void __launch_bounds__(kThreads)
bwd_dq_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
              const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dq,
              int Hq, int Hkv, int Sq, int Sk, int D, int causal, float scale) {
  constexpr int LD = DPAD + 4, LDP = BN + 4, RI = BM / 16, CJ = BN / 16, CD = DPAD / 16;
  extern __shared__ __align__(16) float smem[];
  float* sQ = smem;
  float* sdO = sQ + BM * LD;
  float* sK = sdO + BM * LD;
  float* sV = sK + BN * LD;
  float* sS = sV + BN * LD;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int m0 = blockIdx.x * BM, hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (Hq / Hkv);
  const size_t qoff = ((size_t)b * Hq + hq) * Sq;
  const T* kb = k + ((size_t)b * Hkv + hkv) * Sk * D;
  const T* vb = v + ((size_t)b * Hkv + hkv) * Sk * D;
  const int shift = Sk - Sq;
  const int Kd = (D + 3) & ~3;
  const float scale_log2 = scale * kLog2e;

  load_tile<T, DPAD>(sQ, q + qoff * D, m0, BM, Sq, D, tid);
  load_tile<T, DPAD>(sdO, dout + qoff * D, m0, BM, Sq, D, tid);

  float lse2[RI], dl[RI], acc[RI][CD];
#pragma unroll
  for (int i = 0; i < RI; ++i) {
    const int row = m0 + ty * RI + i;
    lse2[i] = row < Sq ? lse[qoff + row] * kLog2e : 0.f;
    dl[i] = row < Sq ? delta[qoff + row] : 0.f;
#pragma unroll
    for (int j = 0; j < CD; ++j) acc[i][j] = 0.f;
  }
  int n_end = Sk;
  if (causal) n_end = min(Sk, max(0, m0 + BM + shift));

  for (int n0 = 0; n0 < n_end; n0 += BN) {
    __syncthreads();
    load_tile<T, DPAD>(sK, kb, n0, BN, Sk, D, tid);
    load_tile<T, DPAD>(sV, vb, n0, BN, Sk, D, tid);
    __syncthreads();
    float s[RI][CJ], dp[RI][CJ];
#pragma unroll
    for (int i = 0; i < RI; ++i)
#pragma unroll
      for (int j = 0; j < CJ; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
    gemm_nt<RI, CJ>(s, sQ, LD, ty * RI, sK, LD, tx, Kd);
    gemm_nt<RI, CJ>(dp, sdO, LD, ty * RI, sV, LD, tx, Kd);
#pragma unroll
    for (int i = 0; i < RI; ++i) {
      const int row = m0 + ty * RI + i;
#pragma unroll
      for (int j = 0; j < CJ; ++j) {
        const int col = n0 + tx + 16 * j;
        const bool ok = row < Sq && col < Sk && (!causal || col <= row + shift) && lse2[i] != -INFINITY;
        const float p = ok ? exp2f(s[i][j] * scale_log2 - lse2[i]) : 0.f;
        sS[(ty * RI + i) * LDP + tx + 16 * j] = p * (dp[i][j] - dl[i]) * scale;
      }
    }
    __syncthreads();
    gemm_nn<RI, CD>(acc, sS, LDP, ty * RI, sK, LD, tx, BN);
  }
#pragma unroll
  for (int i = 0; i < RI; ++i) {
    const int row = m0 + ty * RI + i;
    if (row >= Sq) continue;
    T* drow = dq + (qoff + row) * D;
#pragma unroll
    for (int j = 0; j < CD; ++j) {
      const int c = tx + 16 * j;
      if (c < D) drow[c] = from_f<T>(acc[i][j]);
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Backward dK/dV: one CTA owns 64 KV rows of one kv head and loops over the query heads of
// its GQA group and over query tiles (single writer, no atomics).
//   dV = sum P^T dO,  dK = sum dS^T Q
// ------------------------------------------------------------------------------------------------
template <typename T, int DPAD, int BM>
__global__ void __launch_bounds__(kThreads)
bwd_dkv_kernel(const T* __restrict__ dout, const T* __restrict__ q, const T* __restrict__ k, const T* __restrict__ v,
               const float* __restrict__ lse, const float* __restrict__ delta, T* __restrict__ dk, T* __restrict__ dv,
               int Hq, int Hkv, int Sq, int Sk, int D, int causal, float scale) {
  constexpr int BN = 64;
  constexpr int LD = DPAD + 4, LDP = BN + 4, RI = BM / 16, CJ = BN / 16, CD = DPAD / 16;
  extern __shared__ __align__(16) float smem[];
  float* sQ = smem;
  float* sdO = sQ + BM * LD;
  float* sK = sdO + BM * LD;
  float* sV = sK + BN * LD;
  float* sP = sV + BN * LD;
  float* sdS = sP + BM * LDP;

  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int n0 = blockIdx.x * BN, hkv = blockIdx.y, b = blockIdx.z;
  const int G = Hq / Hkv;
  const size_t kvoff = ((size_t)b * Hkv + hkv) * Sk;
  const int shift = Sk - Sq;
  const int Kd = (D + 3) & ~3;
  const float scale_log2 = scale * kLog2e;

  load_tile<T, DPAD>(sK, k + kvoff * D, n0, BN, Sk, D, tid);
  load_tile<T, DPAD>(sV, v + kvoff * D, n0, BN, Sk, D, tid);

  float acck[4][CD], accv[4][CD];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < CD; ++j) { acck[i][j] = 0.f; accv[i][j] = 0.f; }

  int m_start = 0;
  if (causal) m_start = (max(0, n0 - shift) / BM) * BM;  // first query row that can see key n0

  for (int g = 0; g < G; ++g) {
    const int hq = hkv * G + g;
    const size_t qoff = ((size_t)b * Hq + hq) * Sq;
    for (int m0 = m_start; m0 < Sq; m0 += BM) {
      __syncthreads();
      load_tile<T, DPAD>(sQ, q + qoff * D, m0, BM, Sq, D, tid);
      load_tile<T, DPAD>(sdO, dout + qoff * D, m0, BM, Sq, D, tid);
      __syncthreads();
      float s[RI][CJ], dp[RI][CJ];
#pragma unroll
      for (int i = 0; i < RI; ++i)
#pragma unroll
        for (int j = 0; j < CJ; ++j) { s[i][j] = 0.f; dp[i][j] = 0.f; }
      gemm_nt<RI, CJ>(s, sQ, LD, ty * RI, sK, LD, tx, Kd);
      gemm_nt<RI, CJ>(dp, sdO, LD, ty * RI, sV, LD, tx, Kd);
#pragma unroll
      for (int i = 0; i < RI; ++i) {
        const int row = m0 + ty * RI + i;
        const float l2 = row < Sq ? lse[qoff + row] * kLog2e : -INFINITY;
        const float dl = row < Sq ? delta[qoff + row] : 0.f;
#pragma unroll
        for (int j = 0; j < CJ; ++j) {
          const int col = n0 + tx + 16 * j;
          const bool ok = row < Sq && col < Sk && (!causal || col <= row + shift) && l2 != -INFINITY;
          const float p = ok ? exp2f(s[i][j] * scale_log2 - l2) : 0.f;
          sP[(ty * RI + i) * LDP + tx + 16 * j] = p;
          sdS[(ty * RI + i) * LDP + tx + 16 * j] = p * (dp[i][j] - dl) * scale;
        }
      }
      __syncthreads();
      gemm_tn<CD>(accv, sP, LDP, ty * 4, sdO, LD, tx, BM);
      gemm_tn<CD>(acck, sdS, LDP, ty * 4, sQ, LD, tx, BM);
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int row = n0 + ty * 4 + i;
    if (row >= Sk) continue;
#pragma unroll
    for (int j = 0; j < CD; ++j) {
      const int c = tx + 16 * j;
      if (c < D) {
        dk[(kvoff + row) * D + c] = from_f<T>(acck[i][j]);
        dv[(kvoff + row) * D + c] = from_f<T>(accv[i][j]);
      }
    }
  }
}

// ------------------------------------------------------------------------------------------------
// Decode, split-KV: one CTA (4 warps) per (split, q head, batch).  A row of D elements is
// spread over LPR lanes with 16-byte loads; each lane group runs its own online softmax and
// the groups are merged through shared memory.  Partials (unnormalised O, max, sum; the max
// in the log2 domain) go to the workspace for the combine kernel.
// ------------------------------------------------------------------------------------------------
constexpr int kDecodeWarps = 4;

template <typename T, int LPR, int NV>
__global__ void __launch_bounds__(kDecodeWarps * 32)
decode_split_kernel(const T* __restrict__ q, const T* __restrict__ kc, const T* __restrict__ vc,
                    const int32_t* __restrict__ seqlens, float* __restrict__ part_o, float2* __restrict__ part_ml,
                    int Hq, int Hkv, int Scap, int D, int nsplit, float scale_log2) {
  constexpr int VE = Vec16<T>::N;
  constexpr int RPW = 32 / LPR;                // rows a warp covers per step
  constexpr int NG = kDecodeWarps * RPW;       // lane groups per CTA
  __shared__ float s_acc[NG][256 + 2];

  const int split = blockIdx.x, hq = blockIdx.y, b = blockIdx.z;
  const int hkv = hq / (Hq / Hkv);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int grp = lane / LPR, gl = lane % LPR;
  int len = seqlens ? min(max(seqlens[b], 0), Scap) : Scap;
  const int chunk = cdiv(cdiv(len, nsplit), 64) * 64;
  const int start = split * chunk;
  const int end = min(len, start + chunk);

  const T* qrow = q + ((size_t)b * Hq + hq) * D;
  const T* kb = kc + ((size_t)b * Hkv + hkv) * Scap * D;
  const T* vb = vc + ((size_t)b * Hkv + hkv) * Scap * D;

  float qv[NV][VE], acc[NV][VE];
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int c = (gl + n * LPR) * VE;
    if (c < D) load_vec16<T>(qrow + c, qv[n]);
#pragma unroll
    for (int i = 0; i < VE; ++i) {
      qv[n][i] = c < D ? qv[n][i] * scale_log2 : 0.f;
      acc[n][i] = 0.f;
    }
  }
  float m = -INFINITY, l = 0.f;

  for (int r0 = start + warp * RPW; r0 < end; r0 += NG) {
    const int r = r0 + grp;
    const bool valid = r < end;
    float kv[NV][VE];
    float s = 0.f;
#pragma unroll
    for (int n = 0; n < NV; ++n) {
      const int c = (gl + n * LPR) * VE;
      if (valid && c < D) {
        load_vec16<T>(kb + (size_t)r * D + c, kv[n]);
#pragma unroll
        for (int i = 0; i < VE; ++i) s += qv[n][i] * kv[n][i];
      }
    }
#pragma unroll
    for (int off = LPR / 2; off >= 1; off >>= 1) s += __shfl_xor_sync(0xffffffffu, s, off);
    if (valid) {
      const float m_new = fmaxf(m, s);
      const float alpha = exp2f(m - m_new);
      const float p = exp2f(s - m_new);
      l = l * alpha + p;
      m = m_new;
#pragma unroll
      for (int n = 0; n < NV; ++n) {
        const int c = (gl + n * LPR) * VE;
        if (c < D) {
          load_vec16<T>(vb + (size_t)r * D + c, kv[n]);
#pragma unroll
          for (int i = 0; i < VE; ++i) acc[n][i] = acc[n][i] * alpha + p * kv[n][i];
        }
      }
    }
  }

  const int g = warp * RPW + grp;
#pragma unroll
  for (int n = 0; n < NV; ++n) {
    const int c = (gl + n * LPR) * VE;
    if (c < D) {
#pragma unroll
      for (int i = 0; i < VE; ++i) s_acc[g][c + i] = acc[n][i];
    }
  }
  if (gl == 0) { s_acc[g][256] = m; s_acc[g][257] = l; }
  __syncthreads();

  float M = -INFINITY;
#pragma unroll
  for (int i = 0; i < NG; ++i) M = fmaxf(M, s_acc[i][256]);
  const size_t pbase = ((size_t)b * Hq + hq) * nsplit + split;
  for (int d = threadIdx.x; d < D; d += kDecodeWarps * 32) {
    float sum = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int i = 0; i < NG; ++i) sum += s_acc[i][d] * exp2f(s_acc[i][256] - M);
    }
    part_o[pbase * D + d] = sum;
  }
  if (threadIdx.x == 0) {
    float L = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int i = 0; i < NG; ++i) L += s_acc[i][257] * exp2f(s_acc[i][256] - M);
    }
    part_ml[pbase] = make_float2(M, L);
  }
}

// ------------------------------------------------------------------------------------------------
// Decode combine: one CTA per (batch, q head).  Warp 0 merges the per-split (max, sum) pairs
// with shuffles, then every thread rescales and sums its output columns.  Also emits LSE.
// ------------------------------------------------------------------------------------------------
constexpr int kMaxSplits = 256;

template <typename T>
__global__ void __launch_bounds__(128)
decode_combine_kernel(const float* __restrict__ part_o, const float2* __restrict__ part_ml, T* __restrict__ o,
                      const Strides o_str, float* __restrict__ lse, int Hq, int D, int nsplit) {
  __shared__ float s_w[kMaxSplits];
  __shared__ float s_ML[2];
  const size_t bh = blockIdx.x;
  const float2* ml = part_ml + bh * nsplit;
  // Launched with programmatic stream serialization: this grid may start while the split kernel is still
  // draining, so that its launch latency is hidden; nothing the split kernel wrote may be read before this wait
  // (it returns once the whole previous grid has finished and its writes are visible).
  asm volatile("griddepcontrol.wait;" ::: "memory");
  if (threadIdx.x < 32) {
    float M = -INFINITY;
    for (int s = threadIdx.x; s < nsplit; s += 32) M = fmaxf(M, ml[s].x);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    float L = 0.f;
    for (int s = threadIdx.x; s < nsplit; s += 32) {
      const float2 x = ml[s];
      const float w = (x.x == -INFINITY) ? 0.f : exp2f(x.x - M);
      s_w[s] = w;
      L += x.y * w;
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    if (threadIdx.x == 0) { s_ML[0] = M; s_ML[1] = L; }
  }
  __syncthreads();
  const float M = s_ML[0], L = s_ML[1];
  const float inv = L > 0.f ? 1.f / L : 0.f;
  T* orow = o + o_str.at((int)(bh / Hq), (int)(bh % Hq), 0);
  for (int d = threadIdx.x; d < D; d += 128) {
    float sum = 0.f;
    for (int s = 0; s < nsplit; ++s) sum += part_o[(bh * nsplit + s) * D + d] * s_w[s];
    orow[d] = from_f<T>(sum * inv);
  }
  if (lse != nullptr && threadIdx.x == 0) lse[bh] = L > 0.f ? (M + log2f(L)) * kLn2 : -INFINITY;
}

}  // namespace general
}  // namespace skb
