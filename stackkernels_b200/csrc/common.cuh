// Shared device helpers for the skb200 attention kernels.
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "skb200.h"

namespace skb {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;

__host__ __device__ constexpr int cdiv(int a, int b) { return (a + b - 1) / b; }

template <typename T> struct DtypeOf;
template <> struct DtypeOf<float> { static constexpr int value = SKB_F32; };
template <> struct DtypeOf<__half> { static constexpr int value = SKB_F16; };
template <> struct DtypeOf<__nv_bfloat16> { static constexpr int value = SKB_BF16; };

__device__ __forceinline__ float to_f(float x) { return x; }
__device__ __forceinline__ float to_f(__half x) { return __half2float(x); }
__device__ __forceinline__ float to_f(__nv_bfloat16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

// Number of elements in one 16-byte vector of T.
// Element strides of the (batch, head, sequence) dimensions of a 4-D tensor whose last dimension is contiguous.
struct Strides {
  long long b, h, s;
  __host__ __device__ size_t at(int ib, int ih, long long is) const {
    return (size_t)((long long)ib * b + (long long)ih * h + is * s);
  }
};
inline Strides contiguous_strides(int H, int S, int D) {
  return Strides{(long long)H * S * D, (long long)S * D, (long long)D};
}

// Paged KV cache: logical row r of sequence b lives in page block_table[b * max_pages + r / page_size] at row
// r % page_size.  block_table == nullptr means a dense cache (page = batch index, row = r).  sub_rows is the
// number of rows one bulk copy fetches: min(page_size, rows of a kernel tile).
struct PagedKv {
  const int32_t* block_table;
  int max_pages, page_size, sub_rows;
};

// Packed variable-length batch: sequence b owns rows [cu_q[b], cu_q[b+1]) of the (total_q, H, D) query-side
// tensors and rows [cu_k[b], cu_k[b+1]) of K and V.  cu_q == nullptr means a dense (B, H, S, D) batch.
// Per-row fp32 statistics of the backward pass are kept per head in a padded row space of total_pad rows in
// which sequence b starts at varlen_pad_off(cu_q[b], b): a multiple of 128, computable without a prefix sum,
// and far enough from its neighbours (floor(a+b) >= floor(a) + floor(b), plus 128 rows per sequence) that every
// sequence has room for its length rounded up to 128.
struct Varlen {
  const int32_t* cu_q;
  const int32_t* cu_k;
  int total_q, total_pad;
};
__host__ __device__ inline int varlen_pad_off(int cu, int b) { return (cu & ~127) + 128 * b; }
inline int varlen_total_pad(int total_q, int B) { return ((total_q + 127) & ~127) + 128 * (B + 1); }

template <typename T> struct Vec16 { static constexpr int N = 16 / sizeof(T); };

// Widen the Vec16<T>::N elements of a 16-byte vector to fp32.
template <typename T>
__device__ __forceinline__ void unpack_vec16(const uint4& raw, float* out) {
  if constexpr (sizeof(T) == 4) {
    out[0] = __uint_as_float(raw.x); out[1] = __uint_as_float(raw.y);
    out[2] = __uint_as_float(raw.z); out[3] = __uint_as_float(raw.w);
  } else {
    const T* e = reinterpret_cast<const T*>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) out[i] = to_f(e[i]);
  }
}

// Load 16 bytes (Vec16<T>::N elements) from global memory and widen to fp32.
template <typename T>
__device__ __forceinline__ void load_vec16(const T* __restrict__ p, float* out) {
  const uint4 raw = __ldg(reinterpret_cast<const uint4*>(p));
  unpack_vec16<T>(raw, out);
}

}  // namespace skb
