// Shared device/host helpers for the sparse-prefill kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "spf_b200.h"

#ifndef __CUDA_ARCH__
#define SPF_HOST_ONLY 1
#endif

namespace spf {

// ---- launch error bookkeeping (per host thread)
void note_cuda_error(cudaError_t e);
inline int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    note_cuda_error(e);
    return SPF_ERR_LAUNCH;
  }
  return SPF_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline bool supported_head_dim(int d) { return d == 64 || d == 128; }
inline bool supported_block_size(int b) { return b == 16 || b == 32 || b == 64 || b == 128; }
inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

// ---- sharing-state layout (device memory owned by the caller)
struct StateView {
  int32_t* pivot_head;     // [S]  global head index of the cluster's pivot, -1 = none yet
  int32_t* pivot_layer;    // [S]
  int32_t* pattern_ready;  // [S]  1 once the pivot's pattern has been built
  float* vs_ratio;         // [S]  NaN = not computed yet
  int32_t* pivot_nv;       // [S]  length of pivot_vlist
  int32_t* pivot_ns;       // [S]
  float* pivot_vertical;   // [S][nb] pooled vertical profile of the pivot
  float* pivot_slash;      // [S][nb]
  int32_t* pivot_vlist;    // [S][nb] the pivot's own vertical column blocks
  int32_t* pivot_slist;    // [S][nb] the pivot's own slash block distances
  uint32_t* pattern;       // [S][nb][nbw]
  float* pivot_attn;       // [S][nb][nb] block-mass matrix of the pivot
};

__host__ __device__ inline int64_t align256(int64_t x) { return (x + 255) & ~int64_t(255); }

__host__ __device__ inline void state_offsets(int S, int nb, int64_t* off /*[13]*/) {
  const int64_t nbw = (nb + 31) / 32;
  int64_t o = 0;
  off[0] = o; o = align256(o + int64_t(S) * 4);
  off[1] = o; o = align256(o + int64_t(S) * 4);
  off[2] = o; o = align256(o + int64_t(S) * 4);
  off[3] = o; o = align256(o + int64_t(S) * 4);
  off[4] = o; o = align256(o + int64_t(S) * 4);
  off[5] = o; o = align256(o + int64_t(S) * 4);
  off[6] = o; o = align256(o + int64_t(S) * nb * 4);
  off[7] = o; o = align256(o + int64_t(S) * nb * 4);
  off[8] = o; o = align256(o + int64_t(S) * nb * 4);
  off[9] = o; o = align256(o + int64_t(S) * nb * 4);
  off[10] = o; o = align256(o + int64_t(S) * nb * nbw * 4);
  off[11] = o; o = align256(o + int64_t(S) * nb * nb * 4);
  off[12] = o;  // total bytes
}

__host__ __device__ inline StateView state_view(void* base, int S, int nb) {
  int64_t off[13];
  state_offsets(S, nb, off);
  char* b = static_cast<char*>(base);
  StateView v;
  v.pivot_head = reinterpret_cast<int32_t*>(b + off[0]);
  v.pivot_layer = reinterpret_cast<int32_t*>(b + off[1]);
  v.pattern_ready = reinterpret_cast<int32_t*>(b + off[2]);
  v.vs_ratio = reinterpret_cast<float*>(b + off[3]);
  v.pivot_nv = reinterpret_cast<int32_t*>(b + off[4]);
  v.pivot_ns = reinterpret_cast<int32_t*>(b + off[5]);
  v.pivot_vertical = reinterpret_cast<float*>(b + off[6]);
  v.pivot_slash = reinterpret_cast<float*>(b + off[7]);
  v.pivot_vlist = reinterpret_cast<int32_t*>(b + off[8]);
  v.pivot_slist = reinterpret_cast<int32_t*>(b + off[9]);
  v.pattern = reinterpret_cast<uint32_t*>(b + off[10]);
  v.pivot_attn = reinterpret_cast<float*>(b + off[11]);
  return v;
}

#ifdef __CUDACC__
// ---- small device helpers
__device__ __forceinline__ float bf16_round(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Block-wide sum in double, deterministic (fixed tree).  `red` holds >= 32 doubles of shared
// memory; every thread of the block must call it.  Result is returned to all threads.
__device__ __forceinline__ double block_sum(double v, double* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  double t = (threadIdx.x < nw) ? red[threadIdx.x] : 0.0;
  if (w == 0) {
    t = warp_sum(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  return t;
}

__device__ __forceinline__ float block_max(float v, float* red) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) red[w] = v;
  __syncthreads();
  float t = (threadIdx.x < nw) ? red[threadIdx.x] : -INFINITY;
  if (w == 0) {
    t = warp_max(t);
    if (lane == 0) red[0] = t;
  }
  __syncthreads();
  t = red[0];
  return t;
}
#endif  // __CUDACC__

}  // namespace spf
