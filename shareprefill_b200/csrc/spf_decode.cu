// Single-query (decode step) attention over a KV cache: out[h] = softmax(q[h] . K^T * scale) V.
// The reference calls flash_attn_func for this step (attn/shareprefill_attn.py:146-153); here it is a
// bandwidth-bound split-K kernel: grid (token splits, query heads), a warp streams token rows with
// 8-byte coalesced loads (a lane owns head_dim/32 elements), keeps an online softmax per warp, the
// warps of a CTA and then the splits are merged with the usual (max, sum, weighted output) rule.
// Query heads of one KV group sit next to each other in the grid, so their K/V reads share L2.
#include "spf_internal.cuh"

namespace spf {

constexpr int DEC_NT = 256;

template <int PER>   // elements per lane: head_dim / 32 (2 or 4)
__device__ __forceinline__ void load_row(const __nv_bfloat16* p, float (&x)[PER]) {
  if (PER == 4) {
    const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
    x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xffff0000u);
    x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xffff0000u);
  } else {
    const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(p));
    x[0] = __uint_as_float(u << 16); x[1] = __uint_as_float(u & 0xffff0000u);
  }
}

template <int PER>
__global__ void __launch_bounds__(DEC_NT) decode_partial_kernel(const DecodeParams p) {
  constexpr int D = PER * 32;
  __shared__ float sm_m[DEC_NT / 32], sm_l[DEC_NT / 32];
  __shared__ float sm_o[DEC_NT / 32][D];
  const int split = blockIdx.x, h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kvh = h / p.group;
  const int chunk = (p.n_keys + p.splits - 1) / p.splits;
  const int t0 = split * chunk, t1 = min(p.n_keys, t0 + chunk);
  float q[PER];
  load_row<PER>(p.q + int64_t(h) * p.q_sh + lane * PER, q);
#pragma unroll
  for (int e = 0; e < PER; ++e) q[e] *= p.scale_log2;
  const __nv_bfloat16* kb = p.k + int64_t(kvh) * p.k_sh + lane * PER;
  const __nv_bfloat16* vb = p.v + int64_t(kvh) * p.v_sh + lane * PER;
  float m = -INFINITY, l = 0.f, acc[PER];
#pragma unroll
  for (int e = 0; e < PER; ++e) acc[e] = 0.f;
  for (int t = t0 + warp * 4; t < t1; t += (DEC_NT / 32) * 4) {
    float s[4], kx[4][PER], vx[4][PER];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int tt = min(t + u, t1 - 1);
      load_row<PER>(kb + int64_t(tt) * p.k_sn, kx[u]);
      load_row<PER>(vb + int64_t(tt) * p.v_sn, vx[u]);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < PER; ++e) d += q[e] * kx[u][e];
      d = warp_sum(d);
      s[u] = (t + u < t1) ? d : -INFINITY;
    }
    const float mx = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
    const float m_new = fmaxf(m, mx);
    const float alpha = exp2f(m - m_new);
    l *= alpha;
#pragma unroll
    for (int e = 0; e < PER; ++e) acc[e] *= alpha;
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const float pr = exp2f(s[u] - m_new);
      l += pr;
#pragma unroll
      for (int e = 0; e < PER; ++e) acc[e] += pr * vx[u][e];
    }
    m = m_new;
  }
  if (lane == 0) { sm_m[warp] = m; sm_l[warp] = l; }
#pragma unroll
  for (int e = 0; e < PER; ++e) sm_o[warp][lane * PER + e] = acc[e];
  __syncthreads();
  if (threadIdx.x < D) {
    float M = -INFINITY;
    for (int w = 0; w < DEC_NT / 32; ++w) M = fmaxf(M, sm_m[w]);
    float L = 0.f, o = 0.f;
    for (int w = 0; w < DEC_NT / 32; ++w) {
      const float sc = (sm_m[w] == -INFINITY) ? 0.f : exp2f(sm_m[w] - M);
      L += sm_l[w] * sc;
      o += sm_o[w][threadIdx.x] * sc;
    }
    float* dst = p.scratch + (int64_t(h) * p.splits + split) * (D + 2);
    dst[2 + threadIdx.x] = o;
    if (threadIdx.x == 0) { dst[0] = M; dst[1] = L; }
  }
}

template <int PER>
__global__ void decode_merge_kernel(const DecodeParams p) {
  constexpr int D = PER * 32;
  const int h = blockIdx.x, d = threadIdx.x;   // D threads
  const float* src = p.scratch + int64_t(h) * p.splits * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < p.splits; ++s) M = fmaxf(M, src[s * (D + 2)]);
  float L = 0.f, o = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = src[s * (D + 2)];
    const float sc = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    L += src[s * (D + 2) + 1] * sc;
    o += src[s * (D + 2) + 2 + d] * sc;
  }
  p.out[int64_t(h) * D + d] = __float2bfloat16_rn(L > 0.f ? o / L : 0.f);
}

int decode_attention(const DecodeParams& p, int head_dim, cudaStream_t st) {
  const dim3 grid(p.splits, p.n_q_heads);
  if (head_dim == 128) {
    decode_partial_kernel<4><<<grid, DEC_NT, 0, st>>>(p);
    decode_merge_kernel<4><<<p.n_q_heads, 128, 0, st>>>(p);
  } else if (head_dim == 64) {
    decode_partial_kernel<2><<<grid, DEC_NT, 0, st>>>(p);
    decode_merge_kernel<2><<<p.n_q_heads, 64, 0, st>>>(p);
  } else {
    return SPF_ERR_SHAPE;
  }
  return check_launch();
}

}  // namespace spf
