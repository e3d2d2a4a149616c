// Single-query (decode step) attention over a KV cache: out[h] = softmax(q[h] . K^T * scale) V.
// The reference calls flash_attn_func for this step (attn/shareprefill_attn.py:146-153); here it is a
// bandwidth-bound split-K pass followed by a merge of the splits with the usual (max, sum, weighted
// output) rule.  Main kernel (query groups of up to 16 heads per KV head): grid (token splits, KV heads);
// the query heads of the group are the 16 rows of an mma.sync m16n8k16 tile, so every K/V row is read
// from HBM once and costs a handful of instructions; each warp streams its own 16-token tiles through a
// private 3-stage cp.async ring.  Larger groups use a scalar kernel (grid over query heads).
#include "spf_internal.cuh"
#include "spf_mma.cuh"

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

constexpr int DTC_NT = 128, DTC_TT = 16, DTC_STAGES = 3;

template <int D>
constexpr int dtc_smem_bytes() { return (DTC_NT / 32) * DTC_STAGES * 2 * DTC_TT * D * 2; }

template <int D>
__global__ void __launch_bounds__(DTC_NT) decode_partial_tc_kernel(const DecodeParams p) {
  constexpr int TT = DTC_TT, CH = D / 8, TILE_B = TT * D * 2, NW = DTC_NT / 32;
  extern __shared__ __align__(128) uint8_t dsm[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kvh = blockIdx.y, g = p.group;
  const int tiles_total = (p.n_keys + TT - 1) / TT;
  const int tps = (tiles_total + p.splits - 1) / p.splits;
  const int tile0 = split * tps, tile1 = min(tiles_total, tile0 + tps);
  const uint32_t ring = smem_u32(dsm) + warp * (DTC_STAGES * 2 * TILE_B);
  const __nv_bfloat16* kb = p.k + int64_t(kvh) * p.k_sh;
  const __nv_bfloat16* vb = p.v + int64_t(kvh) * p.v_sh;
  const int r0 = lane >> 2, r1 = r0 + 8, cq = (lane & 3) * 2;

  // the group's query rows as A fragments (rows past the group are zero)
  uint32_t qa[D / 16][4];
  {
    const __nv_bfloat16* q0 = p.q + int64_t(kvh * g + r0) * p.q_sh + cq;
    const __nv_bfloat16* q1 = p.q + int64_t(kvh * g + r1) * p.q_sh + cq;
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      qa[ks][0] = r0 < g ? __ldg(reinterpret_cast<const uint32_t*>(q0 + ks * 16)) : 0u;
      qa[ks][1] = r1 < g ? __ldg(reinterpret_cast<const uint32_t*>(q1 + ks * 16)) : 0u;
      qa[ks][2] = r0 < g ? __ldg(reinterpret_cast<const uint32_t*>(q0 + ks * 16 + 8)) : 0u;
      qa[ks][3] = r1 < g ? __ldg(reinterpret_cast<const uint32_t*>(q1 + ks * 16 + 8)) : 0u;
    }
  }

  auto issue = [&](int t, int stage) {
    if (t < tile1) {
      const int valid = min(TT, p.n_keys - t * TT);
      const uint32_t ks = ring + stage * (2 * TILE_B), vs = ks + TILE_B;
#pragma unroll
      for (int i = lane; i < TT * CH; i += 32) {
        const int row = i / CH, ch = i % CH;
        const bool ok = row < valid;
        const int64_t tok = ok ? int64_t(t) * TT + row : 0;
        cp_async16(ks + tile_off<D>(row, ch), kb + tok * p.k_sn + ch * 8, ok);
        cp_async16(vs + tile_off<D>(row, ch), vb + tok * p.v_sn + ch * 8, ok);
      }
    }
    cp_async_commit();
  };

  float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
  float o[D / 8][4];
#pragma unroll
  for (int j = 0; j < D / 8; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;

  const int first = tile0 + warp;
  issue(first, 0);
  issue(first + NW, 1);
  int stage = 0;
  for (int t = first; t < tile1; t += NW) {
    int pre = stage + 2; if (pre >= DTC_STAGES) pre -= DTC_STAGES;
    issue(t + 2 * NW, pre);
    cp_async_wait<2>();
    __syncwarp();
    const uint32_t ks_base = ring + stage * (2 * TILE_B), vs_base = ks_base + TILE_B;
    float s[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t b[4];
      ldmatrix_x4(b, ks_base + tile_off<D>((lane & 7) + ((lane >> 4) << 3), ks * 2 + ((lane >> 3) & 1)));
      mma_bf16_16816(s[0], qa[ks], b[0], b[1]);
      mma_bf16_16816(s[1], qa[ks], b[2], b[3]);
    }
    const int valid = p.n_keys - t * TT;
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = j * 8 + cq + (e & 1);
        s[j][e] = col < valid ? s[j][e] * p.scale_log2 : -INFINITY;
      }
    float x0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
    float x1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
    x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 1)); x0 = fmaxf(x0, __shfl_xor_sync(0xffffffffu, x0, 2));
    x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 1)); x1 = fmaxf(x1, __shfl_xor_sync(0xffffffffu, x1, 2));
    const float n0 = fmaxf(m0, x0), n1 = fmaxf(m1, x1);   // finite: token 0 of a tile is always valid
    const float a0 = exp2f(m0 - n0), a1 = exp2f(m1 - n1);
    m0 = n0; m1 = n1;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      s[j][0] = exp2f(s[j][0] - n0); s[j][1] = exp2f(s[j][1] - n0);
      s[j][2] = exp2f(s[j][2] - n1); s[j][3] = exp2f(s[j][3] - n1);
    }
    l0 = l0 * a0 + (s[0][0] + s[0][1]) + (s[1][0] + s[1][1]);
    l1 = l1 * a1 + (s[0][2] + s[0][3]) + (s[1][2] + s[1][3]);
    uint32_t pa[4] = {pack_bf16(s[0][0], s[0][1]), pack_bf16(s[0][2], s[0][3]),
                      pack_bf16(s[1][0], s[1][1]), pack_bf16(s[1][2], s[1][3])};
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] *= a0; o[j][1] *= a0; o[j][2] *= a1; o[j][3] *= a1; }
#pragma unroll
    for (int jj = 0; jj < D / 16; ++jj) {
      uint32_t b[4];
      ldmatrix_x4_trans(b, vs_base + tile_off<D>((lane & 7) + (((lane >> 3) & 1) << 3), jj * 2 + (lane >> 4)));
      mma_bf16_16816(o[jj * 2], pa, b[0], b[1]);
      mma_bf16_16816(o[jj * 2 + 1], pa, b[2], b[3]);
    }
    __syncwarp();
    if (++stage == DTC_STAGES) stage = 0;
  }
  cp_async_wait<0>();
  l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
  l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
  __syncthreads();

  // merge the warps of the CTA through shared memory (the rings are drained)
  constexpr int WSTRIDE = 16 * D + 32;
  float* wbuf = reinterpret_cast<float*>(dsm) + warp * WSTRIDE;
#pragma unroll
  for (int j = 0; j < D / 8; ++j) {
    *reinterpret_cast<float2*>(wbuf + r0 * D + j * 8 + cq) = make_float2(o[j][0], o[j][1]);
    *reinterpret_cast<float2*>(wbuf + r1 * D + j * 8 + cq) = make_float2(o[j][2], o[j][3]);
  }
  if ((lane & 3) == 0) {
    wbuf[16 * D + r0] = m0; wbuf[16 * D + r1] = m1;
    wbuf[16 * D + 16 + r0] = l0; wbuf[16 * D + 16 + r1] = l1;
  }
  __syncthreads();
  const float* all = reinterpret_cast<const float*>(dsm);
  for (int idx = threadIdx.x; idx < g * D; idx += DTC_NT) {
    const int r = idx / D, d = idx % D;
    float M = -INFINITY;
#pragma unroll
    for (int w = 0; w < NW; ++w) M = fmaxf(M, all[w * WSTRIDE + 16 * D + r]);
    float L = 0.f, acc = 0.f;
#pragma unroll
    for (int w = 0; w < NW; ++w) {
      const float mw = all[w * WSTRIDE + 16 * D + r];
      const float sc = (mw == -INFINITY) ? 0.f : exp2f(mw - M);
      L += all[w * WSTRIDE + 16 * D + 16 + r] * sc;
      acc += all[w * WSTRIDE + r * D + d] * sc;
    }
    float* dst = p.scratch + (int64_t(kvh * g + r) * p.splits + split) * (D + 2);
    dst[2 + d] = acc;
    if (d == 0) { dst[0] = M; dst[1] = L; }
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

template <int D>
static int launch_decode_tc(const DecodeParams& p, cudaStream_t st) {
  constexpr int SMEM = dtc_smem_bytes<D>();
  static_assert(SMEM >= (DTC_NT / 32) * (16 * D + 32) * 4, "warp merge buffers must fit in the rings");
  cudaError_t e = cudaFuncSetAttribute(decode_partial_tc_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  decode_partial_tc_kernel<D><<<dim3(p.splits, p.n_q_heads / p.group), DTC_NT, SMEM, st>>>(p);
  decode_merge_kernel<D / 32><<<p.n_q_heads, D, 0, st>>>(p);
  return check_launch();
}

int decode_attention(const DecodeParams& p, int head_dim, cudaStream_t st) {
  if (p.group <= 16) {
    if (head_dim == 128) return launch_decode_tc<128>(p, st);
    if (head_dim == 64) return launch_decode_tc<64>(p, st);
    return SPF_ERR_SHAPE;
  }
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
