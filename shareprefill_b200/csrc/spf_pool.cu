// Block mean pooling of Q and K over tokens: one streaming pass, HBM bound.
//
// A thread owns one 16-byte column chunk (8 bf16 of one head) of the token-major tensor and
// walks the block's tokens, so consecutive threads read consecutive addresses of a token row
// (128-bit coalesced loads) and no cross-thread reduction is needed; eight independent loads
// are kept in flight per thread.  Sums are fp32, rounded to bf16 once.
//
// K follows bnhd_pool_kernel (attn/utils.py:171-187): sum / true block length.
// Q follows attn/attention_sharing.py:350-356: zero padded mean over block_size, and for a
// partial last block the bf16 result is multiplied by block_size and divided by the true
// length, each step rounded to bf16 as torch's bf16 arithmetic does.
#include "spf_internal.cuh"

namespace spf {



constexpr int POOL_NT = 128;
constexpr int POOL_UNROLL = 8;

// bf16 -> fp32 is a 16-bit shift; keeps the 128-bit word in registers
__device__ __forceinline__ void accumulate(float (&acc)[8], const uint4 v) {
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    acc[2 * e] += __uint_as_float(w[e] << 16);
    acc[2 * e + 1] += __uint_as_float(w[e] & 0xffff0000u);
  }
}

__global__ void __launch_bounds__(POOL_NT) pool_blocks_kernel(const PoolParams p) {
  int cy = blockIdx.y;
  const int which = (cy < p.t[0].cta_cols) ? 0 : 1;
  if (which == 1) cy -= p.t[0].cta_cols;
  PoolTensor t;   // field-wise select: indexing the parameter block dynamically would spill it
  t.x = which ? p.t[1].x : p.t[0].x;
  t.sn = which ? p.t[1].sn : p.t[0].sn;
  t.sh = which ? p.t[1].sh : p.t[0].sh;
  t.out = which ? p.t[1].out : p.t[0].out;
  t.heads = which ? p.t[1].heads : p.t[0].heads;
  t.q_style = which ? p.t[1].q_style : p.t[0].q_style;
  const int chunks_per_head = p.head_dim >> 3;
  const int col = cy * POOL_NT + threadIdx.x;
  if (col >= t.heads * chunks_per_head) return;
  const int h = col / chunks_per_head, ch = col % chunks_per_head;
  const int blk = blockIdx.x;
  const int n0 = blk * p.block_size;
  const int cnt = min(p.block_size, p.n_tokens - n0);
  const __nv_bfloat16* src = t.x + int64_t(n0) * t.sn + int64_t(h) * t.sh + ch * 8;

  float acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;
  int i = 0;
  for (; i + POOL_UNROLL <= cnt; i += POOL_UNROLL) {
    uint4 v[POOL_UNROLL];
#pragma unroll
    for (int u = 0; u < POOL_UNROLL; ++u)
      v[u] = __ldg(reinterpret_cast<const uint4*>(src + int64_t(i + u) * t.sn));
#pragma unroll
    for (int u = 0; u < POOL_UNROLL; ++u) accumulate(acc, v[u]);
  }
  for (; i < cnt; ++i) accumulate(acc, __ldg(reinterpret_cast<const uint4*>(src + int64_t(i) * t.sn)));

  uint32_t ow[4];
  const float bs = static_cast<float>(p.block_size), fc = static_cast<float>(cnt);
#pragma unroll
  for (int e = 0; e < 4; ++e) {
    float a = acc[2 * e], b = acc[2 * e + 1];
    if (t.q_style) {
      a = bf16_round(a / bs);
      b = bf16_round(b / bs);
      if (cnt != p.block_size) {
        a = bf16_round(bf16_round(a * bs) / fc);
        b = bf16_round(bf16_round(b * bs) / fc);
      }
    } else {
      a = a / fc;
      b = b / fc;
    }
    const __nv_bfloat162 pk = __floats2bfloat162_rn(a, b);
    ow[e] = (static_cast<uint32_t>(__bfloat16_as_ushort(pk.y)) << 16) | __bfloat16_as_ushort(pk.x);
  }
  const uint4 o = make_uint4(ow[0], ow[1], ow[2], ow[3]);
  *reinterpret_cast<uint4*>(t.out + (int64_t(blk) * t.heads + h) * p.head_dim + ch * 8) = o;
}

int pool_blocks(const PoolParams& p, int nb, cudaStream_t st) {
  const int cta_cols = p.t[0].cta_cols + p.t[1].cta_cols;
  if (cta_cols == 0) return SPF_OK;
  pool_blocks_kernel<<<dim3(nb, cta_cols), POOL_NT, 0, st>>>(p);
  return check_launch();
}

}  // namespace spf
