// Generic block-sparse causal flash attention (mma.sync path).
//
// One CTA owns one (head, query block) pair and walks the set bits of that head's bitmap
// row in ascending key-block order: K/V tiles arrive through a two-stage cp.async pipeline
// into swizzled shared memory, S = Q K^T and O += P V run on mma.sync.m16n8k16, the online
// softmax works in base 2 with scale*log2(e) folded into the scores, P is rounded to bf16
// before P V and the output is bf16 - the arithmetic of block_wise_prefill_attention_kernel
// (attn/shareprefill_attn.py:381-471).  The causal mask is applied on the diagonal block only
// (it is a no-op elsewhere).  Pivot heads run a second sweep over K that writes, per visited
// block, the block's share of the softmax mass averaged over the valid queries
// (attn/shareprefill_attn.py:425-457).
//
// This kernel covers every supported (block_size, head_dim); the tcgen05 kernel takes over
// for block_size = head_dim = 128.
#include "spf_internal.cuh"
#include "spf_mma.cuh"

namespace spf {


// Iterates the set bits of one bitmap row (columns <= row), ascending.
struct RowWalker {
  const uint32_t* words;
  int nwords;   // words that can hold a column <= row
  int row;
  int w;
  uint32_t cur;
  __device__ void init(const uint32_t* row_words, int row_) {
    words = row_words; row = row_; nwords = (row_ >> 5) + 1; w = 0;
    cur = mask(0, __ldg(words));
  }
  __device__ uint32_t mask(int wi, uint32_t x) const {
    const int last = row - (wi << 5);          // highest admissible bit in this word
    return last >= 31 ? x : (x & ((2u << last) - 1u));
  }
  // next column or -1
  __device__ int next() {
    while (cur == 0u) {
      if (++w >= nwords) return -1;
      cur = mask(w, __ldg(words + w));
    }
    const int b = __ffs(cur) - 1;
    cur &= cur - 1u;
    return (w << 5) + b;
  }
};

template <int BS, int D>
__global__ void __launch_bounds__(BS * 2) sparse_attn_generic_kernel(const AttnParams p) {
  constexpr int NW = BS / 16;          // warps; each owns 16 query rows
  constexpr int NT = NW * 32;
  constexpr int KSTEPS = D / 16;       // k-steps of QK^T
  constexpr int NTILES_S = BS / 8;     // n-tiles of S (key columns)
  constexpr int NTILES_O = D / 8;      // n-tiles of O
  constexpr int TILE_BYTES = BS * D * 2;

  extern __shared__ __align__(128) unsigned char smem[];
  // [0] K stage 0, [1] V stage 0, [2] K stage 1, [3] V stage 1; Q is staged in [2] first
  const uint32_t sbase = smem_u32(smem);
  __shared__ float red_sum[NW];

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // heavy (late) query blocks first
  int r, h;
  if (!p.pivot_only) {
    r = p.nb - 1 - static_cast<int>(blockIdx.x / p.n_q_heads);
    h = static_cast<int>(blockIdx.x % p.n_q_heads);
  } else {
    // pivot-only pass: one CTA per (query block, shared cluster); the cluster's pivot of this layer,
    // if any, is the head flagged PIVOT whose slot matches
    r = p.nb - 1 - static_cast<int>(blockIdx.x / p.n_slots);
    const int slot = static_cast<int>(blockIdx.x % p.n_slots);
    h = -1;
    for (int i = 0; i < p.n_q_heads; ++i)
      if ((p.head_flags[i] & SPF_HEAD_PIVOT) && p.slot_of_head[i] == slot) { h = i; break; }
    if (h < 0) return;
  }
  const bool is_pivot = p.head_flags != nullptr && p.pivot_attn != nullptr &&
                        (p.head_flags[h] & SPF_HEAD_PIVOT) && p.slot_of_head[h] >= 0;
  if (p.pivot_only && !is_pivot) return;
  const int kvh = h / p.group;
  const int row0 = r * BS;
  const int rows_valid = min(BS, p.n_tokens - row0);

  const __nv_bfloat16* qg = p.q + int64_t(row0) * p.q_sn + int64_t(h) * p.q_sh;
  const __nv_bfloat16* kg = p.k + int64_t(kvh) * p.k_sh;
  const __nv_bfloat16* vg = p.v + int64_t(kvh) * p.v_sh;
  const uint32_t* brow = p.bitmap + (int64_t(h) * p.nb + r) * p.nbw;

  // ---- Q fragments to registers
  load_tile_async<BS, D, NT>(sbase + 2 * TILE_BYTES, qg, p.q_sn, rows_valid, tid);
  cp_async_commit();
  cp_async_wait<0>();
  __syncthreads();
  uint32_t qf[KSTEPS][4];
  {
    const int qrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks)
      ldmatrix_x4(qf[ks], sbase + 2 * TILE_BYTES + tile_off<D>(qrow, ks * 2 + (lane >> 4)));
  }
  __syncthreads();

  float o_acc[NTILES_O][4];
#pragma unroll
  for (int i = 0; i < NTILES_O; ++i) { o_acc[i][0] = o_acc[i][1] = o_acc[i][2] = o_acc[i][3] = 0.f; }
  float m_run[2] = {-INFINITY, -INFINITY};
  float l_run[2] = {0.f, 0.f};
  const int qpos0 = row0 + warp * 16 + (lane >> 2);  // token index of this thread's first row

  auto issue_kv = [&](int col, int stage, bool with_v) {
    const int c0 = col * BS;
    const int valid = min(BS, p.n_tokens - c0);
    load_tile_async<BS, D, NT>(sbase + (stage * 2) * TILE_BYTES, kg + int64_t(c0) * p.k_sn, p.k_sn,
                               valid, tid);
    if (with_v)
      load_tile_async<BS, D, NT>(sbase + (stage * 2 + 1) * TILE_BYTES, vg + int64_t(c0) * p.v_sn,
                                 p.v_sn, valid, tid);
  };

  // S = Q K^T * scale for the K tile in `stage`; causal mask when `diag`
  auto compute_s = [&](float (&s)[NTILES_S][4], int stage, bool diag, int c0) {
#pragma unroll
    for (int j = 0; j < NTILES_S; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
    const uint32_t kb = sbase + (stage * 2) * TILE_BYTES;
#pragma unroll
    for (int ks = 0; ks < KSTEPS; ++ks) {
#pragma unroll
      for (int jp = 0; jp < NTILES_S / 2; ++jp) {
        uint32_t bf[4];
        const int krow = jp * 16 + (lane & 7) + (lane >> 4) * 8;
        ldmatrix_x4(bf, kb + tile_off<D>(krow, ks * 2 + ((lane >> 3) & 1)));
        mma_bf16_16816(s[2 * jp], qf[ks], bf[0], bf[1]);
        mma_bf16_16816(s[2 * jp + 1], qf[ks], bf[2], bf[3]);
      }
    }
#pragma unroll
    for (int j = 0; j < NTILES_S; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float x = s[j][e] * p.scale_log2;
        if (diag) {
          const int kpos = c0 + j * 8 + (lane & 3) * 2 + (e & 1);
          const int qpos = qpos0 + (e >> 1) * 8;
          if (kpos > qpos) x = -INFINITY;
        }
        s[j][e] = x;
      }
    }
  };

  // the pivot-only pass needs the row statistics (running maximum and sum) of this sweep, not its
  // output: V is not loaded and P V is not computed there
  const bool with_v = !p.pivot_only;
  RowWalker walk;
  walk.init(brow, r);
  int col = walk.next();
  int stage = 0;
  if (col >= 0) issue_kv(col, 0, with_v);
  cp_async_commit();

  while (col >= 0) {
    const int nxt = walk.next();
    if (nxt >= 0) issue_kv(nxt, stage ^ 1, with_v);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();

    float s[NTILES_S][4];
    compute_s(s, stage, col == r, col * BS);

    // online softmax (two rows per thread: lane/4 and lane/4 + 8)
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < NTILES_S; ++j) {
      mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
    float alpha[2], msafe[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
      const float m_new = fmaxf(m_run[i], mx[i]);
      msafe[i] = (m_new == -INFINITY) ? 0.f : m_new;
      alpha[i] = exp2f(m_run[i] - msafe[i]);
      m_run[i] = m_new;
    }
    float rs[2] = {0.f, 0.f};
    uint32_t pf[NTILES_S / 2][4];
#pragma unroll
    for (int j = 0; j < NTILES_S; ++j) {
      const float p0 = exp2f(s[j][0] - msafe[0]);
      const float p1 = exp2f(s[j][1] - msafe[0]);
      const float p2 = exp2f(s[j][2] - msafe[1]);
      const float p3 = exp2f(s[j][3] - msafe[1]);
      rs[0] += p0 + p1;
      rs[1] += p2 + p3;
      pf[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      pf[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 1);
      rs[i] += __shfl_xor_sync(0xffffffffu, rs[i], 2);
      l_run[i] = l_run[i] * alpha[i] + rs[i];
    }
    if (with_v) {
#pragma unroll
      for (int i = 0; i < NTILES_O; ++i) {
        o_acc[i][0] *= alpha[0]; o_acc[i][1] *= alpha[0];
        o_acc[i][2] *= alpha[1]; o_acc[i][3] *= alpha[1];
      }
      // O += P V
      const uint32_t vb = sbase + (stage * 2 + 1) * TILE_BYTES;
#pragma unroll
      for (int kk = 0; kk < BS / 16; ++kk) {
#pragma unroll
        for (int ip = 0; ip < NTILES_O / 2; ++ip) {
          uint32_t bf[4];
          const int vrow = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
          ldmatrix_x4_trans(bf, vb + tile_off<D>(vrow, ip * 2 + (lane >> 4)));
          mma_bf16_16816(o_acc[2 * ip], pf[kk], bf[0], bf[1]);
          mma_bf16_16816(o_acc[2 * ip + 1], pf[kk], bf[2], bf[3]);
        }
      }
    }
    __syncthreads();  // everyone is done with `stage` before it is refilled
    col = nxt;
    stage ^= 1;
  }
  cp_async_wait<0>();

  // ---- epilogue: O / l, bf16, [N][H][D]
  float inv_l[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) inv_l[i] = l_run[i] > 0.f ? 1.f / l_run[i] : 0.f;
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int tok = qpos0 + i * 8;
    if (tok < p.n_tokens && !p.pivot_only) {
      __nv_bfloat16* orow = p.out + (int64_t(tok) * p.n_q_heads + h) * D + (lane & 3) * 2;
#pragma unroll
      for (int t = 0; t < NTILES_O; ++t) {
        *reinterpret_cast<uint32_t*>(orow + t * 8) =
            pack_bf16(o_acc[t][i * 2] * inv_l[i], o_acc[t][i * 2 + 1] * inv_l[i]);
      }
    }
  }

  // ---- pivot heads: block mass matrix
  if (!is_pivot) return;
  const int slot = p.slot_of_head[h];
  float* arow = p.pivot_attn + (int64_t(slot) * p.nb + r) * p.nb;
  float lse[2];
#pragma unroll
  for (int i = 0; i < 2; ++i) lse[i] = (l_run[i] > 0.f) ? m_run[i] + log2f(l_run[i]) : INFINITY;
  bool rvalid[2] = {qpos0 < p.n_tokens, qpos0 + 8 < p.n_tokens};

  __syncthreads();
  walk.init(brow, r);
  col = walk.next();
  stage = 0;
  if (col >= 0) issue_kv(col, 0, false);
  cp_async_commit();
  while (col >= 0) {
    const int nxt = walk.next();
    if (nxt >= 0) issue_kv(nxt, stage ^ 1, false);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    float s[NTILES_S][4];
    compute_s(s, stage, col == r, col * BS);
    float acc = 0.f;
#pragma unroll
    for (int j = 0; j < NTILES_S; ++j) {
      const int kpos = col * BS + j * 8 + (lane & 3) * 2;
      const bool k0 = kpos < p.n_tokens, k1 = kpos + 1 < p.n_tokens;
      if (rvalid[0]) acc += (k0 ? exp2f(s[j][0] - lse[0]) : 0.f) + (k1 ? exp2f(s[j][1] - lse[0]) : 0.f);
      if (rvalid[1]) acc += (k0 ? exp2f(s[j][2] - lse[1]) : 0.f) + (k1 ? exp2f(s[j][3] - lse[1]) : 0.f);
    }
    acc = warp_sum(acc);
    if (lane == 0) red_sum[warp] = acc;
    __syncthreads();
    if (tid == 0) {
      float t = 0.f;
#pragma unroll
      for (int w = 0; w < NW; ++w) t += red_sum[w];
      arow[col] = t / static_cast<float>(rows_valid);
    }
    __syncthreads();
    col = nxt;
    stage ^= 1;
  }
  cp_async_wait<0>();
}

template <int BS, int D>
static int launch_generic(const AttnParams& p, cudaStream_t st) {
  constexpr int NT = (BS / 16) * 32;
  constexpr int SMEM = 4 * BS * D * 2;
  auto kern = sparse_attn_generic_kernel<BS, D>;
  if (SMEM > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM);
    if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  }
  const unsigned grid = static_cast<unsigned>(p.nb) *
                        static_cast<unsigned>(p.pivot_only ? p.n_slots : p.n_q_heads);
  kern<<<grid, NT, SMEM, st>>>(p);
  return check_launch();
}

int sparse_attention_generic(const AttnParams& p, int block_size, int head_dim, cudaStream_t st) {
#define SPF_CASE(BS_, D_) \
  if (block_size == BS_ && head_dim == D_) return launch_generic<BS_, D_>(p, st);
  SPF_CASE(128, 128) SPF_CASE(64, 128) SPF_CASE(32, 128) SPF_CASE(16, 128)
  SPF_CASE(128, 64) SPF_CASE(64, 64) SPF_CASE(32, 64) SPF_CASE(16, 64)
#undef SPF_CASE
  return SPF_ERR_SHAPE;
}

}  // namespace spf
