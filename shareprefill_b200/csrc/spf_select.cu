// Pattern selection on the device: budgets, query-aware test, pivot election / sharing,
// vertical-slash expansion into bitmaps, query-aware block cover, pivot pattern update.
// Everything the reference does between the pooled scores and the block index lists
// (attn/attention_sharing.py:169-364, :94-103; attn/utils.py:26-128) without a host sync:
// decisions live in device flags, patterns in bitmaps.
#include "spf_cover.cuh"
#include "spf_internal.cuh"

namespace spf {

// ------------------------------------------------------------------ budgets + pooled profiles

__global__ void __launch_bounds__(1024) profile_budgets_kernel(const BudgetParams p) {
  __shared__ CoverShared sh;
  const int seg = blockIdx.x;
  const bool is_slash = seg >= p.n_heads;
  const int h = is_slash ? seg - p.n_heads : seg;
  const float* x = (is_slash ? p.slash : p.vertical) + int64_t(h) * p.n_tokens;
  auto load = [x](int i) { return __ldg(x + i); };
  const CoverResult r = cover_select(load, p.n_tokens, p.thr, COVER_PREFIX_LE, 60, &sh);
  if (threadIdx.x == 0) {
    // count(prefix <= thr) + 1, then // block_size + 1, clamped low first, high last
    const long long cnt = static_cast<long long>(r.keep) + 1;
    long long b = cnt / p.block_size + 1;
    if (b < p.min_blocks) b = p.min_blocks;
    if (b > p.max_blocks) b = p.max_blocks;
    (is_slash ? p.ns : p.nv)[h] = static_cast<int32_t>(b);
  }
  // block sums: one warp per block, fixed order
  float* pool = (is_slash ? p.spool : p.vpool) + int64_t(h) * p.nb;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  for (int b = warp; b < p.nb; b += nw) {
    const int n0 = b * p.block_size;
    const int n1 = min(p.n_tokens, n0 + p.block_size);
    double acc = 0.0;
    for (int i = n0 + lane; i < n1; i += 32) acc += static_cast<double>(__ldg(x + i));
    acc = warp_sum(acc);
    if (lane == 0) pool[b] = static_cast<float>(acc);
  }
}

// ------------------------------------------------------------------ pooled last-row estimate

__global__ void __launch_bounds__(256) pooled_last_row_kernel(const LastRowParams p) {
  extern __shared__ float dyn[];         // logits [nb]
  __shared__ float qm[128];
  __shared__ double red_d[32];
  __shared__ float red_f[32];
  const int h = blockIdx.x, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int kvh = h / (p.n_q_heads / p.n_kv_heads);
  const int rows = min(p.block_size, p.n_tokens);
  const int q0 = p.n_tokens - rows;
  // mean over the last `rows` queries of bf16(q / sqrt(D)): warp w takes rows w, w+8, ...; a lane
  // owns head_dim/32 consecutive elements of a row (coalesced), four rows in flight
  {
    const int per = p.head_dim >> 5;   // 2 or 4
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    const __nv_bfloat16* base = p.q + int64_t(q0) * p.q_sn + int64_t(h) * p.q_sh + lane * per;
    for (int i = warp; i < rows; i += 8) {
      const __nv_bfloat16* rp = base + int64_t(i) * p.q_sn;
#pragma unroll
      for (int e = 0; e < 4; ++e)
        if (e < per) acc[e] += bf16_round(__bfloat162float(rp[e]) / p.sqrt_d);
    }
    float* part = dyn;                 // [8 warps][head_dim] scratch, before dyn holds the logits
    for (int e = 0; e < per; ++e) part[warp * p.head_dim + lane * per + e] = acc[e];
    __syncthreads();
    if (tid < p.head_dim) {
      float t = 0.f;
      for (int w = 0; w < 8; ++w) t += part[w * p.head_dim + tid];
      qm[tid] = bf16_round(t / static_cast<float>(rows));
    }
  }
  __syncthreads();
  // one thread per key block: its pooled key row (head_dim bf16, 16-byte loads) against the mean query
  // in shared memory; the blocks of a thread are independent, so their loads overlap
  float lmax = -INFINITY;
  for (int b = tid; b < p.nb; b += 256) {
    const uint4* kr = reinterpret_cast<const uint4*>(p.avg_k + (int64_t(b) * p.n_kv_heads + kvh) * p.head_dim);
    float a0 = 0.f, a1 = 0.f;
    for (int c = 0; c < p.head_dim / 8; ++c) {
      const uint4 v = __ldg(kr + c);
      const float* q8 = qm + c * 8;
      a0 += q8[0] * __uint_as_float(v.x << 16) + q8[2] * __uint_as_float(v.y << 16) +
            q8[4] * __uint_as_float(v.z << 16) + q8[6] * __uint_as_float(v.w << 16);
      a1 += q8[1] * __uint_as_float(v.x & 0xffff0000u) + q8[3] * __uint_as_float(v.y & 0xffff0000u) +
            q8[5] * __uint_as_float(v.z & 0xffff0000u) + q8[7] * __uint_as_float(v.w & 0xffff0000u);
    }
    const float acc = bf16_round(a0 + a1);
    dyn[b] = acc;
    lmax = fmaxf(lmax, acc);
  }
  const float m = block_max(lmax, red_f);
  double part = 0.0;
  for (int b = tid; b < p.nb; b += 256) {
    const float e = expf(dyn[b] - m);
    dyn[b] = e;
    part += static_cast<double>(e);
  }
  const float z = static_cast<float>(block_sum(part, red_d));
  for (int b = tid; b < p.nb; b += 256) p.avg_qk[int64_t(h) * p.nb + b] = dyn[b] / z;
}

// ------------------------------------------------------------------ classification
// sqrt Jensen-Shannon divergence of two length-n fp32 vectors (attn/utils.py:26-30); the
// element terms are fp32 like torch's, summed in double.  0*log(0) stays NaN on purpose.
__device__ float block_sqrt_jsd(const float* a, const float* b, int n, double* red) {
  double sa = 0.0, sb = 0.0;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float pa = a[i], pb = b[i];
    const float m = (pa + pb) / 2.f;
    sa += static_cast<double>(pa * logf(pa / m));
    sb += static_cast<double>(pb * logf(pb / m));
  }
  const float fa = static_cast<float>(block_sum(sa, red));
  const float fb = static_cast<float>(block_sum(sb, red));
  return sqrtf(0.5f * fa + 0.5f * fb);
}


__global__ void __launch_bounds__(256) classify_heads_kernel(const ClassifyParams p) {
  __shared__ double red[32];
  const int h = blockIdx.x;
  const float* vp = p.vpool + int64_t(h) * p.nb;
  const float* sp = p.spool + int64_t(h) * p.nb;
  const float jq = block_sqrt_jsd(p.avg_qk + int64_t(h) * p.nb, vp, p.nb, red);
  float jv = nanf(""), js = nanf("");
  const int slot = p.slot_of_head[h];
  if (slot >= 0 && slot < p.n_slots && p.st.pattern_ready[slot]) {
    jv = block_sqrt_jsd(p.st.pivot_vertical + int64_t(slot) * p.nb, vp, p.nb, red);
    js = block_sqrt_jsd(p.st.pivot_slash + int64_t(slot) * p.nb, sp, p.nb, red);
  }
  if (threadIdx.x == 0) { p.jsd_qa[h] = jq; p.jsd_v[h] = jv; p.jsd_s[h] = js; }
}

// Pairwise divergence of n_vec distributions of length len (offline head clustering): out[i][j] =
// sqrt-JSD(x_i, x_j), same arithmetic as block_sqrt_jsd.  grid (ceil(n_vec / 8), n_vec): a CTA holds row
// i in shared memory and each of its eight warps takes one j.
__global__ void __launch_bounds__(256) pairwise_sqrt_jsd_kernel(const float* x, int n_vec, int len, float* out) {
  extern __shared__ float xi[];
  const int i = blockIdx.y, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int t = threadIdx.x; t < len; t += blockDim.x) xi[t] = x[int64_t(i) * len + t];
  __syncthreads();
  const int j = blockIdx.x * 8 + warp;
  if (j >= n_vec) return;
  const float* xj = x + int64_t(j) * len;
  double sa = 0.0, sb = 0.0;
  for (int t = lane; t < len; t += 32) {
    const float pa = xi[t], pb = __ldg(xj + t);
    const float m = (pa + pb) / 2.f;
    sa += static_cast<double>(pa * logf(pa / m));
    sb += static_cast<double>(pb * logf(pb / m));
  }
  const float fa = static_cast<float>(warp_sum(sa)), fb = static_cast<float>(warp_sum(sb));
  if (lane == 0) out[int64_t(i) * n_vec + j] = sqrtf(0.5f * fa + 0.5f * fb);
}
int launch_pairwise_jsd(const float* x, int n_vec, int len, float* out, cudaStream_t st) {
  pairwise_sqrt_jsd_kernel<<<dim3(ceil_div(n_vec, 8), n_vec), 256, size_t(len) * sizeof(float), st>>>(x, n_vec, len, out);
  return check_launch();
}

// ------------------------------------------------------------------ election / sharing

// One CTA replays the reference's loop over heads in ascending order
// (attn/attention_sharing.py:209-301).  Every rank runs it over ALL heads with identical
// inputs, so all ranks agree on the pivots; profiles are copied only for local pivots.
__global__ void __launch_bounds__(256) elect_and_share_kernel(const ElectParams p) {
  __shared__ int s_new_pivot;
  for (int h = 0; h < p.n_heads_total; ++h) {
    const int hl = h - p.head_offset;
    const bool local = hl >= 0 && hl < p.n_heads;
    int flags = 0;
    const bool qa = p.jsd_qa_all[h] < p.qa_thr;  // NaN -> false
    const int slot = p.slot_of_head_all[h];
    __syncthreads();
    if (threadIdx.x == 0) s_new_pivot = 0;
    __syncthreads();
    if (qa) {
      flags = SPF_HEAD_QUERY_AWARE;
    } else if (slot >= 0 && slot < p.n_slots) {
      if (threadIdx.x == 0) {
        if (p.st.pivot_head[slot] < 0) {
          p.st.pivot_head[slot] = h;
          p.st.pivot_layer[slot] = p.layer;
          s_new_pivot = 1;
        }
      }
      __syncthreads();
      if (s_new_pivot) {
        flags = SPF_HEAD_PIVOT;
        if (local) {
          for (int i = threadIdx.x; i < p.nb; i += blockDim.x) {
            p.st.pivot_vertical[int64_t(slot) * p.nb + i] = p.vpool[int64_t(hl) * p.nb + i];
            p.st.pivot_slash[int64_t(slot) * p.nb + i] = p.spool[int64_t(hl) * p.nb + i];
          }
        }
      } else if (p.st.pattern_ready[slot] && local) {
        const float ratio = p.st.vs_ratio[slot];
        if (p.jsd_v[hl] < p.sim_thr && p.jsd_s[hl] < p.sim_thr && ratio < p.fb_thr)
          flags = SPF_HEAD_SHARED;
      }
    }
    if (local && threadIdx.x == 0) {
      p.head_flags[hl] = flags;
      if (flags & (SPF_HEAD_QUERY_AWARE | SPF_HEAD_SHARED)) {
        p.nv[hl] = p.min_blocks;
        p.ns[hl] = p.min_blocks;
      }
    }
  }
}

// ------------------------------------------------------------------ vertical/slash bitmap

__device__ __forceinline__ uint32_t causal_word_mask(int row, int w) {
  const int last = row - (w << 5);
  if (last < 0) return 0u;
  return last >= 31 ? 0xffffffffu : ((2u << last) - 1u);
}

// bits [lo, lo+32) of a bit array of nwords words (out-of-range bits read 0)
__device__ __forceinline__ uint32_t bit_window(const uint32_t* words, int nwords, int lo) {
  const int wi = lo >> 5;   // arithmetic shift: floor
  const int sh = lo & 31;
  const uint32_t a = (wi >= 0 && wi < nwords) ? words[wi] : 0u;
  const uint32_t b = (wi + 1 >= 0 && wi + 1 < nwords) ? words[wi + 1] : 0u;
  return __funnelshift_r(a, b, sh);
}

__global__ void __launch_bounds__(1024) build_vs_bitmap_kernel(const VsParams p) {
  extern __shared__ unsigned char dyn_raw[];
  float* vv = reinterpret_cast<float*>(dyn_raw);          // [nb]
  float* sv = vv + p.nb;                                   // [nb]
  uint32_t* vmask = reinterpret_cast<uint32_t*>(sv + p.nb);  // [nbw] selected column blocks
  uint32_t* dmask = vmask + p.nbw;                         // [nbw] selected block distances
  const int h = blockIdx.x, nb = p.nb, nbw = p.nbw;
  const int flags = p.head_flags[h];
  const int slot = p.slot_of_head[h];
  const bool pivot = (flags & SPF_HEAD_PIVOT) && slot >= 0 && slot < p.n_slots;
  const bool shared = (flags & SPF_HEAD_SHARED) && slot >= 0 && slot < p.n_slots;
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    vv[i] = (i == 0) ? INFINITY : p.vpool[int64_t(h) * nb + i];
    sv[i] = (i == nb - 1) ? INFINITY : p.spool[int64_t(h) * nb + i];
  }
  for (int i = threadIdx.x; i < 2 * nbw; i += blockDim.x) vmask[i] = 0u;
  __syncthreads();
  const int kv = min(p.nv[h], nb), ks = min(p.ns[h], nb);
  // rank of every element: value descending, lowest index first among equals
  for (int i = threadIdx.x; i < nb; i += blockDim.x) {
    const float xv = vv[i], xs = sv[i];
    int rv = 0, rs = 0;
    for (int j = 0; j < nb; ++j) {
      const float yv = vv[j], ys = sv[j];
      rv += (yv > xv) || (yv == xv && j < i);
      rs += (ys > xs) || (ys == xs && j < i);
    }
    if (rv < kv) {
      atomicOr(&vmask[i >> 5], 1u << (i & 31));
      if (pivot) p.st.pivot_vlist[int64_t(slot) * nb + rv] = i;
    }
    if (rs < ks) {
      const int d = nb - 1 - i;
      atomicOr(&dmask[d >> 5], 1u << (d & 31));
      if (pivot) p.st.pivot_slist[int64_t(slot) * nb + rs] = d;
    }
  }
  if (pivot && threadIdx.x == 0) { p.st.pivot_nv[slot] = kv; p.st.pivot_ns[slot] = ks; }
  __syncthreads();
  uint32_t* out = p.bitmap + int64_t(h) * nb * nbw;
  const uint32_t* pat = shared ? p.st.pattern + int64_t(slot) * nb * nbw : nullptr;
  for (int idx = threadIdx.x; idx < nb * nbw; idx += blockDim.x) {
    const int r = idx / nbw, w = idx % nbw;
    const uint32_t cm = causal_word_mask(r, w);
    uint32_t bits = 0u;
    if (cm) {
      if (pivot) {
        bits = cm;
      } else {
        // column c = 32w + j is on block distance d = r - c; bit j of the result is dmask bit
        // (r - 32w - j): reverse the window that starts at r - 32w - 31
        const uint32_t win = bit_window(dmask, nbw, r - (w << 5) - 31);
        bits = (vmask[w] | __brev(win)) & cm;
        if (pat) bits |= pat[idx];
      }
    }
    out[idx] = bits;
  }
}

// ------------------------------------------------------------------ query-aware scores

// A CTA owns eight query block rows of one head.  A thread takes key blocks c, c + 256, ...: the pooled
// key row is read once (16-byte loads) and used for all eight rows, whose scaled mean queries sit in
// shared memory.  Logits are rounded to bf16 (the reference's bf16 einsum), the softmax over the
// causal prefix runs in fp32, one warp per row; zeros above the diagonal.
// (Four rows per CTA beyond 4096 blocks, where eight rows of logits no longer fit in shared memory.)
template <int QAS_ROWS>
__global__ void __launch_bounds__(256) query_aware_scores_kernel(const QaScoreParams p) {
  extern __shared__ float qa_dyn[];               // logits [QAS_ROWS][nb], then q [QAS_ROWS][D]
  const int h = blockIdx.y;
  if (p.head_flags && !(p.head_flags[h] & SPF_HEAD_QUERY_AWARE)) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r0 = blockIdx.x * QAS_ROWS;
  const int rows = min(QAS_ROWS, p.nb - r0);
  const int kvh = h / (p.n_q_heads / p.n_kv_heads);
  const int D = p.head_dim;
  float* logit = qa_dyn;
  float* qs = qa_dyn + QAS_ROWS * p.nb;
  for (int i = tid; i < QAS_ROWS * D; i += 256) {
    const int rr = i / D, d = i % D;
    qs[i] = rr < rows ? bf16_round(__bfloat162float(p.avg_q[(int64_t(r0 + rr) * p.n_q_heads + h) * D + d]) / p.sqrt_d) : 0.f;
  }
  __syncthreads();
  const int c_end = r0 + rows;                    // key blocks 0 .. r0 + rows - 1 are needed by some row
  for (int c = tid; c < c_end; c += 256) {
    const uint4* kr = reinterpret_cast<const uint4*>(p.avg_k + (int64_t(c) * p.n_kv_heads + kvh) * D);
    float acc[QAS_ROWS];
#pragma unroll
    for (int rr = 0; rr < QAS_ROWS; ++rr) acc[rr] = 0.f;
    for (int ch = 0; ch < D / 8; ++ch) {
      const uint4 v = __ldg(kr + ch);
      const float kf[8] = {__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u),
                           __uint_as_float(v.y << 16), __uint_as_float(v.y & 0xffff0000u),
                           __uint_as_float(v.z << 16), __uint_as_float(v.z & 0xffff0000u),
                           __uint_as_float(v.w << 16), __uint_as_float(v.w & 0xffff0000u)};
#pragma unroll
      for (int rr = 0; rr < QAS_ROWS; ++rr) {
        const float* q8 = qs + rr * D + ch * 8;
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[rr] = fmaf(q8[e], kf[e], acc[rr]);
      }
    }
#pragma unroll
    for (int rr = 0; rr < QAS_ROWS; ++rr) logit[rr * p.nb + c] = bf16_round(acc[rr]);
  }
  __syncthreads();
  if (warp < rows) {
    const int r = r0 + warp;
    const float* lg = logit + warp * p.nb;
    float mx = -INFINITY;
    for (int c = lane; c <= r; c += 32) mx = fmaxf(mx, lg[c]);
    mx = warp_max(mx);
    double z = 0.0;
    for (int c = lane; c <= r; c += 32) z += static_cast<double>(expf(lg[c] - mx));
    const float zf = static_cast<float>(warp_sum(z));
    float* out = p.scores + (int64_t(h) * p.nb + r) * p.nb;
    for (int c = lane; c < p.nb; c += 32) out[c] = (c <= r) ? expf(lg[c] - mx) / zf : 0.f;
  }
}

// ------------------------------------------------------------------ query-aware select

__global__ void __launch_bounds__(1024) query_aware_select_kernel(const QaSelectParams p) {
  __shared__ CoverShared sh;
  const int h = blockIdx.x;
  if (p.head_flags && !(p.head_flags[h] & SPF_HEAD_QUERY_AWARE)) return;
  const float* x = p.scores + int64_t(h) * p.nb * p.nb;
  const int n = p.nb * p.nb;
  auto load = [x](int i) { return __ldg(x + i); };
  const CoverResult r = cover_select<true>(load, n, p.thr, COVER_PREFIX_LE, p.scale_bits, &sh, x);
  uint32_t* bm = p.bitmap + int64_t(h) * p.nb * p.nbw;
  const bool ranked = cover_needs_tie_rank(r);
  if (!ranked && (p.nb & 31) == 0 && (reinterpret_cast<uintptr_t>(x) & 15u) == 0) {
    // no ties to rank: 16 bytes per load; a thread's four elements are four neighbouring bits of a
    // bitmap word and eight neighbouring lanes make up the word
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const int n4 = n >> 2, lane = threadIdx.x & 31;
    const int n4_round = ((n4 + blockDim.x - 1) / blockDim.x) * blockDim.x;
    // (row, column) of the thread's first element, advanced by one block stride per trip: no division
    int row = (threadIdx.x * 4) / p.nb, c0 = (threadIdx.x * 4) % p.nb;
    const int step_rows = (blockDim.x * 4) / p.nb, step_cols = (blockDim.x * 4) % p.nb;
    for (int i = threadIdx.x; i < n4_round; i += blockDim.x, row += step_rows, c0 += step_cols) {
      if (c0 >= p.nb) { c0 -= p.nb; ++row; }
      const bool in = i < n4;
      const float4 v = in ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
      const float vs[4] = {v.x, v.y, v.z, v.w};
      unsigned int nib = 0;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const unsigned int key = __float_as_uint(vs[e]) & 0x7fffffffu;
        const bool keep = in && (c0 + e) <= row && (r.all || (key != 0u && cover_keeps(r, key, 0u)));
        nib |= (keep ? 1u : 0u) << e;
      }
      unsigned int word = nib << (4 * (lane & 7));
      word |= __shfl_xor_sync(0xffffffffu, word, 1);
      word |= __shfl_xor_sync(0xffffffffu, word, 2);
      word |= __shfl_xor_sync(0xffffffffu, word, 4);
      if ((lane & 7) == 0 && word) atomicOr(&bm[int64_t(row) * p.nbw + (c0 >> 5)], word);
    }
    return;
  }
  unsigned int running = 0;
  const int n_round = ((n + blockDim.x - 1) / blockDim.x) * blockDim.x;
  int row = threadIdx.x / p.nb, c = threadIdx.x % p.nb;
  const int step_rows = blockDim.x / p.nb, step_cols = blockDim.x % p.nb;
  for (int i = threadIdx.x; i < n_round; i += blockDim.x, row += step_rows, c += step_cols) {
    if (c >= p.nb) { c -= p.nb; ++row; }
    const bool in = i < n;
    const float v = in ? __ldg(x + i) : 0.f;
    const unsigned int key = __float_as_uint(v) & 0x7fffffffu;
    unsigned int rank = 0;
    if (ranked) rank = block_flag_rank(in && key == r.key_thr && key != 0u, &running, sh.scan_cnt);
    // exact zeros are never part of a cover unless everything is; keep to the causal triangle
    const bool keep = in && c <= row && (r.all || (key != 0u && cover_keeps(r, key, rank)));
    if ((p.nb & 31) == 0) {
      // the 32 elements of a warp are the 32 bits of one bitmap word: one atomic per word
      const unsigned int word = __ballot_sync(0xffffffffu, keep);
      if ((threadIdx.x & 31) == 0 && word) atomicOr(&bm[int64_t(row) * p.nbw + (c >> 5)], word);
    } else if (keep) {
      atomicOr(&bm[int64_t(row) * p.nbw + (c >> 5)], 1u << (c & 31));
    }
  }
}

// ------------------------------------------------------------------ counts
__global__ void __launch_bounds__(256) bitmap_row_counts_kernel(const uint32_t* bitmap, int nb, int nbw,
                                                                int32_t* row_counts,
                                                                unsigned long long* head_totals) {
  __shared__ double red[32];
  const int h = blockIdx.x;
  double tot = 0.0;
  for (int r = threadIdx.x; r < nb; r += blockDim.x) {
    const uint32_t* w = bitmap + (int64_t(h) * nb + r) * nbw;
    int c = 0;
    for (int i = 0; i <= (r >> 5); ++i) c += __popc(w[i] & causal_word_mask(r, i));
    row_counts[int64_t(h) * nb + r] = c;
    tot += c;
  }
  tot = block_sum(tot, red);
  if (threadIdx.x == 0 && head_totals) head_totals[h] = static_cast<unsigned long long>(tot + 0.5);
}

// ------------------------------------------------------------------ pivot update

// grid (nb, H): one CTA per row of a new pivot's block-mass matrix
__global__ void __launch_bounds__(256) pivot_pattern_kernel(const PivotParams p) {
  __shared__ CoverShared sh;
  __shared__ unsigned int s_best;
  const int h = blockIdx.y, r = blockIdx.x;
  if (!(p.head_flags[h] & SPF_HEAD_PIVOT)) return;
  const int slot = p.slot_of_head[h];
  if (slot < 0 || slot >= p.n_slots) return;
  const float* x = p.st.pivot_attn + (int64_t(slot) * p.nb + r) * p.nb;
  uint32_t* prow = p.st.pattern + (int64_t(slot) * p.nb + r) * p.nbw;
  auto load = [x](int i) { return __ldg(x + i); };
  CoverResult res = cover_select(load, p.nb, p.thr, COVER_PREFIX_LT, 58, &sh);
  if (threadIdx.x == 0) s_best = 0xffffffffu;
  for (int w = threadIdx.x; w < p.nbw; w += blockDim.x) prow[w] = (r == 0 && w == 0) ? 1u : 0u;
  __syncthreads();
  if (res.all) {
    // the prefix never reaches the threshold: the reference keeps exactly the largest element
    // (argmax of an all-false mask is 0): largest key, lowest index
    unsigned int best = 0;
    for (int i = threadIdx.x; i < p.nb; i += blockDim.x)
      best = max(best, __float_as_uint(x[i]) & 0x7fffffffu);
    __shared__ unsigned int s_max;
    if (threadIdx.x == 0) s_max = 0;
    __syncthreads();
    atomicMax(&s_max, best);
    __syncthreads();
    for (int i = threadIdx.x; i < p.nb; i += blockDim.x)
      if ((__float_as_uint(x[i]) & 0x7fffffffu) == s_max) atomicMin(&s_best, static_cast<unsigned int>(i));
    __syncthreads();
    if (threadIdx.x == 0) atomicOr(&prow[s_best >> 5], 1u << (s_best & 31));
    return;
  }
  res.ties_keep += 1;   // the element that crosses the threshold is kept too
  const bool ranked = cover_needs_tie_rank(res);
  unsigned int running = 0;
  const int n_round = ((p.nb + blockDim.x - 1) / blockDim.x) * blockDim.x;
  for (int i = threadIdx.x; i < n_round; i += blockDim.x) {
    const bool in = i < p.nb;
    const unsigned int key = in ? (__float_as_uint(x[i]) & 0x7fffffffu) : 0u;
    unsigned int rank = 0;
    if (ranked) rank = block_flag_rank(in && key == res.key_thr && key != 0u, &running, sh.scan_cnt);
    if (in && key != 0u && cover_keeps(res, key, rank)) atomicOr(&prow[i >> 5], 1u << (i & 31));
  }
}

// grid (H): vs_ratio of a new pivot = sum of its block-mass matrix over the MULTISET of its
// own vertical/slash indices (duplicates and the 0 paddings included, as the reference's
// gather-sum does, attn/attention_sharing.py:278-284) divided by the matrix total; then the
// pattern is published to later layers.
__global__ void __launch_bounds__(256) pivot_ratio_kernel(const PivotParams p) {
  __shared__ double red[32];
  const int h = blockIdx.x;
  if (!(p.head_flags[h] & SPF_HEAD_PIVOT)) return;
  const int slot = p.slot_of_head[h];
  if (slot < 0 || slot >= p.n_slots) return;
  const int nb = p.nb;
  const float* A = p.st.pivot_attn + int64_t(slot) * nb * nb;
  const int kv = p.st.pivot_nv[slot], ks = p.st.pivot_ns[slot];
  const int32_t* vl = p.st.pivot_vlist + int64_t(slot) * nb;
  const int32_t* sl = p.st.pivot_slist + int64_t(slot) * nb;
  double tot = 0.0, cov = 0.0;
  for (int64_t i = threadIdx.x; i < int64_t(nb) * nb; i += blockDim.x) tot += static_cast<double>(A[i]);
  const float a00 = A[0];
  for (int64_t i = threadIdx.x; i < int64_t(ks) * nb; i += blockDim.x) {
    const int s = sl[i / nb], r = static_cast<int>(i % nb);
    cov += static_cast<double>((r + s < nb) ? A[int64_t(r + s) * nb + r] : a00);
  }
  for (int64_t i = threadIdx.x; i < int64_t(kv) * nb; i += blockDim.x) {
    const int v = vl[i / nb], r = static_cast<int>(i % nb);
    cov += static_cast<double>((r >= v) ? A[int64_t(r) * nb + v] : a00);
  }
  const float ftot = static_cast<float>(block_sum(tot, red));
  const float fcov = static_cast<float>(block_sum(cov, red));
  if (threadIdx.x == 0) {
    p.st.vs_ratio[slot] = fcov / ftot;
    p.st.pattern_ready[slot] = 1;
  }
}

__global__ void state_reset_kernel(StateView st, int n_slots) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_slots) {
    st.pivot_head[i] = -1;
    st.pivot_layer[i] = -1;
    st.pattern_ready[i] = 0;
    st.vs_ratio[i] = nanf("");
    st.pivot_nv[i] = 0;
    st.pivot_ns[i] = 0;
  }
}

// ------------------------------------------------------------------ host launchers
int launch_budgets(const BudgetParams& p, cudaStream_t st) {
  profile_budgets_kernel<<<2 * p.n_heads, 1024, 0, st>>>(p);
  return check_launch();
}
int launch_last_row(const LastRowParams& p, cudaStream_t st) {
  const size_t dyn_floats = static_cast<size_t>(p.nb > 8 * p.head_dim ? p.nb : 8 * p.head_dim);
  pooled_last_row_kernel<<<p.n_q_heads, 256, dyn_floats * sizeof(float), st>>>(p);
  return check_launch();
}
int launch_classify(const ClassifyParams& p, int n_heads, cudaStream_t st) {
  classify_heads_kernel<<<n_heads, 256, 0, st>>>(p);
  return check_launch();
}
int launch_elect(const ElectParams& p, cudaStream_t st) {
  elect_and_share_kernel<<<1, 256, 0, st>>>(p);
  return check_launch();
}
// ---- pivot summaries for the head-sharded exchange.  One int32 row per slot:
// [flag][vs_ratio bits][vertical nb][slash nb][pattern nb*nbw].  pack fills the rows of pivots elected
// in `layer` among heads [h0, h1) and clears the flag of every other row (their payload is not
// written and not read); merge installs, per slot, the first flagged row among the ranks.
constexpr int SUMMARY_CHUNKS = 8;

__device__ __forceinline__ void copy_words(int32_t* dst, const int32_t* src, int n) {
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < n; i += SUMMARY_CHUNKS * blockDim.x) dst[i] = src[i];
}

__global__ void __launch_bounds__(256) pack_summaries_kernel(StateView st, int nb, int nbw, int layer, int h0,
                                                            int h1, int32_t* out) {
  const int s = blockIdx.x;
  const int64_t width = 2 + 2 * int64_t(nb) + int64_t(nb) * nbw;
  int32_t* row = out + s * width;
  const int ph = st.pivot_head[s];
  const bool mine = st.pivot_layer[s] == layer && ph >= h0 && ph < h1;
  if (blockIdx.y == 0 && threadIdx.x == 0) {
    row[0] = mine ? 1 : 0;
    if (mine) row[1] = __float_as_int(st.vs_ratio[s]);
  }
  if (!mine) return;
  copy_words(row + 2, reinterpret_cast<const int32_t*>(st.pivot_vertical + int64_t(s) * nb), nb);
  copy_words(row + 2 + nb, reinterpret_cast<const int32_t*>(st.pivot_slash + int64_t(s) * nb), nb);
  copy_words(row + 2 + 2 * nb, reinterpret_cast<const int32_t*>(st.pattern + int64_t(s) * nb * nbw), nb * nbw);
}

__global__ void __launch_bounds__(256) merge_summaries_kernel(StateView st, int n_slots, int nb, int nbw,
                                                             const int32_t* gathered, int n_ranks) {
  const int s = blockIdx.x;
  const int64_t width = 2 + 2 * int64_t(nb) + int64_t(nb) * nbw;
  const int32_t* row = nullptr;
  for (int r = 0; r < n_ranks && !row; ++r) {
    const int32_t* cand = gathered + (int64_t(r) * n_slots + s) * width;
    if (cand[0] > 0) row = cand;
  }
  if (!row) return;
  if (blockIdx.y == 0 && threadIdx.x == 0) {
    st.vs_ratio[s] = __int_as_float(row[1]);
    st.pattern_ready[s] = 1;
  }
  copy_words(reinterpret_cast<int32_t*>(st.pivot_vertical + int64_t(s) * nb), row + 2, nb);
  copy_words(reinterpret_cast<int32_t*>(st.pivot_slash + int64_t(s) * nb), row + 2 + nb, nb);
  copy_words(reinterpret_cast<int32_t*>(st.pattern + int64_t(s) * nb * nbw), row + 2 + 2 * nb, nb * nbw);
}

int launch_pack_summaries(void* state, int n_slots, int nb, int layer, int h0, int h1, int32_t* out,
                          cudaStream_t st) {
  pack_summaries_kernel<<<dim3(n_slots, SUMMARY_CHUNKS), 256, 0, st>>>(state_view(state, n_slots, nb), nb,
                                                                      (nb + 31) / 32, layer, h0, h1, out);
  return check_launch();
}
int launch_merge_summaries(void* state, int n_slots, int nb, const int32_t* gathered, int n_ranks,
                           cudaStream_t st) {
  merge_summaries_kernel<<<dim3(n_slots, SUMMARY_CHUNKS), 256, 0, st>>>(state_view(state, n_slots, nb), n_slots,
                                                                       nb, (nb + 31) / 32, gathered, n_ranks);
  return check_launch();
}

int launch_vs_bitmap(const VsParams& p, int n_heads, cudaStream_t st) {
  const size_t smem = size_t(p.nb) * 8 + size_t(p.nbw) * 8;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(build_vs_bitmap_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         static_cast<int>(smem));
    if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  }
  build_vs_bitmap_kernel<<<n_heads, 1024, smem, st>>>(p);
  return check_launch();
}
int launch_qa_scores(const QaScoreParams& p, cudaStream_t st) {
  const int rows = p.nb > 4096 ? 4 : 8;
  const size_t smem = (size_t(rows) * p.nb + size_t(rows) * p.head_dim) * sizeof(float);
  auto kern = rows == 8 ? query_aware_scores_kernel<8> : query_aware_scores_kernel<4>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  }
  kern<<<dim3(ceil_div(p.nb, rows), p.n_q_heads), 256, smem, st>>>(p);
  return check_launch();
}
int launch_qa_select(const QaSelectParams& p, int n_heads, cudaStream_t st) {
  query_aware_select_kernel<<<n_heads, 1024, 0, st>>>(p);
  return check_launch();
}
int launch_row_counts(const uint32_t* bitmap, int n_heads, int nb, int32_t* row_counts,
                      int64_t* head_totals, cudaStream_t st) {
  bitmap_row_counts_kernel<<<n_heads, 256, 0, st>>>(bitmap, nb, (nb + 31) / 32, row_counts,
                                                   reinterpret_cast<unsigned long long*>(head_totals));
  return check_launch();
}
int launch_update_pivots(const PivotParams& p, int n_heads, cudaStream_t st) {
  pivot_pattern_kernel<<<dim3(p.nb, n_heads), 256, 0, st>>>(p);
  pivot_ratio_kernel<<<n_heads, 256, 0, st>>>(p);
  return check_launch();
}
int launch_state_reset(void* state, int n_slots, int nb, cudaStream_t st) {
  int64_t off[13];
  state_offsets(n_slots, nb, off);
  cudaError_t e = cudaMemsetAsync(state, 0, off[12], st);
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  if (n_slots > 0) state_reset_kernel<<<ceil_div(n_slots, 128), 128, 0, st>>>(state_view(state, n_slots, nb), n_slots);
  return check_launch();
}

}  // namespace spf
