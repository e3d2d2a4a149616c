// Cumulative-mass "cover" selection without a sort.
//
// The reference sorts a non-negative fp32 vector in descending order, takes the running sum
// (torch CPU: accumulated in fp64, each prefix rounded to fp32) and keeps the leading
// elements while the prefix stays <= (or <) a threshold:
//   score_cover_topk          attn/utils.py:47-50   count(prefix <= s) + 1
//   score_cover_idx           attn/utils.py:53-57   keep while prefix <= s
//   score_cover_idx_each_row  attn/utils.py:60-76   keep up to and including first prefix >= s
// Only the NUMBER of kept elements K and WHICH elements are the K largest matter, so a
// three-level radix descent over the float bit pattern finds the value at which the prefix
// crosses the threshold: per level a shared-memory histogram of (count, sum) per bin, bins
// scanned from the top.  Sums are exact 64-bit fixed point (2^-scale_bits resolution), so the
// result does not depend on the order of the atomic adds; converted to double and rounded to
// fp32 they reproduce the reference's prefix to ~1e-13, far below an fp32 ulp.
// Ties at the crossing value are resolved lowest index first (torch leaves the order open).
#pragma once

#include "spf_common.cuh"

namespace spf {

constexpr int COVER_BINS = 2048;
constexpr int COVER_LEVELS = 3;

struct CoverShared {
  unsigned long long sum[COVER_BINS];
  unsigned int cnt[COVER_BINS];
  // broadcast slots
  unsigned long long base_sum;
  unsigned int base_cnt;
  int found_bin;
  unsigned int scan_cnt[32];
};

struct CoverResult {
  unsigned int keep;        // K: number of leading sorted elements whose prefix satisfies the rule
  unsigned int key_thr;     // bit pattern of the crossing value
  unsigned int ties_keep;   // how many elements equal to key_thr are among the K
  unsigned int ties_total;  // how many elements equal key_thr
  bool all;                 // every element satisfies the rule (K == n)
};

enum CoverRule { COVER_PREFIX_LE = 0, COVER_PREFIX_LT = 1 };

__device__ __forceinline__ bool cover_ok(unsigned long long fx, double inv_scale, float thr, int rule) {
  const float f = static_cast<float>(static_cast<double>(fx) * inv_scale);
  return rule == COVER_PREFIX_LE ? (f <= thr) : (f < thr);
}

// floor(x * 2^scale_bits) for a positive normal fp32 x (key = its bit pattern), by shifting the
// mantissa: the same value as __double2ull_rz(double(x) * 2^scale_bits) at a fraction of the
// instructions (the histogram passes are bound by instruction issue).
__device__ __forceinline__ unsigned long long cover_fixed(float x, unsigned int key, int scale_bits, double scale) {
  const int eb = static_cast<int>(key >> 23);
  const int sh = eb - 150 + scale_bits;
  const unsigned long long m = static_cast<unsigned long long>((key & 0x7fffffu) | 0x800000u);
  if (eb != 0 && sh >= 0 && sh <= 40) return m << sh;
  if (eb != 0 && sh < 0) return sh > -24 ? (m >> (-sh)) : 0ull;
  return __double2ull_rz(static_cast<double>(x) * scale);   // denormals and values that would overflow
}

// All threads of the block call this with the same arguments.  `load(i)` returns element i
// (non-negative fp32) for i in [0, n).  Exact zeros are skipped (they never move a prefix).
// RUN_LENGTH is for inputs in which the successive elements of a thread (one block stride apart)
// mostly share a bin - a row-major score matrix whose rows are softmaxes over a long causal prefix,
// where a block stride is about one row: a thread then keeps (bin, count, sum) of its current run
// in registers and touches the histogram only when the bin changes.
template <bool RUN_LENGTH = false, class Load>
__device__ CoverResult cover_select(Load load, int n, float thr, int rule, int scale_bits,
                                    CoverShared* sh, const float* contiguous = nullptr) {
  // `contiguous`: the elements as a plain fp32 array (load(i) == contiguous[i]); with n a multiple
  // of 4 and a 16-byte aligned base the passes then read 16 bytes per load, four loads in flight
  const bool vec4 = contiguous != nullptr && (n & 3) == 0 && (reinterpret_cast<uintptr_t>(contiguous) & 15u) == 0;
  const double scale = exp2(static_cast<double>(scale_bits));
  const double inv_scale = exp2(-static_cast<double>(scale_bits));
  const int shifts[COVER_LEVELS] = {20, 9, 0};
  const int widths[COVER_LEVELS] = {11, 11, 9};
  unsigned int prefix = 0;      // key bits decided so far (right aligned)
  unsigned int hi_shift = 31;   // elements with (key >> hi_shift) == prefix are still candidates
  unsigned long long base_sum = 0;
  unsigned int base_cnt = 0;
  CoverResult res;
  res.keep = 0; res.key_thr = 0; res.ties_keep = 0; res.ties_total = 0; res.all = false;

  for (int lvl = 0; lvl < COVER_LEVELS; ++lvl) {
    const int shift = shifts[lvl];
    const int nbins = 1 << widths[lvl];
    __syncthreads();
    for (int b = threadIdx.x; b < nbins; b += blockDim.x) { sh->cnt[b] = 0; sh->sum[b] = 0ull; }
    __syncthreads();
    // eight elements (four 16-byte vectors on the contiguous path) per thread and trip, loaded before any
    // is used (one load in flight per thread leaves the loop waiting on memory); elements past the end
    // read as zero, which is skipped.
    // (Adding up the lanes that share a bin with match_any before touching the histogram was measured
    // slower than the plain shared-memory atomics on the token profiles: 312 against 191 us for 64
    // vectors of 128K elements.)
    unsigned int run_bin = 0xffffffffu, run_cnt = 0;   // RUN_LENGTH: the thread's current run
    unsigned long long run_fx = 0ull;
    auto take = [&](float x) {
      const unsigned int key = __float_as_uint(x) & 0x7fffffffu;
      if (key == 0u || (key >> hi_shift) != prefix) return;
      const unsigned int b = (key >> shift) & (nbins - 1);
      const unsigned long long fx = cover_fixed(x, key, scale_bits, scale);
      if (RUN_LENGTH) {
        if (b != run_bin) {
          if (run_cnt) { atomicAdd(&sh->cnt[run_bin], run_cnt); atomicAdd(&sh->sum[run_bin], run_fx); }
          run_bin = b; run_cnt = 0; run_fx = 0ull;
        }
        ++run_cnt; run_fx += fx;
      } else {
        atomicAdd(&sh->cnt[b], 1u);
        atomicAdd(&sh->sum[b], fx);
      }
    };
    if (vec4) {
      const float4* x4 = reinterpret_cast<const float4*>(contiguous);
      const int n4 = n >> 2;
      for (int i0 = threadIdx.x; i0 < n4; i0 += 4 * blockDim.x) {
        float4 xs[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * blockDim.x;
          xs[u] = i < n4 ? __ldg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) { take(xs[u].x); take(xs[u].y); take(xs[u].z); take(xs[u].w); }
      }
    } else {
      for (int i0 = threadIdx.x; i0 < n; i0 += 8 * blockDim.x) {
        float xs[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int i = i0 + u * blockDim.x;
          xs[u] = i < n ? load(i) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) take(xs[u]);
      }
    }
    if (RUN_LENGTH && run_cnt) { atomicAdd(&sh->cnt[run_bin], run_cnt); atomicAdd(&sh->sum[run_bin], run_fx); }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      unsigned long long run_sum = base_sum;
      unsigned int run_cnt = base_cnt;
      int found = -1;
      unsigned long long fb_sum = 0; unsigned int fb_cnt = 0;
      for (int chunk = nbins - 32; chunk >= 0 && found < 0; chunk -= 32) {
        const int b = chunk + 31 - lane;  // lane 0 holds the highest bin of the chunk
        const unsigned int c = sh->cnt[b];
        const unsigned long long s = sh->sum[b];
        unsigned int ic = c; unsigned long long is = s;
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
          const unsigned int tc = __shfl_up_sync(0xffffffffu, ic, o);
          const unsigned long long ts = __shfl_up_sync(0xffffffffu, is, o);
          if (lane >= o) { ic += tc; is += ts; }
        }
        const unsigned long long cum_sum = run_sum + is;
        const unsigned int cum_cnt = run_cnt + ic;
        const bool fail = (c != 0u) && !cover_ok(cum_sum, inv_scale, thr, rule);
        const unsigned int m = __ballot_sync(0xffffffffu, fail);
        if (m) {
          const int first = __ffs(m) - 1;
          found = chunk + 31 - first;
          fb_sum = __shfl_sync(0xffffffffu, cum_sum - s, first);
          fb_cnt = __shfl_sync(0xffffffffu, cum_cnt - c, first);
        } else {
          run_sum = __shfl_sync(0xffffffffu, cum_sum, 31);
          run_cnt = __shfl_sync(0xffffffffu, cum_cnt, 31);
        }
      }
      if (lane == 0) {
        sh->found_bin = found;
        sh->base_sum = found < 0 ? run_sum : fb_sum;
        sh->base_cnt = found < 0 ? run_cnt : fb_cnt;
      }
    }
    __syncthreads();
    const int found = sh->found_bin;
    base_sum = sh->base_sum;
    base_cnt = sh->base_cnt;
    if (found < 0) {  // the whole candidate range satisfies the rule: every element does
      res.all = true;
      res.keep = static_cast<unsigned int>(n);
      __syncthreads();
      return res;
    }
    prefix = (prefix << widths[lvl]) | static_cast<unsigned int>(found);
    hi_shift = shift;
    if (lvl == COVER_LEVELS - 1) {
      // every element of the bin equals `prefix`; find how many of them still satisfy the rule
      const unsigned int c = sh->cnt[found];
      const unsigned long long fx =
          __double2ull_rz(static_cast<double>(__uint_as_float(prefix)) * scale);
      unsigned int lo = 0, hi = c;  // ok(lo) holds, ok(hi) fails
      while (hi - lo > 1) {
        const unsigned int mid = lo + (hi - lo) / 2;
        if (cover_ok(base_sum + fx * mid, inv_scale, thr, rule)) lo = mid; else hi = mid;
      }
      res.key_thr = prefix;
      res.ties_keep = lo;
      res.ties_total = c;
      res.keep = base_cnt + lo;
    }
  }
  __syncthreads();
  return res;
}

// Does element (key, tie_rank) belong to the K largest?  tie_rank is the element's rank, in
// index order, among the elements whose key equals res.key_thr (only read when needed).
__device__ __forceinline__ bool cover_keeps(const CoverResult& r, unsigned int key, unsigned int tie_rank) {
  if (r.all) return true;
  if (key > r.key_thr) return true;
  if (key == r.key_thr) return tie_rank < r.ties_keep;
  return false;
}
__device__ __forceinline__ bool cover_needs_tie_rank(const CoverResult& r) {
  return !r.all && r.ties_keep > 0u && r.ties_keep < r.ties_total;
}

// Exclusive rank of flagged threads in index order within one pass over a block-strided
// range.  Call from all threads for each chunk; `running` carries the count so far.
__device__ __forceinline__ unsigned int block_flag_rank(bool flag, unsigned int* running,
                                                       unsigned int* scan /*[32] shared*/) {
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  const unsigned int m = __ballot_sync(0xffffffffu, flag);
  // most chunks hold no flagged element: one barrier settles that and nobody needs a rank
  if (!__syncthreads_or(m != 0u)) return *running;
  const unsigned int in_warp = __popc(m & ((1u << lane) - 1u));
  if (lane == 0) scan[w] = __popc(m);
  __syncthreads();
  unsigned int before = 0, total = 0;
  for (int i = 0; i < nw; ++i) {
    const unsigned int c = scan[i];
    if (i < w) before += c;
    total += c;
  }
  const unsigned int rank = *running + before + in_warp;
  *running += total;
  return rank;
}

}  // namespace spf
