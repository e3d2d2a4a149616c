// Last-block profile on the 5th-generation tensor cores (head_dim = 128): the same two passes as
// spf_estimate.cu (attn/attention_sharing.py:127-167, attn/utils.py:79-86 in the reference), with
// the logits on tcgen05.mma into TMEM and the key tiles brought in by TMA.
//
// A CTA owns a run of 128-key tiles of one KV head and up to four query heads of its group, so a
// key tile is fetched once for all of them.  The scaled queries (bf16(q / sqrt(D)), rows past the
// block zero) are written by the CTA itself into 128-byte swizzled tiles; they stay in shared
// memory for the whole run.
//
//   warp 0      TMA producer: key tiles through a 2-deep ring (no multicast)
//   warp 1      MMA issuer: per key tile one 128x128x128 product per head into that head's 128
//               TMEM columns, as soon as the softmax warps have taken the previous tile out of them
//   warps 4-7   heads 0 and 2 of the CTA      warps 8-11  heads 1 and 3
//
//   pass 1 (stats)    S = Q K^T: a TMEM lane is a query row, so a thread owns a row and reduces over
//                     the 128 keys of the tile in registers: tile maximum and sum of exponentials
//   pass 2 (profile)  S^T = K Q^T (operands swapped): a TMEM lane is a key, so a thread owns a key,
//                     sums p = exp(l - M_i) / Z_i over the query rows in registers (vertical); for the
//                     anti-diagonals (slash) row j of a 32-row chunk is rotated by j lanes, which lines
//                     the diagonals up with the lanes; rows are normalised with the per-row constants
//                     of pass 1, staged in shared memory
//
// Rounding points are those of the mma.sync version: logits rounded to bf16, softmax in fp32.
// Every mbarrier wait is bounded; on a timeout the CTA raises an abort flag, all roles drain and
// the kernel returns after recording the event.
#include <type_traits>

#include "spf_tc5.cuh"

namespace spf {

constexpr int ET_THREADS = 384;
constexpr int ET_HEADS = 4;                                   // query heads per CTA (TMEM: 4 x 128 columns)
constexpr int ET_KSTAGES = 2;
constexpr uint32_t ET_SMEM_TABLE = 256;                       // [4][128] per-row constants (pass 2)
constexpr uint32_t ET_SMEM_DPART = ET_SMEM_TABLE + ET_HEADS * 128 * 4;  // [2 warpgroups][2 buffers][4 chunks][4 warps][64] partial anti-diagonal sums
constexpr uint32_t ET_SMEM_Q = 19 * 1024;
constexpr uint32_t ET_SMEM_K = ET_SMEM_Q + ET_HEADS * TC_TILE_BYTES;
constexpr uint32_t ET_SMEM_TOTAL = ET_SMEM_K + ET_KSTAGES * TC_TILE_BYTES;   // 211 KiB
static_assert(ET_SMEM_DPART + 2 * 2 * 4 * 4 * 64 * 4 <= ET_SMEM_Q, "control region overflow");
constexpr float ET_LOG2E = 1.4426950408889634f;

struct EstTc5Params {
  EstParams e;
  int n_kv_heads, subs;        // subs: CTAs per KV head along the group (ceil(group / 4))
  int tiles_per_cta;
};

template <bool PASS2>
__global__ void __launch_bounds__(ET_THREADS, 1)
lastblock_tc5_kernel(const __grid_constant__ CUtensorMap map_k, const EstTc5Params pp) {
  if (*reinterpret_cast<volatile unsigned int*>(&g_tc5_timeouts) > 16u) return;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_addr(smem);
  if (sbase & 1023u) {
    if (threadIdx.x == 0) atomicAdd(&g_tc5_timeouts, 1000u);
    return;
  }
  const EstParams& p = pp.e;
  const uint32_t bar0 = sbase;
  auto bar_kfull = [&](int s) { return bar0 + 8u * (0 + s); };
  auto bar_kempty = [&](int s) { return bar0 + 8u * (2 + s); };
  auto bar_sfull = [&](int h) { return bar0 + 8u * (4 + h); };
  auto bar_sfree = [&](int h) { return bar0 + 8u * (8 + h); };
  const uint32_t bar_qready = bar0 + 8u * 12;
  auto bar_wg = [&](int w) { return bar0 + 8u * (14 + w); };   // the 128 threads of a softmax warpgroup
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + 8 * 13);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + 8 * 13 + 4);
  float* table = reinterpret_cast<float*>(smem + ET_SMEM_TABLE);
  float* dpart_all = reinterpret_cast<float*>(smem + ET_SMEM_DPART);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int sub = blockIdx.y % pp.subs, kvh = blockIdx.y / pp.subs;
  const int h0 = kvh * p.group + sub * ET_HEADS;
  const int nh = min(ET_HEADS, p.group - sub * ET_HEADS);
  const int t_begin = blockIdx.x * pp.tiles_per_cta;
  const int t_end = min(p.ntiles, t_begin + pp.tiles_per_cta);
  const int ntl = t_end - t_begin;
  const int q0 = p.n_tokens - p.rq;

  if (tid == 0) {
    for (int s = 0; s < ET_KSTAGES; ++s) { mbar_init(bar_kfull(s), 1); mbar_init(bar_kempty(s), 1); }
    for (int h = 0; h < ET_HEADS; ++h) { mbar_init(bar_sfull(h), 1); mbar_init(bar_sfree(h), 128); }
    mbar_init(bar_qready, 256);
    mbar_init(bar_wg(0), 128); mbar_init(bar_wg(1), 128);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;

  if (warp < 4) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
    if (warp == 0 && lane == 0) {
      // ------------------------------------------------------------ TMA producer
      bool ok = true;
      int issued = 0;
      for (int i = 0; i < ntl && ok; ++i) {
        const int s = i % ET_KSTAGES;
        ok = mbar_wait(bar_kempty(s), ((i / ET_KSTAGES) & 1) ^ 1, abort_flag);
        if (!ok) break;
        const uint32_t dst = sbase + ET_SMEM_K + s * TC_TILE_BYTES;
        mbar_expect_tx(bar_kfull(s), TC_TILE_BYTES);
        tma_load_3d(dst, &map_k, bar_kfull(s), 0, (t_begin + i) * TC_BS, kvh);
        tma_load_3d(dst + TC_SLAB_BYTES, &map_k, bar_kfull(s), 64, (t_begin + i) * TC_BS, kvh);
        issued = i + 1;
      }
      // every copy this thread started must have landed before the CTA may exit
      for (int j = (issued >= ET_KSTAGES ? issued - ET_KSTAGES : 0); j < issued; ++j)
        mbar_wait(bar_kfull(j % ET_KSTAGES), (j / ET_KSTAGES) & 1, abort_flag, true);
    } else if (warp == 1 && lane == 0) {
      // ------------------------------------------------------------ MMA issuer
      const uint64_t qd0 = desc_kmajor(sbase + ET_SMEM_Q), kd0 = desc_kmajor(sbase + ET_SMEM_K);
      bool ok = mbar_wait(bar_qready, 0, abort_flag);
      for (int i = 0; i < ntl && ok; ++i) {
        const int s = i % ET_KSTAGES;
        ok = mbar_wait(bar_kfull(s), (i / ET_KSTAGES) & 1, abort_flag);
        if (!ok) break;
        const uint64_t kd = kd0 + uint64_t((s * TC_TILE_BYTES) >> 4);
        for (int h = 0; h < nh && ok; ++h) {
          // the softmax warps have taken tile i-1 out of this head's columns
          ok = mbar_wait(bar_sfree(h), (i & 1) ^ 1, abort_flag);
          if (!ok) break;
          tc_fence_after();
          const uint64_t qd = qd0 + uint64_t((h * TC_TILE_BYTES) >> 4);
          if (PASS2) mma_qk_group(tmem + uint32_t(h * 128), kd, qd);   // S^T: lanes are keys
          else mma_qk_group(tmem + uint32_t(h * 128), qd, kd);         // S: lanes are query rows
          tc_commit(bar_sfull(h));
        }
        if (ok) tc_commit(bar_kempty(s));
      }
    }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int wg = (warp - 4) >> 2;
    const int quarter = warp & 3;
    const int ln = quarter * 32 + lane;              // TMEM lane of this thread
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    // ---- scaled queries into the swizzled tiles (rows past the block are zero), per-row constants
    {
      const int t2 = tid - 128;                      // 0..255
      unsigned char* qs = smem + ET_SMEM_Q;
      for (int h = 0; h < nh; ++h) {
        // eight 16-byte pieces per thread and head: all loads first, then scale, round and store
        uint4 vals[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int it = t2 + u * 256, row = it >> 4, ch = it & 15;
          vals[u] = make_uint4(0u, 0u, 0u, 0u);
          if (row < p.rq)
            vals[u] = __ldg(reinterpret_cast<const uint4*>(p.q + int64_t(q0 + row) * p.q_sn + int64_t(h0 + h) * p.q_sh + ch * 8));
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) {
          const int it = t2 + u * 256, row = it >> 4, ch = it & 15;
          __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&vals[u]);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            float2 f = __bfloat1622float2(pr[e]);
            pr[e] = __floats2bfloat162_rn(f.x / p.sqrt_d, f.y / p.sqrt_d);
          }
          const uint32_t off = uint32_t(h) * TC_TILE_BYTES + uint32_t(ch >> 3) * TC_SLAB_BYTES + uint32_t(row) * 128u +
                               (uint32_t((ch & 7) ^ (row & 7)) << 4);
          *reinterpret_cast<uint4*>(qs + off) = vals[u];
        }
        if (PASS2) {
          // p = 2^(l*log2e - c_i) with c_i = M_i*log2e + log2 Z_i; rows past the block contribute nothing
          for (int it = t2; it < 128; it += 256) {
            const float m = p.row_m[(h0 + h) * 128 + it], z = p.row_z[(h0 + h) * 128 + it];
            table[h * 128 + it] = it < p.rq ? m * ET_LOG2E + log2f(z) : INFINITY;
          }
        }
      }
      fence_proxy_async();
      mbar_arrive(bar_qready);
      // the tables are read by both warpgroups
      asm volatile("bar.sync 3, 256;" ::: "memory");
    }
    float* dpart_wg = dpart_all + wg * 2048;         // [2 buffers][4 chunks][4 warps][64]
    // pass 1: running row statistics of the two heads this warpgroup serves
    float run_m0 = -INFINITY, run_m1 = -INFINITY, run_l0 = 0.f, run_l1 = 0.f;
    int nsync = 0;                                   // uses of the warpgroup barrier so far (its phase)
    // bounded like every other wait: a thread that gave up never strands the others at a hardware barrier
    auto wg_sync = [&]() -> bool {
      mbar_arrive(bar_wg(wg));
      return mbar_wait(bar_wg(wg), (nsync++) & 1, abort_flag);
    };
    const float inv_rows = 1.0f / float(p.rq);
    bool ok = true;
    for (int i = 0; i < ntl && ok; ++i) {
      const int tile = t_begin + i, c0 = tile * TC_BS;
      for (int h = wg; h < nh && ok; h += 2) {
        ok = mbar_wait(bar_sfull(h), i & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        const uint32_t tS = tmem + lane_base + uint32_t(h * 128);
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld32_raw(tS + 0, s0);
        tmem_ld32_raw(tS + 32, s1);
        tmem_ld32_raw(tS + 64, s2);
        tmem_ld32_raw(tS + 96, s3);
        tc_wait_ld();
        tc_fence_before();
        mbar_arrive(bar_sfree(h));                   // the issuer may overwrite the columns
        const int head = h0 + h;
        if (!PASS2) {
          // thread = query row ln; columns = keys c0 .. c0+127
          auto round32 = [](uint32_t (&r)[32]) {
#pragma unroll
            for (int j = 0; j < 32; j += 2) {
              const uint32_t pk = bf16x2_from(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
              r[j] = pk << 16; r[j + 1] = pk & 0xffff0000u;
            }
          };
          round32(s0); round32(s1); round32(s2); round32(s3);
          if (c0 + TC_BS - 1 > q0) {                 // keys after a query are masked (also keys past the end)
            const int last = q0 + ln - c0;
            mask_after(s0, last); mask_after(s1, last - 32); mask_after(s2, last - 64); mask_after(s3, last - 96);
          }
          const float mx = fmaxf(fmaxf(row_max(s0), row_max(s1)), fmaxf(row_max(s2), row_max(s3)));
          // running maximum and sum of this row over the CTA's tiles (rescaled when the maximum moves);
          // one partial per head, row and CTA leaves the kernel
          float& run_m = (h < 2) ? run_m0 : run_m1;
          float& run_l = (h < 2) ? run_l0 : run_l1;
          if (mx > run_m) {
            run_l *= fast_exp2((run_m - mx) * ET_LOG2E);   // 0 when run_m is -inf
            run_m = mx;
          }
          const float mref = (run_m == -INFINITY ? 0.f : run_m) * ET_LOG2E;
          float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
          auto add32 = [&](const uint32_t (&r)[32]) {
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              a0 += fast_exp2(fmaf(__uint_as_float(r[j]), ET_LOG2E, -mref));
              a1 += fast_exp2(fmaf(__uint_as_float(r[j + 1]), ET_LOG2E, -mref));
              a2 += fast_exp2(fmaf(__uint_as_float(r[j + 2]), ET_LOG2E, -mref));
              a3 += fast_exp2(fmaf(__uint_as_float(r[j + 3]), ET_LOG2E, -mref));
            }
          };
          add32(s0); add32(s1); add32(s2); add32(s3);
          run_l += (a0 + a1) + (a2 + a3);
          if (i == ntl - 1) {
            const int64_t base = (int64_t(head) * p.n_parts + blockIdx.x) * 128 + ln;
            p.part_m[base] = run_m;
            p.part_l[base] = run_l;
          }
        } else {
          // thread = key c0 + ln; columns = query rows 0..127.  Row i sees this key if kpos <= q0 + i.
          const int kpos = c0 + ln;
          const int first = kpos - q0;               // rows below `first` are masked (all rows for keys past the end)
          const float* tb = table + h * 128;
          // Anti-diagonals without atomics or serial chains.  Slot s = ln + 127 - i holds the tile-local
          // diagonal t = ln + (rq-1) - i (shifted by 128 - rq).  Within a warp (keys 32q + l) and a chunk
          // of 32 rows (i = 32c + j) the slot is 32(q-c) + 127 + (l - j): row j is rotated by j lanes, so
          // that lane m receives the value of lane (m + j) mod 32, whose l - j is m (no wrap) or m - 32
          // (wrap): two running sums per lane, `lo` for slot 32(q-c) + 127 + m and `hi` for 32 less.
          // One shuffle per element, no shared-memory traffic until the chunk is done.
          float vs0 = 0.f, vs1 = 0.f, vs2 = 0.f, vs3 = 0.f;
          float* dpart = dpart_wg + (nsync & 1) * 1024;   // buffers alternate from tile to tile
          float* part = dpart + quarter * 64;        // [chunk][warp][lo 0..31 | hi 0..31]
          // lane m takes the unwrapped values for j < 32 - m and the wrapped ones after: one running
          // sum, `lo` is its value after step 31 - m and `hi` the rest
          auto chunk = [&](const uint32_t (&r)[32], int c, auto masked) {
            float run = 0.f, lo = 0.f;
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              // eight values at a time: exponentials, then the eight rotations, then the running sum, so
              // that no instruction waits for the result of the one just before it
              const float4 ta = *reinterpret_cast<const float4*>(tb + 32 * c + j);
              const float4 tc = *reinterpret_cast<const float4*>(tb + 32 * c + j + 4);
              const float tv[8] = {ta.x, ta.y, ta.z, ta.w, tc.x, tc.y, tc.z, tc.w};
              uint32_t xb[8];
#pragma unroll
              for (int e = 0; e < 8; e += 2) {
                const uint32_t pk = bf16x2_from(__uint_as_float(r[j + e]), __uint_as_float(r[j + e + 1]));
                xb[e] = pk << 16; xb[e + 1] = pk & 0xffff0000u;
              }
              float pv[8], rot[8];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                pv[e] = fast_exp2(fmaf(__uint_as_float(xb[e]), ET_LOG2E, -tv[e]));
                if (decltype(masked)::value && 32 * c + j + e < first) pv[e] = 0.f;
              }
#pragma unroll
              for (int e = 0; e < 8; ++e) rot[e] = __shfl_sync(0xffffffffu, pv[e], lane + j + e);   // source lane modulo 32
              vs0 += pv[0] + pv[4]; vs1 += pv[1] + pv[5]; vs2 += pv[2] + pv[6]; vs3 += pv[3] + pv[7];
#pragma unroll
              for (int e = 0; e < 8; ++e) {
                run += rot[e];
                if (lane == 31 - (j + e)) lo = run;
              }
            }
            part[c * 256 + lane] = lo;
            part[c * 256 + 32 + lane] = run - lo;
          };
          if (c0 + TC_BS - 1 > q0) {   // only the last tiles see the causal mask (and keys past the end)
            chunk(s0, 0, std::true_type{}); chunk(s1, 1, std::true_type{});
            chunk(s2, 2, std::true_type{}); chunk(s3, 3, std::true_type{});
          } else {
            chunk(s0, 0, std::false_type{}); chunk(s1, 1, std::false_type{});
            chunk(s2, 2, std::false_type{}); chunk(s3, 3, std::false_type{});
          }
          if (kpos < p.n_tokens) p.vertical[int64_t(head) * p.n_tokens + kpos] = ((vs0 + vs1) + (vs2 + vs3)) * inv_rows;
          ok = wg_sync();
          if (!ok) break;
          // slot x collects, over chunks c and warps w, lo[m] with m = x - 127 - 32(w-c) and hi[m] with
          // m = x - 95 - 32(w-c), where m falls in 0..31
          for (int x = ln; x < 255; x += 128) {
            float v = 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
#pragma unroll
              for (int w = 0; w < 4; ++w) {
                const int mlo = x - 127 - 32 * (w - c), mhi = mlo + 32;
                if (mlo >= 0 && mlo < 32) v += dpart[c * 256 + w * 64 + mlo];
                if (mhi >= 0 && mhi < 32) v += dpart[c * 256 + w * 64 + 32 + mhi];
              }
            }
            const int t = x - (128 - p.rq);
            const int n = c0 + t;
            if (t >= 0 && n < p.n_tokens && v != 0.f) atomicAdd(&p.slash[int64_t(head) * p.n_tokens + n], v * inv_rows);
          }
          // no second barrier: the next tile of this warpgroup writes the other buffer, and its own barrier
          // orders the rewrite of this one after every thread's reads here
        }
      }
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
}

void launch_lastblock_reduce(const EstParams& p, cudaStream_t st);

// Returns SPF_ERR_SHAPE when the key tensor cannot be described to TMA (the caller then uses the
// mma.sync kernels).  p.slash must be zero on entry.
int lastblock_profile_tc5(const EstParams& e, cudaStream_t st) {
  if (e.k_sn <= 0 || e.k_sh <= 0) return SPF_ERR_SHAPE;
  EstTc5Params pp;
  pp.e = e;
  pp.n_kv_heads = e.n_q_heads / e.group;
  pp.subs = ceil_div(e.group, ET_HEADS);
  CUtensorMap mk;
  if (!make_map(&mk, e.k, e.n_tokens, pp.n_kv_heads, e.k_sn, e.k_sh)) return SPF_ERR_SHAPE;
  const int rows = pp.n_kv_heads * pp.subs;
  // one CTA per SM (one fits at a time, and its set-up - scaled queries, TMEM, first tiles - is not
  // small): runs of key tiles sized so that the grid fills the SMs once
  int sms = 148;
  int dev = 0;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int chunks = sms / rows;
  chunks = chunks < 1 ? 1 : (chunks > e.ntiles ? e.ntiles : chunks);
  const int tpc = ceil_div(e.ntiles, chunks);
  pp.tiles_per_cta = tpc;
  const dim3 grid(ceil_div(e.ntiles, tpc), rows);
  pp.e.n_parts = int(grid.x);   // pass 1 leaves one partial per head, row and CTA
  cudaError_t err = cudaFuncSetAttribute(lastblock_tc5_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         int(ET_SMEM_TOTAL));
  if (err == cudaSuccess)
    err = cudaFuncSetAttribute(lastblock_tc5_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(ET_SMEM_TOTAL));
  if (err != cudaSuccess) { note_cuda_error(err); return SPF_ERR_LAUNCH; }
  lastblock_tc5_kernel<false><<<grid, ET_THREADS, ET_SMEM_TOTAL, st>>>(mk, pp);
  launch_lastblock_reduce(pp.e, st);
  lastblock_tc5_kernel<true><<<grid, ET_THREADS, ET_SMEM_TOTAL, st>>>(mk, pp);
  return check_launch();
}

unsigned int est_tc5_timeout_count() { return tc5_read_timeouts_here(); }
bool est_tc5_reset_timeouts() { return tc5_reset_timeouts_here(); }
bool est_tc5_set_wait_limit(unsigned long long ns) { return tc5_set_wait_limit_here(ns); }

}  // namespace spf
