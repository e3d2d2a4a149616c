// Block-sparse causal flash attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA)
// for block_size = head_dim = 128.
//
// One CTA runs TWO streams that share their K/V tiles: one query block row of two query heads of the
// same KV group (GQA reuse), or - for the last head of an odd-sized group - two consecutive query block
// rows of that head (neighbouring rows visit nearly the same key blocks).  Every K/V tile fetched by TMA
// serves both streams, which ping-pong on the tensor pipe.  Below, "head A / head B" names the streams.
//
//   warp 0      TMA producer: Q tiles once, then K and V tiles of the union of both heads' bitmap
//               rows through a 3-deep K ring and a 2-deep V ring (cp.async.bulk.tensor, 128-byte
//               swizzle, no multicast)
//   warps 1, 2  MMA issuers, one per head: S_h = Q_h K^T (both operands in shared memory) and
//               O_h += P_h V (P_h read from TMEM, V from shared memory) with tcgen05.mma, accumulators
//               in TMEM; completion is signalled to mbarriers with tcgen05.commit.  The sixteen MMAs of
//               a step (P V of the current block, Q K^T of the next) leave the thread back to back,
//               their descriptors fetched from a table in shared memory.  Where the two heads visit
//               (nearly) the same blocks a token passed between the two threads keeps the steps in the
//               order A, B, A, B, which holds the two softmax warpgroups half a period apart; where the
//               lists differ the threads run free, so neither head waits for the other's softmax
//   warp 3      idle (it only completes the control warpgroup, which gives registers to the softmax
//               warpgroups with setmaxnreg)
//   warps 4-7   softmax warpgroup of head A: a thread owns one query row; tcgen05.ld of S, base-2
//               softmax with scale*log2(e) folded in against a reference point that is the maximum
//               of the row's first block and moves only when a score lies more than 2^64 above it
//               (exact: the final normalisation uses the same reference), a quarter of the
//               exponentials as a polynomial on the FMA pipe, P rounded to bf16 and written back
//               over S with tcgen05.st
//   warps 8-11  the same for head B
//
// TMEM (512 columns): S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,384)  O_B [384,512).
// Arithmetic matches block_wise_prefill_attention_kernel (attn/shareprefill_attn.py:381-471):
// fp32 scores, causal mask on the diagonal block, P -> bf16 before P V, fp32 accumulation, bf16
// output.  Every mbarrier wait is bounded; on a timeout the CTA raises a shared abort flag, all
// roles drain and the kernel returns after recording the event in a device-side counter.
#include "spf_tc5.cuh"

namespace spf {

constexpr int TC_THREADS = 384;                             // 3 warpgroups: control, softmax A, softmax B
// setmaxnreg targets.  The CTA owns the registers it was launched with (384 threads x 168) and no more:
// a sum beyond that pool would leave the last setmaxnreg.inc waiting for ever.
constexpr int TC_REGS_CONTROL = 104, TC_REGS_SOFTMAX = 200;
static_assert(4 * TC_REGS_CONTROL + 8 * TC_REGS_SOFTMAX <= 12 * 168, "setmaxnreg targets exceed the CTA's register pool");
constexpr int TC_KSTAGES = 3;
constexpr int TC_VSTAGES = 2;
// shared memory map: 1 KiB of control data, then 1024-byte aligned tiles (Q x2, K x3, V x2)
constexpr uint32_t TC_SMEM_CTRL = 0;                        // mbarriers, TMEM slot, abort flag, descriptor table
constexpr uint32_t TC_SMEM_DTAB = 256;
constexpr uint32_t TC_SMEM_Q = 1024;
constexpr uint32_t TC_SMEM_K = TC_SMEM_Q + 2 * TC_TILE_BYTES;
constexpr uint32_t TC_SMEM_V = TC_SMEM_K + TC_KSTAGES * TC_TILE_BYTES;
constexpr uint32_t TC_SMEM_TOTAL = TC_SMEM_V + TC_VSTAGES * TC_TILE_BYTES;   // 225 KiB of the 227 KiB limit
// The reference point of a row's exponentials moves only when a score lies more than this (in log2
// units) above it; see the softmax warps
constexpr float TC_RESCALE_LOG2 = 64.0f;
constexpr float TC_BLOCK_SUM_LIMIT = 1180591620717411303424.0f;   // 2^70
// of every 8 pairs of exponentials, this many are computed on the FMA pipe (exp_pack_poly)
constexpr int TC_POLY_PAIRS = 2;
// descriptor table: the eight k-step descriptors of Q_A, Q_B, every K stage and every V stage
constexpr int DT_Q = 0, DT_K = 16, DT_V = DT_K + 8 * TC_KSTAGES, DT_N = DT_V + 8 * TC_VSTAGES;
static_assert(TC_SMEM_DTAB + DT_N * 8 <= TC_SMEM_Q, "descriptor table does not fit the control region");

// Timing probe, compiled in only with -DSPF_TC5_TRACE: clock64() stamps of the first CTA's
// first 63 iterations, [role: softmax A, softmax B, MMA issuer A][iteration][slot]; [2][63][*] holds the
// CTA-level stamps (entry, set-up done, Q landed, first Q K^T issued, epilogue begin / end, first K
// requested, exit).
#ifdef SPF_TC5_TRACE
__device__ long long g_tc5_trace[3][64][8];
#define TRACE(role, it, slot) do { if (blockIdx.x == SPF_TC5_TRACE && (it) < 64) g_tc5_trace[role][it][slot] = clock64(); } while (0)
#else
#define TRACE(role, it, slot) do {} while (0)
#endif

struct Tc5Params {
  __nv_bfloat16* out;
  const uint32_t* bitmap;
  int n_tokens, n_q_heads, n_kv_heads, group, pairs, nb, nbw;   // pairs: whole head pairs per KV group
  float scale_log2;
};

// Walks the union of two bitmap rows in ascending column order; flags bit h = head h visits it.
struct PairWalker {
  const uint32_t* wa; const uint32_t* wb;
  int ra, rb, nwords, w;       // last causal column block of stream A / B
  uint32_t ca, cb;
  __device__ static uint32_t lim(int row, int wi, uint32_t x) {
    const int last = row - (wi << 5);
    return last >= 31 ? x : (last < 0 ? 0u : (x & ((2u << last) - 1u)));
  }
  __device__ void load(int wi) {
    ca = wa ? lim(ra, wi, __ldg(wa + wi)) : 0u;
    cb = wb ? lim(rb, wi, __ldg(wb + wi)) : 0u;
  }
  __device__ void init(const uint32_t* a, int row_a, const uint32_t* b, int row_b) {
    wa = a; wb = b; ra = row_a; rb = row_b; w = 0;
    nwords = (max(a ? row_a : 0, b ? row_b : 0) >> 5) + 1;
    load(0);
  }
  __device__ int next(int& flags) {
    while ((ca | cb) == 0u) {
      if (++w >= nwords) { flags = 0; return -1; }
      load(w);
    }
    const int b = __ffs(ca | cb) - 1;
    flags = int((ca >> b) & 1u) | (int((cb >> b) & 1u) << 1);
    const uint32_t clr = ~(1u << b);
    ca &= clr; cb &= clr;
    return (w << 5) + b;
  }
};

__global__ void __launch_bounds__(TC_THREADS, 1)
sparse_attn_tc5_kernel(const __grid_constant__ CUtensorMap map_q, const __grid_constant__ CUtensorMap map_k,
                       const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_o,
                       const Tc5Params p) {
  // once several waits have run out the kernel is not making progress: later CTAs do nothing
  if (*reinterpret_cast<volatile unsigned int*>(&g_tc5_timeouts) > 16u) return;
  extern __shared__ __align__(1024) unsigned char smem[];
  const uint32_t sbase = smem_addr(smem);
  if (sbase & 1023u) {   // the swizzled tiles need a 1024-byte aligned base (no static shared memory here)
    if (threadIdx.x == 0) atomicAdd(&g_tc5_timeouts, 1000u);
    return;
  }
  // control region
  const uint32_t bar0 = sbase + TC_SMEM_CTRL;
  const uint32_t bar_q = bar0;
  auto bar_kfull = [&](int s) { return bar0 + 8u * (1 + s); };
  auto bar_kempty = [&](int s) { return bar0 + 8u * (4 + s); };
  auto bar_vfull = [&](int s) { return bar0 + 8u * (7 + s); };
  auto bar_vempty = [&](int s) { return bar0 + 8u * (9 + s); };
  auto bar_sfull = [&](int h) { return bar0 + 8u * (11 + h); };
  auto bar_pready = [&](int h) { return bar0 + 8u * (13 + h); };
  auto bar_odone = [&](int h) { return bar0 + 8u * (15 + h); };
  auto bar_token = [&](int h) { return bar0 + 8u * (17 + h); };    // issuing thread h may issue its next step
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + TC_SMEM_CTRL + 8 * 19);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + TC_SMEM_CTRL + 8 * 19 + 8);
  // Shared-memory descriptors of all k-steps of every operand tile, written once.  An issuing thread
  // fetches the eight descriptors of a tile with four 16-byte loads instead of deriving them: its
  // instruction stream shares a scheduler with softmax warps that always have something to issue, and
  // an instruction between two MMAs keeps the tensor pipe waiting (four per k-step made a Q K^T group
  // take ~800 clk instead of 512).
  uint64_t* dtab = reinterpret_cast<uint64_t*>(smem + TC_SMEM_DTAB);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTAs that run at the same time belong to the same KV head (its K/V stream stays in L2);
  // within a KV head the heavy (late) query blocks go first
  // Per KV head: nb * pairs CTAs with two heads and one row each, then - if the group size is odd -
  // ceil(nb / 2) CTAs with the last head and two rows each.
  int bid = blockIdx.x;
  const int n_rp = (p.group & 1) ? (p.nb + 1) >> 1 : 0;
  const int per_kvh = p.nb * p.pairs + n_rp;
  const int kvh = bid / per_kvh;
  bid -= kvh * per_kvh;
  int hA, hB, rA, rB;
  if (bid < p.nb * p.pairs) {
    const int pair = bid % p.pairs;
    rA = rB = p.nb - 1 - bid / p.pairs;
    hA = kvh * p.group + pair * 2; hB = hA + 1;
  } else {
    const int rp = n_rp - 1 - (bid - p.nb * p.pairs);
    hA = kvh * p.group + p.group - 1;
    rA = 2 * rp; rB = 2 * rp + 1;
    hB = rB < p.nb ? hA : -1;
  }
  const bool hasB = hB >= 0;
  const uint32_t* rowA = p.bitmap + (int64_t(hA) * p.nb + rA) * p.nbw;
  const uint32_t* rowB = hasB ? p.bitmap + (int64_t(hB) * p.nb + rB) * p.nbw : nullptr;

  if (tid == 0) TRACE(2, 63, 0);
  if (tid == 32) { tma_prefetch_map(&map_q); tma_prefetch_map(&map_k); tma_prefetch_map(&map_v); tma_prefetch_map(&map_o); }
  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < TC_KSTAGES; ++s) { mbar_init(bar_kfull(s), 1); mbar_init(bar_kempty(s), 2); }
    for (int s = 0; s < TC_VSTAGES; ++s) { mbar_init(bar_vfull(s), 1); mbar_init(bar_vempty(s), 2); }
    for (int h = 0; h < 2; ++h) {
      mbar_init(bar_sfull(h), 1); mbar_init(bar_pready(h), 128); mbar_init(bar_odone(h), 1);
      mbar_init(bar_token(h), 1);
    }
    mbar_arrive(bar_token(0));     // head A's thread goes first
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (tid >= 64 && tid < 64 + DT_N) {
    const int e = tid - 64, ks = e & 7;
    const uint64_t kstep = uint64_t(uint32_t(ks >> 2) * (TC_SLAB_BYTES >> 4) + uint32_t(ks & 3) * (32u >> 4));
    uint64_t d;
    if (e < DT_K) d = desc_kmajor(sbase + TC_SMEM_Q + uint32_t(e >> 3) * TC_TILE_BYTES) + kstep;
    else if (e < DT_V) d = desc_kmajor(sbase + TC_SMEM_K + uint32_t((e - DT_K) >> 3) * TC_TILE_BYTES) + kstep;
    else d = desc_mnmajor(sbase + TC_SMEM_V + uint32_t((e - DT_V) >> 3) * TC_TILE_BYTES) + uint64_t(uint32_t(ks) * (2048u >> 4));
    dtab[e] = d;
  }
  if (warp == 0) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)), "r"(512u));
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::);
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem = *tmem_slot;
  if (tid == 0) TRACE(2, 63, 1);

  if (warp < 4) {
    // control warpgroup (producer, MMA issuers, an idle warp) hands registers to the softmax warpgroups
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(TC_REGS_CONTROL));
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar_q, (hasB ? 2u : 1u) * TC_TILE_BYTES);
      for (int h = 0; h < (hasB ? 2 : 1); ++h) {
        const uint32_t dst = sbase + TC_SMEM_Q + h * TC_TILE_BYTES;
        tma_load_3d(dst, &map_q, bar_q, 0, (h == 0 ? rA : rB) * TC_BS, h == 0 ? hA : hB);
        tma_load_3d(dst + TC_SLAB_BYTES, &map_q, bar_q, 64, (h == 0 ? rA : rB) * TC_BS, h == 0 ? hA : hB);
      }
      auto load_k = [&](int i, int col) -> bool {
        const int s = i % TC_KSTAGES;
        if (!mbar_wait(bar_kempty(s), ((i / TC_KSTAGES) & 1) ^ 1, abort_flag)) return false;
        const uint32_t dst = sbase + TC_SMEM_K + s * TC_TILE_BYTES;
        mbar_expect_tx(bar_kfull(s), TC_TILE_BYTES);
        tma_load_3d(dst, &map_k, bar_kfull(s), 0, col * TC_BS, kvh);
        tma_load_3d(dst + TC_SLAB_BYTES, &map_k, bar_kfull(s), 64, col * TC_BS, kvh);
        return true;
      };
      auto load_v = [&](int i, int col) -> bool {
        const int s = i % TC_VSTAGES;
        if (!mbar_wait(bar_vempty(s), ((i / TC_VSTAGES) & 1) ^ 1, abort_flag)) return false;
        const uint32_t dst = sbase + TC_SMEM_V + s * TC_TILE_BYTES;
        mbar_expect_tx(bar_vfull(s), TC_TILE_BYTES);
        tma_load_3d(dst, &map_v, bar_vfull(s), 0, col * TC_BS, kvh);
        tma_load_3d(dst + TC_SLAB_BYTES, &map_v, bar_vfull(s), 64, col * TC_BS, kvh);
        return true;
      };
      // K runs one column ahead of V: K(i+1) is requested before V(i)
      PairWalker wk; wk.init(rowA, rA, rowB, rB);
      int fl, i = 0, k_issued = 0, v_issued = 0;
      int col = wk.next(fl);
      bool ok = true;
      if (col >= 0) { ok = load_k(0, col); k_issued = ok ? 1 : 0; }
      TRACE(2, 63, 6);
      while (ok && col >= 0) {
        const int ncol = wk.next(fl);
        if (ncol >= 0) { ok = load_k(i + 1, ncol); if (ok) k_issued = i + 2; }
        if (ok) { ok = load_v(i, col); if (ok) v_issued = i + 1; }
        col = ncol; ++i;
      }
      // drain: every copy this thread started must have landed before the CTA may exit
      mbar_wait(bar_q, 0, abort_flag, true);
      for (int j = (k_issued >= TC_KSTAGES ? k_issued - TC_KSTAGES : 0); j < k_issued; ++j)
        mbar_wait(bar_kfull(j % TC_KSTAGES), (j / TC_KSTAGES) & 1, abort_flag, true);
      for (int j = (v_issued >= TC_VSTAGES ? v_issued - TC_VSTAGES : 0); j < v_issued; ++j)
        mbar_wait(bar_vfull(j % TC_VSTAGES), (j / TC_VSTAGES) & 1, abort_flag, true);
    }
  } else if (warp <= 2) {
    // ------------------------------------------------------------ MMA issuers (warp 1: head A, warp 2: head B)
    // Both threads walk the union of the two bitmap rows in the producer's order and take part in the
    // hand-shake of every ring stage (two arrivals free a stage; a tile the head does not visit is
    // passed on as soon as it has landed), so the phase of a stage can never run ahead of a thread that
    // skips it.  A CTA with a single head still runs both threads: warp 2 then only passes tiles on.
    // Two ways to run a pair of rows, chosen from the two bitmap rows (the same answer in both warps):
    //  * in step: a token goes back and forth, so the steps leave in the order A, B, A, B - P V of A and
    //    the next Q K^T of A, then the same for B.  That keeps the two softmax warpgroups half a period
    //    apart; best where the heads visit (nearly) the same blocks.  A thread's bookkeeping (ring
    //    hand-shakes, bitmap walk, descriptor fetch) runs under the other thread's MMAs.
    //  * free: no token; a head never waits for the other head's softmax on a block it does not visit;
    //    best where the lists differ.
    // blocks of head A, of head B and of their union in this row (a lane per bitmap word, so the
    // words arrive in one memory latency)
    int cnt_a = 0, cnt_b = 0, cnt_u = 0;
    for (int i = lane; i <= (max(rA, rB) >> 5); i += 32) {
      const uint32_t wa = PairWalker::lim(rA, i, __ldg(rowA + i));
      const uint32_t wb = hasB ? PairWalker::lim(rB, i, __ldg(rowB + i)) : 0u;
      cnt_a += __popc(wa); cnt_b += __popc(wb); cnt_u += __popc(wa | wb);
    }
    cnt_a = __reduce_add_sync(0xffffffffu, cnt_a);
    cnt_b = __reduce_add_sync(0xffffffffu, cnt_b);
    cnt_u = __reduce_add_sync(0xffffffffu, cnt_u);
    if (lane == 0) {
      const int h = warp - 1, mine = 1 << h;
      const bool in_step = hasB && 4 * cnt_u <= 5 * max(cnt_a, cnt_b);
      const uint32_t ts = tmem + (h == 0 ? 0u : 128u), to = tmem + (h == 0 ? 256u : 384u);
      auto fetch = [&](int first, KSteps& o) {
        const ulonglong2* src = reinterpret_cast<const ulonglong2*>(dtab + first);
#pragma unroll
        for (int j = 0; j < 4; ++j) { const ulonglong2 t = src[j]; o.d[2 * j] = t.x; o.d[2 * j + 1] = t.y; }
      };
      int step = 0;
      auto take_token = [&]() { return !in_step || mbar_wait(bar_token(h), step & 1, abort_flag); };
      auto pass_token = [&]() { if (in_step) mbar_arrive(bar_token(h ^ 1)); ++step; };

      bool ok = mbar_wait(bar_q, 0, abort_flag);
      if (h == 0) TRACE(2, 63, 2);
      PairWalker wk; wk.init(rowA, rA, rowB, rB);
      int fl, nfl;
      int col = wk.next(fl);
      int i = 0;
      int np = 0;               // P tiles consumed
      if (ok && col >= 0) {
        ok = mbar_wait(bar_kfull(0), 0, abort_flag);
        if (ok) {
          KSteps qd, kd;
          if (fl & mine) { fetch(DT_Q + 8 * h, qd); fetch(DT_K, kd); }
          ok = take_token();
          if (ok) {
            if (fl & mine) { tc_fence_after(); mma_qk_x8(ts, qd, kd); tc_commit(bar_sfull(h)); }
            if (h == 0) TRACE(2, 63, 3);
            pass_token();
            if (fl & mine) tc_commit(bar_kempty(0)); else mbar_arrive(bar_kempty(0));
          }
        }
      }
      while (ok && col >= 0) {
        const int ncol = wk.next(nfl);
        const int vs = i % TC_VSTAGES, nks = (i + 1) % TC_KSTAGES;
        const bool do_pv = (fl & mine) != 0, do_qk = ncol >= 0 && (nfl & mine) != 0;
        ok = mbar_wait(bar_vfull(vs), (i / TC_VSTAGES) & 1, abort_flag);
        if (ok && ncol >= 0) ok = mbar_wait(bar_kfull(nks), ((i + 1) / TC_KSTAGES) & 1, abort_flag);
        if (!ok) break;
        // everything that is not an MMA comes first, so that between the wait for P and the last MMA of
        // the step there are MMAs only
        KSteps vd, qd, kd;
        if (do_pv) fetch(DT_V + 8 * vs, vd);
        if (do_qk) { fetch(DT_Q + 8 * h, qd); fetch(DT_K + 8 * nks, kd); }
        if (h == 0) TRACE(2, i, 0);
        ok = take_token();
        if (ok && do_pv) ok = mbar_wait(bar_pready(h), np & 1, abort_flag);
        if (!ok) break;
        if (do_pv || do_qk) {
          tc_fence_after();
          if (h == 0) TRACE(2, i, 1);
          if (do_pv) { mma_pv_x8(to, ts, vd, np > 0 ? 1u : 0u); ++np; }
          if (do_qk) { mma_qk_x8(ts, qd, kd); tc_commit(bar_sfull(h)); }
          if (h == 0) TRACE(2, i, 3);
        }
        pass_token();
        // a stage this head used is released when its MMAs are done, one it skipped at once
        if (do_pv) tc_commit(bar_vempty(vs)); else mbar_arrive(bar_vempty(vs));
        if (ncol >= 0) { if (do_qk) tc_commit(bar_kempty(nks)); else mbar_arrive(bar_kempty(nks)); }
        col = ncol; fl = nfl; ++i;
      }
      tc_commit(bar_odone(h));
    }
  }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(TC_REGS_SOFTMAX));
    const int h = (warp - 4) >> 2;                 // 0: head A, 1: head B
    const int quarter = warp & 3;                  // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;           // query row within the block
    const int head = h == 0 ? hA : hB;
    const int r = h == 0 ? rA : rB;                // this stream's query block row
    const int row0 = r * TC_BS;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_base + uint32_t(h * 128);
    const uint32_t tO = tmem + lane_base + uint32_t(256 + h * 128);
    float m_used = -INFINITY, l_sum = 0.f;
    int k = 0;
    bool ok = head >= 0;
    if (ok) {
      PairWalker wk; wk.init(h == 0 ? rowA : rowB, r, nullptr, 0);
      int fl;
      for (int col = wk.next(fl); col >= 0 && ok; col = wk.next(fl), ++k) {
        if (lane == 0 && quarter == 0) TRACE(h, k, 0);
        ok = mbar_wait(bar_sfull(h), k & 1, abort_flag);
        if (!ok) break;
        tc_fence_after();
        if (lane == 0 && quarter == 0) TRACE(h, k, 1);
        const bool diag = (col == r);
        // the whole score row (128 fp32) into registers: four loads in flight, one wait
        uint32_t s0[32], s1[32], s2[32], s3[32];
        tmem_ld32_raw(tS + 0, s0);
        tmem_ld32_raw(tS + 32, s1);
        tmem_ld32_raw(tS + 64, s2);
        tmem_ld32_raw(tS + 96, s3);
        tc_wait_ld();
        if (lane == 0 && quarter == 0) TRACE(h, k, 2);
        if (diag) {   // causal mask inside the diagonal block: key index > query index
          mask_after(s0, row - 0);
          mask_after(s1, row - 32);
          mask_after(s2, row - 64);
          mask_after(s3, row - 96);
        }
        // Only a row's first block needs its maximum before the exponentials: it fixes the reference
        // point m_used.  Later blocks go straight to P = 2^(s*scale - m_used), which keeps the maximum
        // reduction off the chain S -> P -> next S.  A block whose sum of P comes out above 2^70 (a score
        // at least 2^63 above the reference - or the sum is not finite) is redone after the reference has
        // been moved up to its maximum and O rescaled; P, l and O stay far inside the range of bf16 and
        // fp32, and the final normalisation uses the same reference, so the result does not depend on it.
        auto row_max_log2 = [&]() {
          return fmaxf(fmaxf(row_max(s0), row_max(s1)), fmaxf(row_max(s2), row_max(s3))) * p.scale_log2;
        };
        // P as bf16 over the first 64 columns of the S region; returns the sum of the unrounded values
        auto emit_p = [&]() {
          float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
          uint32_t pk[16];
          exp_pack_poly<TC_POLY_PAIRS>(s0, p.scale_log2, m_used, pk, l0); tmem_st16(tS + 0, pk);
          exp_pack_poly<TC_POLY_PAIRS>(s1, p.scale_log2, m_used, pk, l1); tmem_st16(tS + 16, pk);
          exp_pack_poly<TC_POLY_PAIRS>(s2, p.scale_log2, m_used, pk, l2); tmem_st16(tS + 32, pk);
          exp_pack_poly<TC_POLY_PAIRS>(s3, p.scale_log2, m_used, pk, l3); tmem_st16(tS + 48, pk);
          return (l0 + l1) + (l2 + l3);
        };
        if (k == 0) m_used = row_max_log2();
        if (lane == 0 && quarter == 0) TRACE(h, k, 5);
        float blk = emit_p();
        if (k > 0 && __any_sync(0xffffffffu, !(blk <= TC_BLOCK_SUM_LIMIT))) {
          tc_wait_st();
          const float mb = row_max_log2();
          float alpha = 1.f;
          if (mb > m_used + TC_RESCALE_LOG2) {
            alpha = exp2f(m_used - mb);
            m_used = mb;
            l_sum *= alpha;
          }
          // S_h(k) is complete, hence so is every earlier P V of this head: O_h is stable
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float v[32];
            tmem_ld32(tO + c * 32, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= alpha;
            tmem_st32(tO + c * 32, v);
          }
          blk = emit_p();
        }
        l_sum += blk;
        if (lane == 0 && quarter == 0) TRACE(h, k, 3);
        tc_wait_st();
        if (lane == 0 && quarter == 0) TRACE(h, k, 6);
        tc_fence_before();
        mbar_arrive(bar_pready(h));
        if (lane == 0 && quarter == 0) TRACE(h, k, 4);
      }
      // ---- epilogue
      if (h == 0 && lane == 0 && quarter == 0) TRACE(2, 63, 4);
      if (ok && k > 0) ok = mbar_wait(bar_odone(h), 0, abort_flag);
      // O / l as bf16 into this head's Q tile (all its Q K^T products are done), in the swizzled layout
      // of a TMA tile; then one thread stores the two 64-column slabs.  Rows past the end of the
      // sequence are clipped by the copy.
      const uint32_t stage = sbase + TC_SMEM_Q + uint32_t(h) * TC_TILE_BYTES;
      if (ok && k == 0) ok = mbar_wait(bar_q, 0, abort_flag);   // a row that visits nothing: the Q copy may still be landing
      if (ok) {
        tc_fence_after();
        const float inv = (k > 0 && l_sum > 0.f) ? 1.f / l_sum : 0.f;
#pragma unroll 1
        for (int c = 0; c < 4; ++c) {
          float v[32];
          if (k > 0) {
            tmem_ld32(tO + c * 32, v);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = 0.f;
          }
          const uint32_t rbase = stage + uint32_t(c >> 1) * TC_SLAB_BYTES + uint32_t(row) * 128u;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const uint32_t chunk = uint32_t((c & 1) * 4 + j) ^ uint32_t(row & 7);
            asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(rbase + (chunk << 4)),
                         "r"(pack2_bf16(v[8 * j] * inv, v[8 * j + 1] * inv)), "r"(pack2_bf16(v[8 * j + 2] * inv, v[8 * j + 3] * inv)),
                         "r"(pack2_bf16(v[8 * j + 4] * inv, v[8 * j + 5] * inv)), "r"(pack2_bf16(v[8 * j + 6] * inv, v[8 * j + 7] * inv))
                         : "memory");
          }
        }
        fence_proxy_async();
      }
      // every thread of the warpgroup arrives, also one that gave up on a wait: a hardware barrier has no limit
      asm volatile("bar.sync %0, 128;" ::"r"(1 + h) : "memory");
      if (ok && quarter == 0 && lane == 0 && !*abort_flag) {
        tma_store_3d(&map_o, stage, 0, row0, head);
        tma_store_3d(&map_o, stage + TC_SLAB_BYTES, 64, row0, head);
        tma_store_commit_and_wait_read();
      }
      if (h == 0 && lane == 0 && quarter == 0) TRACE(2, 63, 5);
    }
  }
  __syncwarp();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512u));
  }
  if (tid == 0) TRACE(2, 63, 7);
}

// ---------------------------------------------------------------- host side

// Returns SPF_ERR_SHAPE when the tensors cannot be described to TMA (the caller then uses the
// generic kernel).
int sparse_attention_tc5(const AttnParams& a, int n_kv_heads, cudaStream_t st) {
  if (a.q_sn <= 0 || a.k_sn <= 0 || a.v_sn <= 0 || a.q_sh <= 0 || a.k_sh <= 0 || a.v_sh <= 0) return SPF_ERR_SHAPE;
  CUtensorMap mq, mk, mv, mo;
  if (!make_map(&mq, a.q, a.n_tokens, a.n_q_heads, a.q_sn, a.q_sh) ||
      !make_map(&mk, a.k, a.n_tokens, n_kv_heads, a.k_sn, a.k_sh) ||
      !make_map(&mv, a.v, a.n_tokens, n_kv_heads, a.v_sn, a.v_sh) ||
      !make_map(&mo, a.out, a.n_tokens, a.n_q_heads, int64_t(a.n_q_heads) * TC_D, TC_D))
    return SPF_ERR_SHAPE;
  Tc5Params p;
  p.out = a.out; p.bitmap = a.bitmap; p.n_tokens = a.n_tokens; p.n_q_heads = a.n_q_heads;
  p.n_kv_heads = n_kv_heads; p.group = a.group; p.pairs = a.group / 2; p.nb = a.nb; p.nbw = a.nbw;
  p.scale_log2 = a.scale_log2;
  cudaError_t e = cudaFuncSetAttribute(sparse_attn_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(TC_SMEM_TOTAL));
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  const unsigned grid = unsigned(n_kv_heads) * (unsigned(a.nb) * unsigned(p.pairs) + ((a.group & 1) ? unsigned(a.nb + 1) / 2u : 0u));
  sparse_attn_tc5_kernel<<<grid, TC_THREADS, TC_SMEM_TOTAL, st>>>(mq, mk, mv, mo, p);
  return check_launch();
}

#ifdef SPF_TC5_TRACE
extern "C" void spf_tc5_trace_dump(long long* out) { cudaMemcpyFromSymbol(out, g_tc5_trace, sizeof(long long) * 3 * 64 * 8); }
#endif

unsigned int tc5_timeout_count() { return tc5_read_timeouts_here(); }
bool tc5_reset_timeouts() { return tc5_reset_timeouts_here(); }
bool tc5_set_wait_limit(unsigned long long ns) { return tc5_set_wait_limit_here(ns); }

// Self-test of the bounded wait: one thread waits on an mbarrier that nothing ever arrives on.  The
// wait runs out after the configured limit, the event is counted and the kernel returns normally.
__global__ void wait_limit_probe_kernel() {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(smem_addr(&bar), 1);
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) mbar_wait(smem_addr(&bar), 0, &abort_flag);
  __syncthreads();
}
int tc5_wait_limit_selftest(cudaStream_t st) {
  wait_limit_probe_kernel<<<1, 32, 0, st>>>();
  return check_launch();
}

}  // namespace spf
