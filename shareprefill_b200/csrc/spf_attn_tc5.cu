// Block-sparse causal flash attention on the 5th-generation tensor cores (tcgen05 + TMEM + TMA)
// for block_size = head_dim = 128.
//
// One CTA owns one query block row of up to TWO query heads of the same KV group, so every K/V
// tile fetched by TMA serves both heads (GQA reuse); the two heads ping-pong on the tensor pipe.
//
//   warp 0      TMA producer: Q tiles once, then K and V tiles of the union of both heads' bitmap
//               rows through a 3-deep K ring and a 2-deep V ring (cp.async.bulk.tensor, 128-byte
//               swizzle, no multicast)
//   warps 1, 2  MMA issuers: S_h = Q_h K^T (both operands in shared memory) and O_h += P_h V (P_h read
//               from TMEM, V from shared memory) with tcgen05.mma, accumulators in TMEM; completion is
//               signalled to mbarriers with tcgen05.commit.  Warp 1 alone alternates between the
//               heads where they visit the same blocks; where their lists differ each head gets its
//               own issuer, so neither waits for the other's softmax
//   warp 3      idle (it only completes the control warpgroup, which gives most of its registers
//               to the softmax warpgroups with setmaxnreg)
//   warps 4-7   softmax warpgroup of head A: a thread owns one query row; tcgen05.ld of S, base-2
//               online softmax with scale*log2(e) folded in, P rounded to bf16 and written back
//               over S with tcgen05.st, O rescaled in TMEM only when the running maximum moved by
//               more than 2^8 (exact: the final normalisation uses the same reference point)
//   warps 8-11  the same for head B
//
// TMEM (512 columns): S_A/P_A [0,128)  S_B/P_B [128,256)  O_A [256,384)  O_B [384,512).
// Arithmetic matches block_wise_prefill_attention_kernel (attn/shareprefill_attn.py:381-471):
// fp32 scores, causal mask on the diagonal block, P -> bf16 before P V, fp32 accumulation, bf16
// output.  Every mbarrier wait is bounded; on a timeout the CTA raises a shared abort flag, all
// roles drain and the kernel returns after recording the event in a device-side counter.
#include <cuda.h>

#include "spf_internal.cuh"

namespace spf {

constexpr int TC_BS = 128;
constexpr int TC_D = 128;
constexpr int TC_THREADS = 384;                             // 3 warpgroups: control, softmax A, softmax B
constexpr int TC_KSTAGES = 3;
constexpr int TC_VSTAGES = 2;
constexpr uint32_t TC_TILE_BYTES = TC_BS * TC_D * 2;        // 32 KiB: one 128x128 bf16 tile
constexpr uint32_t TC_SLAB_BYTES = TC_TILE_BYTES / 2;       // [128 rows][64 elements]
// shared memory map: 1 KiB of control data, then 1024-byte aligned tiles (Q x2, K x3, V x2)
constexpr uint32_t TC_SMEM_CTRL = 0;                        // mbarriers, TMEM slot, abort flag
constexpr uint32_t TC_SMEM_Q = 1024;
constexpr uint32_t TC_SMEM_K = TC_SMEM_Q + 2 * TC_TILE_BYTES;
constexpr uint32_t TC_SMEM_V = TC_SMEM_K + TC_KSTAGES * TC_TILE_BYTES;
constexpr uint32_t TC_SMEM_TOTAL = TC_SMEM_V + TC_VSTAGES * TC_TILE_BYTES;   // 225 KiB of the 227 KiB limit
constexpr float TC_RESCALE_LOG2 = 8.0f;

static __device__ unsigned int g_tc5_timeouts = 0;

// Timing probe, compiled in only with -DSPF_TC5_TRACE: clock64() stamps of the first CTA's
// first 64 iterations, [role: softmax A, softmax B, MMA issuer][iteration][slot].
#ifdef SPF_TC5_TRACE
__device__ long long g_tc5_trace[3][64][8];
#define TRACE(role, it, slot) do { if (blockIdx.x == 0 && (it) < 64) g_tc5_trace[role][it][slot] = clock64(); } while (0)
#else
#define TRACE(role, it, slot) do {} while (0)
#endif

struct Tc5Params {
  __nv_bfloat16* out;
  const uint32_t* bitmap;
  int n_tokens, n_q_heads, n_kv_heads, group, pairs, nb, nbw;
  float scale_log2;
};

// ---------------------------------------------------------------- PTX wrappers
__device__ __forceinline__ uint32_t smem_addr(const void* p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, 2000;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long global_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
  return t;
}
// Bounded wait: false once the CTA has aborted (unless `drain`) or after ~1 s without completion.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          bool drain = false) {
  if (mbar_try(bar, parity)) return true;
  const unsigned long long t0 = global_ns();
  int spins = 0;
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if ((++spins & 63) == 0) {
      if (*abort_flag && !drain) return false;
      if (global_ns() - t0 > 1000000000ull) {
        *abort_flag = 1;
        atomicAdd(&g_tc5_timeouts, 1u);
        return false;
      }
    }
  }
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y, int z) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
      ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y), "r"(z) : "memory");
}

// D(tmem) (+)= A(smem desc) * B(smem desc)
__device__ __forceinline__ void mma_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}
// D(tmem) (+)= A(tmem) * B(smem desc)
__device__ __forceinline__ void mma_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
      ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(acc) : "memory");
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 32 consecutive columns of this thread's TMEM lane, no wait (pair with tc_wait_ld)
__device__ __forceinline__ void tmem_ld32_raw(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
}
// columns whose index exceeds `last` are masked out (-inf)
__device__ __forceinline__ void mask_after(uint32_t (&r)[32], int last) {
#pragma unroll
  for (int j = 0; j < 32; ++j)
    if (j > last) r[j] = 0xff800000u;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ float row_max(const uint32_t (&r)[32]) {
  float a = __uint_as_float(r[0]), b = __uint_as_float(r[1]);
#pragma unroll
  for (int j = 2; j < 30; j += 4) {
    a = max3(a, __uint_as_float(r[j]), __uint_as_float(r[j + 1]));
    b = max3(b, __uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
  }
  return max3(fmaxf(a, b), __uint_as_float(r[30]), __uint_as_float(r[31]));
}
__device__ __forceinline__ float fast_exp2(float x);
// two fp32 lanes in one 64-bit register (packed fp32x2 arithmetic of sm_100)
__device__ __forceinline__ unsigned long long f2_pack(float lo, float hi) {
  unsigned long long d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "r"(__float_as_uint(lo)), "r"(__float_as_uint(hi)));
  return d;
}
__device__ __forceinline__ void f2_unpack(unsigned long long v, float& lo, float& hi) {
  uint32_t a, b;
  asm("mov.b64 {%0, %1}, %2;" : "=r"(a), "=r"(b) : "l"(v));
  lo = __uint_as_float(a); hi = __uint_as_float(b);
}
__device__ __forceinline__ unsigned long long f2_fma(unsigned long long a, unsigned long long b, unsigned long long c) {
  unsigned long long d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ unsigned long long f2_add(unsigned long long a, unsigned long long b) {
  unsigned long long d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint32_t bf16x2_from(float lo, float hi) {
  uint32_t d;
  asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(d) : "f"(hi), "f"(lo));   // first source -> upper half
  return d;
}
// p = 2^(s*scale - m) for 32 scores: packed to bf16 pairs, unrounded values summed into `sum`
__device__ __forceinline__ void exp_pack(const uint32_t (&r)[32], float scale, float m, uint32_t (&pk)[16], float& sum) {
  const unsigned long long sc2 = f2_pack(scale, scale), nm2 = f2_pack(-m, -m);
  unsigned long long acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    const unsigned long long x = f2_pack(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
    float y0, y1;
    f2_unpack(f2_fma(x, sc2, nm2), y0, y1);
    const float p0 = fast_exp2(y0), p1 = fast_exp2(y1);
    acc[(j >> 1) & 3] = f2_add(acc[(j >> 1) & 3], f2_pack(p0, p1));
    pk[j >> 1] = bf16x2_from(p0, p1);
  }
  float a0, a1;
  f2_unpack(f2_add(f2_add(acc[0], acc[1]), f2_add(acc[2], acc[3])), a0, a1);
  sum += a0 + a1;
}

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr) : "memory");
  tc_wait_ld();
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float (&v)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,"
      "%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,%32};"
      ::"r"(taddr),
        "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])), "r"(__float_as_uint(v[3])),
        "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])), "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])),
        "r"(__float_as_uint(v[8])), "r"(__float_as_uint(v[9])), "r"(__float_as_uint(v[10])), "r"(__float_as_uint(v[11])),
        "r"(__float_as_uint(v[12])), "r"(__float_as_uint(v[13])), "r"(__float_as_uint(v[14])), "r"(__float_as_uint(v[15])),
        "r"(__float_as_uint(v[16])), "r"(__float_as_uint(v[17])), "r"(__float_as_uint(v[18])), "r"(__float_as_uint(v[19])),
        "r"(__float_as_uint(v[20])), "r"(__float_as_uint(v[21])), "r"(__float_as_uint(v[22])), "r"(__float_as_uint(v[23])),
        "r"(__float_as_uint(v[24])), "r"(__float_as_uint(v[25])), "r"(__float_as_uint(v[26])), "r"(__float_as_uint(v[27])),
        "r"(__float_as_uint(v[28])), "r"(__float_as_uint(v[29])), "r"(__float_as_uint(v[30])), "r"(__float_as_uint(v[31]))
      : "memory");
}
// 16 packed bf16x2 words -> 16 consecutive columns
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
      ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]),
        "r"(r[8]), "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
      : "memory");
}

__device__ __forceinline__ uint32_t pack2_bf16(float lo, float hi) {
  const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return (static_cast<uint32_t>(__bfloat16_as_ushort(v.y)) << 16) | __bfloat16_as_ushort(v.x);
}

// shared-memory matrix descriptors, 128-byte swizzle, descriptor version 1
// K-major operand ([rows][64 elements] slabs, 8-row groups 1024 bytes apart)
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t saddr) {
  return (uint64_t((saddr >> 4) & 0x3fff)) | (uint64_t(1) << 16) | (uint64_t(1024 >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// MN-major operand (V: [keys][64 d] slabs; 8-key groups 1024 bytes apart, 64-d slabs 16 KiB apart)
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t saddr) {
  return (uint64_t((saddr >> 4) & 0x3fff)) | (uint64_t(TC_SLAB_BYTES >> 4) << 16) | (uint64_t(1024 >> 4) << 32) |
         (uint64_t(1) << 46) | (uint64_t(2) << 61);
}
// instruction descriptor: bf16 x bf16 -> fp32, M = 128, N = 128
constexpr uint32_t TC_IDESC_QK = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(128 >> 3) << 17) | (uint32_t(128 >> 4) << 24);
constexpr uint32_t TC_IDESC_PV = TC_IDESC_QK | (1u << 16);   // B (V) is MN-major

// The eight k-steps of one 128x128x128 product in a single instruction stream: the descriptors of
// consecutive steps differ only in the 14-bit address field, so each step costs one 32-bit add per
// operand and the tcgen05.mma itself (the issuing warp shares its scheduler with softmax warps).
// S (tmem) = Q (smem) K^T (smem): steps 0-3 walk the first 64-element slab in 32-byte strides, 4-7 the second.
__device__ __forceinline__ void mma_qk_group(uint32_t d_tmem, uint64_t q_desc, uint64_t k_desc) {
  constexpr uint32_t STEP = 32 >> 4, SLAB = (TC_SLAB_BYTES - 3 * 32) >> 4;
  asm volatile(
      "{\n\t.reg .pred pz, po;\n\t.reg .b32 alo, ahi, blo, bhi;\n\t.reg .b64 da, db;\n\t"
      "mov.b64 {alo, ahi}, %1;\n\tmov.b64 {blo, bhi}, %2;\n\t"
      "setp.ne.b32 pz, 0, 0;\n\tsetp.eq.b32 po, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, pz;\n\t"
      "add.u32 alo, alo, %4;\n\tadd.u32 blo, blo, %4;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t"
      "add.u32 alo, alo, %4;\n\tadd.u32 blo, blo, %4;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t"
      "add.u32 alo, alo, %4;\n\tadd.u32 blo, blo, %4;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t"
      "add.u32 alo, alo, %5;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t"
      "add.u32 alo, alo, %4;\n\tadd.u32 blo, blo, %4;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t"
      "add.u32 alo, alo, %4;\n\tadd.u32 blo, blo, %4;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t"
      "add.u32 alo, alo, %4;\n\tadd.u32 blo, blo, %4;\n\tmov.b64 da, {alo, ahi};\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], da, db, %3, po;\n\t}"
      ::"r"(d_tmem), "l"(q_desc), "l"(k_desc), "r"(TC_IDESC_QK), "n"(STEP), "n"(SLAB) : "memory");
}
// O (tmem) (+)= P (tmem, 16 bf16 columns = 8 words per step) V (smem, 16 keys = 2048 bytes per step)
__device__ __forceinline__ void mma_pv_group(uint32_t o_tmem, uint32_t p_tmem, uint64_t v_desc, uint32_t acc) {
  constexpr uint32_t VSTEP = 2048 >> 4;
  asm volatile(
      "{\n\t.reg .pred pa, po;\n\t.reg .b32 blo, bhi, ta;\n\t.reg .b64 db;\n\t"
      "mov.b64 {blo, bhi}, %2;\n\tmov.b32 ta, %1;\n\t"
      "setp.ne.b32 pa, %4, 0;\n\tsetp.eq.b32 po, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], %2, %3, pa;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t"
      "add.u32 ta, ta, 8;\n\tadd.u32 blo, blo, %5;\n\tmov.b64 db, {blo, bhi};\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [ta], db, %3, po;\n\t}"
      ::"r"(o_tmem), "r"(p_tmem), "l"(v_desc), "r"(TC_IDESC_PV), "r"(acc), "n"(VSTEP) : "memory");
}

// Walks the union of two bitmap rows in ascending column order; flags bit h = head h visits it.
struct PairWalker {
  const uint32_t* wa; const uint32_t* wb;
  int row, nwords, w;
  uint32_t ca, cb;
  __device__ uint32_t lim(int wi, uint32_t x) const {
    const int last = row - (wi << 5);
    return last >= 31 ? x : (x & ((2u << last) - 1u));
  }
  __device__ void load(int wi) {
    ca = wa ? lim(wi, __ldg(wa + wi)) : 0u;
    cb = wb ? lim(wi, __ldg(wb + wi)) : 0u;
  }
  __device__ void init(const uint32_t* a, const uint32_t* b, int row_) {
    wa = a; wb = b; row = row_; nwords = (row_ >> 5) + 1; w = 0;
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
                       const __grid_constant__ CUtensorMap map_v, const Tc5Params p) {
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
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + TC_SMEM_CTRL + 8 * 17);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + TC_SMEM_CTRL + 8 * 17 + 8);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // CTAs that run at the same time belong to the same KV head (its K/V stream stays in L2);
  // within a KV head the heavy (late) query blocks go first
  int bid = blockIdx.x;
  const int pair = bid % p.pairs; bid /= p.pairs;
  const int r = p.nb - 1 - (bid % p.nb);
  const int kvh = bid / p.nb;
  const int hA = kvh * p.group + pair * 2;
  const bool hasB = (pair * 2 + 1) < p.group;
  const int hB = hasB ? hA + 1 : -1;
  const int row0 = r * TC_BS;
  const uint32_t* rowA = p.bitmap + (int64_t(hA) * p.nb + r) * p.nbw;
  const uint32_t* rowB = hasB ? p.bitmap + (int64_t(hB) * p.nb + r) * p.nbw : nullptr;

  if (tid == 0) {
    mbar_init(bar_q, 1);
    for (int s = 0; s < TC_KSTAGES; ++s) { mbar_init(bar_kfull(s), 1); mbar_init(bar_kempty(s), 2); }
    for (int s = 0; s < TC_VSTAGES; ++s) { mbar_init(bar_vfull(s), 1); mbar_init(bar_vempty(s), 2); }
    for (int h = 0; h < 2; ++h) { mbar_init(bar_sfull(h), 1); mbar_init(bar_pready(h), 128); mbar_init(bar_odone(h), 1); }
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
    // control warpgroup (producer, MMA issuer, two idle warps) hands registers to the softmax warpgroups
    asm volatile("setmaxnreg.dec.sync.aligned.u32 88;");
  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      mbar_expect_tx(bar_q, (hasB ? 2u : 1u) * TC_TILE_BYTES);
      for (int h = 0; h < (hasB ? 2 : 1); ++h) {
        const uint32_t dst = sbase + TC_SMEM_Q + h * TC_TILE_BYTES;
        tma_load_3d(dst, &map_q, bar_q, 0, row0, hA + h);
        tma_load_3d(dst + TC_SLAB_BYTES, &map_q, bar_q, 64, row0, hA + h);
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
      PairWalker wk; wk.init(rowA, rowB, r);
      int fl, i = 0, k_issued = 0, v_issued = 0;
      int col = wk.next(fl);
      bool ok = true;
      if (col >= 0) { ok = load_k(0, col); k_issued = ok ? 1 : 0; }
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
    // ------------------------------------------------------------ MMA issuers (warp 1, warp 2)
    // Two ways to run the CTA's pair of rows, chosen from the two bitmap rows (the same answer in both
    // warps):
    //  * alternating: warp 1 issues for both heads in the fixed order P V of A, next Q K^T of A, P V of
    //    B, next Q K^T of B, which keeps the two softmax warpgroups half a period apart; best where
    //    the heads visit (nearly) the same blocks.  Warp 2 does nothing.
    //  * split: warp 1 issues for head A and warp 2 for head B, so a head never waits for the other
    //    head's softmax on a block it does not visit; best where the lists differ.  Both walk the
    //    union of the rows in the producer's order and take part in the hand-shake of every tile (a
    //    tile the head does not visit is passed on as soon as it has landed), so the phase of a ring
    //    stage can never run ahead of an issuer that skips it.
    // Every K/V ring stage is released by two arrivals: one per issuer in split mode, both from warp 1
    // in alternating mode.  These warps share their schedulers with the softmax warps, whose
    // instruction issue is the bottleneck of the kernel: every instruction here is paid for there.
    if (lane == 0) {
      const int me = warp - 1;
      // blocks of head A, of head B and of their union in this row; split where the lists differ enough
      int cnt_a = 0, cnt_b = 0, cnt_u = 0;
      for (int i = 0; i <= (r >> 5); ++i) {
        const int last = r - (i << 5);
        const uint32_t m = last >= 31 ? 0xffffffffu : ((2u << last) - 1u);
        const uint32_t wa = __ldg(rowA + i) & m, wb = hasB ? (__ldg(rowB + i) & m) : 0u;
        cnt_a += __popc(wa); cnt_b += __popc(wb); cnt_u += __popc(wa | wb);
      }
      const bool split = hasB && 4 * cnt_u > 5 * max(cnt_a, cnt_b);
      // descriptors differ from a base only in the 14-bit address field: one 64-bit add per operand
      const uint64_t qdA = desc_kmajor(sbase + TC_SMEM_Q), qdB = desc_kmajor(sbase + TC_SMEM_Q + TC_TILE_BYTES);
      const uint64_t kd0 = desc_kmajor(sbase + TC_SMEM_K), vd0 = desc_mnmajor(sbase + TC_SMEM_V);
      auto issue_qk = [&](int h, int ks_stage) {
        const uint64_t kd = kd0 + uint64_t((ks_stage * TC_TILE_BYTES) >> 4);
        const uint64_t qd = h == 0 ? qdA : qdB;
        const uint32_t ts = tmem + (h == 0 ? 0u : 128u);
        mma_qk_group(ts, qd, kd);
        tc_commit(bar_sfull(h));
      };
      auto issue_pv = [&](int h, int vs_stage, bool accumulate) {
        const uint64_t vd = vd0 + uint64_t((vs_stage * TC_TILE_BYTES) >> 4);
        const uint32_t ts = tmem + (h == 0 ? 0u : 128u), to = tmem + (h == 0 ? 256u : 384u);
        mma_pv_group(to, ts, vd, accumulate ? 1u : 0u);
      };
      bool ok = mbar_wait(bar_q, 0, abort_flag);
      PairWalker wk; wk.init(rowA, rowB, r);
      int fl, nfl;
      int col = wk.next(fl);
      int i = 0;
      if (!split && me == 0) {
        // ---- alternating mode: warp 1 for both heads
        int nblk[2] = {0, 0};     // P tiles consumed per head
        if (ok && col >= 0) {
          ok = mbar_wait(bar_kfull(0), 0, abort_flag);
          tc_fence_after();
          if (ok) {
            for (int h = 0; h < 2; ++h) if (fl & (1 << h)) issue_qk(h, 0);
            mbar_arrive(bar_kempty(0));
            tc_commit(bar_kempty(0));
          }
        }
        while (ok && col >= 0) {
          const int ncol = wk.next(nfl);
          const int vs = i % TC_VSTAGES, nks = (i + 1) % TC_KSTAGES;
          bool v_ready = false, nk_ready = false;
          const int last_h = (fl & 2) ? 1 : 0;
          const int nlast_h = (nfl & 2) ? 1 : 0;
          for (int h = 0; h < 2 && ok; ++h) {
            if (fl & (1 << h)) {
              if (!v_ready) { ok = mbar_wait(bar_vfull(vs), (i / TC_VSTAGES) & 1, abort_flag); v_ready = true; }
              if (h == 0) TRACE(2, i, 0); else TRACE(2, i, 4);
              if (ok) ok = mbar_wait(bar_pready(h), nblk[h] & 1, abort_flag);
              if (!ok) break;
              tc_fence_after();
              if (h == 0) TRACE(2, i, 1); else TRACE(2, i, 5);
              issue_pv(h, vs, nblk[h] > 0);
              if (h == 0) TRACE(2, i, 2); else TRACE(2, i, 6);
              ++nblk[h];
              if (h == last_h) { mbar_arrive(bar_vempty(vs)); tc_commit(bar_vempty(vs)); }
            }
            if (ncol >= 0 && (nfl & (1 << h))) {
              if (!nk_ready) { ok = mbar_wait(bar_kfull(nks), ((i + 1) / TC_KSTAGES) & 1, abort_flag); nk_ready = true; }
              if (!ok) break;
              tc_fence_after();
              issue_qk(h, nks);
              if (h == nlast_h) { mbar_arrive(bar_kempty(nks)); tc_commit(bar_kempty(nks)); }
              if (h == 0) TRACE(2, i, 3); else TRACE(2, i, 7);
            }
          }
          col = ncol; fl = nfl; ++i;
        }
        tc_commit(bar_odone(0));
        tc_commit(bar_odone(1));
      } else if (split) {
        // ---- split mode: this thread issues for head `me` and passes the other head's tiles on
        const int h = me, mine = 1 << me;
        int np = 0;               // P tiles consumed
        if (ok && col >= 0) {
          ok = mbar_wait(bar_kfull(0), 0, abort_flag);
          if (ok) {
            if (fl & mine) { tc_fence_after(); issue_qk(h, 0); tc_commit(bar_kempty(0)); }
            else mbar_arrive(bar_kempty(0));
          }
        }
        while (ok && col >= 0) {
          const int ncol = wk.next(nfl);
          const int vs = i % TC_VSTAGES, nks = (i + 1) % TC_KSTAGES;
          ok = mbar_wait(bar_vfull(vs), (i / TC_VSTAGES) & 1, abort_flag);
          if (!ok) break;
          if (fl & mine) {
            ok = mbar_wait(bar_pready(h), np & 1, abort_flag);
            if (!ok) break;
            tc_fence_after();
            issue_pv(h, vs, np > 0);
            ++np;
            tc_commit(bar_vempty(vs));
          } else {
            mbar_arrive(bar_vempty(vs));
          }
          if (ncol >= 0) {
            ok = mbar_wait(bar_kfull(nks), ((i + 1) / TC_KSTAGES) & 1, abort_flag);
            if (!ok) break;
            if (nfl & mine) { tc_fence_after(); issue_qk(h, nks); tc_commit(bar_kempty(nks)); }
            else mbar_arrive(bar_kempty(nks));
          }
          col = ncol; fl = nfl; ++i;
        }
        tc_commit(bar_odone(h));
      }
    }
  }
  } else {
    // ------------------------------------------------------------ softmax warpgroups
    asm volatile("setmaxnreg.inc.sync.aligned.u32 208;");
    const int h = (warp - 4) >> 2;                 // 0: head A, 1: head B
    const int quarter = warp & 3;                  // TMEM lane quarter this warp may touch
    const int row = quarter * 32 + lane;           // query row within the block
    const int head = h == 0 ? hA : hB;
    const uint32_t lane_base = uint32_t(quarter * 32) << 16;
    const uint32_t tS = tmem + lane_base + uint32_t(h * 128);
    const uint32_t tO = tmem + lane_base + uint32_t(256 + h * 128);
    float m_used = -INFINITY, l_sum = 0.f;
    int k = 0;
    bool ok = head >= 0;
    if (ok) {
      PairWalker wk; wk.init(h == 0 ? rowA : rowB, nullptr, r);
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
        const float mx = fmaxf(fmaxf(row_max(s0), row_max(s1)), fmaxf(row_max(s2), row_max(s3)));
        const float mb = mx * p.scale_log2;
        float alpha = 1.f;
        bool grow = false;
        if (k == 0) {
          m_used = mb;
        } else if (mb > m_used + TC_RESCALE_LOG2) {
          alpha = exp2f(m_used - mb);
          m_used = mb;
          l_sum *= alpha;
          grow = true;
        }
        if (__any_sync(0xffffffffu, grow)) {
          // S_h(k) is complete, hence so is every earlier P V of this head: O_h is stable
#pragma unroll 1
          for (int c = 0; c < 4; ++c) {
            float v[32];
            tmem_ld32(tO + c * 32, v);
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= alpha;
            tmem_st32(tO + c * 32, v);
          }
        }
        // P = 2^(s*scale - m) as bf16 over the first 64 columns of the S region
        float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f;
        uint32_t pk[16];
        exp_pack(s0, p.scale_log2, m_used, pk, l0); tmem_st16(tS + 0, pk);
        exp_pack(s1, p.scale_log2, m_used, pk, l1); tmem_st16(tS + 16, pk);
        exp_pack(s2, p.scale_log2, m_used, pk, l2); tmem_st16(tS + 32, pk);
        exp_pack(s3, p.scale_log2, m_used, pk, l3); tmem_st16(tS + 48, pk);
        l_sum += (l0 + l1) + (l2 + l3);
        if (lane == 0 && quarter == 0) TRACE(h, k, 3);
        tc_wait_st();
        tc_fence_before();
        mbar_arrive(bar_pready(h));
        if (lane == 0 && quarter == 0) TRACE(h, k, 4);
      }
      // ---- epilogue
      const int tok = row0 + row;
      __nv_bfloat16* orow = p.out + (int64_t(tok) * p.n_q_heads + head) * TC_D;
      if (ok && k > 0) ok = mbar_wait(bar_odone(h), 0, abort_flag);
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
          if (tok < p.n_tokens) {
#pragma unroll
            for (int j = 0; j < 32; j += 8) {
              uint4 o;
              o.x = pack2_bf16(v[j] * inv, v[j + 1] * inv);
              o.y = pack2_bf16(v[j + 2] * inv, v[j + 3] * inv);
              o.z = pack2_bf16(v[j + 4] * inv, v[j + 5] * inv);
              o.w = pack2_bf16(v[j + 6] * inv, v[j + 7] * inv);
              *reinterpret_cast<uint4*>(orow + c * 32 + j) = o;
            }
          }
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

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (!fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// [N][heads][128] bf16 view (strides in elements) as a 3-D tensor (d, token, head); box 64 x 128 x 1
static bool make_map(CUtensorMap* m, const void* base, int n_tokens, int heads, int64_t sn, int64_t sh) {
  EncodeTiledFn fn = encode_fn();
  if (!fn) return false;
  const cuuint64_t dims[3] = {cuuint64_t(TC_D), cuuint64_t(n_tokens), cuuint64_t(heads)};
  const cuuint64_t strides[2] = {cuuint64_t(sn) * 2, cuuint64_t(sh) * 2};
  const cuuint32_t box[3] = {64, TC_BS, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  return fn(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
            CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
            CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

// Returns SPF_ERR_SHAPE when the tensors cannot be described to TMA (the caller then uses the
// generic kernel).
int sparse_attention_tc5(const AttnParams& a, int n_kv_heads, cudaStream_t st) {
  if (a.q_sn <= 0 || a.k_sn <= 0 || a.v_sn <= 0 || a.q_sh <= 0 || a.k_sh <= 0 || a.v_sh <= 0) return SPF_ERR_SHAPE;
  CUtensorMap mq, mk, mv;
  if (!make_map(&mq, a.q, a.n_tokens, a.n_q_heads, a.q_sn, a.q_sh) ||
      !make_map(&mk, a.k, a.n_tokens, n_kv_heads, a.k_sn, a.k_sh) ||
      !make_map(&mv, a.v, a.n_tokens, n_kv_heads, a.v_sn, a.v_sh))
    return SPF_ERR_SHAPE;
  Tc5Params p;
  p.out = a.out; p.bitmap = a.bitmap; p.n_tokens = a.n_tokens; p.n_q_heads = a.n_q_heads;
  p.n_kv_heads = n_kv_heads; p.group = a.group; p.pairs = (a.group + 1) / 2; p.nb = a.nb; p.nbw = a.nbw;
  p.scale_log2 = a.scale_log2;
  cudaError_t e = cudaFuncSetAttribute(sparse_attn_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                       int(TC_SMEM_TOTAL));
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  const unsigned grid = unsigned(a.nb) * unsigned(n_kv_heads) * unsigned(p.pairs);
  sparse_attn_tc5_kernel<<<grid, TC_THREADS, TC_SMEM_TOTAL, st>>>(mq, mk, mv, p);
  return check_launch();
}

#ifdef SPF_TC5_TRACE
extern "C" void spf_tc5_trace_dump(long long* out) { cudaMemcpyFromSymbol(out, g_tc5_trace, sizeof(long long) * 3 * 64 * 8); }
#endif

unsigned int tc5_timeout_count() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc5_timeouts, sizeof(v));
  return v;
}

}  // namespace spf
