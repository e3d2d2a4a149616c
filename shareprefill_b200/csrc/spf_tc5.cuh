// tcgen05 / TMEM / TMA building blocks shared by the sm_100a kernels (block-sparse attention,
// last-block profile): mbarrier and TMA wrappers with bounded waits, TMEM loads and stores,
// shared-memory matrix descriptors for 128-byte swizzled [128][64]-element bf16 slabs, grouped
// tcgen05.mma issue, and the host-side tensor-map encoder.  Every translation unit that includes
// this header gets its own timeout counter.
#pragma once

#include <cuda.h>

#include "spf_internal.cuh"

namespace spf {

constexpr int TC_BS = 128;
constexpr int TC_D = 128;
constexpr uint32_t TC_TILE_BYTES = TC_BS * TC_D * 2;        // 32 KiB: one 128x128 bf16 tile
constexpr uint32_t TC_SLAB_BYTES = TC_TILE_BYTES / 2;       // [128 rows][64 elements]

// bounded device-side waits that gave up (read back by the host after a run)
static __device__ unsigned int g_tc5_timeouts = 0;
// how long a wait may spin before it gives up (1 s; tests shorten it)
static __constant__ unsigned long long c_tc5_wait_limit_ns = 1000000000ull;

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
// Bounded wait: false once the CTA has aborted (unless `drain`) or after the wait limit has been spent
// SPINNING.  Time is added up between consecutive looks at the clock and a single gap counts for at
// most 1 ms, so a CTA that was not running for a while (a time slice taken by another context, a
// profiler replay) is not mistaken for one that hangs.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag,
                                          bool drain = false) {
  if (mbar_try(bar, parity)) return true;
  unsigned long long last = global_ns(), spent = 0;
  int spins = 0;
  while (true) {
    if (mbar_try(bar, parity)) return true;
    if ((++spins & 63) == 0) {
      if (*abort_flag && !drain) return false;
      const unsigned long long now = global_ns(), gap = now - last;
      last = now;
      spent += gap < 1000000ull ? gap : 1000000ull;
      if (spent > c_tc5_wait_limit_ns) {
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

// the first copy through a tensor map otherwise waits for the map itself to be fetched
__device__ __forceinline__ void tma_prefetch_map(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}
// store of a shared-memory tile (the layout a load with the same map produces) to global memory; the
// issuing thread commits the group and waits until the tile has been read out of shared memory
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(map), "r"(src), "r"(x), "r"(y), "r"(z) : "memory");
}
__device__ __forceinline__ void tma_store_commit_and_wait_read() {
  asm volatile("cp.async.bulk.commit_group;" ::: "memory");
  asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
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
// p = 2^(s*scale - m) for 32 scores: packed to bf16 pairs, unrounded values summed into `sum`.
// POLY of every 8 element pairs are taken off the exponential unit (16 exponentials per clock and
// SM): their 2^y comes from a range reduction and a degree-3 polynomial on the FMA pipe
// (relative error 7.5e-5, far below the bf16 rounding of P).
//   u = sat((y + 57) / 128)         y = s*scale - m clamped to [-57, 71]: the reference point m never
//                                   exceeds the row's true maximum, so 2^-57 is noise against l >= 1
//   n = round(128u - 57) by the 1.5 * 2^23 trick;  f = 128u - 57 - n in [-0.5, 0.5]
//   2^y = poly(f) * 2^n             n is added to the exponent field of poly(f)
template <int POLY>
__device__ __forceinline__ void exp_pack_poly(const uint32_t (&r)[32], float scale, float m, uint32_t (&pk)[16], float& sum) {
  const unsigned long long sc2 = f2_pack(scale, scale), nm2 = f2_pack(-m, -m);
  const float sc128 = scale * 0.0078125f, b128 = (57.f - m) * 0.0078125f;
  constexpr float MAGIC = 12582912.f - 57.f;      // 1.5 * 2^23 - 57
  const unsigned long long k128 = f2_pack(128.f, 128.f), kmag = f2_pack(MAGIC, MAGIC), kneg = f2_pack(-1.f, -1.f);
  const unsigned long long c0 = f2_pack(0.99992806f, 0.99992806f), c1 = f2_pack(0.69326097f, 0.69326097f),
                           c2 = f2_pack(0.24261113f, 0.24261113f), c3 = f2_pack(0.05517167f, 0.05517167f);
  unsigned long long acc[4] = {0ull, 0ull, 0ull, 0ull};
#pragma unroll
  for (int j = 0; j < 32; j += 2) {
    float p0, p1;
    if (((j >> 1) & 7) < POLY) {
      const float u0 = __saturatef(fmaf(__uint_as_float(r[j]), sc128, b128));
      const float u1 = __saturatef(fmaf(__uint_as_float(r[j + 1]), sc128, b128));
      const unsigned long long u = f2_pack(u0, u1);
      const unsigned long long xf = f2_fma(u, k128, kmag);          // MAGIC + n (n in the low mantissa bits)
      const unsigned long long c = f2_fma(xf, kneg, kmag);          // -(57 + n)
      const unsigned long long f = f2_fma(u, k128, c);
      unsigned long long pl = f2_fma(f, c3, c2);
      pl = f2_fma(pl, f, c1);
      pl = f2_fma(pl, f, c0);
      float q0, q1, x0, x1;
      f2_unpack(pl, q0, q1);
      f2_unpack(xf, x0, x1);
      p0 = __uint_as_float(__float_as_uint(q0) + (__float_as_uint(x0) << 23));
      p1 = __uint_as_float(__float_as_uint(q1) + (__float_as_uint(x1) << 23));
    } else {
      const unsigned long long x = f2_pack(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
      float y0, y1;
      f2_unpack(f2_fma(x, sc2, nm2), y0, y1);
      p0 = fast_exp2(y0); p1 = fast_exp2(y1);
    }
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
// The same products with every descriptor prepared BEFORE the first tcgen05.mma, so that the eight
// instructions leave the issuing thread back to back (the attention kernel keeps the descriptors of
// every tile in a shared-memory table).
struct KSteps { uint64_t d[8]; };
__device__ __forceinline__ void mma_qk_x8(uint32_t d_tmem, const KSteps& a, const KSteps& b) {
  asm volatile(
      "{\n\t.reg .pred pz, po;\n\t"
      "setp.ne.b32 pz, 0, 0;\n\tsetp.eq.b32 po, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %2, %10, %1, pz;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %3, %11, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %4, %12, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %5, %13, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %6, %14, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %7, %15, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %8, %16, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %9, %17, %1, po;\n\t}"
      ::"r"(d_tmem), "r"(TC_IDESC_QK),
        "l"(a.d[0]), "l"(a.d[1]), "l"(a.d[2]), "l"(a.d[3]), "l"(a.d[4]), "l"(a.d[5]), "l"(a.d[6]), "l"(a.d[7]),
        "l"(b.d[0]), "l"(b.d[1]), "l"(b.d[2]), "l"(b.d[3]), "l"(b.d[4]), "l"(b.d[5]), "l"(b.d[6]), "l"(b.d[7])
      : "memory");
}
// O (+)= P V with P at p_tmem + 8 i (16 bf16 columns per step)
__device__ __forceinline__ void mma_pv_x8(uint32_t o_tmem, uint32_t p_tmem, const KSteps& v, uint32_t acc) {
  asm volatile(
      "{\n\t.reg .pred pa, po;\n\t"
      "setp.ne.b32 pa, %2, 0;\n\tsetp.eq.b32 po, 0, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%3], %11, %1, pa;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%4], %12, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%5], %13, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%6], %14, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%7], %15, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%8], %16, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%9], %17, %1, po;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%10], %18, %1, po;\n\t}"
      ::"r"(o_tmem), "r"(TC_IDESC_PV), "r"(acc),
        "r"(p_tmem), "r"(p_tmem + 8u), "r"(p_tmem + 16u), "r"(p_tmem + 24u), "r"(p_tmem + 32u), "r"(p_tmem + 40u),
        "r"(p_tmem + 48u), "r"(p_tmem + 56u),
        "l"(v.d[0]), "l"(v.d[1]), "l"(v.d[2]), "l"(v.d[3]), "l"(v.d[4]), "l"(v.d[5]), "l"(v.d[6]), "l"(v.d[7])
      : "memory");
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

// the counter and the wait limit exist once per translation unit that includes this header
static unsigned int tc5_read_timeouts_here() {
  unsigned int v = 0;
  cudaMemcpyFromSymbol(&v, g_tc5_timeouts, sizeof(v));
  return v;
}
static bool tc5_reset_timeouts_here() {
  const unsigned int z = 0;
  return cudaMemcpyToSymbol(g_tc5_timeouts, &z, sizeof(z)) == cudaSuccess;
}
static bool tc5_set_wait_limit_here(unsigned long long ns) {
  return cudaMemcpyToSymbol(c_tc5_wait_limit_ns, &ns, sizeof(ns)) == cudaSuccess;
}

}  // namespace spf
