// Last-block profile: softmax of the last `block_size` queries of every head against all
// keys, reduced to the vertical profile (mean over the queries) and the slash profile (mean
// over the queries along each anti-diagonal).  Restates attn/attention_sharing.py:127-167 and
// sum_all_diagonal_matrix (attn/utils.py:79-86) as a streaming two-pass computation that never
// materialises the [H, block, N] score tensor:
//   pass 1  per (key tile, head): logits on mma.sync, per-row tile max and sum of exp
//   reduce  per head: global row max M_i and normaliser Z_i
//   pass 2  per (key tile, head): recompute logits, p = exp(l - M_i) / Z_i into shared memory,
//           column sums -> vertical, anti-diagonal sums -> slash
// Rounding points follow the reference's bf16 path: q / sqrt(D) is rounded to bf16, logits are
// rounded to bf16 (its einsum output dtype) and the softmax runs in fp32.
// Each slash element receives at most two addends (from two adjacent key tiles) on a zeroed
// buffer, so the atomic adds are order independent.
#include <cstdlib>
#include <cstring>

#include "spf_internal.cuh"
#include "spf_mma.cuh"

namespace spf {

constexpr int EST_ROWS = 128;   // query rows per tile (block_size <= 128, padded)
constexpr int EST_COLS = 128;   // keys per tile
constexpr int EST_NT = 256;


// Stage bf16(q / sqrt(D)) for the last rq queries of head h (rows >= rq are zero) in shared
// memory and pull this warp's 16 rows into A fragments.  The staging area may be reused after
// the trailing barrier.
template <int D>
__device__ __forceinline__ void est_load_q(const EstParams& p, int h, uint32_t sq,
                                           uint32_t (&qf)[D / 16][4]) {
  constexpr int CHUNKS = D / 8;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int q0 = p.n_tokens - p.rq;
  unsigned char* sq_ptr = reinterpret_cast<unsigned char*>(__cvta_shared_to_generic(sq));
  for (int i = tid; i < EST_ROWS * CHUNKS; i += EST_NT) {
    const int row = i / CHUNKS, ch = i % CHUNKS;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (row < p.rq) {
      val = *reinterpret_cast<const uint4*>(p.q + int64_t(q0 + row) * p.q_sn + int64_t(h) * p.q_sh + ch * 8);
      __nv_bfloat162* pr = reinterpret_cast<__nv_bfloat162*>(&val);
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 f = __bfloat1622float2(pr[e]);
        pr[e] = __floats2bfloat162_rn(f.x / p.sqrt_d, f.y / p.sqrt_d);
      }
    }
    *reinterpret_cast<uint4*>(sq_ptr + tile_off<D>(row, ch)) = val;
  }
  __syncthreads();
  const int qrow = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) ldmatrix_x4(qf[ks], sq + tile_off<D>(qrow, ks * 2 + (lane >> 4)));
  __syncthreads();
}

// exp(x) through ex2.approx: the logits were rounded to bf16 already, a 2-ulp exponential is ample
__device__ __forceinline__ float est_exp(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x * 1.4426950408889634f));
  return y;
}

// Start the asynchronous copy of key tile `tile` of the head's KV head into shared memory at sk.
template <int D>
__device__ __forceinline__ void est_issue_tile(const EstParams& p, int h, int tile, uint32_t sk) {
  const int kvh = h / p.group;
  const int c0 = tile * EST_COLS;
  load_tile_async<EST_COLS, D, EST_NT>(sk, p.k + int64_t(kvh) * p.k_sh + int64_t(c0) * p.k_sn, p.k_sn,
                                       min(EST_COLS, p.n_tokens - c0), threadIdx.x);
}

// S = Q K^T for the key tile resident at sk, rounded to bf16, with the causal mask.
template <int D>
__device__ __forceinline__ void est_tile_scores(const EstParams& p, int tile, uint32_t sk,
                                                const uint32_t (&qf)[D / 16][4],
                                                float (&s)[EST_COLS / 8][4]) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int c0 = tile * EST_COLS;
  const int q0 = p.n_tokens - p.rq;
#pragma unroll
  for (int j = 0; j < EST_COLS / 8; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f; }
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
#pragma unroll
    for (int jp = 0; jp < EST_COLS / 16; ++jp) {
      uint32_t bf[4];
      const int krow = jp * 16 + (lane & 7) + (lane >> 4) * 8;
      ldmatrix_x4(bf, sk + tile_off<D>(krow, ks * 2 + ((lane >> 3) & 1)));
      mma_bf16_16816(s[2 * jp], qf[ks], bf[0], bf[1]);
      mma_bf16_16816(s[2 * jp + 1], qf[ks], bf[2], bf[3]);
    }
  }
  const int row_lo = warp * 16 + (lane >> 2);
  if (c0 + EST_COLS - 1 <= q0) {   // tile entirely before the first query: no mask needed
#pragma unroll
    for (int j = 0; j < EST_COLS / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) s[j][e] = bf16_round(s[j][e]);
    }
  } else {
#pragma unroll
    for (int j = 0; j < EST_COLS / 8; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kpos = c0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const int qpos = q0 + row_lo + (e >> 1) * 8;
        s[j][e] = (kpos > qpos) ? -INFINITY : bf16_round(s[j][e]);
      }
    }
  }
}

template <int D>
__global__ void __launch_bounds__(EST_NT) lastblock_stats_kernel(const EstParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr uint32_t TILE = EST_ROWS * D * 2;
  const uint32_t sbase = smem_u32(smem);      // two key tile buffers; the second stages Q first
  const int h = blockIdx.y;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t_begin = blockIdx.x * p.tiles_per_cta;
  const int t_end = min(p.ntiles, t_begin + p.tiles_per_cta);
  est_issue_tile<D>(p, h, t_begin, sbase);
  cp_async_commit();
  uint32_t qf[D / 16][4];
  est_load_q<D>(p, h, sbase + TILE, qf);
  for (int tile = t_begin; tile < t_end; ++tile) {
    const int buf = (tile - t_begin) & 1;
    if (tile + 1 < t_end) est_issue_tile<D>(p, h, tile + 1, sbase + (buf ^ 1) * TILE);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    float s[EST_COLS / 8][4];
    est_tile_scores<D>(p, tile, sbase + buf * TILE, qf, s);
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < EST_COLS / 8; ++j) {
      mx[0] = fmaxf(mx[0], fmaxf(s[j][0], s[j][1]));
      mx[1] = fmaxf(mx[1], fmaxf(s[j][2], s[j][3]));
    }
    float sum[2] = {0.f, 0.f};
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 1));
      mx[i] = fmaxf(mx[i], __shfl_xor_sync(0xffffffffu, mx[i], 2));
    }
    const float m0 = (mx[0] == -INFINITY) ? 0.f : mx[0];
    const float m1 = (mx[1] == -INFINITY) ? 0.f : mx[1];
#pragma unroll
    for (int j = 0; j < EST_COLS / 8; ++j) {
      sum[0] += est_exp(s[j][0] - m0) + est_exp(s[j][1] - m0);
      sum[1] += est_exp(s[j][2] - m1) + est_exp(s[j][3] - m1);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 1);
      sum[i] += __shfl_xor_sync(0xffffffffu, sum[i], 2);
    }
    if ((lane & 3) == 0) {
      const int row = warp * 16 + (lane >> 2);
      const int64_t base = (int64_t(h) * p.ntiles + tile) * EST_ROWS;
      p.part_m[base + row] = mx[0];
      p.part_l[base + row] = sum[0];
      p.part_m[base + row + 8] = mx[1];
      p.part_l[base + row + 8] = sum[1];
    }
    __syncthreads();   // everyone is done with this buffer before it is refilled
  }
  cp_async_wait<0>();
}

constexpr int RED_SLICES = 8;   // tile slices per head, one warpgroup-sized slice of threads each

__global__ void __launch_bounds__(EST_ROWS * RED_SLICES) lastblock_reduce_kernel(const EstParams p) {
  // thread (slice, row): running (max, sum) over the tiles slice, slice + 8, ...; slices merged in shared memory
  __shared__ float sm_m[RED_SLICES][EST_ROWS];
  __shared__ double sm_z[RED_SLICES][EST_ROWS];
  const int h = blockIdx.x, row = threadIdx.x % EST_ROWS, slice = threadIdx.x / EST_ROWS;
  const float* pm = p.part_m + int64_t(h) * p.n_parts * EST_ROWS + row;
  const float* pl = p.part_l + int64_t(h) * p.n_parts * EST_ROWS + row;
  float m = -INFINITY;
  for (int t = slice; t < p.n_parts; t += RED_SLICES) m = fmaxf(m, pm[int64_t(t) * EST_ROWS]);
  double z = 0.0;
  for (int t = slice; t < p.n_parts; t += RED_SLICES) {
    const float mt = pm[int64_t(t) * EST_ROWS];
    if (mt != -INFINITY) z += static_cast<double>(pl[int64_t(t) * EST_ROWS]) * static_cast<double>(est_exp(mt - m));
  }
  sm_m[slice][row] = m;
  sm_z[slice][row] = z;
  __syncthreads();
  if (slice == 0) {
    float mm = -INFINITY;
    for (int s = 0; s < RED_SLICES; ++s) mm = fmaxf(mm, sm_m[s][row]);
    double zz = 0.0;
    for (int s = 0; s < RED_SLICES; ++s)
      if (sm_m[s][row] != -INFINITY) zz += sm_z[s][row] * static_cast<double>(est_exp(sm_m[s][row] - mm));
    p.row_m[h * EST_ROWS + row] = mm;
    p.row_z[h * EST_ROWS + row] = static_cast<float>(zz);
  }
}

template <int D>
__global__ void __launch_bounds__(EST_NT, 2) lastblock_profile_kernel(const EstParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  // P rows are 136 floats apart: the 8-byte stores of the MMA fragment layout (4 rows x 8 columns per
  // half warp) then fall into distinct banks; column and anti-diagonal reads are conflict free anyway.
  // One key tile buffer only: two CTAs share an SM and cover each other's load and reduction phases.
  constexpr int LD = EST_COLS + 8;
  constexpr uint32_t P_BYTES = EST_ROWS * LD * 4;
  float* P = reinterpret_cast<float*>(smem);            // [128][136] fp32
  __shared__ float colpart[EST_COLS];
  const uint32_t sk = smem_u32(smem) + P_BYTES;         // key tile; stages Q first
  const int h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int t_begin = blockIdx.x * p.tiles_per_cta;
  const int t_end = min(p.ntiles, t_begin + p.tiles_per_cta);
  uint32_t qf[D / 16][4];
  est_load_q<D>(p, h, sk, qf);
  const int row_lo = warp * 16 + (lane >> 2);
  const float M0 = p.row_m[h * EST_ROWS + row_lo], M1 = p.row_m[h * EST_ROWS + row_lo + 8];
  const float R0 = 1.0f / p.row_z[h * EST_ROWS + row_lo], R1 = 1.0f / p.row_z[h * EST_ROWS + row_lo + 8];
  const int rq = p.rq;
  const float inv_rows = 1.0f / static_cast<float>(rq);
  for (int tile = t_begin; tile < t_end; ++tile) {
    est_issue_tile<D>(p, h, tile, sk);
    cp_async_commit();
    cp_async_wait<0>();
    __syncthreads();   // the tile has landed; the previous tile's sums are done reading P
    float s[EST_COLS / 8][4];
    est_tile_scores<D>(p, tile, sk, qf, s);
#pragma unroll
    for (int j = 0; j < EST_COLS / 8; ++j) {
      const int c = j * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(&P[row_lo * LD + c]) =
          make_float2(est_exp(s[j][0] - M0) * R0, est_exp(s[j][1] - M0) * R0);
      *reinterpret_cast<float2*>(&P[(row_lo + 8) * LD + c]) =
          make_float2(est_exp(s[j][2] - M1) * R1, est_exp(s[j][3] - M1) * R1);
    }
    __syncthreads();   // P complete; every warp is also done reading the key tile
    const int c0 = tile * EST_COLS;
    // anti-diagonals first (255 of them): element (i, jj) lands on tile-local index t = jj + (rq-1) - i
    for (int t = tid; t < EST_COLS + rq - 1; t += EST_NT) {
      const int i_lo = max(0, rq - 1 - t);
      const int i_hi = min(rq - 1, EST_COLS - 1 + rq - 1 - t);
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
      const float* base = P + (t - (rq - 1));
      int i = i_lo;
      for (; i + 3 <= i_hi; i += 4) {
        a0 += base[i * (LD + 1)];
        a1 += base[(i + 1) * (LD + 1)];
        a2 += base[(i + 2) * (LD + 1)];
        a3 += base[(i + 3) * (LD + 1)];
      }
      for (; i <= i_hi; ++i) a0 += base[i * (LD + 1)];
      const int n = c0 + t;
      if (n < p.n_tokens) atomicAdd(&p.slash[int64_t(h) * p.n_tokens + n], ((a0 + a1) + (a2 + a3)) * inv_rows);
    }
    // column sums: warps 0-3 take the even rows, warps 4-7 the odd rows (consecutive lanes read
    // consecutive columns), halves combined through shared memory
    {
      const int col = tid & (EST_COLS - 1), par = tid >> 7;
      float b0 = 0.f, b1 = 0.f;
      int i = par;
      for (; i + 2 < rq; i += 4) { b0 += P[i * LD + col]; b1 += P[(i + 2) * LD + col]; }
      for (; i < rq; i += 2) b0 += P[i * LD + col];
      const float acc = b0 + b1;
      if (par == 1) colpart[col] = acc;
      __syncthreads();
      if (par == 0 && c0 + col < p.n_tokens)
        p.vertical[int64_t(h) * p.n_tokens + c0 + col] = (acc + colpart[col]) * inv_rows;
    }
  }
}

void launch_lastblock_reduce(const EstParams& p, cudaStream_t st) {
  lastblock_reduce_kernel<<<p.n_q_heads, EST_ROWS * RED_SLICES, 0, st>>>(p);
}

template <int D>
static int launch_estimate(const EstParams& p, cudaStream_t st) {
  const dim3 grid(ceil_div(p.ntiles, p.tiles_per_cta), p.n_q_heads);
  constexpr int TILE = EST_ROWS * D * 2;
  constexpr int P_BYTES = EST_ROWS * (EST_COLS + 8) * 4;
  cudaError_t e;
  e = cudaFuncSetAttribute(lastblock_stats_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * TILE);
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  e = cudaFuncSetAttribute(lastblock_profile_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, P_BYTES + TILE);
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  lastblock_stats_kernel<D><<<grid, EST_NT, 2 * TILE, st>>>(p);
  lastblock_reduce_kernel<<<p.n_q_heads, EST_ROWS * RED_SLICES, 0, st>>>(p);
  lastblock_profile_kernel<D><<<grid, EST_NT, P_BYTES + TILE, st>>>(p);
  return check_launch();
}

int lastblock_profile(const EstParams& p, int head_dim, cudaStream_t st) {
  cudaError_t e = cudaMemsetAsync(p.slash, 0, sizeof(float) * int64_t(p.n_q_heads) * p.n_tokens, st);
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  if (head_dim == 128) {
    // tcgen05 kernels unless spf_force_generic_kernels asks for the mma.sync ones (used by the tests
    // to compare the two) or the key tensor cannot be described to TMA
    if (!force_generic_profile()) {
      const int rc = lastblock_profile_tc5(p, st);
      if (rc != SPF_ERR_SHAPE) return rc;
    }
    return launch_estimate<128>(p, st);
  }
  if (head_dim == 64) return launch_estimate<64>(p, st);
  return SPF_ERR_SHAPE;
}

}  // namespace spf

// ------------------------------------------------------------------------------------------
// Entry point for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc (or torch's allocator) at the point where
// the profile is needed: a plugin running inside another framework's memory plan that hands it
// only the input and output buffers, or a serving loop whose allocator is frozen once warm-up
// ends.  For them the pass-1 scratch lives in the fixed array below instead of a caller buffer.
// The array is part of the library image: every GPU that loads the library holds
// SPF_STATIC_SCRATCH_BYTES of it until the process exits.
//
// In host code `g_static_scratch` is only a stand-in for the symbol, not a device address: the
// address each device uses is looked up with cudaGetSymbolAddress while that device is current,
// once per device, and that pointer is what the kernels receive.
#include <mutex>

namespace spf {
constexpr int64_t STATIC_SCRATCH_BYTES = SPF_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[STATIC_SCRATCH_BYTES];

constexpr int MAX_DEVICES = 64;
static void* g_scratch_addr[MAX_DEVICES] = {nullptr};
static std::mutex g_scratch_mutex;

// Device address of the static scratch on the current device (looked up on first use).
static int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) { note_cuda_error(e); return SPF_ERR_LAUNCH; }
  if (dev < 0 || dev >= MAX_DEVICES) return SPF_ERR_RANGE;
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_addr[dev] == nullptr) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_static_scratch);
    if (e != cudaSuccess || p == nullptr) {
      note_cuda_error(e);
      return SPF_ERR_LAUNCH;
    }
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return SPF_OK;
}
}  // namespace spf

extern "C" int spf_lastblock_profile_static(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                                            const void* k, int64_t k_stride_n, int64_t k_stride_h,
                                            int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                                            int block_size, float* vertical, float* slash, void* stream) {
  using namespace spf;
  if (!q || !k || !vertical || !slash) return SPF_ERR_NULL;
  if (!supported_head_dim(head_dim) || !supported_block_size(block_size)) return SPF_ERR_SHAPE;
  if (n_tokens < block_size || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return SPF_ERR_SHAPE;
  if (n_q_heads > SPF_MAX_HEADS || ceil_div(n_tokens, block_size) > SPF_MAX_BLOCKS) return SPF_ERR_TOO_LARGE;
  if ((q_stride_n | q_stride_h | k_stride_n | k_stride_h) % 8 != 0 || !aligned16(q) || !aligned16(k))
    return SPF_ERR_ALIGN;
  // same scratch layout as spf_lastblock_profile: two [H][tiles][128] and two [H][128] fp32 arrays
  const int ntiles = ceil_div(n_tokens, EST_COLS);
  const int64_t part = align256(int64_t(n_q_heads) * ntiles * EST_ROWS * 4);
  const int64_t rows = align256(int64_t(n_q_heads) * EST_ROWS * 4);
  if (2 * part + 2 * rows > STATIC_SCRATCH_BYTES) return SPF_ERR_TOO_LARGE;  // heads x tokens too big for the fixed scratch
  void* base = nullptr;
  const int rc = static_scratch_for_current_device(&base);
  if (rc != SPF_OK) return rc;
  EstParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_sn = q_stride_n; p.q_sh = q_stride_h;
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_sn = k_stride_n; p.k_sh = k_stride_h;
  p.n_tokens = n_tokens; p.n_q_heads = n_q_heads; p.group = n_q_heads / n_kv_heads;
  p.rq = block_size; p.ntiles = ntiles; p.n_parts = ntiles;
  const int tpc = (ntiles * n_q_heads) / (148 * 8);
  p.tiles_per_cta = tpc < 1 ? 1 : (tpc > 8 ? 8 : tpc);
  p.sqrt_d = sqrtf(static_cast<float>(head_dim));
  char* s = static_cast<char*>(base);
  p.part_m = reinterpret_cast<float*>(s);
  p.part_l = reinterpret_cast<float*>(s + part);
  p.row_m = reinterpret_cast<float*>(s + 2 * part);
  p.row_z = reinterpret_cast<float*>(s + 2 * part + rows);
  p.vertical = vertical; p.slash = slash;
  return lastblock_profile(p, head_dim, static_cast<cudaStream_t>(stream));
}
