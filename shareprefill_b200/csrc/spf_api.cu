// C ABI of libspf_b200.so: argument validation and dispatch.  See include/spf_b200.h.
#include <atomic>
#include <cmath>
#include <cstdlib>
#include <cstring>

#include "spf_internal.cuh"

namespace spf {
static thread_local cudaError_t g_last_error = cudaSuccess;
// the value spf_device_timeouts() last returned: lets a launcher refuse work without a synchronisation
static std::atomic<unsigned int> g_known_timeouts{0};
static inline bool timeouts_tripped() { return g_known_timeouts.load(std::memory_order_relaxed) > 16u; }
// test hooks (spf_force_generic_kernels): run the mma.sync kernels where the tcgen05 ones would
static std::atomic<int> g_force_generic_attention{0}, g_force_generic_profile{0};
bool force_generic_profile() { return g_force_generic_profile.load(std::memory_order_relaxed) != 0; }
void note_cuda_error(cudaError_t e) { g_last_error = e; }

static inline bool strides_ok(int64_t sn, int64_t sh) { return (sn % 8 == 0) && (sh % 8 == 0); }
static inline int log2_ceil(int x) { int b = 0; while ((1 << b) < x) ++b; return b; }
}  // namespace spf

using namespace spf;

extern "C" {

const char* spf_status_string(int status) {
  switch (status) {
    case SPF_OK: return "ok";
    case SPF_ERR_NULL: return "a required pointer is NULL";
    case SPF_ERR_SHAPE: return "unsupported shape (head_dim in {64,128}, block_size in {16,32,64,128}, n_tokens >= block_size, q heads a multiple of kv heads)";
    case SPF_ERR_ALIGN: return "pointer or stride is not 16-byte aligned";
    case SPF_ERR_RANGE: return "argument out of range";
    case SPF_ERR_LAUNCH: return "CUDA launch error (see spf_last_cuda_error)";
    case SPF_ERR_TOO_LARGE: return "size beyond a compiled-in maximum";
    case SPF_ERR_TIMEOUT: return "bounded device-side waits gave up earlier (spf_device_timeouts); reset with spf_reset_device_timeouts";
    default: return "unknown status";
  }
}

const char* spf_last_cuda_error(void) { return cudaGetErrorString(g_last_error); }
int spf_version(void) { return 100; }

static int check_shape(int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int block_size) {
  if (!supported_head_dim(head_dim) || !supported_block_size(block_size)) return SPF_ERR_SHAPE;
  if (n_tokens < block_size || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return SPF_ERR_SHAPE;
  if (n_q_heads > SPF_MAX_HEADS) return SPF_ERR_TOO_LARGE;
  if (ceil_div(n_tokens, block_size) > SPF_MAX_BLOCKS) return SPF_ERR_TOO_LARGE;
  return SPF_OK;
}

int spf_pool_qk(const void* q, int64_t q_stride_n, int64_t q_stride_h, const void* k, int64_t k_stride_n,
                int64_t k_stride_h, int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                int block_size, void* avg_q, void* avg_k, void* stream) {
  if ((q == nullptr) != (avg_q == nullptr) || (k == nullptr) != (avg_k == nullptr)) return SPF_ERR_NULL;
  if (!q && !k) return SPF_ERR_NULL;
  if (!supported_head_dim(head_dim) || n_tokens <= 0 || block_size <= 0 || block_size > 512) return SPF_ERR_SHAPE;
  if (ceil_div(n_tokens, block_size) > 65535 * 16) return SPF_ERR_TOO_LARGE;
  PoolParams p;
  std::memset(&p, 0, sizeof(p));
  p.n_tokens = n_tokens; p.head_dim = head_dim; p.block_size = block_size;
  const int cph = head_dim / 8;
  if (q) {
    if (!aligned16(q) || !aligned16(avg_q) || !strides_ok(q_stride_n, q_stride_h)) return SPF_ERR_ALIGN;
    if (n_q_heads <= 0) return SPF_ERR_SHAPE;
    p.t[0] = PoolTensor{static_cast<const __nv_bfloat16*>(q), q_stride_n, q_stride_h,
                        static_cast<__nv_bfloat16*>(avg_q), n_q_heads, ceil_div(n_q_heads * cph, 128), 1};
  }
  if (k) {
    if (!aligned16(k) || !aligned16(avg_k) || !strides_ok(k_stride_n, k_stride_h)) return SPF_ERR_ALIGN;
    if (n_kv_heads <= 0) return SPF_ERR_SHAPE;
    p.t[1] = PoolTensor{static_cast<const __nv_bfloat16*>(k), k_stride_n, k_stride_h,
                        static_cast<__nv_bfloat16*>(avg_k), n_kv_heads, ceil_div(n_kv_heads * cph, 128), 0};
  }
  return pool_blocks(p, ceil_div(n_tokens, block_size), static_cast<cudaStream_t>(stream));
}

int64_t spf_lastblock_scratch_bytes(int n_tokens, int n_q_heads, int block_size) {
  (void)block_size;
  if (n_tokens <= 0 || n_q_heads <= 0) return 0;
  const int64_t ntiles = ceil_div(n_tokens, 128);
  return align256(int64_t(n_q_heads) * ntiles * 128 * 4) * 2 + align256(int64_t(n_q_heads) * 128 * 4) * 2;
}

int spf_lastblock_profile(const void* q, int64_t q_stride_n, int64_t q_stride_h, const void* k,
                          int64_t k_stride_n, int64_t k_stride_h, int n_tokens, int n_q_heads,
                          int n_kv_heads, int head_dim, int block_size, float* vertical, float* slash,
                          void* scratch, int64_t scratch_bytes, void* stream) {
  if (!q || !k || !vertical || !slash || !scratch) return SPF_ERR_NULL;
  if (timeouts_tripped()) return SPF_ERR_TIMEOUT;
  int rc = check_shape(n_tokens, n_q_heads, n_kv_heads, head_dim, block_size);
  if (rc) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(scratch) || !strides_ok(q_stride_n, q_stride_h) ||
      !strides_ok(k_stride_n, k_stride_h))
    return SPF_ERR_ALIGN;
  if (scratch_bytes < spf_lastblock_scratch_bytes(n_tokens, n_q_heads, block_size)) return SPF_ERR_RANGE;
  EstParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_sn = q_stride_n; p.q_sh = q_stride_h;
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_sn = k_stride_n; p.k_sh = k_stride_h;
  p.n_tokens = n_tokens; p.n_q_heads = n_q_heads; p.group = n_q_heads / n_kv_heads;
  p.rq = block_size; p.ntiles = ceil_div(n_tokens, 128); p.n_parts = p.ntiles;
  int tpc = (p.ntiles * n_q_heads) / (148 * 8);
  p.tiles_per_cta = tpc < 1 ? 1 : (tpc > 8 ? 8 : tpc);
  p.sqrt_d = static_cast<float>(std::sqrt(static_cast<double>(head_dim)));
  char* s = static_cast<char*>(scratch);
  const int64_t part = align256(int64_t(n_q_heads) * p.ntiles * 128 * 4);
  const int64_t rows = align256(int64_t(n_q_heads) * 128 * 4);
  p.part_m = reinterpret_cast<float*>(s);
  p.part_l = reinterpret_cast<float*>(s + part);
  p.row_m = reinterpret_cast<float*>(s + 2 * part);
  p.row_z = reinterpret_cast<float*>(s + 2 * part + rows);
  p.vertical = vertical; p.slash = slash;
  return lastblock_profile(p, head_dim, static_cast<cudaStream_t>(stream));
}

int spf_profile_budgets(const float* vertical, const float* slash, int n_heads, int n_tokens, int block_size,
                        double pattern_threshold, int min_blocks, int max_blocks, int32_t* nv, int32_t* ns,
                        float* vpool, float* spool, void* stream) {
  if (!vertical || !slash || !nv || !ns || !vpool || !spool) return SPF_ERR_NULL;
  if (n_heads <= 0 || n_tokens <= 0 || block_size <= 0) return SPF_ERR_SHAPE;
  if (n_heads > SPF_MAX_HEADS || ceil_div(n_tokens, block_size) > SPF_MAX_BLOCKS) return SPF_ERR_TOO_LARGE;
  BudgetParams p;
  p.vertical = vertical; p.slash = slash; p.n_heads = n_heads; p.n_tokens = n_tokens;
  p.block_size = block_size; p.nb = ceil_div(n_tokens, block_size);
  p.thr = static_cast<float>(pattern_threshold);
  p.min_blocks = min_blocks; p.max_blocks = max_blocks < p.nb ? max_blocks : p.nb;
  p.nv = nv; p.ns = ns; p.vpool = vpool; p.spool = spool;
  return launch_budgets(p, static_cast<cudaStream_t>(stream));
}

int spf_pooled_last_row(const void* q, int64_t q_stride_n, int64_t q_stride_h, const void* avg_k, int n_tokens,
                        int n_q_heads, int n_kv_heads, int head_dim, int block_size, float* avg_qk,
                        void* stream) {
  if (!q || !avg_k || !avg_qk) return SPF_ERR_NULL;
  int rc = check_shape(n_tokens, n_q_heads, n_kv_heads, head_dim, block_size);
  if (rc) return rc;
  if (!aligned16(avg_k)) return SPF_ERR_ALIGN;   // pooled key rows are read 16 bytes at a time
  LastRowParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_sn = q_stride_n; p.q_sh = q_stride_h;
  p.avg_k = static_cast<const __nv_bfloat16*>(avg_k);
  p.n_tokens = n_tokens; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
  p.block_size = block_size; p.nb = ceil_div(n_tokens, block_size);
  p.sqrt_d = static_cast<float>(std::sqrt(static_cast<double>(head_dim)));
  p.avg_qk = avg_qk;
  return launch_last_row(p, static_cast<cudaStream_t>(stream));
}

int64_t spf_sharing_state_bytes(int n_slots, int nb) {
  if (n_slots < 0 || nb <= 0 || nb > SPF_MAX_BLOCKS) return 0;
  int64_t off[13];
  state_offsets(n_slots > 0 ? n_slots : 1, nb, off);
  return off[12];
}

int spf_sharing_state_layout(int n_slots, int nb, int64_t* offsets) {
  if (!offsets) return SPF_ERR_NULL;
  if (n_slots < 0 || nb <= 0 || nb > SPF_MAX_BLOCKS) return SPF_ERR_RANGE;
  int64_t off[13];
  state_offsets(n_slots > 0 ? n_slots : 1, nb, off);
  for (int i = 0; i < 12; ++i) offsets[i] = off[i];
  return SPF_OK;
}

int spf_sharing_state_reset(void* state, int n_slots, int nb, void* stream) {
  if (!state) return SPF_ERR_NULL;
  if (n_slots < 0 || nb <= 0 || nb > SPF_MAX_BLOCKS) return SPF_ERR_RANGE;
  return launch_state_reset(state, n_slots > 0 ? n_slots : 1, nb, static_cast<cudaStream_t>(stream));
}

int spf_classify_heads(const float* avg_qk, const float* vpool, const float* spool, const int32_t* slot_of_head,
                       const void* state, int n_slots, int n_heads, int nb, float* jsd_qa, float* jsd_v,
                       float* jsd_s, void* stream) {
  if (!avg_qk || !vpool || !spool || !slot_of_head || !state || !jsd_qa || !jsd_v || !jsd_s) return SPF_ERR_NULL;
  if (n_heads <= 0 || n_heads > SPF_MAX_HEADS || nb <= 0 || nb > SPF_MAX_BLOCKS || n_slots < 0) return SPF_ERR_RANGE;
  ClassifyParams p;
  p.avg_qk = avg_qk; p.vpool = vpool; p.spool = spool; p.slot_of_head = slot_of_head;
  p.st = state_view(const_cast<void*>(state), n_slots > 0 ? n_slots : 1, nb);
  p.n_slots = n_slots; p.nb = nb; p.jsd_qa = jsd_qa; p.jsd_v = jsd_v; p.jsd_s = jsd_s;
  return launch_classify(p, n_heads, static_cast<cudaStream_t>(stream));
}

int spf_pairwise_sqrt_jsd(const float* x, int n_vec, int len, float* out, void* stream) {
  if (!x || !out) return SPF_ERR_NULL;
  if (n_vec <= 0 || n_vec > 65535 || len <= 0 || len > 2 * SPF_MAX_BLOCKS) return SPF_ERR_RANGE;
  return launch_pairwise_jsd(x, n_vec, len, out, static_cast<cudaStream_t>(stream));
}

int spf_elect_and_share(const float* jsd_qa_all, const int32_t* slot_of_head_all, int n_heads_total,
                        int head_offset, int n_heads, const float* jsd_v, const float* jsd_s,
                        const float* vpool, const float* spool, void* state, int n_slots, int nb, int layer,
                        double queryaware_threshold, double similarity_threshold, double fallback_threshold,
                        int min_blocks, int32_t* nv, int32_t* ns, int32_t* head_flags, void* stream) {
  if (!jsd_qa_all || !slot_of_head_all || !jsd_v || !jsd_s || !vpool || !spool || !state || !nv || !ns || !head_flags)
    return SPF_ERR_NULL;
  if (n_heads <= 0 || n_heads_total < n_heads || head_offset < 0 || head_offset + n_heads > n_heads_total ||
      n_heads_total > SPF_MAX_HEADS || nb <= 0 || nb > SPF_MAX_BLOCKS || n_slots < 0)
    return SPF_ERR_RANGE;
  ElectParams p;
  p.jsd_qa_all = jsd_qa_all; p.slot_of_head_all = slot_of_head_all; p.jsd_v = jsd_v; p.jsd_s = jsd_s;
  p.vpool = vpool; p.spool = spool;
  p.st = state_view(state, n_slots > 0 ? n_slots : 1, nb);
  p.n_slots = n_slots; p.nb = nb; p.layer = layer;
  p.n_heads_total = n_heads_total; p.head_offset = head_offset; p.n_heads = n_heads;
  p.qa_thr = static_cast<float>(queryaware_threshold);
  p.sim_thr = static_cast<float>(similarity_threshold);
  p.fb_thr = static_cast<float>(fallback_threshold);
  p.min_blocks = min_blocks; p.nv = nv; p.ns = ns; p.head_flags = head_flags;
  return launch_elect(p, static_cast<cudaStream_t>(stream));
}

int spf_build_vs_bitmap(const float* vpool, const float* spool, const int32_t* nv, const int32_t* ns,
                        const int32_t* head_flags, const int32_t* slot_of_head, void* state, int n_slots,
                        int n_heads, int nb, uint32_t* bitmap, void* stream) {
  if (!vpool || !spool || !nv || !ns || !head_flags || !slot_of_head || !state || !bitmap) return SPF_ERR_NULL;
  if (n_heads <= 0 || n_heads > SPF_MAX_HEADS || nb <= 0 || nb > SPF_MAX_BLOCKS || n_slots < 0) return SPF_ERR_RANGE;
  VsParams p;
  p.vpool = vpool; p.spool = spool; p.nv = nv; p.ns = ns; p.head_flags = head_flags;
  p.slot_of_head = slot_of_head; p.st = state_view(state, n_slots > 0 ? n_slots : 1, nb);
  p.n_slots = n_slots; p.nb = nb; p.nbw = (nb + 31) / 32; p.bitmap = bitmap;
  return launch_vs_bitmap(p, n_heads, static_cast<cudaStream_t>(stream));
}

int spf_query_aware_scores(const void* avg_q, const void* avg_k, const int32_t* head_flags, int n_q_heads,
                           int n_kv_heads, int head_dim, int nb, float* scores, void* stream) {
  if (!avg_q || !avg_k || !scores) return SPF_ERR_NULL;
  if (!supported_head_dim(head_dim) || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads) return SPF_ERR_SHAPE;
  if (n_q_heads > SPF_MAX_HEADS || nb <= 0 || nb > SPF_MAX_BLOCKS) return SPF_ERR_TOO_LARGE;
  if (!aligned16(avg_k)) return SPF_ERR_ALIGN;   // pooled key rows are read 16 bytes at a time
  QaScoreParams p;
  p.avg_q = static_cast<const __nv_bfloat16*>(avg_q); p.avg_k = static_cast<const __nv_bfloat16*>(avg_k);
  p.head_flags = head_flags; p.n_q_heads = n_q_heads; p.n_kv_heads = n_kv_heads; p.head_dim = head_dim;
  p.nb = nb; p.sqrt_d = static_cast<float>(std::sqrt(static_cast<double>(head_dim))); p.scores = scores;
  return launch_qa_scores(p, static_cast<cudaStream_t>(stream));
}

int spf_query_aware_select(const float* scores, const int32_t* head_flags, int n_heads, int nb,
                           double pattern_threshold, uint32_t* bitmap, void* stream) {
  if (!scores || !bitmap) return SPF_ERR_NULL;
  if (n_heads <= 0 || n_heads > SPF_MAX_HEADS || nb <= 0 || nb > SPF_MAX_BLOCKS) return SPF_ERR_RANGE;
  QaSelectParams p;
  p.scores = scores; p.head_flags = head_flags; p.nb = nb; p.nbw = (nb + 31) / 32;
  p.thr = static_cast<float>(pattern_threshold * static_cast<double>(nb));
  p.scale_bits = 60 - log2_ceil(nb) - 1;
  p.bitmap = bitmap;
  return launch_qa_select(p, n_heads, static_cast<cudaStream_t>(stream));
}

int spf_bitmap_row_counts(const uint32_t* bitmap, int n_heads, int nb, int32_t* row_counts, int64_t* head_totals,
                          void* stream) {
  if (!bitmap || !row_counts) return SPF_ERR_NULL;
  if (n_heads <= 0 || nb <= 0 || nb > SPF_MAX_BLOCKS) return SPF_ERR_RANGE;
  return launch_row_counts(bitmap, n_heads, nb, row_counts, head_totals, static_cast<cudaStream_t>(stream));
}

int spf_sparse_attention(const void* q, int64_t q_stride_n, int64_t q_stride_h, const void* k, int64_t k_stride_n,
                         int64_t k_stride_h, const void* v, int64_t v_stride_n, int64_t v_stride_h, int n_tokens,
                         int n_q_heads, int n_kv_heads, int head_dim, int block_size, double softmax_scale,
                         const uint32_t* bitmap, const int32_t* head_flags, const int32_t* slot_of_head,
                         void* state, int n_slots, void* out, void* stream) {
  if (!q || !k || !v || !bitmap || !out) return SPF_ERR_NULL;
  if (timeouts_tripped()) return SPF_ERR_TIMEOUT;
  int rc = check_shape(n_tokens, n_q_heads, n_kv_heads, head_dim, block_size);
  if (rc) return rc;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !strides_ok(q_stride_n, q_stride_h) ||
      !strides_ok(k_stride_n, k_stride_h) || !strides_ok(v_stride_n, v_stride_h))
    return SPF_ERR_ALIGN;
  AttnParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_sn = q_stride_n; p.q_sh = q_stride_h;
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_sn = k_stride_n; p.k_sh = k_stride_h;
  p.v = static_cast<const __nv_bfloat16*>(v); p.v_sn = v_stride_n; p.v_sh = v_stride_h;
  p.out = static_cast<__nv_bfloat16*>(out); p.bitmap = bitmap;
  const bool with_state = head_flags && slot_of_head && state && n_slots > 0;
  p.head_flags = with_state ? head_flags : nullptr;
  p.slot_of_head = with_state ? slot_of_head : nullptr;
  p.pivot_attn = with_state ? state_view(state, n_slots, ceil_div(n_tokens, block_size)).pivot_attn : nullptr;
  p.n_tokens = n_tokens; p.n_q_heads = n_q_heads; p.group = n_q_heads / n_kv_heads;
  p.nb = ceil_div(n_tokens, block_size); p.nbw = (p.nb + 31) / 32;
  p.scale_log2 = static_cast<float>(softmax_scale * 1.4426950408889634);
  p.pivot_only = 0;
  p.n_slots = with_state ? n_slots : 0;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // block_size = head_dim = 128 runs on the tcgen05 kernel; spf_force_generic_kernels (a test hook)
  // keeps the mma.sync kernel, which also serves every other supported shape
  const bool want_tc5 = block_size == 128 && head_dim == 128 &&
                        g_force_generic_attention.load(std::memory_order_relaxed) == 0;
  if (want_tc5) {
    rc = sparse_attention_tc5(p, n_kv_heads, st);
    if (rc == SPF_OK) {
      if (!with_state) return SPF_OK;
      p.pivot_only = 1;   // pivot heads: the block-mass matrix comes from the two-sweep kernel
      return sparse_attention_generic(p, block_size, head_dim, st);
    }
    if (rc != SPF_ERR_SHAPE) return rc;
  }
  return sparse_attention_generic(p, block_size, head_dim, st);
}

// Token splits of the decode pass: about two CTAs per SM over (splits x CTA rows), at least four
// 16-token tiles per split, every split non-empty.
static int decode_splits(int n_keys, int n_q_heads, int n_kv_heads) {
  const int rows = (n_q_heads / n_kv_heads <= 16) ? n_kv_heads : n_q_heads;   // CTA rows of the grid
  const int tiles = (n_keys + 15) / 16;
  int s = (2 * 148 + rows - 1) / rows;
  if (s > (tiles + 3) / 4) s = (tiles + 3) / 4;
  if (s > 256) s = 256;
  if (s < 1) s = 1;
  const int per = (tiles + s - 1) / s;
  return (tiles + per - 1) / per;
}

int64_t spf_decode_scratch_bytes(int n_keys, int n_q_heads, int n_kv_heads, int head_dim) {
  if (n_keys <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads || !supported_head_dim(head_dim))
    return 0;
  return align256(int64_t(n_q_heads) * decode_splits(n_keys, n_q_heads, n_kv_heads) * (head_dim + 2) * 4);
}

int spf_decode_attention(const void* q, int64_t q_stride_h, const void* k, int64_t k_stride_n, int64_t k_stride_h,
                         const void* v, int64_t v_stride_n, int64_t v_stride_h, int n_keys, int n_q_heads,
                         int n_kv_heads, int head_dim, double softmax_scale, void* out, void* scratch,
                         int64_t scratch_bytes, void* stream) {
  if (!q || !k || !v || !out || !scratch) return SPF_ERR_NULL;
  if (!supported_head_dim(head_dim) || n_keys <= 0 || n_q_heads <= 0 || n_kv_heads <= 0 || n_q_heads % n_kv_heads)
    return SPF_ERR_SHAPE;
  if (n_q_heads > SPF_MAX_HEADS) return SPF_ERR_TOO_LARGE;
  if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(out) || !aligned16(scratch) ||
      q_stride_h % 8 || !strides_ok(k_stride_n, k_stride_h) || !strides_ok(v_stride_n, v_stride_h))
    return SPF_ERR_ALIGN;
  if (scratch_bytes < spf_decode_scratch_bytes(n_keys, n_q_heads, n_kv_heads, head_dim)) return SPF_ERR_RANGE;
  DecodeParams p;
  p.q = static_cast<const __nv_bfloat16*>(q); p.q_sh = q_stride_h;
  p.k = static_cast<const __nv_bfloat16*>(k); p.k_sn = k_stride_n; p.k_sh = k_stride_h;
  p.v = static_cast<const __nv_bfloat16*>(v); p.v_sn = v_stride_n; p.v_sh = v_stride_h;
  p.out = static_cast<__nv_bfloat16*>(out); p.scratch = static_cast<float*>(scratch);
  p.n_keys = n_keys; p.n_q_heads = n_q_heads; p.group = n_q_heads / n_kv_heads;
  p.splits = decode_splits(n_keys, n_q_heads, n_kv_heads);
  p.scale_log2 = static_cast<float>(softmax_scale * 1.4426950408889634);
  return decode_attention(p, head_dim, static_cast<cudaStream_t>(stream));
}

int spf_device_timeouts(void) {
  const unsigned int n = tc5_timeout_count() + est_tc5_timeout_count();
  g_known_timeouts.store(n, std::memory_order_relaxed);
  return static_cast<int>(n);
}

int spf_reset_device_timeouts(void) {
  if (!tc5_reset_timeouts() || !est_tc5_reset_timeouts()) return SPF_ERR_LAUNCH;
  g_known_timeouts.store(0, std::memory_order_relaxed);
  return SPF_OK;
}

int spf_set_device_wait_limit_ns(uint64_t ns) {
  if (ns == 0) return SPF_ERR_RANGE;
  return (tc5_set_wait_limit(ns) && est_tc5_set_wait_limit(ns)) ? SPF_OK : SPF_ERR_LAUNCH;
}

int spf_force_generic_kernels(int attention, int profile) {
  g_force_generic_attention.store(attention ? 1 : 0, std::memory_order_relaxed);
  g_force_generic_profile.store(profile ? 1 : 0, std::memory_order_relaxed);
  return SPF_OK;
}

int spf_wait_limit_selftest(void* stream) { return tc5_wait_limit_selftest(static_cast<cudaStream_t>(stream)); }

int spf_update_pivots(const int32_t* head_flags, const int32_t* slot_of_head, void* state, int n_slots, int n_heads,
                      int nb, double pattern_threshold, void* stream) {
  if (!head_flags || !slot_of_head || !state) return SPF_ERR_NULL;
  if (n_heads <= 0 || n_heads > SPF_MAX_HEADS || nb <= 0 || nb > SPF_MAX_BLOCKS || n_slots < 0) return SPF_ERR_RANGE;
  if (n_slots == 0) return SPF_OK;
  PivotParams p;
  p.head_flags = head_flags; p.slot_of_head = slot_of_head; p.st = state_view(state, n_slots, nb);
  p.n_slots = n_slots; p.nb = nb; p.nbw = (nb + 31) / 32; p.thr = static_cast<float>(pattern_threshold);
  return launch_update_pivots(p, n_heads, static_cast<cudaStream_t>(stream));
}

int64_t spf_pivot_summary_width(int nb) {
  if (nb <= 0 || nb > SPF_MAX_BLOCKS) return 0;
  return 2 + 2 * int64_t(nb) + int64_t(nb) * ((nb + 31) / 32);
}

int spf_pack_pivot_summaries(void* state, int n_slots, int nb, int layer, int head_begin, int head_end,
                             int32_t* packed, void* stream) {
  if (!state || !packed) return SPF_ERR_NULL;
  if (nb <= 0 || nb > SPF_MAX_BLOCKS || n_slots < 0 || head_begin < 0 || head_end < head_begin) return SPF_ERR_RANGE;
  if (n_slots == 0) return SPF_OK;
  return launch_pack_summaries(state, n_slots, nb, layer, head_begin, head_end, packed,
                               static_cast<cudaStream_t>(stream));
}

int spf_merge_pivot_summaries(void* state, int n_slots, int nb, const int32_t* gathered, int n_ranks,
                              void* stream) {
  if (!state || !gathered) return SPF_ERR_NULL;
  if (nb <= 0 || nb > SPF_MAX_BLOCKS || n_slots < 0 || n_ranks <= 0) return SPF_ERR_RANGE;
  if (n_slots == 0) return SPF_OK;
  return launch_merge_summaries(state, n_slots, nb, gathered, n_ranks, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
