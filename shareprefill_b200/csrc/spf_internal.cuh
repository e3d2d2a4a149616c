// Parameter blocks and launcher prototypes shared between the kernels and the C ABI.
#pragma once

#include "spf_common.cuh"

namespace spf {

struct AttnParams {
  const __nv_bfloat16* q; int64_t q_sn, q_sh;
  const __nv_bfloat16* k; int64_t k_sn, k_sh;
  const __nv_bfloat16* v; int64_t v_sn, v_sh;
  __nv_bfloat16* out;      // [N][H][D]
  const uint32_t* bitmap;  // [H][nb][nbw]
  const int32_t* head_flags;
  const int32_t* slot_of_head;
  float* pivot_attn;       // state.pivot_attn or nullptr
  int n_tokens, n_q_heads, group, nb, nbw;
  float scale_log2;        // softmax_scale * log2(e)
  int pivot_only;          // 1: only pivot heads run, only their block-mass matrix is written
  int n_slots;             // shared clusters (grid of the pivot-only pass is nb x n_slots)
};

struct EstParams {
  const __nv_bfloat16* q; int64_t q_sn, q_sh;
  const __nv_bfloat16* k; int64_t k_sn, k_sh;
  int n_tokens, n_q_heads, group, rq, ntiles, tiles_per_cta;
  int n_parts;            // partial (max, sum) pairs per head and row that pass 1 leaves (mma.sync path: ntiles)
  float sqrt_d;           // queries are divided by it
  float* part_m;          // [H][n_parts][128] (allocated for ntiles)
  float* part_l;          // [H][n_parts][128]
  float* row_m;           // [H][128]
  float* row_z;           // [H][128]
  float* vertical;        // [H][N]
  float* slash;           // [H][N]
};

struct PoolTensor {
  const __nv_bfloat16* x;
  int64_t sn, sh;
  __nv_bfloat16* out;   // [nb][heads][D]
  int heads;
  int cta_cols;         // CTAs along the column axis for this tensor
  int q_style;
};

struct PoolParams {
  PoolTensor t[2];
  int n_tokens, head_dim, block_size;
};

struct BudgetParams {
  const float* vertical; const float* slash;
  int n_heads, n_tokens, block_size, nb;
  float thr; int min_blocks, max_blocks;
  int32_t* nv; int32_t* ns; float* vpool; float* spool;
};

struct LastRowParams {
  const __nv_bfloat16* q; int64_t q_sn, q_sh;
  const __nv_bfloat16* avg_k;   // [nb][Hkv][D]
  int n_tokens, n_q_heads, n_kv_heads, head_dim, block_size, nb;
  float sqrt_d;
  float* avg_qk;                // [H][nb]
};

struct ClassifyParams {
  const float* avg_qk; const float* vpool; const float* spool;
  const int32_t* slot_of_head;   // local heads
  StateView st; int n_slots, nb;
  float* jsd_qa; float* jsd_v; float* jsd_s;
};

struct ElectParams {
  const float* jsd_qa_all;          // [n_heads_total] gathered over all ranks
  const int32_t* slot_of_head_all;  // [n_heads_total]
  const float* jsd_v; const float* jsd_s;   // local heads
  const float* vpool; const float* spool;   // local heads
  StateView st; int n_slots, nb, layer;
  int n_heads_total, head_offset, n_heads;
  float qa_thr, sim_thr, fb_thr; int min_blocks;
  int32_t* nv; int32_t* ns; int32_t* head_flags;  // local heads
};

struct VsParams {
  const float* vpool; const float* spool;
  const int32_t* nv; const int32_t* ns; const int32_t* head_flags; const int32_t* slot_of_head;
  StateView st; int n_slots, nb, nbw;
  uint32_t* bitmap;
};

struct QaScoreParams {
  const __nv_bfloat16* avg_q;   // [nb][H][D]
  const __nv_bfloat16* avg_k;   // [nb][Hkv][D]
  const int32_t* head_flags;
  int n_q_heads, n_kv_heads, head_dim, nb;
  float sqrt_d;
  float* scores;                // [H][nb][nb]
};

struct QaSelectParams {
  const float* scores; const int32_t* head_flags;
  int nb, nbw; float thr; int scale_bits;
  uint32_t* bitmap;
};

struct PivotParams {
  const int32_t* head_flags; const int32_t* slot_of_head;
  StateView st; int n_slots, nb, nbw; float thr;
};

struct DecodeParams {
  const __nv_bfloat16* q; int64_t q_sh;
  const __nv_bfloat16* k; int64_t k_sn, k_sh;
  const __nv_bfloat16* v; int64_t v_sn, v_sh;
  __nv_bfloat16* out;      // [H][D]
  float* scratch;          // [H][splits][D + 2]
  int n_keys, n_q_heads, group, splits;
  float scale_log2;
};

int decode_attention(const DecodeParams& p, int head_dim, cudaStream_t st);
int lastblock_profile_tc5(const EstParams& p, cudaStream_t st);
bool force_generic_profile();
unsigned int est_tc5_timeout_count();
bool est_tc5_reset_timeouts();
bool est_tc5_set_wait_limit(unsigned long long ns);
int sparse_attention_generic(const AttnParams& p, int block_size, int head_dim, cudaStream_t st);
int sparse_attention_tc5(const AttnParams& p, int n_kv_heads, cudaStream_t st);
unsigned int tc5_timeout_count();
bool tc5_reset_timeouts();
bool tc5_set_wait_limit(unsigned long long ns);
int tc5_wait_limit_selftest(cudaStream_t st);
int lastblock_profile(const EstParams& p, int head_dim, cudaStream_t st);
int pool_blocks(const PoolParams& p, int nb, cudaStream_t st);
int launch_budgets(const BudgetParams& p, cudaStream_t st);
int launch_last_row(const LastRowParams& p, cudaStream_t st);
int launch_classify(const ClassifyParams& p, int n_heads, cudaStream_t st);
int launch_pairwise_jsd(const float* x, int n_vec, int len, float* out, cudaStream_t st);
int launch_elect(const ElectParams& p, cudaStream_t st);
int launch_vs_bitmap(const VsParams& p, int n_heads, cudaStream_t st);
int launch_qa_scores(const QaScoreParams& p, cudaStream_t st);
int launch_qa_select(const QaSelectParams& p, int n_heads, cudaStream_t st);
int launch_row_counts(const uint32_t* bitmap, int n_heads, int nb, int32_t* row_counts,
                      int64_t* head_totals, cudaStream_t st);
int launch_update_pivots(const PivotParams& p, int n_heads, cudaStream_t st);
int launch_state_reset(void* state, int n_slots, int nb, cudaStream_t st);
int launch_pack_summaries(void* state, int n_slots, int nb, int layer, int h0, int h1, int32_t* out,
                          cudaStream_t st);
int launch_merge_summaries(void* state, int n_slots, int nb, const int32_t* gathered, int n_ranks,
                           cudaStream_t st);

}  // namespace spf
