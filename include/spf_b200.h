/*
 * spf_b200.h - C ABI of the B200 sparse-prefill attention library (libspf_b200.so).
 *
 * The reference (opas-lab/SharePrefill) is pure Python and has no FFI; every entry
 * point below replaces a Python function of the reference's prefill attention path,
 * cited as file:line within that project.
 *
 * Conventions
 *   - Batch is 1 per call (the reference's sharing state assumes it,
 *     attn/attention_sharing.py:42-44); callers loop over the batch.
 *   - All pointers are DEVICE pointers unless marked "host".  The caller owns every
 *     buffer (inputs, outputs, scratch, sharing state); nothing here allocates.
 *   - q/k/v/avg tensors are bf16 with the head dimension contiguous; token and head
 *     strides are given in ELEMENTS and must be multiples of 8 (16-byte rows).
 *   - `stream` is a cudaStream_t passed as void*; work is enqueued, never synchronised.
 *   - Every function returns SPF_OK (0) or a negative spf_status; nothing throws,
 *     exits or aborts.  spf_status_string() names a code.
 *   - head_dim in {64,128}; block_size in {16,32,64,128}; num_blocks <= SPF_MAX_BLOCKS.
 *
 * Bitmaps: a block pattern is `uint32_t[heads][nb][nbw]`, nbw = spf_bitmap_words(nb);
 * bit (c & 31) of word c >> 5 in row r is set when key block c is visited by query
 * block r.  This replaces the reference's per-head sorted lists of flat indices
 * r*nb + c (attn/attention_sharing.py:204-207,333-337).
 */
#ifndef SPF_B200_H_
#define SPF_B200_H_

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SPF_MAX_BLOCKS 8192
#define SPF_MAX_HEADS 256

typedef enum spf_status {
  SPF_OK = 0,
  SPF_ERR_NULL = -1,        /* a required pointer is NULL */
  SPF_ERR_SHAPE = -2,       /* unsupported head_dim / block_size / head counts / sizes */
  SPF_ERR_ALIGN = -3,       /* pointer or stride not 16-byte aligned */
  SPF_ERR_RANGE = -4,       /* argument out of range (thresholds, budgets, layer, slots) */
  SPF_ERR_LAUNCH = -5,      /* CUDA reported an error at launch; see spf_last_cuda_error */
  SPF_ERR_TOO_LARGE = -6,   /* size beyond a compiled-in maximum */
  SPF_ERR_TIMEOUT = -7      /* bounded device-side waits gave up earlier in this process; the tcgen05
                               kernels refuse to run until spf_reset_device_timeouts() */
} spf_status;

/* head flag bits written by spf_elect_and_share */
#define SPF_HEAD_QUERY_AWARE 1
#define SPF_HEAD_PIVOT 2
#define SPF_HEAD_SHARED 4

const char* spf_status_string(int status);
/* cudaGetErrorString of the last launch error seen by this library on this thread. */
const char* spf_last_cuda_error(void);
int spf_version(void);
static inline int spf_bitmap_words(int nb) { return (nb + 31) / 32; }

/* ---------------------------------------------------------------- pooling
 * Block mean of Q and K over tokens.  Replaces triton_bnhd_pool / bnhd_pool_kernel
 * (attn/utils.py:131-261, pool type "avg") for K and the padded view().mean() of Q
 * (attn/attention_sharing.py:350-356).  avg_q is [nb][H][D], avg_k is [nb][Hkv][D], bf16.
 * The last, partial block of K divides by its true length; the last block of Q follows
 * the reference's mean-over-block_size then rescale, with its bf16 roundings.
 * Either of (q, avg_q) or (k, avg_k) may be NULL together to skip that tensor.
 */
int spf_pool_qk(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                const void* k, int64_t k_stride_n, int64_t k_stride_h,
                int n_tokens, int n_q_heads, int n_kv_heads, int head_dim, int block_size,
                void* avg_q, void* avg_k, void* stream);

/* ---------------------------------------------------------------- last-block profile
 * Softmax of the last `block_size` queries against all keys, reduced to the vertical
 * profile (mean over queries) and the slash profile (mean over queries per
 * anti-diagonal): attn/attention_sharing.py:127-167, attn/utils.py:79-86.
 * vertical, slash: fp32 [H][n_tokens].  Logits are rounded to bf16 before the fp32
 * softmax, as the reference's bf16 einsum does.
 * scratch: at least spf_lastblock_scratch_bytes() bytes; contents are overwritten.
 */
int64_t spf_lastblock_scratch_bytes(int n_tokens, int n_q_heads, int block_size);
int spf_lastblock_profile(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                          const void* k, int64_t k_stride_n, int64_t k_stride_h,
                          int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                          int block_size, float* vertical, float* slash,
                          void* scratch, int64_t scratch_bytes, void* stream);

/* spf_lastblock_profile_static: the same computation for callers that cannot allocate
 * device memory.  (No counterpart in the reference; added for such callers.)
 *
 * Who needs it: code that runs where cudaMalloc / a framework allocator is off limits, e.g. a
 * plugin living inside another runtime's fixed memory plan that is handed only its input and
 * output buffers, or a serving loop whose memory pool is frozen after warm-up.  They pass
 * inputs and outputs only; the pass-1 scratch is a fixed array inside the library.
 *
 * Limits and rules:
 *   - The array is SPF_STATIC_SCRATCH_BYTES (8 MiB + 128 KiB) and is resident on every GPU
 *     that loads the library until the process exits.  A call whose scratch need (the value
 *     spf_lastblock_scratch_bytes reports) exceeds it returns SPF_ERR_TOO_LARGE.  The array
 *     covers n_q_heads * (ceil(n_tokens/128) + 1) <= 8320, e.g. 32 heads x 32K tokens or
 *     8 heads x 128K tokens.
 *   - The first call on a device looks up the array's device address (that device must be
 *     current); make that first call outside any stream capture.  The address is kept for the
 *     life of the process and is only valid while that device's context lives: do not call this
 *     function again after cudaDeviceReset() (or after the primary context was released).
 *   - The function calls no cudaMalloc / cudaFree and no allocating library routine.
 *   - All calls on a device share the one array: calls that may overlap on the GPU (different
 *     streams, threads or processes sharing a context) race; serialise them.  Nothing in the
 *     array needs to start at zero - every word is written before it is read - and the
 *     previous call's contents are simply overwritten.
 */
#define SPF_STATIC_SCRATCH_BYTES (8 * 1024 * 1024 + 128 * 1024)
int spf_lastblock_profile_static(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                                 const void* k, int64_t k_stride_n, int64_t k_stride_h,
                                 int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                                 int block_size, float* vertical, float* slash, void* stream);

/* ---------------------------------------------------------------- budgets + pooled profiles
 * Per head: number of vertical / slash blocks from the cumulative-mass rule
 * (score_cover_topk, attn/utils.py:47-50; attn/attention_sharing.py:169-176) and the
 * block sums of both profiles (torch_bhn_sumpool, attn/utils.py:33-44).
 * nv, ns: int32 [H] (clamped to [min_blocks, min(max_blocks, nb)]);
 * vpool, spool: fp32 [H][nb].
 */
int spf_profile_budgets(const float* vertical, const float* slash, int n_heads, int n_tokens,
                        int block_size, double pattern_threshold, int min_blocks, int max_blocks,
                        int32_t* nv, int32_t* ns, float* vpool, float* spool, void* stream);

/* ---------------------------------------------------------------- pooled last-row estimate
 * avg_qk[h][b] = softmax_b( mean(last queries / sqrt(D)) . avg_k[b] )
 * (attn/attention_sharing.py:197-200).  avg_qk: fp32 [H][nb].  avg_k: the pooled keys of
 * spf_pool_qk, bf16 [nb][Hkv][D] contiguous, 16-byte aligned.
 */
int spf_pooled_last_row(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                        const void* avg_k, int n_tokens, int n_q_heads, int n_kv_heads,
                        int head_dim, int block_size, float* avg_qk, void* stream);

/* ---------------------------------------------------------------- sharing state
 * Device-resident per-forward state of the shared clusters; replaces the dictionaries of
 * AttentionSharing (attn/attention_sharing.py:41-78).  The caller allocates
 * spf_sharing_state_bytes(n_slots, nb) bytes, 256-byte aligned, and calls
 * spf_sharing_state_reset before every forward (shareprefill_patch.py:156-160).
 * A "slot" is the index of a cluster within the lookup's shared_clusters list.
 */
int64_t spf_sharing_state_bytes(int n_slots, int nb);
int spf_sharing_state_reset(void* state, int n_slots, int nb, void* stream);
/* Byte offsets of the state's arrays, for tests and for exchanging pivot summaries
 * between GPUs: pivot_head[int32 S], pivot_layer[int32 S], pattern_ready[int32 S],
 * vs_ratio[f32 S], pivot_nv[int32 S], pivot_ns[int32 S], pivot_vertical[f32 S*nb],
 * pivot_slash[f32 S*nb], pivot_vlist[int32 S*nb], pivot_slist[int32 S*nb],
 * pattern[u32 S*nb*nbw], pivot_attn[f32 S*nb*nb].  offsets: host int64[12]. */
int spf_sharing_state_layout(int n_slots, int nb, int64_t* offsets /* host */);

/* ---------------------------------------------------------------- classify + elect
 * spf_classify_heads: query-aware test and similarity to the cluster's pivot
 * (attn/attention_sharing.py:201-202,271-276; attn/utils.py:26-30).
 *   slot_of_head: int32 [H], slot of the head's cluster for THIS layer or -1.
 *   out: jsd_qa, jsd_v, jsd_s fp32 [H] (NaN where not computed).
 * spf_elect_and_share: the sequential per-head decision (attn/attention_sharing.py:209-301):
 * pivot election, share test incl. the vs_ratio fallback, budget reset for query-aware
 * and shared heads.  head_flags: int32 [H] (SPF_HEAD_*), nv/ns updated in place.
 * A rank may own heads [head_offset, head_offset+n_heads) of a model with n_heads_total
 * heads: jsd_qa_all / slot_of_head_all cover ALL heads (gathered by the caller), every
 * other array covers the local heads.  Thresholds are doubles and are rounded to fp32
 * where torch compares an fp32 tensor with a Python float.
 */
int spf_classify_heads(const float* avg_qk, const float* vpool, const float* spool,
                       const int32_t* slot_of_head, const void* state, int n_slots,
                       int n_heads, int nb, float* jsd_qa, float* jsd_v, float* jsd_s,
                       void* stream);
int spf_elect_and_share(const float* jsd_qa_all, const int32_t* slot_of_head_all, int n_heads_total,
                        int head_offset, int n_heads, const float* jsd_v, const float* jsd_s,
                        const float* vpool, const float* spool, void* state, int n_slots, int nb,
                        int layer, double queryaware_threshold, double similarity_threshold,
                        double fallback_threshold, int min_blocks,
                        int32_t* nv, int32_t* ns, int32_t* head_flags, void* stream);

/* Offline head clustering (no counterpart in the reference, which ships a finished lookup file but
 * not the program that made it): out[i][j] = sqrt Jensen-Shannon divergence of x[i] and x[j], the
 * measure of attn/utils.py:26-30, for n_vec fp32 distributions of length len (<= 2 * SPF_MAX_BLOCKS);
 * out is fp32 [n_vec][n_vec].  Used by shareprefill_b200.clusters.build_lookup. */
int spf_pairwise_sqrt_jsd(const float* x, int n_vec, int len, float* out, void* stream);

/* ---------------------------------------------------------------- pattern bitmap
 * spf_build_vs_bitmap: top-k vertical columns / slash distances with the forced sink and
 * diagonal blocks, expanded to blocks, unioned with the full triangle (pivot) or the
 * cluster's shared pattern (attn/attention_sharing.py:303-337, attn/utils.py:99-128).
 * Overwrites bitmap[H][nb][nbw].  For pivot heads also stores the head's own
 * vertical / slash lists in the state (attn/attention_sharing.py:229-263).
 */
int spf_build_vs_bitmap(const float* vpool, const float* spool, const int32_t* nv,
                        const int32_t* ns, const int32_t* head_flags,
                        const int32_t* slot_of_head, void* state, int n_slots,
                        int n_heads, int nb, uint32_t* bitmap, void* stream);

/* spf_query_aware_scores: causal block-level softmax of pooled Q . pooled K for heads whose
 * SPF_HEAD_QUERY_AWARE flag is set (attn/attention_sharing.py:350-360).
 * scores: fp32 [H][nb][nb]; rows of other heads are left untouched.
 * spf_query_aware_select: global cumulative-mass rule over a head's nb*nb scores, crossing
 * element excluded (score_cover_idx, attn/utils.py:53-57; attn/attention_sharing.py:361-364);
 * selected blocks are OR-ed into the bitmap.  head_flags may be NULL to process every head.
 */
int spf_query_aware_scores(const void* avg_q, const void* avg_k, const int32_t* head_flags,
                           int n_q_heads, int n_kv_heads, int head_dim, int nb,
                           float* scores, void* stream);
int spf_query_aware_select(const float* scores, const int32_t* head_flags, int n_heads, int nb,
                           double pattern_threshold, uint32_t* bitmap, void* stream);

/* Visited key blocks per (head, query block): int32 [H][nb]; totals int64 [H]. */
int spf_bitmap_row_counts(const uint32_t* bitmap, int n_heads, int nb, int32_t* row_counts,
                          int64_t* head_totals, void* stream);

/* ---------------------------------------------------------------- block-sparse attention
 * Causal flash attention over the blocks set in `bitmap`; replaces
 * triton_block_wise_prefill_attention / block_wise_prefill_attention_kernel
 * (attn/shareprefill_attn.py:272-620): base-2 online softmax with
 * softmax_scale*log2(e), P rounded to bf16 before P.V, fp32 accumulation, bf16 output.
 * out: bf16 [n_tokens][H][D] contiguous.
 * For heads with SPF_HEAD_PIVOT set a second pass writes the per-block mean attention mass
 * into state.pivot_attn[slot] (attn/shareprefill_attn.py:425-457).  head_flags /
 * slot_of_head / state may be NULL when no head needs that.
 */
int spf_sparse_attention(const void* q, int64_t q_stride_n, int64_t q_stride_h,
                         const void* k, int64_t k_stride_n, int64_t k_stride_h,
                         const void* v, int64_t v_stride_n, int64_t v_stride_h,
                         int n_tokens, int n_q_heads, int n_kv_heads, int head_dim,
                         int block_size, double softmax_scale, const uint32_t* bitmap,
                         const int32_t* head_flags, const int32_t* slot_of_head, void* state,
                         int n_slots, void* out, void* stream);

/* ---------------------------------------------------------------- head-sharded exchange
 * With the heads of a layer split over several GPUs, the owner of a pivot elected in `layer` sends
 * its summary to the other ranks (the reference keeps all heads in one process,
 * attn/attention_sharing.py:94-103, so these have no counterpart there).  One int32 row of
 * spf_pivot_summary_width(nb) words per slot: [flag][vs_ratio bits][vertical nb][slash nb]
 * [pattern nb*ceil(nb/32)].  pack: rows of pivots elected in `layer` among heads
 * [head_begin, head_end) are filled and flagged, the flag of every other row is cleared (payload
 * untouched).  merge: `gathered` is [n_ranks][n_slots][width], as an all-gather of the packed rows
 * leaves it; per slot the first flagged row is installed and the pattern marked ready.
 */
int64_t spf_pivot_summary_width(int nb);
int spf_pack_pivot_summaries(void* state, int n_slots, int nb, int layer, int head_begin, int head_end,
                             int32_t* packed, void* stream);
int spf_merge_pivot_summaries(void* state, int n_slots, int nb, const int32_t* gathered, int n_ranks,
                              void* stream);

/* ---------------------------------------------------------------- decode step
 * One query token per head against the KV cache (q_len == 1): dense softmax attention, the step
 * the reference hands to flash_attn_func (attn/shareprefill_attn.py:146-153).
 * q: bf16 [H][D] (head stride q_stride_h); k, v: bf16 [n_keys][Hkv][D] views; out: bf16 [H][D].
 * scratch: spf_decode_scratch_bytes() bytes of split-K partials, overwritten.
 */
int64_t spf_decode_scratch_bytes(int n_keys, int n_q_heads, int n_kv_heads, int head_dim);
int spf_decode_attention(const void* q, int64_t q_stride_h,
                         const void* k, int64_t k_stride_n, int64_t k_stride_h,
                         const void* v, int64_t v_stride_n, int64_t v_stride_h,
                         int n_keys, int n_q_heads, int n_kv_heads, int head_dim,
                         double softmax_scale, void* out, void* scratch, int64_t scratch_bytes,
                         void* stream);

/* ---------------------------------------------------------------- bounded device-side waits
 * The tcgen05 kernels never spin without a limit: a wait (on an mbarrier) that has been spinning for
 * longer than the wait limit makes its CTA drain and return - its rows of the output stay unwritten -
 * and is counted.  The reference has no counterpart (its Triton kernels have no such waits); the
 * caller is expected to read the counter at a point where a device synchronisation is cheap (the
 * Python host does so at the start of every forward and raises).
 *   spf_device_timeouts        waits that gave up since the library was loaded or the counter was
 *                              reset (0 in a healthy run).  Synchronises the device.  Once it has
 *                              returned more than 16, spf_sparse_attention and spf_lastblock_profile
 *                              return SPF_ERR_TIMEOUT instead of launching.
 *   spf_reset_device_timeouts  zero the counter (after the caller has dealt with the event).
 *   spf_set_device_wait_limit_ns  the limit, default 1e9 ns; time during which the CTA was not
 *                              running is not counted.  Meant for tests.
 *   spf_wait_limit_selftest    launches one tiny kernel whose only wait can never complete: it returns
 *                              after the limit and the counter goes up by one.  Meant for tests. */
int spf_device_timeouts(void);
int spf_reset_device_timeouts(void);
int spf_set_device_wait_limit_ns(uint64_t ns);
int spf_wait_limit_selftest(void* stream);

/* Test hook (no counterpart in the reference): two kernels serve block_size = head_dim = 128 - the
 * tcgen05 ones and the mma.sync ones that also cover every other shape.  A non-zero `attention` /
 * `profile` makes spf_sparse_attention / spf_lastblock_profile take the mma.sync kernel from now on,
 * so that a test can run both on the same inputs.  Process-wide; deployments never call it. */
int spf_force_generic_kernels(int attention, int profile);

/* ---------------------------------------------------------------- pivot update
 * For every head elected pivot in this layer: per-row cumulative-mass cover of its
 * block-mass matrix, crossing element included (score_cover_idx_each_row,
 * attn/utils.py:60-76; update_pivotal_attns, attn/attention_sharing.py:94-103), stored as
 * the cluster's shared pattern; marks the pattern ready for later layers.
 */
int spf_update_pivots(const int32_t* head_flags, const int32_t* slot_of_head, void* state,
                      int n_slots, int n_heads, int nb, double pattern_threshold, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPF_B200_H_ */
