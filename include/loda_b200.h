/*
 * loda_b200 — C ABI of the B200 (sm_100a) decode hot path of LoDA-SA / NFA
 * two-level sparse attention: paged KV append with page metadata and packed
 * 4-bit tail keys, L1 page scoring + top-k, L2 token scoring + top-k + union,
 * split-K gather attention.
 *
 * Conventions (they mirror what the reference's CUDA-graph decode requires of
 * its operators, sparse_attn/indexer/nfa_layer_batch_selector.py:2769-2783 and
 * sparse_attn/engine/graph_runner.py:78-133):
 *   - every pointer is a DEVICE pointer owned by the caller, at a fixed address
 *     for the lifetime of a captured graph; the library allocates nothing;
 *   - calls are stream-ordered on `stream` (a cudaStream_t passed as void*),
 *     never synchronise the host and never copy to the host;
 *   - lengths, block tables, slot mappings and request ids are read on the
 *     device at run time, so a captured call can be replayed after they change;
 *   - functions return 0 on success and a negative code on an argument error
 *     (loda_last_error() gives the message); kernels never trap: a row that
 *     cannot be processed produces an empty selection / zero output and sets a
 *     bit in the optional device status word.
 */
#ifndef LODA_B200_H_
#define LODA_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define LODA_DTYPE_BF16 0
#define LODA_DTYPE_FP32 1

#define LODA_OK 0
#define LODA_ERR_ARGUMENT (-1)
#define LODA_ERR_UNSUPPORTED (-2)
#define LODA_ERR_LAUNCH (-3)

/* device status word bits (sparse_attn/ops/eager_decoding.py:7-35 keeps the
 * same "deferred error flag" convention) */
#define LODA_STATUS_BAD_SLOT 1u
#define LODA_STATUS_BAD_PAGE 2u
#define LODA_STATUS_TRUNCATED 4u
#define LODA_STATUS_BAD_REQ 8u   /* an active row's request slot is outside [0, max_requests): treated as a padding row */
#define LODA_STATUS_TIMEOUT 16u  /* a bounded wait (on an asynchronous copy, or on a row's scores in the level-1 launch of a large batch) gave up: the row's result is not valid */

/* Static geometry of one attention layer's cache and selector.
 * Mirrors GraphReadyPagedRegionCache.__init__ (sparse_attn/cache/
 * paged_region_cache.py:128-244), RegionGeometry (sparse_attn/policies/
 * region_geometry.py:5-23) and the NFAIndexer constants
 * (sparse_attn/indexer/nfa_indexer.py:28-121). */
typedef struct loda_geometry {
  int32_t dtype;          /* LODA_DTYPE_*: KV pool, query and output dtype */
  int32_t num_q_heads;
  int32_t num_kv_heads;
  int32_t head_dim;       /* K head dim */
  int32_t head_dim_v;
  int32_t sub_dims;       /* d': size of the scoring subspace (multiple of 16) */
  int32_t sub_lo0;        /* subspace = [sub_lo0, sub_lo0 + d'/2) U          */
  int32_t sub_lo1;        /*            [sub_lo1, sub_lo1 + d'/2)            */
  int32_t page;           /* tokens per page == selector block size */
  int32_t num_pages;      /* physical pages including the trailing PAD page */
  int32_t max_blocks;     /* block-table row length (logical pages per request) */
  int32_t max_requests;
  int32_t max_query_tokens; /* most batch rows / query rows of one call */
  int32_t max_visible;    /* row length of the gather list */
  int32_t k_far;          /* far pages kept by L1  (level1_topk - near_pages) */
  int32_t k_near;         /* near pages kept by L1 */
  int32_t level2_topk;    /* K2: token budget including sink and window */
  int32_t sink;
  int32_t swa;            /* sliding window, a multiple of `page` */
  int32_t near_len;       /* region geometry `near` */
  int32_t pool_near_len;  /* near candidate-pool span in tokens */
  int32_t shard_rank;     /* sequence sharding: this GPU owns the logical pages p with        */
  int32_t shard_count;    /* p % shard_count == shard_rank; 0 or 1 = not sharded              */
  int32_t near_tokens_p1; /* numeric near-token quota of level 2 (nfa_near_tokens, nfa_layer_batch_selector.py:
                           * 872-920): 0 = "off" (one quota over the whole middle range, the default); n + 1 =
                           * n tokens reserved for the near region, the far and near regions then select separately */
  int32_t far_method;     /* LODA_FAR_*: level-1 score of the far pool (nfa_far_method) */
  int32_t near_minmax;    /* 0: near pool scored by the page mean (nfa_near_method "avg", the default); 1: by the
                           * min/max bound */
  int32_t reserved;
} loda_geometry;

/* loda_geometry.far_method (nfa_layer_batch_selector.py:290-354, 2412-2427) */
#define LODA_FAR_MINMAX 0    /* min/max upper bound, mean over the GQA group (default) */
#define LODA_FAR_AVG 1       /* page mean, mean over the group */
#define LODA_FAR_AVG_TOP2 2  /* page mean, mean of the two best heads of the group */

/* Per-layer device buffers.
 *   pool_k / pool_v  [num_pages, num_kv_heads, page, head_dim(_v)]   (the
 *        reference arena [pages+1, 1, Hkv, PAGE, D], paged_region_cache.py:89-98)
 *   page_mm   per (request slot, kv head) row the min and the max of the subspace keys over the visible
 *        tokens of every logical page; page_sum: the sum of the same (replace P_MIN / P_MAX / P_SUM,
 *        nfa_layer_batch_selector.py:2103-2118).  Layout of a row: the logical pages in groups of 32;
 *        a group stores 16-byte chunk c of its 32 pages, then chunk c + 1, ... — for page_mm the d'/8
 *        chunks of the min row followed by the d'/8 chunks of the max row (d'/4 chunks, 128 d' bytes per
 *        group), for page_sum d'/8 chunks (64 d' bytes per group).  Byte offset of chunk c of page p in a
 *        row: ((p / 32) * CH + c) * 512 + (p % 32) * 16 with CH chunks per page; a row has
 *        ceil(max_blocks / 32) groups; rows follow each other [max_requests, num_kv_heads].  (32 threads
 *        reading one chunk of 32 consecutive pages read 512 contiguous bytes, and a run of groups is one
 *        contiguous block for a bulk copy.)
 *   tail_code [num_pages, num_kv_heads, page, d'/2] bytes: two 4-bit codes per
 *        byte, dim 2i in the low nibble
 *   tail_sz   [num_pages, num_kv_heads, page, 2]: quantisation scale and zero
 *   block_table [max_requests, max_blocks] int32 logical -> physical page      */
typedef struct loda_layer {
  void* pool_k;
  void* pool_v;
  void* page_mm;
  void* page_sum;
  uint8_t* tail_code;
  void* tail_sz;
  const int32_t* block_table;
  /* region skip decisions of this layer per request slot, [max_requests] int32, nonzero = the far /
   * near region of the request is neither scored nor selected (skip_far_layer_buf / skip_near_layer_buf,
   * sparse_attn/cache/paged_region_cache.py:293-296, 540-559).  NULL = nothing is skipped. */
  const int32_t* skip_far;
  const int32_t* skip_near;
} loda_layer;

/* Per-step batch metadata (paged_region_cache.py:214-231). */
typedef struct loda_batch {
  int32_t batch;                  /* rows in this step */
  const int32_t* lengths;         /* [batch] length including the current token */
  const int64_t* valid_req_ids;   /* [batch] request slot of each row (pad rows: 0) */
  const int64_t* active_req_ids;  /* [batch] < 0 marks a padding row */
} loda_batch;

/* Selection outputs (workspace tensors of the reference selector).
 *   i_far [batch, Hkv, k_far], i_near [batch, Hkv, k_near]: page ids, best first,
 *   then fillers; n_far / n_near [batch, Hkv]: how many leading entries carry a
 *   finite score.  These four are OPTIONAL (all NULL or all given): the page
 *   list travels from L1 to L2 inside the workspace in ascending page order,
 *   and the best-first lists are only written when asked for (parity checks).
 *   gather [>=batch, Hkv, max_visible] physical slots in ascending logical order
 *   visible_lens [>=batch, Hkv]
 *   middle / middle_counts (optional, may be NULL): the L2 survivors as logical
 *   token ids [batch, Hkv, level2_topk] before the union                        */
typedef struct loda_selection {
  int32_t* i_far;
  int32_t* n_far;
  int32_t* i_near;
  int32_t* n_near;
  int32_t* gather;
  int32_t* visible_lens;
  int32_t* middle;
  int32_t* middle_counts;
  int32_t middle_only;    /* 1: gather / visible_lens receive the level-2 survivors only, without the sink
                           * and window tokens (select_topk_for_layer_batched(middle_only=True),
                           * nfa_layer_batch_selector.py:2649-2671) */
  int32_t flags;          /* LODA_SEL_* bits, 0 by default */
} loda_selection;

/* loda_selection.flags.
 * LODA_SEL_CHAINED: the caller guarantees that (1) the kernel launched before this call on the same
 * stream is a loda_decode_step / loda_select_step of this library, and (2) everything this call reads
 * besides the query — b->lengths / valid_req_ids / active_req_ids, the skip flags and the page
 * statistics of pages outside the sliding window — was complete before THAT launch started.  This is
 * the decode of one token through the layers of a model: set the flag for every layer but the first.
 * The one-launch kernel then fetches the batch metadata and stages page statistics while the previous
 * launch drains.  Without the flag nothing but launch parameters is read before the launch's
 * dependency wait, and the call is safe behind any kernel (one that advances lengths on the device, an
 * index build, a foreign kernel that releases its dependents early). */
#define LODA_SEL_CHAINED 1

const char* loda_version(void);
const char* loda_last_error(void);

/* Scratch bytes needed by the calls below (sized by g->max_query_tokens).  The
 * scratch must be zero-filled once before first use; kernels leave it zeroed
 * where that matters.  Returns 0 if the geometry is not supported. */
size_t loda_workspace_bytes(const loda_geometry* g);

/* Append one decode token per row: K/V rows into the pool, packed 4-bit tail
 * key of the token, and min/max/sum of its logical page.
 * Replaces paged_write_decode (sparse_attn/ops/paged_region_kernels.py:665-724)
 * and the fused owner write + page-stats body
 * (nfa_layer_batch_selector.py:31-131, 1005-1078).
 *   k_new [batch, Hkv, head_dim], v_new [batch, Hkv, head_dim_v], slots [batch]
 *   (-1 routes the row to the PAD page and skips the metadata).
 *   k_new == v_new == NULL: the rows are already in the pool; only the packed
 *   key of the newest token (position lengths[row] - 1) and the statistics of
 *   its page are refreshed. */
int loda_append_decode(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                       const void* k_new, const void* v_new, const int32_t* slots,
                       uint32_t* status, void* stream);

/* Scatter a prefill [Hkv, n_tokens, head_dim] through one block-table row.
 * Replaces paged_write_prefill (paged_region_kernels.py:610-662). */
int loda_write_prefill(const loda_geometry* g, const loda_layer* layer,
                       const void* k, const void* v, const int32_t* block_table_row,
                       int32_t n_tokens, void* stream);

/* (Re)build page metadata and packed tail keys of logical pages
 * [first_block, first_block + n_blocks) of request slot `req_id` whose length
 * is `length`, reading the keys from the pool.  Replaces the full page-stats
 * rebuild after freeze (nfa_layer_batch_selector.py:2121-2145). */
int loda_build_index(const loda_geometry* g, const loda_layer* layer, int32_t req_id,
                     int32_t length, int32_t first_block, int32_t n_blocks, void* stream);

/* L1: page scores from the min/max bound (far pool) and page mean (near pool),
 * exact top-k per pool with ties toward the lower page id.  Replaces
 * _l1_scores + the L1 top-k kernels (nfa_layer_batch_selector.py:174-354,
 * 1473-1863).  q [batch, Hq, head_dim].  Leaves the surviving pages of every
 * row (ascending, bypass pages included, with their physical page ids) in the
 * workspace for loda_select_l2. */
int loda_select_l1(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                   const void* q, float scale, const loda_selection* out,
                   void* workspace, void* stream);

/* L2: grouped-query logits on the packed 4-bit tail keys of the surviving
 * pages, exact top-quota with ties toward the lower token id, hole fill, union
 * with sink and window tokens, logical -> physical slots.  Must follow
 * loda_select_l1 of the same batch on the same workspace.  Replaces candidate
 * expansion, fine scores, filtered top-k and the final union
 * (nfa_layer_batch_selector.py:422-848, 1116-1437). */
int loda_select_l2(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                   const void* q, float scale, const loda_selection* sel,
                   uint32_t* status, void* workspace, void* stream);

/* Append + L1 + L2 of one layer in two launches: the append (or, with k_new ==
 * v_new == NULL, the index refresh) rides in extra CTAs of the L1 launch — it
 * only touches the newest token and its page, which this step's selection
 * never reads.  This is what select_topk_for_layer_batched(decode_write=...)
 * does in the reference with its fused owner write
 * (nfa_layer_batch_selector.py:1005-1078, 2649-2720). */
int loda_select_step(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                     const void* q, const void* k_new, const void* v_new, const int32_t* slots,
                     float scale, const loda_selection* sel, uint32_t* status,
                     void* workspace, void* stream);

/* Gather attention over the selected slots with split-K and a log-sum-exp
 * merge.  Replaces sparse_paged_attention_gather (paged_region_kernels.py:
 * 800-1041).  q [n_query, Hq, head_dim], query_to_req [n_query] (<0: output
 * row of zeros), out [n_query, Hq, head_dim_v]. */
int loda_gather_attend(const loda_geometry* g, const loda_layer* layer,
                       const void* q, const int32_t* gather, const int32_t* visible_lens,
                       const int32_t* query_to_req, int32_t n_query, int32_t n_req_rows,
                       float scale, void* out, void* workspace, void* stream);

/* Same as loda_gather_attend, additionally writing lse [n_query, Hq, 2] float:
 * the row maximum of the scaled scores in the exp2 domain and the softmax sum.
 * Partial attentions over disjoint token sets (pages of one long request held
 * by different GPUs) merge exactly from (out, lse): see lse_merge in
 * two-level-attention_b200/sharding.py.  Extends the split combine of the
 * reference (paged_region_kernels.py:578-607) across devices. */
int loda_gather_attend_lse(const loda_geometry* g, const loda_layer* layer,
                           const void* q, const int32_t* gather, const int32_t* visible_lens,
                           const int32_t* query_to_req, int32_t n_query, int32_t n_req_rows,
                           float scale, void* out, float* lse, void* workspace, void* stream);

/* Gather attention without a caller-provided workspace and without any
 * allocation.  (No counterpart in the reference: its Triton operators always
 * allocate their split buffers through torch.)
 * Meant for hosts that cannot allocate device memory where they call this
 * library — a plugin inside another framework's fixed memory plan, a process
 * whose device memory was handed out at start-up, code under a no-allocation
 * guard.  The split-K partials and tickets live in a fixed array inside the
 * library (about 4.1 MiB on every GPU that loads it, held until exit), which
 * limits the call to n_query * num_kv_heads <= 64, num_q_heads / num_kv_heads
 * <= 8 and head_dim_v <= 128; larger calls return LODA_ERR_UNSUPPORTED.
 * The first call on each device looks up the array's device address; make that
 * first call before any stream capture.  All calls on a device share the one
 * array: calls that overlap on the GPU (different streams) race on it.
 * Same arguments and results as loda_gather_attend otherwise. */
int loda_gather_attend_static(const loda_geometry* g, const loda_layer* layer,
                              const void* q, const int32_t* gather, const int32_t* visible_lens,
                              const int32_t* query_to_req, int32_t n_query, int32_t n_req_rows,
                              float scale, void* out, void* stream);

/* The whole decode step of one layer on one stream: append, L1, L2, attend.
 * One kernel launch where a thread-block cluster per (request, kv head) row fits
 * the GPU (batch 1 at long context) and head_dim = head_dim_v = 128: the clusters
 * that selected the tokens attend over them.  Otherwise the launches of
 * loda_select_step followed by the attention launch.  Same results either way:
 * identical lists, attention within the bf16 tolerance of the path.
 * With sel->flags & LODA_SEL_CHAINED (see there) the one-launch kernel reads
 * b->lengths / valid_req_ids / active_req_ids and the page statistics of pages
 * outside the sliding window before it waits for the launch before it; without
 * the flag every read follows the wait.
 *
 * Replaces select_topk_for_layer_batched(decode_write=...) followed by
 * decode_graph_ready (nfa_layer_batch_selector.py:2649-2720,
 * sparse_attn/ops/paged_region_kernels_nfa.py:122-162).  One query per row
 * (query_to_req is the identity over the batch rows). */
int loda_decode_step(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                     const void* q, const void* k_new, const void* v_new, const int32_t* slots,
                     float scale, const loda_selection* sel, const int32_t* query_to_req,
                     void* out, uint32_t* status, void* workspace, void* stream);

/* How many kernels the latest loda_decode_step of this process launched: 1 (selection and
 * attention in one launch: batch 1 at long context, head dimensions 128), 2 (one-launch
 * selection, then attention) or 3 (L1, L2, attention).  For benchmarks and logs. */
int loda_last_decode_launches(void);

/* CTAs per (request, kv head) row of the one-launch kernel as the latest call of this thread launched it
 * (16, or 8 where the GPU cannot hold a cluster of 16 for every row), 0 if the
 * call ran the separate launches.  For benchmarks and logs. */
int loda_last_decode_cluster(void);

/* gather / visible_lens = the protected tokens only: sink ++ sliding window as physical
 * slots, per (batch row, kv head).  Replaces build_protected_gather
 * (sparse_attn/ops/paged_region_kernels_nfa.py:84-119).  With loda_selection.middle_only
 * and loda_gather_attend_lse on the two lists, the partial attentions merge by
 * log-sum-exp (the reference's "disjoint protected / middle" operator mode). */
int loda_protected_gather(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                          int32_t* gather, int32_t* visible_lens, uint32_t* status, void* stream);

/* ---- sequence sharding (batch-1 long context over several GPUs) ---------------
 * No counterpart in the reference's code (its runs are single-GPU): logical page p belongs to GPU p % shard_count (geometry.shard_rank /
 * shard_count), whose block table holds -1 for the pages of the others.  The selector
 * runs in four stages; between the stages the caller combines the score rows of the
 * GPUs with a bitwise OR (every page / slot is scored by exactly one GPU, the others
 * hold 0), e.g. an all-gather over NCCL.  With identical combined scores every GPU
 * selects the same pages and tokens as a single GPU would; its gather list holds -1
 * for tokens on pages it does not own, its attention (loda_gather_attend_lse) covers
 * its own tokens, and the partial outputs merge by log-sum-exp. */

/* out[0], out[1] = byte offset and size of the level-1 score rows in the workspace,
 * out[2], out[3] = of the level-2 score rows (both uint16, 0 = not scored here). */
int loda_shard_workspace_regions(const loda_geometry* g, int64_t* out);

/* level 1: scores of this GPU's pages -> workspace | selection on the combined scores */
int loda_shard_l1_scores(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                         const void* q, float scale, const loda_selection* sel, void* workspace,
                         void* stream);
/* gathered (may be NULL): the score rows of all shard_count GPUs after an all-gather, shard_count blocks of
 * the size loda_shard_workspace_regions reports for the level, in rank order; the selection ORs them while it
 * loads the row.  NULL: the caller has already combined the rows inside the workspace. */
int loda_shard_l1_select(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                         const void* q, float scale, const loda_selection* sel, const void* gathered,
                         void* workspace, void* stream);
/* level 2: logits of the candidate slots on this GPU's pages -> workspace | quota
 * selection, hole fill and union on the combined logits -> gather, visible_lens */
int loda_shard_l2_scores(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                         const void* q, float scale, const loda_selection* sel, uint32_t* status,
                         void* workspace, void* stream);
int loda_shard_l2_select(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                         const void* q, float scale, const loda_selection* sel, uint32_t* status,
                         const void* gathered, void* workspace, void* stream);

/* Fixed-order log-sum-exp merge of n_parts partial attentions (loda_gather_attend_lse on disjoint token
 * sets, e.g. the GPUs of a sequence-sharded request after an all-gather): part r lies part_stride_bytes
 * after part r - 1 and holds out [n_rows, dv] bf16 at byte 0 and lse [n_rows, 2] float at lse_offset_bytes;
 * out [n_rows, dv] float.  Parts merge in index order, so every GPU that merges the same parts gets the same
 * bits; a part with sum 0 contributes nothing; all sums 0 give zeros. */
int loda_lse_merge(const void* parts, int64_t part_stride_bytes, int64_t lse_offset_bytes, int32_t n_parts,
                   int32_t n_rows, int32_t dv, float* out, void* stream);

/* ---- kernels under the TIA indexer's method surface -------------------------
 * (sparse_attn/indexer/tia_indexer.py; tensors bf16 or fp32, dtype = LODA_DTYPE_*) */

/* y = 4-bit per-token quantise + de-quantise of n_rows rows of `dim` <= 128
 * values (row strides in elements).  Replaces TIAIndexer.min_max_per_token_quant
 * (tia_indexer.py:22-31), bit for bit. */
int loda_tia_quant4(const void* x, void* y, int64_t n_rows, int32_t dim, int64_t x_stride,
                    int64_t y_stride, int32_t dtype, void* stream);

/* k [S, H, D] -> kmin, kmax [ceil(S / block_size), H, D]; the ragged last block
 * is padded with zeros before reducing.  Replaces the amin / amax of
 * TIAIndexer.prepare_index (tia_indexer.py:39-46). */
int loda_tia_block_minmax(const void* k, void* kmin, void* kmax, int32_t S, int32_t H, int32_t D,
                          int32_t block_size, int32_t dtype, void* stream);

/* coarse [Hq, T] = sum_d min(q s, 0) kmin + max(q s, 0) kmax and
 * fine [Hq, S] = sum_d (q s) kqat for q [Hq, D], kmin / kmax [T, Hkv, D],
 * kqat [S, Hkv, D], s = scale; fp32 accumulate, one rounding to the dtype.
 * Replaces TIAIndexer.compute_score (tia_indexer.py:64-99). */
int loda_tia_scores(const void* q, const void* kmin, const void* kmax, const void* kqat,
                    void* coarse, void* fine, int32_t Hq, int32_t Hkv, int32_t D, int32_t T,
                    int32_t S, float scale, int32_t dtype, void* stream);

/* ---- the prototype chain on a contiguous KV cache (tls_attn/ops) ---------------
 * All tensors bf16 unless stated, caches [max_batch, max_seqlen, Hkv, D] token-major
 * as in the reference; scores fp32; indices int32. */

/* decode = 0: cache[b, s] = x[b, offsets[b] + s] for s < seqlen - offsets[b], for
 * k [batch, seqlen, Hkv, dim_k] and v [.., dim_v]; decode = 1: x is [batch, 1, Hkv, D]
 * and lands at cache[b, lengths[b] - 1].  Replaces MHAStoreKVInterface.prefill_forward /
 * decode_forward (tls_attn/ops/mha_store_kv.py:123-141). */
int loda_tls_store_kv(const void* k, const void* v, const int32_t* offsets_or_lengths,
                      void* k_cache, void* v_cache, int32_t batch, int32_t seqlen,
                      int32_t max_seqlen, int32_t num_kv_heads, int32_t dim_k, int32_t dim_v,
                      int32_t decode, void* stream);

/* Index of the keys: per block of `block` tokens the min and max over the tokens of the
 * full key (l1_min, l1_max [max_batch, l1_len, Hkv, dim_k]; a ragged last block is padded
 * with zeros) and per token the tail sub-dimensions [D/2 - c, D/2) ++ [D - c, D),
 * c = D / 2 / cmp_ratio (l2_k [max_batch, l2_len, Hkv, 2c]).  decode = 0: k is
 * [batch, src_len, Hkv, dim_k], tokens from offsets[b] on are indexed at positions 0..;
 * decode = 1: k is the cache [max_batch, src_len, Hkv, dim_k], the token lengths[b] - 1
 * is indexed (its block's min / max only when it completes the block).  Replaces
 * MHAStoreKIndexInterface.prefill_forward / decode_forward
 * (tls_attn/ops/mha_store_k_index.py:167-185). */
int loda_tls_store_k_index(const void* k, const int32_t* offsets_or_lengths, void* l1_min,
                           void* l1_max, void* l2_k, int32_t batch, int32_t src_len,
                           int32_t num_kv_heads, int32_t dim_k, int32_t block, int32_t cmp_ratio,
                           int32_t l1_len, int32_t l2_len, int32_t decode, void* stream);

/* scores [batch, Hkv, max_length] = sum over the group's heads of max(q s, 0) . k_max +
 * min(q s, 0) . k_min per block (q [batch, 1, Hq, dim_k]; q s rounded to bf16; lengths in
 * blocks), -inf from lengths[b] - sliding_blocks on; then the topk best blocks, sorted
 * (score descending, lower block first), missing entries (-inf, -1).  Replaces
 * MHAIndexerLevel1Interface.forward_with_buffer (tls_attn/ops/mha_indexer_level1.py:237-249). */
int loda_tls_level1(const void* q, const void* k_min, const void* k_max, const int32_t* lengths,
                    float* scores, float* topk_scores, int32_t* topk_indices, int32_t batch,
                    int32_t num_heads, int32_t num_kv_heads, int32_t dim_k, int32_t l1_len,
                    int32_t max_length, int32_t topk, int32_t sliding_blocks, float scaling,
                    void* stream);

/* For every token of the blocks block_indices [batch, Hkv, level1_topk] (-1 = hole):
 * scores = sum over the group's heads of exp(s_g - M), s_g = (q_g s) . k_token on the
 * sub-dimensions (k [max_batch, k_len, Hkv, dim_k]), M the maximum over the row; indices =
 * token ids (-1 for holes); cummax_scores (may be NULL) is filled with M.  Then the
 * level2_topk best tokens, the tokens of the last sliding_blocks blocks of the sequence
 * (lengths in tokens) first with score +inf.  Replaces
 * MHAIndexerLevel2Interface.forward_with_buffer (tls_attn/ops/mha_indexer_level2.py:277-290). */
int loda_tls_level2(const void* q, const void* k, const int32_t* block_indices,
                    const int32_t* lengths, float* scores, float* cummax_scores, int32_t* indices,
                    float* topk_scores, int32_t* topk_indices, int32_t batch, int32_t num_heads,
                    int32_t num_kv_heads, int32_t dim_k, int32_t k_len, int32_t level1_topk,
                    int32_t level2_topk, int32_t block, int32_t sliding_blocks, float scaling,
                    void* stream);

#ifdef __cplusplus
}
#endif
#endif /* LODA_B200_H_ */
