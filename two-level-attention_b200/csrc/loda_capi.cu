// C ABI of loda_b200 (declared in include/loda_b200.h): argument validation,
// scratch layout and kernel launches.  No allocation, no host synchronisation.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "loda_common.cuh"

namespace loda {

cudaError_t launch_append_decode(const loda_geometry&, const loda_layer&, const loda_batch&, const void*,
                                 const void*, const int32_t*, uint32_t*, cudaStream_t);
cudaError_t launch_build_index(const loda_geometry&, const loda_layer&, int, int, int, int, cudaStream_t);
cudaError_t launch_write_prefill(const loda_geometry&, const loda_layer&, const void*, const void*,
                                 const int32_t*, int, cudaStream_t);
cudaError_t launch_l1(const loda_geometry&, const loda_layer&, const loda_batch&, const void*, float,
                      const loda_selection&, const SelectWorkspace&, const AppendArgs&, int, cudaStream_t);
cudaError_t launch_l2(const loda_geometry&, const loda_layer&, const loda_batch&, const void*, float,
                      const loda_selection&, const SelectWorkspace&, uint32_t*, bool, int, cudaStream_t);
int l1_score_stride(const loda_geometry&);
cudaError_t launch_protected_gather(const loda_geometry&, const loda_layer&, const loda_batch&, int32_t*, int32_t*,
                                    uint32_t*, cudaStream_t);
bool select_fused_applicable(const loda_geometry&, int);
void select_fused_refuse(int);
int select_fused_last_cluster();
cudaError_t launch_decode_fused(const loda_geometry&, const loda_layer&, const loda_batch&, const void*, float,
                                const loda_selection&, uint32_t*, const AppendArgs&, const int32_t*, void*, cudaStream_t);
cudaError_t launch_select_fused(const loda_geometry&, const loda_layer&, const loda_batch&, const void*, float,
                                const loda_selection&, uint32_t*, const AppendArgs&, cudaStream_t);
cudaError_t launch_attn(const loda_geometry&, const loda_layer&, const void*, const int32_t*, const int32_t*,
                        const int32_t*, int, int, float, void*, float*, const AttnWorkspace&, bool, bool, bool, cudaStream_t);
cudaError_t launch_attn_mla(const loda_geometry&, const loda_layer&, const void*, const int32_t*, const int32_t*,
                            const int32_t*, int, int, float, void*, float*, const AttnWorkspace&, bool, bool, uint32_t*,
                            cudaStream_t);
size_t l1_smem_bytes(const loda_geometry&);
size_t l2_smem_bytes(const loda_geometry&);
int attn_nsplit(const loda_geometry&, int);

static thread_local char g_error[512] = "";

static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_error, sizeof(g_error), fmt, ap);
  va_end(ap);
  return code;
}

static int check_cuda(cudaError_t e, const char* what) {
  if (e == cudaSuccess) return LODA_OK;
  return fail(LODA_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
}

static size_t align_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// Properties of the current device, looked up once per device ordinal.
int device_ordinal() {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess) { (void)cudaGetLastError(); return -1; }
  return dev;
}

int device_sm_count() {
  constexpr int kMax = 64;
  static int sms[kMax] = {};
  const int dev = device_ordinal();
  if (dev < 0 || dev >= kMax) return 148;
  if (sms[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      (void)cudaGetLastError();
      n = 148;
    }
    sms[dev] = n;
  }
  return sms[dev];
}

constexpr int kAttnMaxSplit = 16;

struct WsLayout {
  size_t l1_ticket, l2_ticket, at_ticket, l1_scores, pages, phys, np, l2_scores;
  size_t at_m, at_z, at_o, total;
};

static WsLayout ws_layout(const loda_geometry& g) {
  WsLayout w;
  const size_t rows = (size_t)g.max_query_tokens * g.num_kv_heads;
  const size_t pairs = rows;
  const size_t G = g.num_q_heads / g.num_kv_heads;
  const size_t np_max = g.k_far + g.k_near + 2;
  size_t off = 0;
  w.l1_ticket = off; off = align_up(off + (rows + 2) * 4, 256);
  w.l2_ticket = off; off = align_up(off + rows * 4, 256);
  w.at_ticket = off; off = align_up(off + pairs * 4, 256);
  w.np = off; off = align_up(off + rows * 4, 256);
  w.pages = off; off = align_up(off + rows * np_max * 4, 256);
  w.phys = off; off = align_up(off + rows * np_max * 4, 256);
  w.l1_scores = off; off = align_up(off + rows * (size_t)l1_score_stride(g) * 2, 256);
  w.l2_scores = off; off = align_up(off + rows * np_max * g.page * 2, 256);
  w.at_m = off; off = align_up(off + pairs * kAttnMaxSplit * G * 4, 256);
  w.at_z = off; off = align_up(off + pairs * kAttnMaxSplit * G * 4, 256);
  w.at_o = off; off = align_up(off + pairs * kAttnMaxSplit * G * g.head_dim_v * 4, 256);
  w.total = off;
  return w;
}

static SelectWorkspace select_ws(const loda_geometry& g, void* workspace) {
  const WsLayout w = ws_layout(g);
  char* base = (char*)workspace;
  SelectWorkspace ws;
  ws.l1_ticket = (int*)(base + w.l1_ticket);
  ws.ticket_rows = g.max_query_tokens * g.num_kv_heads;
  ws.l2_ticket = (int*)(base + w.l2_ticket);
  ws.l1_scores = (uint16_t*)(base + w.l1_scores);
  ws.score_stride = l1_score_stride(g);
  ws.pages = (int*)(base + w.pages);
  ws.phys = (int*)(base + w.phys);
  ws.np = (int*)(base + w.np);
  ws.l2_scores = (uint16_t*)(base + w.l2_scores);
  return ws;
}

static int check_geometry(const loda_geometry* g) {
  if (!g) return fail(LODA_ERR_ARGUMENT, "geometry is NULL");
  if (g->dtype != LODA_DTYPE_BF16)
    return fail(LODA_ERR_UNSUPPORTED, "only bf16 KV pools are implemented (dtype=%d)", g->dtype);
  if (g->shard_count < 0 || (g->shard_count > 1 && (g->shard_rank < 0 || g->shard_rank >= g->shard_count)))
    return fail(LODA_ERR_ARGUMENT, "shard_rank must be in [0, shard_count)");
  if (g->num_kv_heads < 1 || g->num_q_heads % g->num_kv_heads)
    return fail(LODA_ERR_ARGUMENT, "GQA requires num_q_heads %% num_kv_heads == 0");
  const int G = g->num_q_heads / g->num_kv_heads;
  if (G > 16) return fail(LODA_ERR_UNSUPPORTED, "GQA group %d > 16", G);
  if (g->head_dim % 16 || g->head_dim_v % 16) return fail(LODA_ERR_ARGUMENT, "head dims must be multiples of 16");
  if (g->sub_dims != 16 && g->sub_dims != 32 && g->sub_dims != 64)
    return fail(LODA_ERR_UNSUPPORTED, "subspace size %d not in {16, 32, 64}", g->sub_dims);
  const int half = g->sub_dims / 2;
  if (g->sub_lo0 < 0 || g->sub_lo1 < 0 || g->sub_lo0 + half > g->head_dim || g->sub_lo1 + half > g->head_dim)
    return fail(LODA_ERR_ARGUMENT, "subspace ranges outside the head");
  if (g->page < 1 || (g->page & (g->page - 1))) return fail(LODA_ERR_ARGUMENT, "page must be a power of two");
  if (g->swa < 1 || g->swa % g->page) return fail(LODA_ERR_ARGUMENT, "swa must be a positive multiple of page");
  if (g->max_blocks < 1 || g->max_blocks > 65536) return fail(LODA_ERR_UNSUPPORTED, "max_blocks must be in [1, 65536]");
  if (g->max_requests < 1 || g->max_query_tokens < 1)
    return fail(LODA_ERR_ARGUMENT, "max_requests / max_query_tokens must be >= 1");
  if (g->num_pages < 2) return fail(LODA_ERR_ARGUMENT, "num_pages must include the PAD page");
  if (g->k_far < 0 || g->k_near < 0 || g->k_far > 512 || g->k_near > 512)
    return fail(LODA_ERR_UNSUPPORTED, "k_far / k_near must be in [0, 512]");
  if (g->k_far > g->max_blocks || g->k_near > g->max_blocks)
    return fail(LODA_ERR_ARGUMENT, "k_far / k_near exceed max_blocks");
  if ((size_t)(g->k_far + g->k_near + 2) * g->page > 32768)
    return fail(LODA_ERR_UNSUPPORTED, "more than 32768 L2 candidate slots per row");
  if (g->page < 8 && g->k_far + g->k_near > 0)
    return fail(LODA_ERR_UNSUPPORTED, "the selector needs pages of at least 8 tokens");
  if (g->pool_near_len / g->page + 8 > 512)
    return fail(LODA_ERR_UNSUPPORTED, "near pool wider than 512 pages");
  if (g->level2_topk < g->sink + g->swa) return fail(LODA_ERR_ARGUMENT, "level2_topk < sink + swa");
  if (g->far_method < LODA_FAR_MINMAX || g->far_method > LODA_FAR_AVG_TOP2 || g->near_minmax < 0 || g->near_minmax > 1)
    return fail(LODA_ERR_ARGUMENT, "far_method must be LODA_FAR_*, near_minmax 0 or 1");
  if (g->near_tokens_p1 < 0 || (g->near_tokens_p1 > 0 && g->near_tokens_p1 - 1 > g->k_near * g->page))
    return fail(LODA_ERR_ARGUMENT, "near_tokens_p1 must be 0 (off) or 1 + a count of at most k_near * page tokens");
  if (g->far_method == LODA_FAR_AVG_TOP2 && g->num_q_heads / g->num_kv_heads < 2)
    return fail(LODA_ERR_ARGUMENT, "far method avg_top2 needs a GQA group of at least two heads");
  if (g->shard_count > 1 && (g->near_tokens_p1 > 0 || g->far_method != LODA_FAR_MINMAX || g->near_minmax))
    return fail(LODA_ERR_UNSUPPORTED, "sequence sharding serves the default level-1 methods and quota");
  if (g->max_visible < g->level2_topk) return fail(LODA_ERR_ARGUMENT, "max_visible < level2_topk");
  if (g->sink < 0 || g->near_len < 0 || g->pool_near_len < g->page)
    return fail(LODA_ERR_ARGUMENT, "bad sink / near_len / pool_near_len");
  if ((size_t)g->max_blocks * 2 + 16 > 40 * 1024)
    return fail(LODA_ERR_UNSUPPORTED, "max_blocks too large: a row's page scores must fit in shared memory");
  if (l1_smem_bytes(*g) > 200 * 1024 || l2_smem_bytes(*g) > 200 * 1024)
    return fail(LODA_ERR_UNSUPPORTED, "geometry needs more than 200 KB of shared memory");
  return LODA_OK;
}

static int check_layer(const loda_layer* l, bool need_index = true) {
  if (!l || !l->pool_k || !l->pool_v) return fail(LODA_ERR_ARGUMENT, "layer pools must be non-NULL");
  if (need_index &&
      (!l->page_mm || !l->page_sum || !l->tail_code || !l->tail_sz || !l->block_table))
    return fail(LODA_ERR_ARGUMENT, "layer index buffers and block table must be non-NULL");
  return LODA_OK;
}

static int check_batch(const loda_geometry* g, const loda_batch* b) {
  if (!b || b->batch < 0 || b->batch > g->max_query_tokens)
    return fail(LODA_ERR_ARGUMENT, "batch must be in [0, max_query_tokens]");
  if (b->batch > 0 && (!b->lengths || !b->valid_req_ids || !b->active_req_ids))
    return fail(LODA_ERR_ARGUMENT, "batch metadata pointers must be non-NULL");
  return LODA_OK;
}

// Shared with entry points that live next to their kernels.
int report_error(int code, const char* message) { return fail(code, "%s", message); }

int check_gather_attend_args(const loda_geometry* g, const loda_layer* layer, const void* q,
                             const int32_t* gather, const int32_t* visible_lens, const int32_t* query_to_req,
                             int32_t n_query, int32_t n_req_rows, const void* out) {
  int rc = check_geometry(g);
  if (rc != LODA_OK) return rc;
  rc = check_layer(layer, false);
  if (rc != LODA_OK) return rc;
  if (n_query < 0 || n_query > g->max_query_tokens)
    return fail(LODA_ERR_ARGUMENT, "n_query must be in [0, max_query_tokens]");
  if (n_query > 0 && (!q || !gather || !visible_lens || !query_to_req || !out || n_req_rows < 1))
    return fail(LODA_ERR_ARGUMENT, "gather attention needs q, gather, visible_lens, query_to_req and out");
  if (g->head_dim == 576 && g->head_dim_v == 512) {
    // shared-latent layout: the value row is the first 512 dims of the key row
    if (layer->pool_v != layer->pool_k || g->num_kv_heads != 1 || g->num_q_heads > 16)
      return fail(LODA_ERR_UNSUPPORTED, "head dims 576 / 512 are served for the shared-latent layout only: "
                                        "pool_v == pool_k, one kv head, at most 16 query heads");
    return LODA_OK;
  }
  if (!((g->head_dim == 128 && g->head_dim_v == 128) || (g->head_dim == 64 && g->head_dim_v == 64)))
    return fail(LODA_ERR_UNSUPPORTED, "gather attention supports head dims 64 and 128, and 576 / 512 with a shared latent");
  return LODA_OK;
}

}  // namespace loda

using namespace loda;

#define LODA_TRY(expr)          \
  do {                          \
    int rc_ = (expr);           \
    if (rc_ != LODA_OK) return rc_; \
  } while (0)

extern "C" {

const char* loda_version(void) { return "loda_b200 0.1 (sm_100a)"; }

const char* loda_last_error(void) { return g_error; }

size_t loda_workspace_bytes(const loda_geometry* g) {
  if (check_geometry(g) != LODA_OK) return 0;
  return ws_layout(*g).total;
}

int loda_append_decode(const loda_geometry* g, const loda_layer* layer, const loda_batch* b,
                       const void* k_new, const void* v_new, const int32_t* slots, uint32_t* status,
                       void* stream) {
  LODA_TRY(check_geometry(g));
  // a layer without index buffers may only be used for a plain K/V write: the
  // kernel touches the index only for rows whose active_req_ids entry is >= 0
  LODA_TRY(check_layer(layer, layer && layer->page_mm != nullptr));
  LODA_TRY(check_batch(g, b));
  if (b->batch == 0) return LODA_OK;
  if ((k_new == nullptr) != (v_new == nullptr) || (k_new && !slots))
    return fail(LODA_ERR_ARGUMENT, "k_new, v_new and slots go together (all NULL = refresh the index only)");
  return check_cuda(launch_append_decode(*g, *layer, *b, k_new, v_new, slots, status, (cudaStream_t)stream),
                    "append_decode");
}

int loda_write_prefill(const loda_geometry* g, const loda_layer* layer, const void* k, const void* v,
                       const int32_t* block_table_row, int32_t n_tokens, void* stream) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer, false));
  if (n_tokens < 0 || n_tokens > g->max_blocks * g->page)
    return fail(LODA_ERR_ARGUMENT, "prefill length exceeds block-table capacity");
  if (!k || !v || !block_table_row) return fail(LODA_ERR_ARGUMENT, "k / v / block_table_row must be non-NULL");
  return check_cuda(launch_write_prefill(*g, *layer, k, v, block_table_row, n_tokens, (cudaStream_t)stream),
                    "write_prefill");
}

int loda_build_index(const loda_geometry* g, const loda_layer* layer, int32_t req_id, int32_t length,
                     int32_t first_block, int32_t n_blocks, void* stream) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer));
  if (req_id < 0 || req_id >= g->max_requests) return fail(LODA_ERR_ARGUMENT, "req_id out of range");
  if (length < 0 || first_block < 0 || n_blocks < 0 || first_block + n_blocks > g->max_blocks)
    return fail(LODA_ERR_ARGUMENT, "block range out of range");
  return check_cuda(launch_build_index(*g, *layer, req_id, length, first_block, n_blocks, (cudaStream_t)stream),
                    "build_index");
}

int loda_select_l1(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                   float scale, const loda_selection* out, void* workspace, void* stream) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer));
  LODA_TRY(check_batch(g, b));
  if (b->batch == 0) return LODA_OK;
  if (!q || !out || !workspace) return fail(LODA_ERR_ARGUMENT, "L1 needs q, a selection struct and a workspace");
  if (out->i_far && (!out->i_near || !out->n_far || !out->n_near))
    return fail(LODA_ERR_ARGUMENT, "i_far, n_far, i_near, n_near are given together or not at all");
  const AppendArgs none{nullptr, nullptr, nullptr, nullptr, 0};
  return check_cuda(launch_l1(*g, *layer, *b, q, scale, *out, select_ws(*g, workspace), none, 0, (cudaStream_t)stream),
                    "select_l1");
}

// kernels the latest loda_select_step / loda_decode_step of the calling thread launched
static thread_local int g_last_select_launches = 0;

int loda_select_step(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                     const void* k_new, const void* v_new, const int32_t* slots, float scale,
                     const loda_selection* sel, uint32_t* status, void* workspace, void* stream) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer));
  LODA_TRY(check_batch(g, b));
  if (b->batch == 0) return LODA_OK;
  if (!q || !sel || !sel->gather || !sel->visible_lens || !workspace)
    return fail(LODA_ERR_ARGUMENT, "select_step needs q, gather, visible_lens and a workspace");
  if (sel->i_far && (!sel->i_near || !sel->n_far || !sel->n_near))
    return fail(LODA_ERR_ARGUMENT, "i_far, n_far, i_near, n_near are given together or not at all");
  if ((sel->middle == nullptr) != (sel->middle_counts == nullptr))
    return fail(LODA_ERR_ARGUMENT, "middle and middle_counts must be given together");
  if ((k_new == nullptr) != (v_new == nullptr) || (k_new && !slots))
    return fail(LODA_ERR_ARGUMENT, "k_new, v_new and slots go together (all NULL = refresh the index only)");
  const SelectWorkspace ws = select_ws(*g, workspace);
  const AppendArgs ap{(const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, slots, status, 1};
  if (g->shard_count > 1)
    return fail(LODA_ERR_ARGUMENT, "sequence-sharded geometries use the staged selector (loda_shard_*)");
  if (select_fused_applicable(*g, b->batch * g->num_kv_heads)) {
    // one launch for both levels (a cluster per row); refused shapes fall through to the two-launch chain
    const cudaError_t e = launch_select_fused(*g, *layer, *b, q, scale, *sel, status, ap, (cudaStream_t)stream);
    if (e == cudaSuccess) { g_last_select_launches = 1; return LODA_OK; }
    if (e != cudaErrorNotSupported) {                    // NotSupported: nothing was launched, the GPU cannot hold the clusters
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing((cudaStream_t)stream, &cap);
      if (cap != cudaStreamCaptureStatusNone) return check_cuda(e, "select_step/fused");   // cannot retry inside a capture
      (void)cudaGetLastError();
      select_fused_refuse(g->sub_dims);
    }
  }
  g_last_select_launches = 2;
  LODA_TRY(check_cuda(launch_l1(*g, *layer, *b, q, scale, *sel, ws, ap, 0, (cudaStream_t)stream), "select_step/l1"));
  return check_cuda(launch_l2(*g, *layer, *b, q, scale, *sel, ws, status, /*chained=*/true, 0, (cudaStream_t)stream),
                    "select_step/l2");
}

int loda_select_l2(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                   float scale, const loda_selection* sel, uint32_t* status, void* workspace, void* stream) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer));
  LODA_TRY(check_batch(g, b));
  if (b->batch == 0) return LODA_OK;
  if (!q || !sel || !sel->gather || !sel->visible_lens || !workspace)
    return fail(LODA_ERR_ARGUMENT, "L2 needs q, gather, visible_lens and the workspace L1 ran on");
  if ((sel->middle == nullptr) != (sel->middle_counts == nullptr))
    return fail(LODA_ERR_ARGUMENT, "middle and middle_counts must be given together");
  return check_cuda(launch_l2(*g, *layer, *b, q, scale, *sel, select_ws(*g, workspace), status, /*chained=*/false, 0,
                              (cudaStream_t)stream),
                    "select_l2");
}

// chained: the launch directly follows the selector launches of the same call
static int gather_attend_impl(const loda_geometry* g, const loda_layer* layer, const void* q, const int32_t* gather,
                              const int32_t* visible_lens, const int32_t* query_to_req, int32_t n_query,
                              int32_t n_req_rows, float scale, void* out, float* lse, void* workspace,
                              bool chained, void* stream, bool identity = false) {
  LODA_TRY(check_gather_attend_args(g, layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, out));
  if (n_query == 0) return LODA_OK;
  if (!workspace) return fail(LODA_ERR_ARGUMENT, "gather attention needs a workspace");
  const WsLayout w = ws_layout(*g);
  char* base = (char*)workspace;
  const AttnWorkspace ws{(int*)(base + w.at_ticket), (float*)(base + w.at_m), (float*)(base + w.at_z),
                         (float*)(base + w.at_o)};
  if (g->head_dim == 576)
    return check_cuda(launch_attn_mla(*g, *layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale, out,
                                      lse, ws, chained, identity, nullptr, (cudaStream_t)stream),
                      "gather_attend/latent");
  return check_cuda(launch_attn(*g, *layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale,
                                out, lse, ws, /*allow_cluster=*/true, chained, identity, (cudaStream_t)stream),
                    "gather_attend");
}

int loda_gather_attend_lse(const loda_geometry* g, const loda_layer* layer, const void* q, const int32_t* gather,
                           const int32_t* visible_lens, const int32_t* query_to_req, int32_t n_query,
                           int32_t n_req_rows, float scale, void* out, float* lse, void* workspace,
                           void* stream) {
  return gather_attend_impl(g, layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale, out, lse,
                            workspace, /*chained=*/false, stream);
}

int loda_gather_attend(const loda_geometry* g, const loda_layer* layer, const void* q, const int32_t* gather,
                       const int32_t* visible_lens, const int32_t* query_to_req, int32_t n_query,
                       int32_t n_req_rows, float scale, void* out, void* workspace, void* stream) {
  return gather_attend_impl(g, layer, q, gather, visible_lens, query_to_req, n_query, n_req_rows, scale, out,
                            nullptr, workspace, /*chained=*/false, stream);
}

int loda_protected_gather(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, int32_t* gather,
                          int32_t* visible_lens, uint32_t* status, void* stream) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer));
  LODA_TRY(check_batch(g, b));
  if (b->batch == 0) return LODA_OK;
  if (!gather || !visible_lens) return fail(LODA_ERR_ARGUMENT, "protected_gather needs gather and visible_lens");
  if (g->sink + g->swa > g->max_visible) return fail(LODA_ERR_ARGUMENT, "max_visible < sink + swa");
  return check_cuda(launch_protected_gather(*g, *layer, *b, gather, visible_lens, status, (cudaStream_t)stream),
                    "protected_gather");
}

// ---- sequence sharding: the selector in four stages, the caller combines the score rows of the
// ---- GPUs (bitwise OR: every page and every slot is scored by exactly one of them) in between
int loda_shard_workspace_regions(const loda_geometry* g, int64_t* out) {
  LODA_TRY(check_geometry(g));
  if (!out) return fail(LODA_ERR_ARGUMENT, "out is NULL");
  const WsLayout w = ws_layout(*g);
  const size_t rows = (size_t)g->max_query_tokens * g->num_kv_heads;
  out[0] = (int64_t)w.l1_scores;
  out[1] = (int64_t)(rows * (size_t)l1_score_stride(*g) * 2);
  out[2] = (int64_t)w.l2_scores;
  out[3] = (int64_t)(rows * (size_t)(g->k_far + g->k_near + 2) * g->page * 2);
  return LODA_OK;
}

static int shard_stage(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q, float scale,
                       const loda_selection* sel, uint32_t* status, void* workspace, void* stream, int level,
                       int phase, const void* gathered = nullptr) {
  LODA_TRY(check_geometry(g));
  LODA_TRY(check_layer(layer));
  LODA_TRY(check_batch(g, b));
  if (g->shard_count < 2) return fail(LODA_ERR_ARGUMENT, "the staged selector is for shard_count >= 2");
  if (b->batch == 0) return LODA_OK;
  if (!q || !sel || !workspace) return fail(LODA_ERR_ARGUMENT, "staged selector needs q, a selection struct and a workspace");
  if (level == 2 && phase == 2 && (!sel->gather || !sel->visible_lens))
    return fail(LODA_ERR_ARGUMENT, "the level-2 selection needs gather and visible_lens");
  SelectWorkspace ws = select_ws(*g, workspace);
  if (gathered != nullptr) {      // the score rows of all GPUs, stacked: ORed by the selecting CTA while loading
    const size_t rows = (size_t)g->max_query_tokens * g->num_kv_heads;
    ws.gathered = (const uint16_t*)gathered;
    ws.n_gathered = g->shard_count;
    ws.gathered_stride = level == 1 ? rows * (size_t)l1_score_stride(*g) : rows * (size_t)(g->k_far + g->k_near + 2) * g->page;
  }
  if (level == 1) {
    const AppendArgs none{nullptr, nullptr, nullptr, nullptr, 0};
    loda_selection no_lists = *sel;
    no_lists.i_far = nullptr;                            // the best-first lists are not produced in this mode
    return check_cuda(launch_l1(*g, *layer, *b, q, scale, no_lists, ws, none, phase, (cudaStream_t)stream), "shard/l1");
  }
  return check_cuda(launch_l2(*g, *layer, *b, q, scale, *sel, ws, status, /*chained=*/false, phase, (cudaStream_t)stream),
                    "shard/l2");
}

int loda_shard_l1_scores(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                         float scale, const loda_selection* sel, void* workspace, void* stream) {
  return shard_stage(g, layer, b, q, scale, sel, nullptr, workspace, stream, 1, 1);
}
int loda_shard_l1_select(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                         float scale, const loda_selection* sel, const void* gathered, void* workspace, void* stream) {
  return shard_stage(g, layer, b, q, scale, sel, nullptr, workspace, stream, 1, 2, gathered);
}
int loda_shard_l2_scores(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                         float scale, const loda_selection* sel, uint32_t* status, void* workspace, void* stream) {
  return shard_stage(g, layer, b, q, scale, sel, status, workspace, stream, 2, 1);
}
int loda_shard_l2_select(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                         float scale, const loda_selection* sel, uint32_t* status, const void* gathered, void* workspace,
                         void* stream) {
  return shard_stage(g, layer, b, q, scale, sel, status, workspace, stream, 2, 2, gathered);
}

static thread_local int g_last_decode_launches = 0;
int loda_last_decode_launches(void) { return g_last_decode_launches; }
int loda_last_decode_cluster(void) { return g_last_decode_launches == 1 || g_last_select_launches == 1 ? select_fused_last_cluster() : 0; }

int loda_decode_step(const loda_geometry* g, const loda_layer* layer, const loda_batch* b, const void* q,
                     const void* k_new, const void* v_new, const int32_t* slots, float scale,
                     const loda_selection* sel, const int32_t* query_to_req, void* out, uint32_t* status,
                     void* workspace, void* stream) {
  // One launch for the whole step where a cluster per row fits the GPU (batch 1 at long context)
  // and the head dimensions are the attention phase's; everything else, and every argument error,
  // goes through the two entry points below, which validate their arguments themselves.
  if (g && layer && b && sel && q && out && query_to_req && workspace && k_new && v_new && slots && sel->gather &&
      sel->visible_lens && b->batch > 0 && check_geometry(g) == LODA_OK && check_layer(layer) == LODA_OK &&
      check_batch(g, b) == LODA_OK && g->shard_count <= 1 && (sel->i_far == nullptr || (sel->i_near && sel->n_far && sel->n_near)) &&
      (sel->middle == nullptr) == (sel->middle_counts == nullptr) && !sel->middle_only &&
      select_fused_applicable(*g, b->batch * g->num_kv_heads)) {
    const AppendArgs ap{(const __nv_bfloat16*)k_new, (const __nv_bfloat16*)v_new, slots, status, 1};
    const cudaError_t e = launch_decode_fused(*g, *layer, *b, q, scale, *sel, status, ap, query_to_req, out,
                                              (cudaStream_t)stream);
    if (e == cudaSuccess) { g_last_decode_launches = 1; return LODA_OK; }
    if (e != cudaErrorNotSupported) {
      cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
      cudaStreamIsCapturing((cudaStream_t)stream, &cap);
      if (cap != cudaStreamCaptureStatusNone) return check_cuda(e, "decode_step/fused");   // cannot retry inside a capture
      (void)cudaGetLastError();
      select_fused_refuse(g->sub_dims);
    }
  }
  LODA_TRY(loda_select_step(g, layer, b, q, k_new, v_new, slots, scale, sel, status, workspace, stream));
  if (b->batch == 0) return LODA_OK;
  g_last_decode_launches = 1 + g_last_select_launches;
  // one query per batch row: the gather list has one row per batch row, and a query_to_req entry other
  // than the row's own index (or < 0) gives a row of zeros, exactly as in the one-launch kernel
  return gather_attend_impl(g, layer, q, sel->gather, sel->visible_lens, query_to_req, b->batch, b->batch,
                            scale, out, nullptr, workspace, /*chained=*/true, stream, /*identity=*/true);
}

}  // extern "C"
