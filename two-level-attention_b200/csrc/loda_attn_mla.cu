// Gather attention for a shared-latent KV layout (multi-head latent attention in its absorbed form):
// one KV head whose key row is the whole latent (head_dim = 576: 512 compressed dims + 64 rotary dims)
// and whose value row is the first head_dim_v = 512 dims of the SAME row — the layer's pool_v aliases
// pool_k — attended by a group of up to 16 query heads.
//
// Same contract as the general kernel (sparse_paged_attention_gather, sparse_attn/ops/
// paged_region_kernels.py:800-1041): exact softmax over the slots gather[req, 0, 0:visible_lens], slots
// < 0 skipped, empty list or query_to_req < 0 gives zeros.  The closest reference code is the
// materialised GLM path (sparse_attn/patches/glm4_moe_lite_attn_patch.py:44-59), which expands the
// latent to per-head keys first; attending in the latent space reads 1 152 bytes per token instead.
//
// Why not the general kernel: with D = 576 and Dv = 512 a warp that owned 16 tokens and all output
// columns would carry 256 accumulator registers.  Here the 16 query heads fill the 16 rows of
// mma.sync m16n8k16 exactly; per tile of 64 tokens every warp computes S = Q K^T for its own 16 tokens
// (Q fragments from shared memory), the tile's softmax statistics are combined through shared memory, P
// goes to shared memory as bf16, and every warp accumulates O += P V for its own quarter of the 512
// output columns over all 64 tokens.  K rows double as V rows, so a token is staged once: one bulk
// asynchronous copy per token row (1 152 B) on an mbarrier, two tiles in flight.  (A tcgen05 tile needs
// M >= 64 rows per CTA pair and the requests of a batch attend over different token lists, so the 16
// heads of one request are all the M there is: the 16-row mma.sync tile is the one without padding.)
#include "loda_attn.cuh"
#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;

constexpr int MLA_D = 576, MLA_DV = 512;
constexpr int MLA_TILE = 64, MLA_WARPS = 4, MLA_NT = 32 * MLA_WARPS;
constexpr int MLA_KSTR = MLA_D + 8;              // padded rows: conflict-free ldmatrix, 16-byte multiple
constexpr int MLA_PSTR = MLA_TILE + 8;
constexpr int MLA_MAX_SPLIT = 16;
constexpr int MLA_COLS = MLA_DV / MLA_WARPS;     // output columns per warp
constexpr int MLA_NTV = MLA_COLS / 8;            // n-tiles of 8 columns per warp

struct MlaSmem {
  static constexpr size_t K = 0;                                               // [2][TILE][KSTR] bf16
  static constexpr size_t Q = K + (size_t)2 * MLA_TILE * MLA_KSTR * 2;         // [16][KSTR] bf16
  static constexpr size_t P = Q + (size_t)16 * MLA_KSTR * 2;                   // [16][PSTR] bf16
  static constexpr size_t WMAX = P + (size_t)16 * MLA_PSTR * 2;                // [WARPS][16] float
  static constexpr size_t WSUM = WMAX + MLA_WARPS * 16 * 4;                    // [WARPS][16] float
  static constexpr size_t SLOT = WSUM + MLA_WARPS * 16 * 4;                    // [2][TILE] int
  static constexpr size_t BAR = SLOT + 2 * MLA_TILE * 4;                       // [2] mbarrier
  static constexpr size_t SH = BAR + 16;                                       // 4 ints
  static constexpr size_t TOTAL = SH + 16;
};

__global__ void __launch_bounds__(MLA_NT) attn_mla_kernel(
    loda_geometry g, loda_layer L, const bf16* __restrict__ q, const int32_t* gather, const int32_t* visible_lens,
    const int32_t* query_to_req, int n_req_rows, float scale_log2, bf16* __restrict__ out, float* __restrict__ lse,
    AttnWorkspace ws, int nsplit, int chained, int identity, uint32_t* status) {
  extern __shared__ __align__(128) unsigned char smem[];
  bf16* Ks = (bf16*)(smem + MlaSmem::K);
  bf16* Qs = (bf16*)(smem + MlaSmem::Q);
  bf16* Ps = (bf16*)(smem + MlaSmem::P);
  float* wmax = (float*)(smem + MlaSmem::WMAX);
  float* wsum = (float*)(smem + MlaSmem::WSUM);
  int* slot_s = (int*)(smem + MlaSmem::SLOT);
  uint64_t* bars = (uint64_t*)(smem + MlaSmem::BAR);
  int* sh = (int*)(smem + MlaSmem::SH);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x, t = blockIdx.z;
  const int G = g.num_q_heads;                       // one kv head: the group is all the query heads
  const int page_log2 = 31 - __clz(g.page);
  if (tid == 0) {
    mbar_init(bars, 2);                              // one arrival per issuing warp
    mbar_init(bars + 1, 2);
    mbar_init_fence();
  }
  // the query rows (heads beyond G are zero rows): read before the dependency wait only when this launch is
  // chained behind the selector launches of the same step, which read the query themselves
  auto load_q = [&]() {
    for (int c = tid; c < 16 * (MLA_D / 8); c += MLA_NT) {
      const int r = c / (MLA_D / 8), cc = c % (MLA_D / 8);
      uint4 v = make_uint4(0u, 0u, 0u, 0u);
      if (r < G) v = *(const uint4*)(q + ((size_t)t * g.num_q_heads + r) * MLA_D + cc * 8);
      *(uint4*)(Qs + (size_t)r * MLA_KSTR + cc * 8) = v;
    }
  };
  if (chained) load_q();
  pdl_wait();
  if (!chained) load_q();
  int req = __ldcg(query_to_req + t);
  if (identity && req != t) req = -1;
  int n = 0;
  if (req >= 0 && req < n_req_rows) n = min(max(__ldcg(visible_lens + (size_t)req * g.num_kv_heads), 0), g.max_visible);
  const int c0 = (int)(((long long)split * n) / nsplit);
  const int c1 = (int)(((long long)(split + 1) * n) / nsplit);
  const int32_t* list = gather + (size_t)max(req, 0) * g.num_kv_heads * g.max_visible;
  const int slot_end = g.num_pages * g.page;
  const int ntiles = (c1 - c0 + MLA_TILE - 1) / MLA_TILE;
  __syncthreads();                                   // barriers initialised, Q staged

  // Stage tile `tile` into buffer `st`: threads 0..63 own one token row each — a bulk copy of the row, or
  // zeros for a skipped slot and for the rows that pad the tile to a multiple of 16.
  auto issue = [&](int tile, int st) {
    if (warp >= 2) return;
    bf16* Kb = Ks + (size_t)st * MLA_TILE * MLA_KSTR;
    const int ntok = min(MLA_TILE, c1 - c0 - tile * MLA_TILE);
    const int nrow = (ntok + 15) & ~15;
    const int r = tid;
    int s = -1;
    if (tile < ntiles && r < ntok) {
      s = __ldcg(list + c0 + tile * MLA_TILE + r);
      if (s >= slot_end) s = -1;
    }
    if (tile < ntiles && r < MLA_TILE) slot_s[st * MLA_TILE + r] = s;
    const uint32_t bytes = s >= 0 ? MLA_D * 2 : 0;
    const uint32_t total = __reduce_add_sync(0xffffffffu, bytes);
    if (tile < ntiles && s < 0 && r < nrow) {
      for (int c = 0; c < MLA_D / 8; ++c) *(uint4*)(Kb + (size_t)r * MLA_KSTR + c * 8) = make_uint4(0u, 0u, 0u, 0u);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");      // earlier generic writes to the buffer, then async writes
    if (lane == 0) mbar_arrive_expect_tx(bars + st, tile < ntiles ? total : 0u);
    __syncwarp();
    if (s >= 0) {
      const size_t row = ((size_t)(s >> page_log2) * g.num_kv_heads) * g.page + (s & (g.page - 1));
      bulk_copy_g2s(Kb + (size_t)r * MLA_KSTR, (const bf16*)L.pool_k + row * MLA_D, MLA_D * 2, bars + st);
    }
  };
  issue(0, 0);
  issue(1, 1);

  float oacc[MLA_NTV][4];
#pragma unroll
  for (int i = 0; i < MLA_NTV; ++i) { oacc[i][0] = oacc[i][1] = oacc[i][2] = oacc[i][3] = 0.0f; }
  float m_run[2] = {-INFINITY, -INFINITY}, z_run[2] = {0.0f, 0.0f};   // rows lane / 4 and lane / 4 + 8
  const int r0 = lane >> 2;
  bool timed_out = false;
#pragma unroll 1
  for (int it = 0; it < ntiles; ++it) {
    const int st = it & 1;
    const int ntok = min(MLA_TILE, c1 - c0 - it * MLA_TILE);
    const int nrow = (ntok + 15) & ~15;
    if (!mbar_wait(bars + st, (uint32_t)(it >> 1) & 1u)) timed_out = true;
    __syncthreads();                                 // zero-filled rows and the slot table are visible
    const bf16* Kt = Ks + (size_t)st * MLA_TILE * MLA_KSTR;
    const int* slot_t = slot_s + st * MLA_TILE;
    // ---- S = Q K^T for this warp's 16 tokens -------------------------------------------------------
    const int tok0 = warp * 16;
    float sacc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
    if (tok0 < nrow) {
#pragma unroll 4
      for (int ks = 0; ks < MLA_D / 16; ++ks) {
        uint32_t qa[4], kb[4];
        ldmatrix_x4(qa, Qs + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * MLA_KSTR + ks * 16 + ((lane >> 4) & 1) * 8);
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4(kb, Kt + (size_t)(tok0 + (mi >> 1) * 8 + r) * MLA_KSTR + ks * 16 + (mi & 1) * 8);
        mma_bf16(sacc[0], qa, kb[0], kb[1]);
        mma_bf16(sacc[1], qa, kb[2], kb[3]);
      }
    }
    float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < 2; ++j) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int tk = tok0 + j * 8 + (lane & 3) * 2 + (e & 1);
        const bool ok = tk < ntok && slot_t[tk] >= 0;
        const float v = ok ? sacc[j][e] * scale_log2 : -INFINITY;
        sacc[j][e] = v;
        mx[e >> 1] = fmaxf(mx[e >> 1], v);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
      mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
    }
    if ((lane & 3) == 0) { wmax[warp * 16 + r0] = mx[0]; wmax[warp * 16 + r0 + 8] = mx[1]; }
    __syncthreads();
    // ---- tile statistics, P to shared memory -------------------------------------------------------
    float alpha[2], msafe[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float tm = -INFINITY;
#pragma unroll
      for (int w = 0; w < MLA_WARPS; ++w) tm = fmaxf(tm, wmax[w * 16 + r0 + 8 * h]);
      const float m_new = fmaxf(m_run[h], tm);
      msafe[h] = m_new == -INFINITY ? 0.0f : m_new;
      alpha[h] = exp2f(m_run[h] - msafe[h]);
      m_run[h] = m_new;
    }
    float zs[2] = {0.0f, 0.0f};
    if (tok0 < nrow) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const float p0 = exp2f(sacc[j][0] - msafe[0]), p1 = exp2f(sacc[j][1] - msafe[0]);
        const float p2 = exp2f(sacc[j][2] - msafe[1]), p3 = exp2f(sacc[j][3] - msafe[1]);
        zs[0] += p0 + p1;
        zs[1] += p2 + p3;
        const int col = tok0 + j * 8 + (lane & 3) * 2;
        *(uint32_t*)(Ps + (size_t)r0 * MLA_PSTR + col) = pack_bf16(p0, p1);
        *(uint32_t*)(Ps + (size_t)(r0 + 8) * MLA_PSTR + col) = pack_bf16(p2, p3);
      }
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      zs[h] += __shfl_xor_sync(0xffffffffu, zs[h], 1);
      zs[h] += __shfl_xor_sync(0xffffffffu, zs[h], 2);
    }
    if ((lane & 3) == 0) { wsum[warp * 16 + r0] = zs[0]; wsum[warp * 16 + r0 + 8] = zs[1]; }
    __syncthreads();
    // ---- O += P V on this warp's output columns, all tokens of the tile ----------------------------
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      float zt = 0.0f;
#pragma unroll
      for (int w = 0; w < MLA_WARPS; ++w) zt += wsum[w * 16 + r0 + 8 * h];
      z_run[h] = z_run[h] * alpha[h] + zt;
    }
#pragma unroll
    for (int i = 0; i < MLA_NTV; ++i) {
      oacc[i][0] *= alpha[0]; oacc[i][1] *= alpha[0];
      oacc[i][2] *= alpha[1]; oacc[i][3] *= alpha[1];
    }
    const int colbase = warp * MLA_COLS;
#pragma unroll 1
    for (int kt = 0; kt < nrow; kt += 16) {
      uint32_t pa[4];
      ldmatrix_x4(pa, Ps + (size_t)((lane & 7) + ((lane >> 3) & 1) * 8) * MLA_PSTR + kt + ((lane >> 4) & 1) * 8);
#pragma unroll
      for (int i = 0; i < MLA_NTV; i += 2) {
        uint32_t vb[4];
        const int mi = lane >> 3, r = lane & 7;
        ldmatrix_x4_trans(vb, Kt + (size_t)(kt + (mi & 1) * 8 + r) * MLA_KSTR + colbase + i * 8 + (mi >> 1) * 8);
        mma_bf16(oacc[i], pa, vb[0], vb[1]);
        mma_bf16(oacc[i + 1], pa, vb[2], vb[3]);
      }
    }
    __syncthreads();                                 // the buffer and P are free
    issue(it + 2, st);
  }
  if (timed_out && tid == 0 && status) atomicOr(status, LODA_STATUS_TIMEOUT);
  pdl_launch_dependents();

  // ---- this CTA's result: every warp owns its output columns, no merge inside the CTA -------------
  const size_t pair = (size_t)t * g.num_kv_heads;                      // one kv head
  const size_t orow = (size_t)t * g.num_q_heads;
  const int colbase = warp * MLA_COLS;
  if (nsplit == 1) {
    const float inv0 = z_run[0] == 0.0f ? 0.0f : 1.0f / z_run[0], inv1 = z_run[1] == 0.0f ? 0.0f : 1.0f / z_run[1];
#pragma unroll
    for (int i = 0; i < MLA_NTV; ++i) {
      const int col = colbase + i * 8 + (lane & 3) * 2;
      if (r0 < G) *(uint32_t*)(out + (orow + r0) * MLA_DV + col) = pack_bf16(oacc[i][0] * inv0, oacc[i][1] * inv0);
      if (r0 + 8 < G) *(uint32_t*)(out + (orow + r0 + 8) * MLA_DV + col) = pack_bf16(oacc[i][2] * inv1, oacc[i][3] * inv1);
    }
    if (lse != nullptr && warp == 0 && (lane & 3) == 0) {
      if (r0 < G) { lse[(orow + r0) * 2] = m_run[0]; lse[(orow + r0) * 2 + 1] = z_run[0]; }
      if (r0 + 8 < G) { lse[(orow + r0 + 8) * 2] = m_run[1]; lse[(orow + r0 + 8) * 2 + 1] = z_run[1]; }
    }
    return;
  }
  {
    const size_t ps = pair * nsplit + split;
#pragma unroll
    for (int i = 0; i < MLA_NTV; ++i) {
      const int col = colbase + i * 8 + (lane & 3) * 2;
      if (r0 < G) *(float2*)(ws.part_o + (ps * G + r0) * MLA_DV + col) = make_float2(oacc[i][0], oacc[i][1]);
      if (r0 + 8 < G) *(float2*)(ws.part_o + (ps * G + r0 + 8) * MLA_DV + col) = make_float2(oacc[i][2], oacc[i][3]);
    }
    if (warp == 0 && (lane & 3) == 0) {
      if (r0 < G) { ws.part_m[ps * G + r0] = m_run[0]; ws.part_z[ps * G + r0] = z_run[0]; }
      if (r0 + 8 < G) { ws.part_m[ps * G + r0 + 8] = m_run[1]; ws.part_z[ps * G + r0 + 8] = z_run[1]; }
    }
  }
  // ---- last CTA of the query row merges the splits in split order (atomic ticket, no spinning) ----
  __threadfence();
  __syncthreads();
  if (tid == 0) sh[0] = (atomicAdd(ws.ticket + pair, 1) == nsplit - 1);
  __syncthreads();
  if (!sh[0]) return;
  __threadfence();
  float* sm_w = (float*)(smem + MlaSmem::K);           // [nsplit][16] weight of each split (the K buffers are consumed)
  float* sm_zt = sm_w + MLA_MAX_SPLIT * 16;            // [16]
  if (tid < G) {
    float M = -INFINITY;
    for (int s = 0; s < nsplit; ++s) M = fmaxf(M, __ldcg(ws.part_m + (pair * nsplit + s) * G + tid));
    float z = 0.0f;
    for (int s = 0; s < nsplit; ++s) {
      const float a = M == -INFINITY ? 0.0f : exp2f(__ldcg(ws.part_m + (pair * nsplit + s) * G + tid) - M);
      sm_w[s * 16 + tid] = a;
      z += __ldcg(ws.part_z + (pair * nsplit + s) * G + tid) * a;
    }
    sm_zt[tid] = z;
    if (lse != nullptr) { lse[(orow + tid) * 2] = M; lse[(orow + tid) * 2 + 1] = z; }
  }
  __syncthreads();
  const float* po = ws.part_o + pair * nsplit * G * MLA_DV;
  for (int e = tid; e < G * MLA_DV / 4; e += MLA_NT) {
    const int gi = e / (MLA_DV / 4), dv = (e % (MLA_DV / 4)) * 4;
    float4 o = make_float4(0, 0, 0, 0);
#pragma unroll 4
    for (int s = 0; s < nsplit; ++s) {
      const float4 v = __ldcg((const float4*)(po + ((size_t)s * G + gi) * MLA_DV + dv));
      const float a = sm_w[s * 16 + gi];
      o.x += v.x * a; o.y += v.y * a; o.z += v.z * a; o.w += v.w * a;
    }
    const float z = sm_zt[gi];
    const float inv = z == 0.0f ? 0.0f : 1.0f / z;
    uint2 packed;
    packed.x = pack_bf16(o.x * inv, o.y * inv);
    packed.y = pack_bf16(o.z * inv, o.w * inv);
    *(uint2*)(out + (orow + gi) * MLA_DV + dv) = packed;
  }
  if (tid == 0) ws.ticket[pair] = 0;
}

int attn_nsplit(const loda_geometry&, int);

// Launch for a layer whose values alias its keys (layer.pool_v == layer.pool_k), head_dim 576, head_dim_v 512,
// one kv head, at most 16 query heads.  The split partials go through the caller's workspace.
cudaError_t launch_attn_mla(const loda_geometry& g, const loda_layer& L, const void* q, const int32_t* gather,
                            const int32_t* visible_lens, const int32_t* query_to_req, int n_query, int n_req_rows,
                            float scale, void* out, float* lse, const AttnWorkspace& ws, bool chained, bool identity,
                            uint32_t* status, cudaStream_t st) {
  if (n_query <= 0) return cudaSuccess;
  int nsplit = attn_nsplit(g, n_query);
  if (nsplit > MLA_MAX_SPLIT) nsplit = MLA_MAX_SPLIT;
  const dim3 grid(nsplit, 1, n_query);
  cudaError_t e = set_kernel_smem(attn_mla_kernel, MlaSmem::TOTAL);
  if (e != cudaSuccess) return e;
  return launch_pdl(attn_mla_kernel, grid, dim3(MLA_NT), MlaSmem::TOTAL, st, g, L, (const bf16*)q, gather, visible_lens,
                    query_to_req, n_req_rows, scale * 1.4426950408889634f, (bf16*)out, lse, ws, nsplit, (int)chained,
                    (int)identity, status);
}

}  // namespace loda
