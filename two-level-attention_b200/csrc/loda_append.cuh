// One-warp append of a decode token: K/V rows, packed 4-bit tail key and the
// statistics of the token's page.  Shared by the stand-alone append kernel and
// by the L1 kernel, which carries the append in extra CTAs of the same launch.
#pragma once

#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;

struct QuantOut {
  float scale, zero;
};

// One warp quantises one token: lane l holds dims l, l + 32, ...  (NV per lane).
template <int DSUB>
__device__ __forceinline__ QuantOut warp_quant4(const float (&x)[(DSUB + 31) / 32], int lane,
                                                uint32_t (&code)[(DSUB + 31) / 32]) {
  constexpr int NV = (DSUB + 31) / 32;
  float mx = -INFINITY, mn = INFINITY;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    if (lane + 32 * j < DSUB) { mx = fmaxf(mx, x[j]); mn = fminf(mn, x[j]); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  const float floor_v = bf16r(1e-9f);
  float range = bf16r(__fsub_rn(mx, mn));
  range = range < floor_v ? floor_v : range;
  QuantOut q;
  q.scale = bf16r(__fdiv_rn(range, 15.0f));
  q.zero = -mn;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    float t = bf16r(__fdiv_rn(bf16r(__fadd_rn(x[j], q.zero)), q.scale));
    t = fminf(fmaxf(rintf(t), 0.0f), 15.0f);
    code[j] = (uint32_t)t;
  }
  return q;
}

// Pack the warp's 4-bit codes (dim d in lane d % 32, register d / 32) into
// DSUB / 2 bytes: dim 2i in the low nibble of byte i.
template <int DSUB>
__device__ __forceinline__ void warp_store_codes(const uint32_t (&code)[(DSUB + 31) / 32], int lane,
                                                 uint8_t* dst) {
  constexpr int NV = (DSUB + 31) / 32;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const uint32_t lo = __shfl_sync(0xffffffffu, code[j], (2 * lane) & 31);
    const uint32_t hi = __shfl_sync(0xffffffffu, code[j], (2 * lane + 1) & 31);
    // lanes 0..15 hold bytes of dims [32 j, 32 j + 32)
    if (lane < 16 && 32 * j + 2 * lane < DSUB) dst[16 * j + lane] = (uint8_t)(lo | (hi << 4));
  }
}

// Store min / max / sum of subspace dim d of logical page blk of (request slot req, kv head kv)
// into the interleaved statistics layout (STAT_GROUP in loda_common.cuh): dim d lives in 16-byte
// chunk d / 8 of the page's min row, chunk d' / 8 + d / 8 of its max row, chunk d / 8 of its sum row.
template <int DSUB>
__device__ __forceinline__ void store_page_stats(const loda_geometry& g, const loda_layer& L, int req, int kv, int blk,
                                                 int d, float mn, float mx, float sum) {
  constexpr int NC = DSUB / 8, CPR = 2 * NC;
  const size_t rowi = (size_t)req * g.num_kv_heads + kv;
  unsigned char* mm_row = (unsigned char*)L.page_mm + rowi * stat_row_bytes(g.max_blocks, CPR);
  unsigned char* sum_row = (unsigned char*)L.page_sum + rowi * stat_row_bytes(g.max_blocks, NC);
  const int c = d / 8, e = d % 8;
  *(bf16*)(mm_row + stat_chunk_offset(blk, c, CPR) + e * 2) = __float2bfloat16_rn(mn);
  *(bf16*)(mm_row + stat_chunk_offset(blk, NC + c, CPR) + e * 2) = __float2bfloat16_rn(mx);
  *(bf16*)(sum_row + stat_chunk_offset(blk, c, NC) + e * 2) = __float2bfloat16_rn(sum);
}

// Append (or refresh) one (row, kv head) with one warp.
template <int DSUB>
__device__ __forceinline__ void append_row(
    const loda_geometry& g, const loda_layer& L, const loda_batch& B, const bf16* __restrict__ k_new,
    const bf16* __restrict__ v_new, const int32_t* __restrict__ slots, uint32_t* status, int row, int kv,
    int lane) {
  constexpr int NV = (DSUB + 31) / 32;
  // k_new == NULL: the K/V rows are already in the pool (written by a plain paged
  // write); only the index of the newest token and of its page is refreshed.
  const bool refresh = k_new == nullptr;
  int phys = -1, off = 0;
  const bf16* ksrc = nullptr;
  if (!refresh) {
    int slot = slots[row];
    const bool pad = slot < 0;
    if (pad) slot = (g.num_pages - 1) * g.page;
    phys = slot / g.page;
    off = slot % g.page;
    if (phys >= g.num_pages) {
      if (lane == 0 && status) atomicOr(status, LODA_STATUS_BAD_SLOT);
      return;
    }
    const size_t dst_row = ((size_t)phys * g.num_kv_heads + kv) * g.page + off;
    ksrc = k_new + ((size_t)row * g.num_kv_heads + kv) * g.head_dim;
    const bf16* vsrc = v_new + ((size_t)row * g.num_kv_heads + kv) * g.head_dim_v;
    bf16* kdst = (bf16*)L.pool_k + dst_row * g.head_dim;
    bf16* vdst = (bf16*)L.pool_v + dst_row * g.head_dim_v;
    for (int c = lane; c < g.head_dim / 8; c += 32) ((uint4*)kdst)[c] = ((const uint4*)ksrc)[c];
    // shared-latent layout (pool_v aliases pool_k): the value is the head of the key row just written
    if (L.pool_v != L.pool_k)
      for (int c = lane; c < g.head_dim_v / 8; c += 32) ((uint4*)vdst)[c] = ((const uint4*)vsrc)[c];
    if (pad) return;
  }
  if (L.page_mm == nullptr || B.active_req_ids[row] < 0) return;
  const int length = B.lengths[row];
  if (length <= 0) return;
  const long long req64 = B.valid_req_ids[row];
  if (req64 < 0 || req64 >= g.max_requests) {          // never address the index with a slot outside the cache
    if (lane == 0 && status) atomicOr(status, LODA_STATUS_BAD_REQ);
    return;
  }
  const int req = (int)req64;
  const int tok = length - 1;
  const int blk = tok / g.page;
  if (blk >= g.max_blocks) {
    if (lane == 0 && status) atomicOr(status, LODA_STATUS_BAD_PAGE);
    return;
  }
  if (refresh) {
    phys = L.block_table[(size_t)req * g.max_blocks + blk];
    off = tok % g.page;
    if (phys < 0 || phys >= g.num_pages) {
      if (lane == 0 && status) atomicOr(status, LODA_STATUS_BAD_PAGE);
      return;
    }
    ksrc = (const bf16*)L.pool_k + (((size_t)phys * g.num_kv_heads + kv) * g.page + off) * g.head_dim;
  }
  const size_t tok_row = ((size_t)phys * g.num_kv_heads + kv) * g.page + off;

  // packed 4-bit key of the new token
  float x[NV];
  int dim[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int d = lane + 32 * j;
    dim[j] = d < DSUB ? sub_dim(g, d) : 0;
    x[j] = d < DSUB ? __bfloat162float(ksrc[dim[j]]) : 0.0f;
  }
  uint32_t code[NV];
  const QuantOut qo = warp_quant4<DSUB>(x, lane, code);
  warp_store_codes<DSUB>(code, lane, L.tail_code + tok_row * (DSUB / 2));
  if (lane == 0) {
    bf16* sz = (bf16*)L.tail_sz + tok_row * 2;
    sz[0] = __float2bfloat16_rn(qo.scale);
    sz[1] = __float2bfloat16_rn(qo.zero);
  }

  // statistics of the token's logical page: older tokens from the pool (ascending
  // order), the new token last
  const int n_old = tok - blk * g.page;
  const bf16* page_k = (const bf16*)L.pool_k + ((size_t)phys * g.num_kv_heads + kv) * g.page * g.head_dim;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int d = lane + 32 * j;
    if (d >= DSUB) continue;
    float mn = INFINITY, mx = -INFINITY, sum = 0.0f;
    // eight independent loads in flight per round, reduced in token order
    for (int i0 = 0; i0 < n_old; i0 += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u)
        v[u] = (i0 + u < n_old) ? __bfloat162float(page_k[(size_t)(i0 + u) * g.head_dim + dim[j]]) : 0.0f;
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        if (i0 + u < n_old) {
          mn = fminf(mn, v[u]);
          mx = fmaxf(mx, v[u]);
          sum = __fadd_rn(sum, v[u]);
        }
      }
    }
    mn = fminf(mn, x[j]);
    mx = fmaxf(mx, x[j]);
    sum = __fadd_rn(sum, x[j]);
    store_page_stats<DSUB>(g, L, req, kv, blk, d, mn, mx, sum);
  }
}

}  // namespace loda
