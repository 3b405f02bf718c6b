// Append-time maintenance of the paged KV cache index: K/V row scatter, per-page
// min / max / sum on the scoring subspace and packed 4-bit tail keys.
//
// Arithmetic contract (bit exact with the reference's PyTorch quantiser,
// sparse_attn/indexer/tia_indexer.py:22-31, in bf16: every torch op is one
// rounding to bf16):
//   range = bf16(max - min) clamped below at bf16(1e-9); scale = bf16(range / 15)
//   zero = -min; code = clamp(rint(bf16(bf16(x + zero) / scale)), 0, 15)
// Page statistics follow nfa_layer_batch_selector.py:87-131: min / max over the
// visible tokens only, sum in fp32 in ascending token order, each stored in the
// pool dtype.
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

template <int DSUB>
__global__ void __launch_bounds__(32) append_decode_kernel(
    loda_geometry g, loda_layer L, loda_batch B, const bf16* __restrict__ k_new,
    const bf16* __restrict__ v_new, const int32_t* __restrict__ slots, uint32_t* status) {
  constexpr int NV = (DSUB + 31) / 32;
  const int row = blockIdx.x / g.num_kv_heads;
  const int kv = blockIdx.x % g.num_kv_heads;
  const int lane = threadIdx.x;
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
    for (int c = lane; c < g.head_dim_v / 8; c += 32) ((uint4*)vdst)[c] = ((const uint4*)vsrc)[c];
    if (pad) return;
  }
  if (L.page_mm == nullptr || B.active_req_ids[row] < 0) return;
  const int length = B.lengths[row];
  if (length <= 0) return;
  const int req = (int)B.valid_req_ids[row];
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
    for (int i = 0; i < n_old; ++i) {
      const float v = __bfloat162float(page_k[(size_t)i * g.head_dim + dim[j]]);
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
      sum = __fadd_rn(sum, v);
    }
    mn = fminf(mn, x[j]);
    mx = fmaxf(mx, x[j]);
    sum = __fadd_rn(sum, x[j]);
    const size_t pg = ((size_t)req * g.num_kv_heads + kv) * g.max_blocks + blk;
    bf16* mm = (bf16*)L.page_mm + pg * 2 * DSUB;
    mm[d] = __float2bfloat16_rn(mn);
    mm[DSUB + d] = __float2bfloat16_rn(mx);
    ((bf16*)L.page_sum)[pg * DSUB + d] = __float2bfloat16_rn(sum);
  }
}

// One warp per (logical page, kv head): quantise every visible token of the
// page and reduce its statistics.
template <int DSUB, int WARPS>
__global__ void __launch_bounds__(32 * WARPS) build_index_kernel(
    loda_geometry g, loda_layer L, int req, int length, int first_block, int n_blocks) {
  constexpr int NV = (DSUB + 31) / 32;
  const int lane = threadIdx.x & 31;
  const int blk = first_block + blockIdx.x * WARPS + (threadIdx.x >> 5);
  const int kv = blockIdx.y;
  if (blk >= first_block + n_blocks || blk >= g.max_blocks) return;
  const int n_vis = min(g.page, length - blk * g.page);
  if (n_vis <= 0) return;
  const int phys = L.block_table[(size_t)req * g.max_blocks + blk];
  if (phys < 0 || phys >= g.num_pages) return;
  const size_t row0 = ((size_t)phys * g.num_kv_heads + kv) * g.page;
  const bf16* page_k = (const bf16*)L.pool_k + row0 * g.head_dim;
  int dim[NV];
  float mn[NV], mx[NV], sum[NV];
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int d = lane + 32 * j;
    dim[j] = d < DSUB ? sub_dim(g, d) : 0;
    mn[j] = INFINITY; mx[j] = -INFINITY; sum[j] = 0.0f;
  }
  for (int i = 0; i < n_vis; ++i) {
    float x[NV];
#pragma unroll
    for (int j = 0; j < NV; ++j) {
      x[j] = (lane + 32 * j < DSUB) ? __bfloat162float(page_k[(size_t)i * g.head_dim + dim[j]]) : 0.0f;
      mn[j] = fminf(mn[j], x[j]);
      mx[j] = fmaxf(mx[j], x[j]);
      sum[j] = __fadd_rn(sum[j], x[j]);
    }
    uint32_t code[NV];
    const QuantOut qo = warp_quant4<DSUB>(x, lane, code);
    warp_store_codes<DSUB>(code, lane, L.tail_code + (row0 + i) * (DSUB / 2));
    if (lane == 0) {
      bf16* sz = (bf16*)L.tail_sz + (row0 + i) * 2;
      sz[0] = __float2bfloat16_rn(qo.scale);
      sz[1] = __float2bfloat16_rn(qo.zero);
    }
  }
  const size_t pg = ((size_t)req * g.num_kv_heads + kv) * g.max_blocks + blk;
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int d = lane + 32 * j;
    if (d >= DSUB) continue;
    bf16* mm = (bf16*)L.page_mm + pg * 2 * DSUB;
    mm[d] = __float2bfloat16_rn(mn[j]);
    mm[DSUB + d] = __float2bfloat16_rn(mx[j]);
    ((bf16*)L.page_sum)[pg * DSUB + d] = __float2bfloat16_rn(sum[j]);
  }
}

// Scatter [Hkv, N, D] rows through a block-table row, 16 bytes per thread.
__global__ void __launch_bounds__(256) write_prefill_kernel(
    loda_geometry g, loda_layer L, const bf16* __restrict__ k, const bf16* __restrict__ v,
    const int32_t* __restrict__ table, int n_tokens) {
  const int ck = g.head_dim / 8, cv = g.head_dim_v / 8;
  const size_t per_tok = (size_t)ck + cv;
  const size_t total = (size_t)g.num_kv_heads * n_tokens * per_tok;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
       i += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(i % per_tok);
    const size_t t = i / per_tok;
    const int n = (int)(t % n_tokens);
    const int kv = (int)(t / n_tokens);
    const int phys = table[n / g.page];
    if (phys < 0 || phys >= g.num_pages) continue;
    const size_t dst_row = ((size_t)phys * g.num_kv_heads + kv) * g.page + n % g.page;
    const size_t src_row = (size_t)kv * n_tokens + n;
    if (c < ck)
      ((uint4*)((bf16*)L.pool_k + dst_row * g.head_dim))[c] = ((const uint4*)(k + src_row * g.head_dim))[c];
    else
      ((uint4*)((bf16*)L.pool_v + dst_row * g.head_dim_v))[c - ck] =
          ((const uint4*)(v + src_row * g.head_dim_v))[c - ck];
  }
}

// ---------------------------------------------------------------------------
// host launchers
// ---------------------------------------------------------------------------
cudaError_t launch_append_decode(const loda_geometry& g, const loda_layer& L, const loda_batch& B,
                                 const void* k_new, const void* v_new, const int32_t* slots,
                                 uint32_t* status, cudaStream_t st) {
  const dim3 grid(B.batch * g.num_kv_heads);
  switch (g.sub_dims) {
    case 16: append_decode_kernel<16><<<grid, 32, 0, st>>>(g, L, B, (const bf16*)k_new, (const bf16*)v_new, slots, status); break;
    case 32: append_decode_kernel<32><<<grid, 32, 0, st>>>(g, L, B, (const bf16*)k_new, (const bf16*)v_new, slots, status); break;
    case 64: append_decode_kernel<64><<<grid, 32, 0, st>>>(g, L, B, (const bf16*)k_new, (const bf16*)v_new, slots, status); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_build_index(const loda_geometry& g, const loda_layer& L, int req, int length,
                               int first_block, int n_blocks, cudaStream_t st) {
  constexpr int WARPS = 4;
  if (n_blocks <= 0) return cudaSuccess;
  const dim3 grid((n_blocks + WARPS - 1) / WARPS, g.num_kv_heads);
  switch (g.sub_dims) {
    case 16: build_index_kernel<16, WARPS><<<grid, 32 * WARPS, 0, st>>>(g, L, req, length, first_block, n_blocks); break;
    case 32: build_index_kernel<32, WARPS><<<grid, 32 * WARPS, 0, st>>>(g, L, req, length, first_block, n_blocks); break;
    case 64: build_index_kernel<64, WARPS><<<grid, 32 * WARPS, 0, st>>>(g, L, req, length, first_block, n_blocks); break;
    default: return cudaErrorInvalidValue;
  }
  return cudaGetLastError();
}

cudaError_t launch_write_prefill(const loda_geometry& g, const loda_layer& L, const void* k,
                                 const void* v, const int32_t* table, int n_tokens, cudaStream_t st) {
  if (n_tokens <= 0) return cudaSuccess;
  const size_t total = (size_t)g.num_kv_heads * n_tokens * (g.head_dim / 8 + g.head_dim_v / 8);
  const int blocks = (int)((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
  write_prefill_kernel<<<blocks, 256, 0, st>>>(g, L, (const bf16*)k, (const bf16*)v, table, n_tokens);
  return cudaGetLastError();
}

}  // namespace loda
