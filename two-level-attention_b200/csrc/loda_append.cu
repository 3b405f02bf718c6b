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
#include "loda_append.cuh"

namespace loda {

template <int DSUB>
__global__ void __launch_bounds__(32) append_decode_kernel(
    loda_geometry g, loda_layer L, loda_batch B, const bf16* __restrict__ k_new,
    const bf16* __restrict__ v_new, const int32_t* __restrict__ slots, uint32_t* status) {
  pdl_wait();
  append_row<DSUB>(g, L, B, k_new, v_new, slots, status, blockIdx.x / g.num_kv_heads,
                   blockIdx.x % g.num_kv_heads, threadIdx.x);
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
#pragma unroll
  for (int j = 0; j < NV; ++j) {
    const int d = lane + 32 * j;
    if (d >= DSUB) continue;
    store_page_stats<DSUB>(g, L, req, kv, blk, d, mn[j], mx[j], sum[j]);
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
    else if (L.pool_v != L.pool_k)      // shared-latent layout: no separate value rows
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
    case 16: return launch_pdl(append_decode_kernel<16>, grid, dim3(32), 0, st, g, L, B, (const bf16*)k_new, (const bf16*)v_new, slots, status);
    case 32: return launch_pdl(append_decode_kernel<32>, grid, dim3(32), 0, st, g, L, B, (const bf16*)k_new, (const bf16*)v_new, slots, status);
    case 64: return launch_pdl(append_decode_kernel<64>, grid, dim3(32), 0, st, g, L, B, (const bf16*)k_new, (const bf16*)v_new, slots, status);
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
  const int blocks = (int)((total + 255) / 256 < (size_t)device_sm_count() * 16 ? (total + 255) / 256 : (size_t)device_sm_count() * 16);
  write_prefill_kernel<<<blocks, 256, 0, st>>>(g, L, (const bf16*)k, (const bf16*)v, table, n_tokens);
  return cudaGetLastError();
}

}  // namespace loda
