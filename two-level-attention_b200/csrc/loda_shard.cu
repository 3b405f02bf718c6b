// Sequence sharding helpers: the fixed-order log-sum-exp merge of the GPUs' partial attentions as one
// kernel.  Every rank attends over the selected tokens that live on its own pages and reports
// (out bf16 [rows, Dv] normalised by its own sum, lse float [rows, 2] = row maximum in the exp2 domain and
// sum); after an all-gather each rank merges the parts in rank order, so every rank gets the same bits.
// Extends the split combine of the reference (sparse_attn/ops/paged_region_kernels.py:578-607) across
// devices; the arithmetic is that of lse_merge in two-level-attention_b200/sharding.py.
#include "loda_common.cuh"

namespace loda {

constexpr int MERGE_MAX_PARTS = 16;

// parts: n_parts blocks `part_stride` bytes apart; inside a block the outputs start at byte 0 and the
// (max, sum) pairs at byte `lse_offset`.  One CTA per row.
__global__ void __launch_bounds__(128) lse_merge_kernel(const unsigned char* parts, long long part_stride,
                                                        long long lse_offset, int n_parts, int n_rows, int dv,
                                                        float* __restrict__ out) {
  const int row = blockIdx.x;
  pdl_wait();
  float w[MERGE_MAX_PARTS];
  float M = -INFINITY;
#pragma unroll
  for (int r = 0; r < MERGE_MAX_PARTS; ++r) {
    w[r] = -INFINITY;
    if (r < n_parts) {
      const float* lse = (const float*)(parts + r * part_stride + lse_offset) + (size_t)row * 2;
      w[r] = __ldcg(lse);
      M = fmaxf(M, w[r]);
    }
  }
  const float safe = M == -INFINITY ? 0.0f : M;
  float z = 0.0f;
#pragma unroll
  for (int r = 0; r < MERGE_MAX_PARTS; ++r) {
    if (r < n_parts) {
      const float* lse = (const float*)(parts + r * part_stride + lse_offset) + (size_t)row * 2;
      w[r] = exp2f(w[r] - safe) * __ldcg(lse + 1);      // weight of the part: exp2(m_r - M) z_r
      z += w[r];
    } else {
      w[r] = 0.0f;
    }
  }
  const float inv = z > 0.0f ? 1.0f / fmaxf(z, 1e-38f) : 0.0f;
  for (int c = threadIdx.x; c < dv; c += blockDim.x) {
    float o = 0.0f;
#pragma unroll
    for (int r = 0; r < MERGE_MAX_PARTS; ++r) {
      if (r < n_parts) {
        const __nv_bfloat16* po = (const __nv_bfloat16*)(parts + r * part_stride) + (size_t)row * dv;
        o += __bfloat162float(po[c]) * w[r];
      }
    }
    out[(size_t)row * dv + c] = o * inv;
  }
}

int report_error(int code, const char* message);

}  // namespace loda

extern "C" int loda_lse_merge(const void* parts, int64_t part_stride_bytes, int64_t lse_offset_bytes, int32_t n_parts,
                              int32_t n_rows, int32_t dv, float* out, void* stream) {
  using namespace loda;
  if (!parts || !out || n_parts < 1 || n_parts > MERGE_MAX_PARTS || n_rows < 0 || dv < 1 || (lse_offset_bytes & 3))
    return report_error(LODA_ERR_ARGUMENT, "lse_merge: 1..16 parts, non-NULL buffers, 4-byte aligned lse offset");
  if (n_rows == 0) return LODA_OK;
  const cudaError_t e = launch_pdl(lse_merge_kernel, dim3(n_rows), dim3(128), 0, (cudaStream_t)stream,
                                   (const unsigned char*)parts, (long long)part_stride_bytes, (long long)lse_offset_bytes,
                                   (int)n_parts, (int)n_rows, (int)dv, out);
  if (e != cudaSuccess) return report_error(LODA_ERR_LAUNCH, cudaGetErrorString(e));
  return LODA_OK;
}
