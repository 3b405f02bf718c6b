// Pieces of the gather attention shared by its stand-alone kernel and by the one-launch decode
// step: tensor-core fragments (mma.sync m16n8k16, bf16 operands, fp32 accumulate) and the online
// softmax step of one warp over 16 staged tokens.
// Restates the inner loop of the reference's grouped gather kernel
// (sparse_attn/ops/paged_region_kernels.py:251-363).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace loda {

__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], const void* smem_ptr) {
  const uint32_t a = (uint32_t)__cvta_generic_to_shared(smem_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *(uint32_t*)&v;
}


// Q fragments of one (query row, kv head): A operand, rows = heads of the group (zero beyond G).
// q0 points at the first head of the group, rows D elements apart.
template <int D>
__device__ __forceinline__ void attn_load_q(uint32_t (&qa)[D / 16][4], const __nv_bfloat16* qg, int G, int lane) {
  const int r0 = lane >> 2, r1 = r0 + 8, kc = (lane & 3) * 2;
  const __nv_bfloat16* q0 = qg + (size_t)r0 * D;
  const __nv_bfloat16* q1 = qg + (size_t)r1 * D;
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    qa[ks][0] = r0 < G ? *(const uint32_t*)(q0 + ks * 16 + kc) : 0u;
    qa[ks][1] = r1 < G ? *(const uint32_t*)(q1 + ks * 16 + kc) : 0u;
    qa[ks][2] = r0 < G ? *(const uint32_t*)(q0 + ks * 16 + kc + 8) : 0u;
    qa[ks][3] = r1 < G ? *(const uint32_t*)(q1 + ks * 16 + kc + 8) : 0u;
  }
}

// One warp, 16 staged tokens [tok0, tok0 + 16) of a tile of ntok tokens: S = Q K^T, fp32 online
// softmax in the exp2 domain (tokens with slot < 0 or beyond ntok masked), O += P V with P rounded
// to bf16.  Kt / Vt: the tile's rows, D + 8 and DV + 8 elements apart (conflict-free ldmatrix).
// The state (oacc, m_run, z_run) covers rows lane / 4 and lane / 4 + 8 of the group.
template <int D, int DV>
__device__ __forceinline__ void attn_warp_step(const __nv_bfloat16* Kt, const __nv_bfloat16* Vt, const int* slot_t,
                                               int tok0, int ntok, const uint32_t (&qa)[D / 16][4], float scale_log2,
                                               float (&oacc)[DV / 8][4], float (&m_run)[2], float (&z_run)[2]) {
  constexpr int KSTR = D + 8, VSTR = DV + 8, KSTEPS = D / 16, NTV = DV / 8;
  const int lane = threadIdx.x & 31;
  // S = Q K^T for this warp's 16 tokens: two n-tiles of 8 tokens
  float sacc[2][4] = {{0, 0, 0, 0}, {0, 0, 0, 0}};
#pragma unroll
  for (int ks = 0; ks < KSTEPS; ++ks) {
    uint32_t kb[4];
    const int mi = lane >> 3, r = lane & 7;
    ldmatrix_x4(kb, Kt + (tok0 + (mi >> 1) * 8 + r) * KSTR + ks * 16 + (mi & 1) * 8);
    mma_bf16(sacc[0], qa[ks], kb[0], kb[1]);
    mma_bf16(sacc[1], qa[ks], kb[2], kb[3]);
  }
  // mask, scale (log2 domain), per-row max over this warp's tokens
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
  float alpha[2], msafe[2];
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    const float m_new = fmaxf(m_run[h], mx[h]);
    msafe[h] = m_new == -INFINITY ? 0.0f : m_new;
    alpha[h] = exp2f(m_run[h] - msafe[h]);     // m_run = -inf -> 0
    m_run[h] = m_new;
  }
  uint32_t pa[4];
  float zs[2] = {0.0f, 0.0f};
  {
    float p[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        p[j][e] = exp2f(sacc[j][e] - msafe[e >> 1]);
        zs[e >> 1] += p[j][e];
      }
    pa[0] = pack_bf16(p[0][0], p[0][1]);   // row r,   tokens 0..7
    pa[1] = pack_bf16(p[0][2], p[0][3]);   // row r+8, tokens 0..7
    pa[2] = pack_bf16(p[1][0], p[1][1]);   // row r,   tokens 8..15
    pa[3] = pack_bf16(p[1][2], p[1][3]);   // row r+8, tokens 8..15
  }
#pragma unroll
  for (int h = 0; h < 2; ++h) {
    zs[h] += __shfl_xor_sync(0xffffffffu, zs[h], 1);
    zs[h] += __shfl_xor_sync(0xffffffffu, zs[h], 2);
    z_run[h] = z_run[h] * alpha[h] + zs[h];
  }
#pragma unroll
  for (int i = 0; i < NTV; ++i) {
    oacc[i][0] *= alpha[0]; oacc[i][1] *= alpha[0];
    oacc[i][2] *= alpha[1]; oacc[i][3] *= alpha[1];
  }
  // O += P V: V^T fragments by transposed ldmatrix, two dv n-tiles per load
#pragma unroll
  for (int i = 0; i < NTV; i += 2) {
    uint32_t vb[4];
    const int mi = lane >> 3, r = lane & 7;
    ldmatrix_x4_trans(vb, Vt + (tok0 + (mi & 1) * 8 + r) * VSTR + i * 8 + (mi >> 1) * 8);
    mma_bf16(oacc[i], pa, vb[0], vb[1]);
    mma_bf16(oacc[i + 1], pa, vb[2], vb[3]);
  }
}

}  // namespace loda
