// Kernels under the TIA indexer's method surface (sparse_attn/indexer/tia_indexer.py):
//   min_max_per_token_quant  :22-31   4-bit per-token fake quantisation (round trip)
//   prepare_index            :33-62   per-block min / max over the full head dim
//   compute_score            :64-99   min/max bound per block and fine score per token
// bf16 and fp32 tensors.  Every torch op of the reference is one rounding to the
// tensor dtype; the quantiser reproduces its bits, the block min/max are exact,
// the scores accumulate in fp32 and are rounded once (the reference leaves the
// summation order to the BLAS, so scores agree to fp32 re-association).
#include "loda_common.cuh"

namespace loda {

using bf16 = __nv_bfloat16;

template <typename T> struct Num;
template <> struct Num<bf16> {
  static __device__ __forceinline__ float load(const bf16* p) { return __bfloat162float(*p); }
  static __device__ __forceinline__ void store(bf16* p, float v) { *p = __float2bfloat16_rn(v); }
  static __device__ __forceinline__ float round(float v) { return bf16r(v); }
};
template <> struct Num<float> {
  static __device__ __forceinline__ float load(const float* p) { return *p; }
  static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
  static __device__ __forceinline__ float round(float v) { return v; }
};

// one warp per row of `dim` <= 128 values: y = dequant(quant(x))
template <typename T>
__global__ void __launch_bounds__(128) tia_quant4_kernel(const T* __restrict__ x, T* __restrict__ y, long long n_rows,
                                                         int dim, long long x_stride, long long y_stride) {
  const long long row = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= n_rows) return;
  float v[4];
  float mx = -INFINITY, mn = INFINITY;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane + 32 * j;
    v[j] = d < dim ? Num<T>::load(x + row * x_stride + d) : 0.0f;
    if (d < dim) { mx = fmaxf(mx, v[j]); mn = fminf(mn, v[j]); }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
  }
  const float floor_v = Num<T>::round(1e-9f);
  float range = Num<T>::round(__fsub_rn(mx, mn));
  range = range < floor_v ? floor_v : range;
  const float scale = Num<T>::round(__fdiv_rn(range, 15.0f));
  const float zero = -mn;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int d = lane + 32 * j;
    if (d >= dim) continue;
    float t = Num<T>::round(__fdiv_rn(Num<T>::round(__fadd_rn(v[j], zero)), scale));
    t = fminf(fmaxf(rintf(t), 0.0f), 15.0f);
    Num<T>::store(y + row * y_stride + d, Num<T>::round(__fsub_rn(Num<T>::round(__fmul_rn(t, scale)), zero)));
  }
}

// k [S, H, D] -> kmin / kmax [T, H, D]; a ragged last block is padded with zeros
// as the reference pads before reducing (tia_indexer.py:39-46)
template <typename T>
__global__ void __launch_bounds__(128) tia_block_minmax_kernel(const T* __restrict__ k, T* __restrict__ kmin,
                                                               T* __restrict__ kmax, int S, int H, int D, int bs) {
  const int t = blockIdx.x, h = blockIdx.y;
  for (int d = threadIdx.x; d < D; d += blockDim.x) {
    float mn = INFINITY, mx = -INFINITY;
    for (int i = 0; i < bs; ++i) {
      const int tok = t * bs + i;
      const float v = tok < S ? Num<T>::load(k + ((size_t)tok * H + h) * D + d) : 0.0f;
      mn = fminf(mn, v);
      mx = fmaxf(mx, v);
    }
    Num<T>::store(kmin + ((size_t)t * H + h) * D + d, mn);
    Num<T>::store(kmax + ((size_t)t * H + h) * D + d, mx);
  }
}

// one warp per (query head, block): coarse = sum_d min(qs,0) kmin + max(qs,0) kmax, qs = q * scale
template <typename T>
__global__ void __launch_bounds__(128) tia_coarse_kernel(const T* __restrict__ q, const T* __restrict__ kmin,
                                                         const T* __restrict__ kmax, T* __restrict__ out, int Hq,
                                                         int Hkv, int D, int Tn, float scale) {
  const int warp = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (warp >= Hq * Tn) return;
  const int h = warp / Tn, t = warp % Tn, kv = h / (Hq / Hkv);
  float acc = 0.0f;
  for (int d = lane; d < D; d += 32) {
    const float qs = __fmul_rn(Num<T>::load(q + (size_t)h * D + d), scale);
    const size_t o = ((size_t)t * Hkv + kv) * D + d;
    acc = fmaf(fminf(qs, 0.0f), Num<T>::load(kmin + o), acc);
    acc = fmaf(fmaxf(qs, 0.0f), Num<T>::load(kmax + o), acc);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) Num<T>::store(out + (size_t)h * Tn + t, acc);
}

// one warp per (query head, token): fine = sum_d qs kqat
template <typename T>
__global__ void __launch_bounds__(128) tia_fine_kernel(const T* __restrict__ q, const T* __restrict__ kqat,
                                                       T* __restrict__ out, int Hq, int Hkv, int D, int S, float scale) {
  const long long warp = (long long)blockIdx.x * 4 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (warp >= (long long)Hq * S) return;
  const int h = (int)(warp / S), s = (int)(warp % S), kv = h / (Hq / Hkv);
  float acc = 0.0f;
  for (int d = lane; d < D; d += 32)
    acc = fmaf(__fmul_rn(Num<T>::load(q + (size_t)h * D + d), scale), Num<T>::load(kqat + ((size_t)s * Hkv + kv) * D + d), acc);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if (lane == 0) Num<T>::store(out + (size_t)h * S + s, acc);
}

int report_error(int code, const char* message);

}  // namespace loda

using namespace loda;

extern "C" {

int loda_tia_quant4(const void* x, void* y, int64_t n_rows, int32_t dim, int64_t x_stride, int64_t y_stride,
                    int32_t dtype, void* stream) {
  if (!x || !y || n_rows < 0 || dim < 1 || dim > 128) return report_error(LODA_ERR_ARGUMENT, "quant4: dim must be in [1, 128]");
  if (n_rows == 0) return LODA_OK;
  const unsigned blocks = (unsigned)((n_rows + 3) / 4);
  if (dtype == LODA_DTYPE_BF16)
    tia_quant4_kernel<bf16><<<blocks, 128, 0, (cudaStream_t)stream>>>((const bf16*)x, (bf16*)y, n_rows, dim, x_stride, y_stride);
  else if (dtype == LODA_DTYPE_FP32)
    tia_quant4_kernel<float><<<blocks, 128, 0, (cudaStream_t)stream>>>((const float*)x, (float*)y, n_rows, dim, x_stride, y_stride);
  else
    return report_error(LODA_ERR_UNSUPPORTED, "quant4: dtype must be bf16 or fp32");
  return cudaGetLastError() == cudaSuccess ? LODA_OK : report_error(LODA_ERR_LAUNCH, "quant4 launch failed");
}

int loda_tia_block_minmax(const void* k, void* kmin, void* kmax, int32_t S, int32_t H, int32_t D, int32_t block_size,
                          int32_t dtype, void* stream) {
  if (!k || !kmin || !kmax || S < 1 || H < 1 || D < 1 || block_size < 1)
    return report_error(LODA_ERR_ARGUMENT, "block_minmax: bad arguments");
  const dim3 grid((S + block_size - 1) / block_size, H);
  if (dtype == LODA_DTYPE_BF16)
    tia_block_minmax_kernel<bf16><<<grid, 128, 0, (cudaStream_t)stream>>>((const bf16*)k, (bf16*)kmin, (bf16*)kmax, S, H, D, block_size);
  else if (dtype == LODA_DTYPE_FP32)
    tia_block_minmax_kernel<float><<<grid, 128, 0, (cudaStream_t)stream>>>((const float*)k, (float*)kmin, (float*)kmax, S, H, D, block_size);
  else
    return report_error(LODA_ERR_UNSUPPORTED, "block_minmax: dtype must be bf16 or fp32");
  return cudaGetLastError() == cudaSuccess ? LODA_OK : report_error(LODA_ERR_LAUNCH, "block_minmax launch failed");
}

int loda_tia_scores(const void* q, const void* kmin, const void* kmax, const void* kqat, void* coarse, void* fine,
                    int32_t Hq, int32_t Hkv, int32_t D, int32_t T, int32_t S, float scale, int32_t dtype, void* stream) {
  if (!q || !kmin || !kmax || !kqat || !coarse || !fine || Hq < 1 || Hkv < 1 || Hq % Hkv || T < 1 || S < 1)
    return report_error(LODA_ERR_ARGUMENT, "tia_scores: bad arguments");
  const unsigned cb = (unsigned)(((long long)Hq * T + 3) / 4), fb = (unsigned)(((long long)Hq * S + 3) / 4);
  cudaStream_t st = (cudaStream_t)stream;
  if (dtype == LODA_DTYPE_BF16) {
    tia_coarse_kernel<bf16><<<cb, 128, 0, st>>>((const bf16*)q, (const bf16*)kmin, (const bf16*)kmax, (bf16*)coarse, Hq, Hkv, D, T, scale);
    tia_fine_kernel<bf16><<<fb, 128, 0, st>>>((const bf16*)q, (const bf16*)kqat, (bf16*)fine, Hq, Hkv, D, S, scale);
  } else if (dtype == LODA_DTYPE_FP32) {
    tia_coarse_kernel<float><<<cb, 128, 0, st>>>((const float*)q, (const float*)kmin, (const float*)kmax, (float*)coarse, Hq, Hkv, D, T, scale);
    tia_fine_kernel<float><<<fb, 128, 0, st>>>((const float*)q, (const float*)kqat, (float*)fine, Hq, Hkv, D, S, scale);
  } else {
    return report_error(LODA_ERR_UNSUPPORTED, "tia_scores: dtype must be bf16 or fp32");
  }
  return cudaGetLastError() == cudaSuccess ? LODA_OK : report_error(LODA_ERR_LAUNCH, "tia_scores launch failed");
}

}  // extern "C"
