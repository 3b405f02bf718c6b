// Shared device helpers of the loda_b200 kernels: bf16 rounding, ordered score
// keys, region geometry, block-wide radix select and scans.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "loda_b200.h"

namespace loda {

// ---------------------------------------------------------------------------
// numerics
// ---------------------------------------------------------------------------
__device__ __forceinline__ float bf16r(float x) {
  return __bfloat162float(__float2bfloat16_rn(x));
}

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
  return __uint_as_float(bits16 << 16);
}

// Monotone 16-bit key of a bf16-representable score: larger score -> larger
// key; NaN is canonicalised to the positive quiet NaN and sorts highest; -inf
// maps to ORD16_NEG_INF.  Same construction as the packed keys of
// nfa_layer_batch_selector.py:1482-1485.
__device__ __forceinline__ uint32_t ord16(float r) {
  uint32_t b = __float_as_uint(r) >> 16;
  if (r != r) b = 0x7FC0u;
  return (b & 0x8000u) ? ((~b) & 0xFFFFu) : (b | 0x8000u);
}
constexpr uint32_t ORD16_NEG_INF = 0x007Fu;

// index of subspace dim d inside the head: two contiguous halves
__device__ __forceinline__ int sub_dim(const loda_geometry& g, int d) {
  const int half = g.sub_dims >> 1;
  return d < half ? g.sub_lo0 + d : g.sub_lo1 + d - half;
}

// ---------------------------------------------------------------------------
// region geometry of one request (nfa_layer_batch_selector.py:209-262,
// 1136-1163, 1971-1986); no region is skipped
// ---------------------------------------------------------------------------
struct Regions {
  int length, kt_eff, near_blks, spl;
  int far_lo, far_hi;       // far pool = pages [far_lo, far_hi)
  int swa_lo_blk, swa_lo_tok, swa_byp_blk;
  bool swa_byp, sink_byp;
  int lower, upper, quota, kt_cap;
};

__device__ __forceinline__ int cdiv_trunc(int a, int b) { return a / b; }  // C division truncates

__device__ __forceinline__ Regions make_regions(const loda_geometry& g, int length) {
  Regions r;
  const int bs = g.page, w = g.swa;
  r.length = length;
  r.kt_cap = g.max_blocks;
  r.spl = g.sink / bs;
  r.kt_eff = (length + bs - 1) / bs;
  r.near_blks = max(cdiv_trunc(length - w - g.pool_near_len, bs), r.spl);
  r.sink_byp = (g.sink % bs) != 0;
  r.far_lo = r.spl + (r.sink_byp ? 1 : 0);
  r.far_hi = min(min(r.near_blks, r.kt_eff), g.max_blocks);
  r.swa_lo_blk = max(r.near_blks, r.kt_eff - max(1, w / bs));
  r.swa_lo_tok = max(length - w, 0);
  r.swa_byp_blk = r.swa_lo_tok / bs;
  r.swa_byp = (r.swa_lo_tok % bs != 0) && (r.swa_byp_blk >= r.spl);
  if (r.sink_byp) r.swa_byp = r.swa_byp && (r.swa_byp_blk != r.spl);
  r.lower = r.spl * bs;
  r.upper = max(r.lower, r.swa_lo_tok);
  int q = max(min(length, g.level2_topk) - g.sink - (length - r.swa_lo_tok), 0);
  r.quota = min(q, r.upper - r.lower);
  return r;
}

__device__ __forceinline__ bool in_far_pool(const Regions& r, int t) {
  return t >= r.far_lo && t < r.far_hi;
}

__device__ __forceinline__ bool in_near_pool(const Regions& r, int t) {
  if (t < r.near_blks || t >= r.swa_lo_blk || t >= r.kt_eff || t >= r.kt_cap) return false;
  if (r.swa_byp && t == r.swa_byp_blk) return false;
  if (r.sink_byp && t == r.spl) return false;
  return true;
}

// ---------------------------------------------------------------------------
// block-wide primitives (NT threads, all must call)
// ---------------------------------------------------------------------------

// Exclusive prefix sum of one int per thread; *total gets the block sum.
// scratch: 33 ints of shared memory.
template <int NT>
__device__ __forceinline__ int block_exclusive_scan(int v, int* scratch, int* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int n = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += n;
  }
  __syncthreads();
  if (lane == 31) scratch[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    int w = lane < NT / 32 ? scratch[lane] : 0;
    int wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int n = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += n;
    }
    scratch[lane] = wi - w;
    if (lane == 31) scratch[32] = wi;
  }
  __syncthreads();
  *total = scratch[32];
  return scratch[warp] + incl - v;
}

// k-th largest of n unique non-zero 32-bit keys held in shared memory (zeros
// are "no key" and must number at most n - k).  Four 8-bit radix passes from
// the most significant byte.  hist: 258 ints of shared memory.
template <int NT>
__device__ __forceinline__ uint32_t block_kth_largest(const uint32_t* keys, int n, int k, int* hist) {
  uint32_t prefix = 0, mask = 0;
#pragma unroll 1
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = threadIdx.x; i < 256; i += NT) hist[i] = 0;
    __syncthreads();
    // warp-aggregated histogram: lanes holding the same digit elect one lane to
    // add their count (scores share their leading bits, so un-aggregated atomics
    // would serialise 32-way on one shared-memory word)
    for (int base = 0; base < n; base += NT) {
      const int i = base + threadIdx.x;
      const uint32_t key = i < n ? keys[i] : 0u;
      const bool live = i < n && (key & mask) == prefix;
      const unsigned active = __ballot_sync(0xffffffffu, live);
      if (live) {
        const uint32_t digit = (key >> shift) & 255u;
        const unsigned peers = __match_any_sync(active, digit);
        if ((threadIdx.x & 31) == __ffs(peers) - 1) atomicAdd(&hist[digit], __popc(peers));
      }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
      const int lane = threadIdx.x;
      int c[8], s = 0;
#pragma unroll
      for (int i = 0; i < 8; ++i) { c[i] = hist[lane * 8 + i]; s += c[i]; }
      int above = 0;  // sum over the lanes holding larger digits
      int acc = s;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        int nb = __shfl_down_sync(0xffffffffu, acc, o);
        if (lane + o < 32) acc += nb;
      }
      above = acc - s;
      if (above < k && k <= above + s) {
        int run = above;
#pragma unroll
        for (int i = 7; i >= 0; --i) {
          if (run < k && k <= run + c[i]) { hist[256] = lane * 8 + i; hist[257] = k - run; }
          run += c[i];
        }
      }
    }
    __syncthreads();
    prefix |= (uint32_t)hist[256] << shift;
    mask |= 255u << shift;
    k = hist[257];
    __syncthreads();
  }
  return prefix;
}

// ---------------------------------------------------------------------------
// async copy
// ---------------------------------------------------------------------------
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src, bool valid) {
  const uint32_t dst = (uint32_t)__cvta_generic_to_shared(smem_dst);
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(dst), "l"(gmem_src), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// ---------------------------------------------------------------------------
// programmatic dependent launch: a kernel of the chain may be scheduled while
// its predecessor in the stream still runs; it must not touch memory before
// pdl_wait(), which returns once the predecessor has completed and flushed.
// Both are no-ops for a kernel launched without the attribute.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

// decode append carried by extra CTAs of the L1 launch (enabled == 0: none)
struct AppendArgs {
  const __nv_bfloat16* k_new;   // NULL with enabled != 0: refresh the index only
  const __nv_bfloat16* v_new;
  const int32_t* slots;
  uint32_t* status;
  int enabled;
};

// scratch views handed to the kernels (carved out of the caller's workspace)
struct L1Workspace {
  int* ticket;          // [rows], zero between launches
  int* cnt_far;         // [rows, nsplit]
  int* cnt_near;        // [rows, nsplit]
  uint32_t* part_far;   // [rows, nsplit, k_far]
  uint32_t* part_near;  // [rows, nsplit, k_near]
};
struct AttnWorkspace {
  int* ticket;    // [n_query * Hkv], zero between launches
  float* part_m;  // [n_query * Hkv, nsplit, G]
  float* part_z;  // [n_query * Hkv, nsplit, G]
  float* part_o;  // [n_query * Hkv, nsplit, G, DV]
};

}  // namespace loda
