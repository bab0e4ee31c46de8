// Device helpers shared by the top-k kernels: monotone score keys, digit picking, block scan.
#pragma once

#include "common.cuh"

namespace mxb {

constexpr int kSmemRowMax = 45056;  // 176 KB of keys
constexpr int kBigBins = 2048;      // top 11 bits

__device__ __forceinline__ uint32_t score_key_full(float x) {
  if (!(fabsf(x) <= 3.402823466e38f)) return 0u;  // NaN and +-inf are never selected
  uint32_t b = __float_as_uint(x + 0.0f);         // -0 + 0 = +0
  return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}

// Find, scanning digits from 255 down, the digit where the running count reaches `want`.
// hist[256] in shared memory; executed by warp 0; results through shared scalars.
__device__ __forceinline__ void pick_digit_256(const uint32_t* hist, uint32_t want, uint32_t* out_digit,
                                               uint32_t* out_above) {
  const int lane = threadIdx.x & 31;
  // lane l owns digits [255 - 8l - 7, 255 - 8l], highest first
  uint32_t loc[8];
  uint32_t s = 0;
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    loc[j] = hist[255 - (lane * 8 + j)];
    s += loc[j];
  }
  uint32_t incl = s;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  const uint32_t excl = incl - s;
  const bool mine = excl < want && incl >= want;
  if (mine) {
    uint32_t run = excl;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (run + loc[j] >= want) {
        *out_digit = 255 - (lane * 8 + j);
        *out_above = run;
        break;
      }
      run += loc[j];
    }
  }
}

// block-wide exclusive scan of one uint per thread (1024 threads max); returns exclusive prefix,
// total through *total.
__device__ __forceinline__ uint32_t block_excl_scan(uint32_t v, uint32_t* warp_sums, uint32_t* total) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  uint32_t incl = v;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    uint32_t t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_sums[warp] = incl;
  __syncthreads();
  if (warp == 0) {
    uint32_t w = (lane < (int)(blockDim.x >> 5)) ? warp_sums[lane] : 0;
    uint32_t wi = w;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      uint32_t t = __shfl_up_sync(0xffffffffu, wi, o);
      if (lane >= o) wi += t;
    }
    warp_sums[lane] = wi - w;
    if (lane == 31) *total = wi;
  }
  __syncthreads();
  uint32_t r = warp_sums[warp] + incl - v;
  __syncthreads();
  return r;
}

// Threshold bin of a 2048-bin histogram (global or shared memory): the bin, counted from the top,
// where the running count reaches min(k, total).  All 512 or 1024 threads of the CTA take part;
// s_out must be zero on entry.
// Thread t owns bins top-down in groups of `per` = 2048 / blockDim.x.
__device__ __forceinline__ void row_threshold(const uint32_t* g, int k, uint32_t* warp_sums, uint32_t* s_total,
                                              uint32_t* s_out /* k_eff, bin, above, cnt */) {
  const int tid = threadIdx.x;
  const int per = kBigBins / (int)blockDim.x;   // 4 (512 threads) or 2 (1024 threads)
  uint32_t loc[4];
  uint32_t s = 0;
  for (int j = 0; j < per; ++j) {
    loc[j] = g[kBigBins - 1 - (tid * per + j)];
    s += loc[j];
  }
  const uint32_t excl = block_excl_scan(s, warp_sums, s_total);
  const uint32_t ke = min((uint32_t)k, *s_total);
  if (tid == 0) s_out[0] = ke;
  if (ke > 0 && excl < ke && excl + s >= ke) {
    uint32_t run = excl;
    for (int j = 0; j < per; ++j) {
      if (run + loc[j] >= ke) {
        s_out[1] = kBigBins - 1 - (tid * per + j);
        s_out[2] = run;
        s_out[3] = loc[j];
        break;
      }
      run += loc[j];
    }
  }
  __syncthreads();
}

}  // namespace mxb
