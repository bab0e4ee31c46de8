// Shared host/device helpers for the sm_100a attention kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/moespresso_b200.h"

namespace mxb {

// ---- error reporting (thread-local message behind mxb_last_error) ----------
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);

#define MXB_REQUIRE(cond, code, ...)                 \
  do {                                               \
    if (!(cond)) return ::mxb::fail((code), __VA_ARGS__); \
  } while (0)

#define MXB_CUDA_OK(expr)                                                        \
  do {                                                                           \
    cudaError_t e__ = (expr);                                                    \
    if (e__ != cudaSuccess)                                                      \
      return ::mxb::fail(MXB_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e__)); \
  } while (0)

__host__ __device__ inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }
__host__ __device__ inline int64_t round_up(int64_t a, int64_t b) { return ceil_div(a, b) * b; }

int sm_count();
void note_launch(int n = 1);   // counts kernels enqueued by this library (mxb_kernel_launches)


// ---- element loads as float -------------------------------------------------
template <int DT>
struct ElemBytes;
template <> struct ElemBytes<MXB_F32> { static constexpr int v = 4; };
template <> struct ElemBytes<MXB_F16> { static constexpr int v = 2; };
template <> struct ElemBytes<MXB_BF16> { static constexpr int v = 2; };
template <> struct ElemBytes<MXB_F8E4M3> { static constexpr int v = 1; };
template <> struct ElemBytes<MXB_I8> { static constexpr int v = 1; };

__host__ __device__ inline int dtype_bytes(int dt) {
  return dt == MXB_F32 ? 4 : (dt == MXB_F16 || dt == MXB_BF16) ? 2 : 1;
}

__device__ __forceinline__ float e4m3_to_float(uint8_t b) {
  __half_raw h = __nv_cvt_fp8_to_halfraw((__nv_fp8_storage_t)b, __NV_E4M3);
  return __half2float(__half(h));
}

template <int DT>
__device__ __forceinline__ float load_elem(const void* p, int64_t i) {
  if constexpr (DT == MXB_F32) return reinterpret_cast<const float*>(p)[i];
  else if constexpr (DT == MXB_F16) return __half2float(reinterpret_cast<const __half*>(p)[i]);
  else if constexpr (DT == MXB_BF16) return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
  else if constexpr (DT == MXB_F8E4M3) return e4m3_to_float(reinterpret_cast<const uint8_t*>(p)[i]);
  else return (float)reinterpret_cast<const int8_t*>(p)[i];
}

// Convert the 16 bytes in `v` (8 / 4 / 16 elements of type DT) to floats.
template <int DT>
__device__ __forceinline__ void unpack16(const uint4& v, float* f) {
  if constexpr (DT == MXB_F32) {
    f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
    f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
  } else if constexpr (DT == MXB_F16) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __half22float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  } else if constexpr (DT == MXB_BF16) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) { float2 t = __bfloat1622float2(h[i]); f[2 * i] = t.x; f[2 * i + 1] = t.y; }
  } else if constexpr (DT == MXB_F8E4M3) {
    const uint8_t* b = reinterpret_cast<const uint8_t*>(&v);
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = e4m3_to_float(b[i]);
  } else {
    const int8_t* b = reinterpret_cast<const int8_t*>(&v);
#pragma unroll
    for (int i = 0; i < 16; ++i) f[i] = (float)b[i];
  }
}

template <int DT>
__device__ __forceinline__ void store_elem(void* p, int64_t i, float x) {
  if constexpr (DT == MXB_F32) reinterpret_cast<float*>(p)[i] = x;
  else if constexpr (DT == MXB_F16) reinterpret_cast<__half*>(p)[i] = __float2half_rn(x);
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(x);
}

// one rounding from float64 to the element type
template <int DT>
__device__ __forceinline__ void store_elem_f64(void* p, int64_t i, double x) {
  if constexpr (DT == MXB_F32) reinterpret_cast<float*>(p)[i] = __double2float_rn(x);
  else if constexpr (DT == MXB_F16) reinterpret_cast<__half*>(p)[i] = __double2half(x);
  else reinterpret_cast<__nv_bfloat16*>(p)[i] = __double2bfloat16(x);
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

}  // namespace mxb
