// Cache-row formats either side of the attention path.
//
//  * fp8_kv_rows_kernel — DeepSeek-V4's E4M3FN round trip of the non-rotary prefix of 512-wide
//    compressed-KV rows: dims [0, 448) in blocks of 64, block scale
//    exp(ceil(log(max(amax, 1e-4) / 448) / ln 2) * ln 2) in float32 steps, values clipped to
//    [-448, 448], snapped to the nearest of the 127 non-negative E4M3FN magnitudes (ties to the LOWER
//    one), sign restored (NaN -> 0), multiplied back; dims [448, 512) pass through.  One warp per row,
//    lane l holds dims [16l, 16l + 16), the layout and operation order of the reference's kernel
//    (src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:149-176, 536-560).  The nearest
//    magnitude is found arithmetically (grid step of the value's binade, ceil(t - 1/2)), which selects
//    the same table entry as the reference's first-wins scan of the table.
//  * quant_i8_rows_kernel — the per-token int8 quantiser that produces the int8 + fp16-scale cache the
//    sparse decode kernels read: scale = fp16(amax / 127) (rounded up when the rounding would let a
//    value exceed 127), q = clamp(rint(x / scale), -127, 127).  No counterpart in the reference.
#include "common.cuh"

namespace mxb {

__device__ __forceinline__ float e4m3_nearest_lower_tie(float absn) {
  // absn in [0, 448]
  float step;
  if (absn < 0.015625f) {
    step = 0.001953125f;   // subnormal spacing 2^-9
  } else {
    const int e = (int)((__float_as_uint(absn) >> 23) & 0xff) - 127;   // floor(log2(absn)), -6 .. 8
    step = __uint_as_float((uint32_t)(e - 3 + 127) << 23);
  }
  const float t = __fdiv_rn(absn, step);             // exact: step is a power of two
  return __fmul_rn(fabsf(ceilf(__fsub_rn(t, 0.5f))), step);  // exact; a tie (t = k + 1/2) goes to k; fabsf: ceil(-0.3) = -0
}

// nearest E4M3FN magnitude with ties to the even code: within a binade the code's parity is the parity of the
// grid multiple, so this is round-half-even on t
__device__ __forceinline__ float e4m3_nearest_even_tie(float absn) {
  float step;
  if (absn < 0.015625f) {
    step = 0.001953125f;
  } else {
    const int e = (int)((__float_as_uint(absn) >> 23) & 0xff) - 127;
    step = __uint_as_float((uint32_t)(e - 3 + 127) << 23);
  }
  return __fmul_rn(rintf(__fdiv_rn(absn, step)), step);
}

// REPLAY = false: the served transcription; true: the reference's NumPy replay form (exact power-of-two scale,
// ties to the even code)
template <bool REPLAY>
__global__ void __launch_bounds__(128) fp8_kv_rows_kernel(const float* __restrict__ x, float* __restrict__ out,
                                                          int64_t n_rows) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const float4* src = reinterpret_cast<const float4*>(x + row * 512 + 16 * lane);
  float4* dst = reinterpret_cast<float4*>(out + row * 512 + 16 * lane);
  float xv[16];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float4 v = src[j];
    xv[4 * j] = v.x; xv[4 * j + 1] = v.y; xv[4 * j + 2] = v.z; xv[4 * j + 3] = v.w;
  }
  // lanes 28 .. 31 hold the rotary tail: they take part in the shuffles and store their input back
  float amax = 0.0f;   // the maximum skips NaN elements (fmax), as the reference kernel's does
#pragma unroll
  for (int j = 0; j < 16; ++j) amax = fmaxf(amax, fabsf(xv[j]));
#pragma unroll
  for (int m = 1; m <= 2; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  if (lane < 28) {
    if (!(amax > 1.0e-4f)) amax = 1.0e-4f;
    float scale;
    if (REPLAY) {
      int e;
      const double m = frexp((double)amax / 448.0, &e);   // amax / 448 = m * 2^e, m in [0.5, 1)
      scale = ldexpf(1.0f, m == 0.5 ? e - 1 : e);         // 2^ceil(log2(amax / 448)), exactly
    } else {
      const float kLn2 = 0.6931471805599453f;
      const float lg = (float)log((double)__fdiv_rn(amax, 448.0f));   // correctly rounded float32 log
      const float arg = __fmul_rn(ceilf(__fdiv_rn(lg, kLn2)), kLn2);
      scale = (float)exp((double)arg);                                // correctly rounded float32 exp
    }
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      float n = __fdiv_rn(xv[j], scale);
      n = (isnan(n) || n > -448.0f) ? n : -448.0f;
      n = (isnan(n) || n < 448.0f) ? n : 448.0f;
      const float qv = isnan(n) ? 0.0f : (REPLAY ? e4m3_nearest_even_tie(fabsf(n)) : e4m3_nearest_lower_tie(fabsf(n)));
      const float sign = n < 0.0f ? -1.0f : (n > 0.0f ? 1.0f : 0.0f);
      xv[j] = __fmul_rn(__fmul_rn(sign, qv), scale);
    }
  }
#pragma unroll
  for (int j = 0; j < 4; ++j) dst[j] = make_float4(xv[4 * j], xv[4 * j + 1], xv[4 * j + 2], xv[4 * j + 3]);
}

template <int XT>
__global__ void __launch_bounds__(128) quant_i8_rows_kernel(const void* __restrict__ x, int8_t* __restrict__ q,
                                                            __half* __restrict__ scales, int64_t n_rows, int width) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  float amax = 0.0f;
  for (int i = lane; i < width; i += 32) amax = fmaxf(amax, fabsf(load_elem<XT>(x, row * width + i)));
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  __half hs = __float2half_rn(amax / 127.0f);
  if (__half2float(hs) * 127.0f < amax) hs = __ushort_as_half((unsigned short)(__half_as_ushort(hs) + 1));  // next fp16 up
  if (__half2float(hs) == 0.0f) hs = __ushort_as_half((unsigned short)1);   // all-zero row: any scale will do
  const float s = __half2float(hs);
  for (int i = lane; i < width; i += 32) {
    const float v = rintf(load_elem<XT>(x, row * width + i) / s);
    q[row * width + i] = (int8_t)fminf(fmaxf(v, -127.0f), 127.0f);
  }
  if (lane == 0) scales[row] = hs;
}

}  // namespace mxb

using namespace mxb;

extern "C" int mxb_fp8_kv_rows(const mxb_fp8_kv_rows_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "fp8 rows: null args");
  MXB_REQUIRE(a->width == 512, MXB_ERR_INVALID, "fp8 rows expect 512-wide rows");
  MXB_REQUIRE(a->n_rows > 0, MXB_ERR_INVALID, "fp8 rows expect at least one row");
  MXB_REQUIRE(a->x && a->out, MXB_ERR_INVALID, "fp8 rows: null tensor");
  MXB_REQUIRE(a->mode == MXB_FP8KV_SERVED || a->mode == MXB_FP8KV_REPLAY, MXB_ERR_INVALID, "fp8 rows: unknown mode");
  MXB_REQUIRE(((reinterpret_cast<uintptr_t>(a->x) | reinterpret_cast<uintptr_t>(a->out)) & 15) == 0, MXB_ERR_INVALID,
              "fp8 rows must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (a->mode == MXB_FP8KV_REPLAY)
    fp8_kv_rows_kernel<true><<<(unsigned)ceil_div(a->n_rows, 4), 128, 0, st>>>(a->x, a->out, a->n_rows);
  else
    fp8_kv_rows_kernel<false><<<(unsigned)ceil_div(a->n_rows, 4), 128, 0, st>>>(a->x, a->out, a->n_rows);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_quantize_kv_int8(const mxb_quantize_kv_int8_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "int8 quantiser: null args");
  MXB_REQUIRE(a->n_rows > 0 && a->width > 0, MXB_ERR_INVALID, "int8 quantiser expects at least one row and column");
  MXB_REQUIRE(a->x && a->q && a->scales, MXB_ERR_INVALID, "int8 quantiser: null tensor");
  MXB_REQUIRE(a->x_dtype == MXB_F32 || a->x_dtype == MXB_F16 || a->x_dtype == MXB_BF16, MXB_ERR_INVALID,
              "int8 quantiser rows must be float32, float16, or bfloat16");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
  __half* sc = reinterpret_cast<__half*>(a->scales);
  if (a->x_dtype == MXB_F32) quant_i8_rows_kernel<MXB_F32><<<grid, 128, 0, st>>>(a->x, a->q, sc, a->n_rows, a->width);
  else if (a->x_dtype == MXB_F16) quant_i8_rows_kernel<MXB_F16><<<grid, 128, 0, st>>>(a->x, a->q, sc, a->n_rows, a->width);
  else quant_i8_rows_kernel<MXB_BF16><<<grid, 128, 0, st>>>(a->x, a->q, sc, a->n_rows, a->width);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

// ---------------------------------------------------------------------------------------------
// Partial rotary embedding of the last `rope_dim` channels of every row (interleaved pairs), forward or
// inverse: the seam either side of the attention call
// (src/moespresso/runtime/deepseek_v4/attention.py:114-156; in-kernel forms
//  src/moespresso/runtime/deepseek_v4/decode_attention_kernel.py:398-422, 504-521).
// Row r sits at sequence index r % seq_len (the sequence axis is the second-to-last).  Angles are
// position * inverse frequency in float64, as in the NumPy definition; the result is rounded once to
// the row type.  Leading channels are copied.
// ---------------------------------------------------------------------------------------------
namespace mxb {

template <int XT>
__global__ void __launch_bounds__(128) rope_tail_kernel(const void* __restrict__ x, void* __restrict__ out,
                                                        const int64_t* __restrict__ positions,
                                                        const double* __restrict__ inv_freq, int64_t n_rows,
                                                        int seq_len, int width, int rope_dim, int inverse,
                                                        int half_chain) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  const int64_t base = row * width;
  const int lead = width - rope_dim;
  if (x != out)
    for (int i = lane; i < lead; i += 32) store_elem<XT>(out, base + i, load_elem<XT>(x, base + i));
  const double pos = (double)positions[row % seq_len];
  if constexpr (XT == MXB_F16) {
    if (half_chain) {
      // the fused decode kernels' float16 form: float32 angle, cos / sin rounded to float16, every product and
      // sum rounded to float16 (decode_attention_kernel.py:120-147, 398-422)
      const int64_t ipos = positions[row % seq_len];
      for (int pr = lane; pr < rope_dim / 2; pr += 32) {
        const float theta = __fmul_rn((float)ipos, (float)inv_freq[pr]);
        const __half c = __float2half_rn((float)cos((double)theta));
        __half s = __float2half_rn((float)sin((double)theta));
        if (inverse) s = __hneg(s);
        const __half x0 = reinterpret_cast<const __half*>(x)[base + lead + 2 * pr];
        const __half x1 = reinterpret_cast<const __half*>(x)[base + lead + 2 * pr + 1];
        // the _rn forms are never contracted into a fused multiply-add: every product is rounded on its own
        const __half m0 = __hmul_rn(x0, c), m1 = __hmul_rn(x1, s), m2 = __hmul_rn(x0, s), m3 = __hmul_rn(x1, c);
        reinterpret_cast<__half*>(out)[base + lead + 2 * pr] = __hsub_rn(m0, m1);
        reinterpret_cast<__half*>(out)[base + lead + 2 * pr + 1] = __hadd_rn(m2, m3);
      }
      return;
    }
  }
  for (int pr = lane; pr < rope_dim / 2; pr += 32) {
    double s, c;
    sincos(pos * inv_freq[pr], &s, &c);
    if (inverse) s = -s;
    const double x0 = (double)load_elem<XT>(x, base + lead + 2 * pr);
    const double x1 = (double)load_elem<XT>(x, base + lead + 2 * pr + 1);
    store_elem_f64<XT>(out, base + lead + 2 * pr, x0 * c - x1 * s);
    store_elem_f64<XT>(out, base + lead + 2 * pr + 1, x0 * s + x1 * c);
  }
}

}  // namespace mxb

extern "C" int mxb_rope_tail(const mxb_rope_tail_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "rope: null args");
  MXB_REQUIRE(a->n_rows > 0 && a->seq_len > 0 && a->n_rows % a->seq_len == 0, MXB_ERR_INVALID,
              "x must have at least sequence and feature dimensions");
  MXB_REQUIRE(a->rope_dim > 0 && a->rope_dim % 2 == 0, MXB_ERR_INVALID, "rope_dim must be a positive even integer");
  MXB_REQUIRE(a->width >= a->rope_dim, MXB_ERR_INVALID, "rope_dim cannot exceed the feature dimension");
  MXB_REQUIRE(a->x && a->out && a->positions && a->inv_freq, MXB_ERR_INVALID, "rope: null tensor");
  MXB_REQUIRE(a->x_dtype == MXB_F32 || a->x_dtype == MXB_F16 || a->x_dtype == MXB_BF16, MXB_ERR_INVALID,
              "rope rows must be float32, float16, or bfloat16");
  MXB_REQUIRE(!a->half_chain || a->x_dtype == MXB_F16, MXB_ERR_INVALID, "the float16 rope chain takes float16 rows");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
#define MXB_ROPE(XT)                                                                                          \
  rope_tail_kernel<XT><<<grid, 128, 0, st>>>(a->x, a->out, a->positions, a->inv_freq, a->n_rows, a->seq_len, \
                                             a->width, a->rope_dim, a->inverse, a->half_chain)
  if (a->x_dtype == MXB_F32) MXB_ROPE(MXB_F32);
  else if (a->x_dtype == MXB_F16) MXB_ROPE(MXB_F16);
  else MXB_ROPE(MXB_BF16);
#undef MXB_ROPE
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
