// Affine 8-bit KV format of the Qwen full-attention cache (group 64) and the long-context decode attention
// over it.
//
// The reference keeps the Qwen KV cache in MLX's affine quantised form (mlx-lm QuantizedKVCache, bits 8, group
// size 64: src/moespresso/runtime/qwen/full_attention.py:200-236) and hands it to two third-party kernels:
// sdpa_fa_prefill_q8 (:372-382) and sdpa_decode_q8 (:323-335).  The format as MLX documents it for mx.quantize:
// every group of 64 consecutive features of a row has beta = min, alpha = max, scale = (alpha - beta) / 255,
// bias = beta; element = round((w - bias) / scale) in [0, 255]; w ~= element * scale + bias.  Four elements per
// uint32 word, lowest byte first; scales and biases in the row's floating type.
//
//  * affine_q8_quantize_kernel / affine_q8_dequantize_kernel — the format, one warp per row (any width that is
//    a multiple of 64); the dequantiser writes with a caller-chosen row stride so that a past can be expanded
//    straight into the front of a [past + chunk] operand of the flash prefill kernel.
//  * q8_decode_kernel — one query token over a q8 cache, split over the keys: a CTA owns (split, KV head), its
//    eight warps take keys four at a time, round-robin, and keep an online softmax for each of the KV head's query heads; the
//    warps' states are merged in shared memory and every split writes (o, m, l) partials for the log-sum-exp
//    merge kernel (mxb_merge_partials).  HBM-bound: 2 x (256 + 16) bytes per key and KV head are read once.
#include "common.cuh"

namespace mxb {

constexpr int Q8_GROUP = 64;

template <int XT>
__global__ void __launch_bounds__(128) affine_q8_quantize_kernel(const void* __restrict__ x, int64_t x_row_stride,
                                                                 uint32_t* __restrict__ packed, void* __restrict__ scales,
                                                                 void* __restrict__ biases, int64_t n_rows, int width) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  // 8 lanes share a group of 64 features: lane l of a 256-feature span holds features 8 l .. 8 l + 7
  for (int f0 = 0; f0 < width; f0 += 256) {
    const int f = f0 + lane * 8;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = f < width ? load_elem<XT>(x, row * x_row_stride + f + e) : 0.f;
    float lo = v[0], hi = v[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) {
      lo = fminf(lo, v[e]);
      hi = fmaxf(hi, v[e]);
    }
#pragma unroll
    for (int m = 4; m >= 1; m >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, m));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, m));
    }
    if (f >= width) continue;
    // scale and bias are stored in the row's type; the elements are taken against the STORED values
    // (every step is a single correctly rounded float32 operation, no contraction: the packed words are compared
    // bit for bit with the CPU restatement)
    float scale = __fdiv_rn(__fsub_rn(hi, lo), 255.f), bias = lo;
    if constexpr (XT == MXB_F16) {
      scale = __half2float(__float2half_rn(scale));
      bias = __half2float(__float2half_rn(bias));
    } else if constexpr (XT == MXB_BF16) {
      scale = __bfloat162float(__float2bfloat16_rn(scale));
      bias = __bfloat162float(__float2bfloat16_rn(bias));
    }
    const float inv = scale > 0.f ? __fdiv_rn(1.f, scale) : 0.f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float q = fminf(fmaxf(floorf(__fadd_rn(__fmul_rn(__fsub_rn(v[e], bias), inv), 0.5f)), 0.f), 255.f);
      w[e >> 2] |= (uint32_t)q << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(packed + row * (width / 4) + f / 4) = make_uint2(w[0], w[1]);
    if ((lane & 7) == 0) {
      const int64_t g = row * (width / Q8_GROUP) + f / Q8_GROUP;
      store_elem<XT>(scales, g, scale);
      store_elem<XT>(biases, g, bias);
    }
  }
}

template <int ST, int OT>
__global__ void __launch_bounds__(128) affine_q8_dequantize_kernel(const uint32_t* __restrict__ packed,
                                                                   const void* __restrict__ scales,
                                                                   const void* __restrict__ biases, void* __restrict__ out,
                                                                   int64_t out_row_stride, int64_t n_rows, int width) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  for (int f = lane * 8; f < width; f += 256) {
    const uint2 w = *reinterpret_cast<const uint2*>(packed + row * (width / 4) + f / 4);
    const int64_t g = row * (width / Q8_GROUP) + f / Q8_GROUP;
    const float scale = load_elem<ST>(scales, g), bias = load_elem<ST>(biases, g);
    const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
    for (int e = 0; e < 8; ++e)
      store_elem<OT>(out, row * out_row_stride + f + e, fmaf((float)((ww[e >> 2] >> (8 * (e & 3))) & 0xffu), scale, bias));
  }
}

// ---------------------------------------------------------------------------------------------
// decode: one query token, head_dim 256, GQA group of up to 8 query heads per KV head
// ---------------------------------------------------------------------------------------------
constexpr int QD_D = 256, QD_WARPS = 8, QD_MAXG = 8, QD_BATCH = 4;

struct Q8DecodeParams {
  const void* q;           // [Hq, 256]
  int32_t q_dtype;
  const uint32_t* kp; const void* ks; const void* kb;   // keys   [Hkv, P, 64] u32, [Hkv, P, 4], [Hkv, P, 4]
  const uint32_t* vp; const void* vs; const void* vb;   // values, same
  int64_t head_stride_rows;   // rows between consecutive KV heads (the cache capacity)
  int32_t sb_dtype;        // type of the scales and biases
  int32_t P, Hq, Hkv, nsplit;
  float scale_log2;
  float* o_parts;          // [nsplit, Hq, 256]
  float* ml_parts;         // [nsplit, Hq, 2]
};

template <int ST>
__global__ void __launch_bounds__(QD_WARPS * 32) q8_decode_kernel(Q8DecodeParams p) {
  extern __shared__ float q8_smem[];
  float (*q_s)[QD_D] = reinterpret_cast<float (*)[QD_D]>(q8_smem);                                   // [QD_MAXG][QD_D]
  float (*o_s)[QD_MAXG][QD_D] = reinterpret_cast<float (*)[QD_MAXG][QD_D]>(q8_smem + QD_MAXG * QD_D);   // the warps' accumulators at the end
  __shared__ float m_s[QD_WARPS][QD_MAXG], l_s[QD_WARPS][QD_MAXG];
  const int split = blockIdx.x, kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int G = p.Hq / p.Hkv;
  for (int i = tid; i < G * QD_D; i += QD_WARPS * 32) {
    const int g = i / QD_D, d = i % QD_D;
    const int64_t off = (int64_t)(kvh * G + g) * QD_D + d;
    q_s[g][d] = p.q_dtype == MXB_F32 ? load_elem<MXB_F32>(p.q, off)
                : p.q_dtype == MXB_F16 ? load_elem<MXB_F16>(p.q, off) : load_elem<MXB_BF16>(p.q, off);
  }
  __syncthreads();
  const int per = (p.P + p.nsplit - 1) / p.nsplit;
  const int k_lo = min(split * per, p.P), k_hi = min(k_lo + per, p.P);
  // lane l holds features 8 l .. 8 l + 7 of a row: one 8-byte word pair, group l / 8
  float qv[QD_MAXG][8];
#pragma unroll
  for (int g = 0; g < QD_MAXG; ++g)
#pragma unroll
    for (int e = 0; e < 8; ++e) qv[g][e] = g < G ? q_s[g][lane * 8 + e] : 0.f;
  float m[QD_MAXG], l[QD_MAXG], o[QD_MAXG][8];
#pragma unroll
  for (int g = 0; g < QD_MAXG; ++g) {
    m[g] = -INFINITY;
    l[g] = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) o[g][e] = 0.f;
  }
  const int64_t hb = (int64_t)kvh * p.head_stride_rows;
  // a warp takes QD_BATCH keys per trip and issues all of their loads before the arithmetic (bytes in flight)
  for (int key0 = k_lo + warp * QD_BATCH; key0 < k_hi; key0 += QD_WARPS * QD_BATCH) {
    uint2 kw[QD_BATCH], vw[QD_BATCH];
    float ksc[QD_BATCH], kbi[QD_BATCH], vsc[QD_BATCH], vbi[QD_BATCH];
#pragma unroll
    for (int b = 0; b < QD_BATCH; ++b) {
      const int64_t r = hb + min(key0 + b, k_hi - 1);
      kw[b] = __ldg(reinterpret_cast<const uint2*>(p.kp + r * 64) + lane);
      vw[b] = __ldg(reinterpret_cast<const uint2*>(p.vp + r * 64) + lane);
      const int64_t gi = r * 4 + (lane >> 3);
      ksc[b] = load_elem<ST>(p.ks, gi);
      kbi[b] = load_elem<ST>(p.kb, gi);
      vsc[b] = load_elem<ST>(p.vs, gi);
      vbi[b] = load_elem<ST>(p.vb, gi);
    }
#pragma unroll
    for (int b = 0; b < QD_BATCH; ++b) {
      if (key0 + b >= k_hi) break;
      float kf[8], vf[8];
      const uint32_t kww[2] = {kw[b].x, kw[b].y}, vww[2] = {vw[b].x, vw[b].y};
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        kf[e] = fmaf((float)((kww[e >> 2] >> (8 * (e & 3))) & 0xffu), ksc[b], kbi[b]);
        vf[e] = fmaf((float)((vww[e >> 2] >> (8 * (e & 3))) & 0xffu), vsc[b], vbi[b]);
      }
#pragma unroll
      for (int g = 0; g < QD_MAXG; ++g) {
        if (g < G) {
          float s = 0.f;
#pragma unroll
          for (int e = 0; e < 8; ++e) s = fmaf(qv[g][e], kf[e], s);
          s = warp_sum(s) * p.scale_log2;
          const float mn = fmaxf(m[g], s);
          const float corr = exp2f(m[g] - mn), pw = exp2f(s - mn);   // m = -inf: corr = 0
          l[g] = l[g] * corr + pw;
#pragma unroll
          for (int e = 0; e < 8; ++e) o[g][e] = fmaf(o[g][e], corr, pw * vf[e]);
          m[g] = mn;
        }
      }
    }
  }
  // merge the eight warps in warp order
#pragma unroll
  for (int g = 0; g < QD_MAXG; ++g) {
    if (g < G) {
      if (lane == 0) {
        m_s[warp][g] = m[g];
        l_s[warp][g] = l[g];
      }
#pragma unroll
      for (int e = 0; e < 8; ++e) o_s[warp][g][lane * 8 + e] = o[g][e];
    }
  }
  __syncthreads();
  for (int i = tid; i < G * QD_D; i += QD_WARPS * 32) {
    const int g = i / QD_D, d = i % QD_D;
    float mm = -INFINITY;
    for (int w = 0; w < QD_WARPS; ++w) mm = fmaxf(mm, m_s[w][g]);
    float acc = 0.f, ll = 0.f;
    for (int w = 0; w < QD_WARPS; ++w) {
      const float f = m_s[w][g] == -INFINITY ? 0.f : exp2f(m_s[w][g] - mm);
      acc = fmaf(o_s[w][g][d], f, acc);
      ll = fmaf(l_s[w][g], f, ll);
    }
    const int h = kvh * G + g;
    p.o_parts[((int64_t)split * p.Hq + h) * QD_D + d] = acc;
    if (d == 0) {
      // (m, l) in natural-log units for the merge kernel
      p.ml_parts[((int64_t)split * p.Hq + h) * 2] = mm == -INFINITY ? -INFINITY : mm * 0.6931471805599453f;
      p.ml_parts[((int64_t)split * p.Hq + h) * 2 + 1] = ll;
    }
  }
}

}  // namespace mxb

using namespace mxb;

static int q8_check(const mxb_affine_q8_args* a, const char* what) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "%s: null args", what);
  MXB_REQUIRE(a->n_rows > 0 && a->width > 0 && a->width % Q8_GROUP == 0, MXB_ERR_INVALID,
              "%s: rows must be non-empty and their width a multiple of the group size 64", what);
  MXB_REQUIRE(a->x && a->packed && a->scales && a->biases, MXB_ERR_INVALID, "%s: null tensor", what);
  MXB_REQUIRE(a->x_dtype == MXB_F32 || a->x_dtype == MXB_F16 || a->x_dtype == MXB_BF16, MXB_ERR_INVALID,
              "%s: rows must be float32, float16 or bfloat16", what);
  MXB_REQUIRE(a->sb_dtype == MXB_F32 || a->sb_dtype == MXB_F16 || a->sb_dtype == MXB_BF16, MXB_ERR_INVALID,
              "%s: scales and biases must be float32, float16 or bfloat16", what);
  MXB_REQUIRE((reinterpret_cast<uintptr_t>(a->packed) & 7) == 0, MXB_ERR_INVALID, "%s: packed words must be 8-byte aligned", what);
  return MXB_OK;
}

extern "C" int mxb_affine_q8_quantize(const mxb_affine_q8_args* a, void* stream) {
  int rc = q8_check(a, "affine q8 quantise");
  if (rc != MXB_OK) return rc;
  MXB_REQUIRE(a->sb_dtype == a->x_dtype, MXB_ERR_INVALID, "affine q8 quantise: scales and biases take the rows' type");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
  uint32_t* pk = reinterpret_cast<uint32_t*>(a->packed);
#define MXB_Q(XT) affine_q8_quantize_kernel<XT><<<grid, 128, 0, st>>>(a->x, a->x_row_stride, pk, a->scales, a->biases, a->n_rows, a->width)
  if (a->x_dtype == MXB_F32) MXB_Q(MXB_F32);
  else if (a->x_dtype == MXB_F16) MXB_Q(MXB_F16);
  else MXB_Q(MXB_BF16);
#undef MXB_Q
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_affine_q8_dequantize(const mxb_affine_q8_args* a, void* stream) {
  int rc = q8_check(a, "affine q8 dequantise");
  if (rc != MXB_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
  const uint32_t* pk = reinterpret_cast<const uint32_t*>(a->packed);
  void* out = const_cast<void*>(a->x);
#define MXB_DQ(ST, OT) \
  if (a->sb_dtype == ST && a->x_dtype == OT)                                                                          \
    affine_q8_dequantize_kernel<ST, OT><<<grid, 128, 0, st>>>(pk, a->scales, a->biases, out, a->x_row_stride, a->n_rows, a->width); \
  else
  MXB_DQ(MXB_F32, MXB_F32) MXB_DQ(MXB_F32, MXB_F16) MXB_DQ(MXB_F32, MXB_BF16)
  MXB_DQ(MXB_F16, MXB_F32) MXB_DQ(MXB_F16, MXB_F16) MXB_DQ(MXB_F16, MXB_BF16)
  MXB_DQ(MXB_BF16, MXB_F32) MXB_DQ(MXB_BF16, MXB_F16) MXB_DQ(MXB_BF16, MXB_BF16)
  return fail(MXB_ERR_UNSUPPORTED, "affine q8 dequantise: unsupported type pair");
#undef MXB_DQ
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_sdpa_decode_q8(const mxb_sdpa_decode_q8_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "q8 decode: null args");
  MXB_REQUIRE(a->D == QD_D, MXB_ERR_INVALID, "q8 decode requires head_dim=256");
  MXB_REQUIRE(a->Hq > 0 && a->Hkv > 0 && a->Hq % a->Hkv == 0 && a->Hq / a->Hkv <= QD_MAXG, MXB_ERR_INVALID,
              "q8 decode: query heads must be a multiple (at most 8x) of kv heads");
  MXB_REQUIRE(a->P >= 1, MXB_ERR_INVALID, "q8 decode needs at least one cached key");
  MXB_REQUIRE(a->n_splits >= 1 && a->n_splits <= 1024, MXB_ERR_INVALID, "q8 decode: splits must be between 1 and 1024");
  MXB_REQUIRE(a->q && a->k_packed && a->k_scales && a->k_biases && a->v_packed && a->v_scales && a->v_biases &&
                  a->o_parts && a->ml_parts,
              MXB_ERR_INVALID, "q8 decode: null tensor");
  MXB_REQUIRE(((reinterpret_cast<uintptr_t>(a->k_packed) | reinterpret_cast<uintptr_t>(a->v_packed)) & 7) == 0,
              MXB_ERR_INVALID, "q8 decode: packed words must be 8-byte aligned");
  Q8DecodeParams p{};
  p.q = a->q; p.q_dtype = a->q_dtype;
  p.kp = reinterpret_cast<const uint32_t*>(a->k_packed); p.ks = a->k_scales; p.kb = a->k_biases;
  p.vp = reinterpret_cast<const uint32_t*>(a->v_packed); p.vs = a->v_scales; p.vb = a->v_biases;
  p.head_stride_rows = a->head_stride_rows; p.sb_dtype = a->sb_dtype;
  p.P = a->P; p.Hq = a->Hq; p.Hkv = a->Hkv; p.nsplit = a->n_splits;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.o_parts = a->o_parts; p.ml_parts = a->ml_parts;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)a->n_splits, (unsigned)a->Hkv);
  const int smem = (QD_MAXG * QD_D + QD_WARPS * QD_MAXG * QD_D) * (int)sizeof(float);   // 72 KB
#define MXB_QD(ST)                                                                                            \
  {                                                                                                           \
    MXB_CUDA_OK(cudaFuncSetAttribute(q8_decode_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    q8_decode_kernel<ST><<<grid, QD_WARPS * 32, smem, st>>>(p);                                               \
  }
  if (a->sb_dtype == MXB_F32) MXB_QD(MXB_F32)
  else if (a->sb_dtype == MXB_F16) MXB_QD(MXB_F16)
  else if (a->sb_dtype == MXB_BF16) MXB_QD(MXB_BF16)
  else return fail(MXB_ERR_INVALID, "q8 decode: scales and biases must be float32, float16 or bfloat16");
#undef MXB_QD
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
