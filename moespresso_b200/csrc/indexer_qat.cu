// Indexer pre- and post-ops of the DeepSeek-V4 decode chain.
//
//  * indexer_qat_kernel — the query / pool-row "QAT" that precedes the indexer score: a size-128
//    Walsh-Hadamard transform (radix-2 butterflies in increasing-stride order, float32, scaled by
//    128^-0.5) followed by an e2m1 round trip over 32-element groups: group scale
//    exp(ceil(log(amax / 6) / ln 2) * ln 2) evaluated in float32 steps, values clipped to
//    [-6, 6], snapped to the nearest of {0, .5, 1, 1.5, 2, 3, 4, 6} (ties to the LOWER lattice
//    value), sign restored, multiplied back by the scale.  One warp per row, lane l holds
//    elements 4l .. 4l+3, exactly the data layout and operation order of the reference's kernel
//    (src/moespresso/runtime/deepseek_v4/indexer_score_kernel.py:78-134), with every float32
//    operation rounded on its own (no fused multiply-add).  log and exp are evaluated in double
//    and rounded once to float32.
//  * score_tail_kernel — the tail of the composed score chain over per-head score rows: relu,
//    x scale, x (w_raw * H^-0.5), head sum with lane l owning heads l, l+32, ... followed by an
//    xor-butterfly over the 32 partials, invalid tail = +inf, result negated
//    (src/moespresso/runtime/deepseek_v4/indexer_score_kernel.py:472-490).  One thread per
//    column evaluates the same expression tree, so consecutive threads read consecutive columns.
#include "common.cuh"

namespace mxb {

struct QatParams {
  const void* x;
  float* out;
  int64_t n_rows;
};

__device__ __forceinline__ float lattice_snap(float n) {
  // nearest of the eight e2m1 magnitudes; the first (lower) value wins a tie
  const float values[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
  const float absn = fabsf(n);
  float best = fabsf(__fsub_rn(absn, values[0]));
  float dq = values[0];
#pragma unroll
  for (int k = 1; k < 8; ++k) {
    const float d = fabsf(__fsub_rn(absn, values[k]));
    if (d < best) {
      best = d;
      dq = values[k];
    }
  }
  return n < 0.0f ? -dq : dq;
}

template <int XT>
__global__ void __launch_bounds__(128) indexer_qat_kernel(QatParams p) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= p.n_rows) return;   // whole warps leave together
  float v[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) v[j] = load_elem<XT>(p.x, row * 128 + 4 * lane + j);

  // strides 1 and 2 inside the lane
  const float a0 = __fadd_rn(v[0], v[1]), a1 = __fsub_rn(v[0], v[1]);
  const float a2 = __fadd_rn(v[2], v[3]), a3 = __fsub_rn(v[2], v[3]);
  float x[4] = {__fadd_rn(a0, a2), __fadd_rn(a1, a3), __fsub_rn(a0, a2), __fsub_rn(a1, a3)};
  // strides 4 .. 64 pair lanes
#pragma unroll
  for (int m = 1; m <= 16; m <<= 1) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float other = __shfl_xor_sync(0xffffffffu, x[j], m);
      x[j] = (lane & m) ? __fsub_rn(other, x[j]) : __fadd_rn(x[j], other);
    }
  }
  const float kHadamardScale = 0.08838834764831845f;
#pragma unroll
  for (int j = 0; j < 4; ++j) x[j] = __fmul_rn(x[j], kHadamardScale);

  // e2m1 round trip over groups of 32 elements = 8 lanes
  // the maximum skips NaN elements (fmax), as the reference kernel's does; a group of nothing but NaN keeps NaN
  float amax = fmaxf(fmaxf(fabsf(x[0]), fabsf(x[1])), fmaxf(fabsf(x[2]), fabsf(x[3])));
#pragma unroll
  for (int m = 1; m <= 4; m <<= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, m));
  const float kAmaxFloor = 7.052966104933725e-38f;
  if (!isnan(amax) && !(amax > kAmaxFloor)) amax = kAmaxFloor;
  const float kLn2 = 0.6931471805599453f;           // ln 2 rounded to float32, as the float32 chain sees it
  const float ratio = __fdiv_rn(amax, 6.0f);
  const float lg = (float)log((double)ratio);        // correctly rounded float32 log
  const float log2_scale = __fdiv_rn(lg, kLn2);
  const float arg = __fmul_rn(ceilf(log2_scale), kLn2);
  const float scale = (float)exp((double)arg);       // correctly rounded float32 exp

  float* o = p.out + row * 128 + 4 * lane;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    float n = __fdiv_rn(x[j], scale);
    n = (isnan(n) || n > -6.0f) ? n : -6.0f;
    n = (isnan(n) || n < 6.0f) ? n : 6.0f;
    o[j] = __fmul_rn(lattice_snap(n), scale);
  }
}

struct TailParams {
  const float* scores;    // [H, capacity]
  const void* wraw;       // [H]
  const int32_t* params;  // [>= 2]; params[1] = valid columns
  float* neg;             // [capacity]
  int32_t H;
  int64_t capacity;
  float scale, head_norm;
};

template <int WT>
__global__ void __launch_bounds__(256) score_tail_kernel(TailParams p) {
  const int64_t col = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (col >= p.capacity) return;
  const int valid = p.params[1];
  float part[32];
#pragma unroll
  for (int l = 0; l < 32; ++l) {
    float acc = 0.0f;
    for (int h = l; h < p.H; h += 32) {
      const float w = __fmul_rn(load_elem<WT>(p.wraw, h), p.head_norm);
      float t = p.scores[(int64_t)h * p.capacity + col];
      t = isnan(t) ? t : (t > 0.0f ? t : 0.0f);
      t = __fmul_rn(t, p.scale);
      t = __fmul_rn(t, w);
      acc = __fadd_rn(acc, t);
    }
    part[l] = acc;
  }
  // the 32-lane xor butterfly, strides 16, 8, 4, 2, 1, on one thread
#pragma unroll
  for (int m = 16; m >= 1; m >>= 1) {
#pragma unroll
    for (int l = 0; l < 32; ++l)
      if ((l & m) == 0) part[l] = __fadd_rn(part[l], part[l | m]);
  }
  p.neg[col] = col < valid ? -part[0] : __int_as_float(0x7f800000);
}

}  // namespace mxb

using namespace mxb;

extern "C" int mxb_indexer_qat(const mxb_indexer_qat_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "indexer QAT: null args");
  MXB_REQUIRE(a->width == 128, MXB_ERR_INVALID, "indexer QAT expects 128-wide rows");
  MXB_REQUIRE(a->n_rows > 0, MXB_ERR_INVALID, "indexer QAT expects at least one row");
  MXB_REQUIRE(a->x && a->out, MXB_ERR_INVALID, "indexer QAT: null tensor");
  MXB_REQUIRE(a->x_dtype == MXB_F32 || a->x_dtype == MXB_F16 || a->x_dtype == MXB_BF16, MXB_ERR_INVALID,
              "indexer QAT rows must be float32, float16, or bfloat16");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  QatParams p{a->x, a->out, a->n_rows};
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
  if (a->x_dtype == MXB_F32) indexer_qat_kernel<MXB_F32><<<grid, 128, 0, st>>>(p);
  else if (a->x_dtype == MXB_F16) indexer_qat_kernel<MXB_F16><<<grid, 128, 0, st>>>(p);
  else indexer_qat_kernel<MXB_BF16><<<grid, 128, 0, st>>>(p);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_score_tail(const mxb_score_tail_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "score tail: null args");
  MXB_REQUIRE(a->capacity > 0, MXB_ERR_INVALID, "scores must cover at least one capacity column");
  MXB_REQUIRE(a->H >= 32 && a->H <= 64, MXB_ERR_INVALID, "the score tail transcription covers 32 to 64 index heads");
  MXB_REQUIRE(a->scores && a->weights_raw && a->params && a->out, MXB_ERR_INVALID, "score tail: null tensor");
  MXB_REQUIRE(a->w_dtype == MXB_F32 || a->w_dtype == MXB_F16 || a->w_dtype == MXB_BF16, MXB_ERR_INVALID,
              "weights_raw must be float32, float16, or bfloat16");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TailParams p{a->scores, a->weights_raw, a->params, a->out, a->H, a->capacity, a->scale,
               1.0f / sqrtf((float)a->H)};
  // H^-0.5 as the host's float32 power would give it (correctly rounded for 32 .. 64)
  p.head_norm = (float)(1.0 / sqrt((double)a->H));
  const unsigned grid = (unsigned)ceil_div(a->capacity, 256);
  if (a->w_dtype == MXB_F32) score_tail_kernel<MXB_F32><<<grid, 256, 0, st>>>(p);
  else if (a->w_dtype == MXB_F16) score_tail_kernel<MXB_F16><<<grid, 256, 0, st>>>(p);
  else score_tail_kernel<MXB_BF16><<<grid, 256, 0, st>>>(p);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
