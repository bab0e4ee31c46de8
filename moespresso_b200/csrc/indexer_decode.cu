// Indexer score, decode form (one query token per sequence) over FP8-E4M3 key tables.
//
// A pure bandwidth scan: 64 (or 128) key bytes in, 4 score bytes out, per row.  Every warp
// works alone on 16-row tiles, straight from global memory into registers:
//
//   * lane (g = lane / 4, t = lane % 4) loads the t-th quarter of key rows g and g + 8 of the
//     tile (16-byte vector loads; a warp reads 2 x 512 contiguous bytes per 64-byte-row tile);
//   * the quarter is widened to fp16 pairs (cvt.f16x2.e4m3x2, exact) which ARE the A fragment
//     of mma.sync.m16n8k16 under a permutation of the feature axis: MMA step s, slots
//     (2t, 2t+1, 2t+8, 2t+9) stand for features t*D/4 + 4s + (0..3).  The query (B fragment)
//     is loaded once per warp under the same permutation, so no shuffle or shared-memory
//     transpose is needed;
//   * the query is scaled per head by a power of two (max |q| * 2^a in [2^13, 2^14)), which
//     makes every bf16 value within 2^-27 of the head's maximum an exact fp16 value; the head
//     weight carries 2^-a.  Products are exact, accumulation is fp32;
//   * relu, weights and the head sum happen on the accumulator fragment (two shuffles per
//     quad, same order for every row, so a row's score does not depend on the partition).
//
// No shared memory, no barriers: latency is hidden by the loads of several tiles in flight
// per warp and by occupancy.  The tensor work is tiny (32 flop per byte); this kernel is
// bound by HBM, which is why it uses warp-level MMA rather than the tcgen05 pipeline the
// prefill form needs.
#include "common.cuh"

namespace mxb {

struct DecodeIdxParams {
  const uint8_t* keys;
  const void* q;
  int q_is_bf16;
  int64_t q_sb, q_sh;
  const float* weights;   // [B, H]
  float* scores;
  int64_t s_sb;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t B, H;
  int64_t n_rows;
  int32_t rows_per_cta;   // multiple of 8 warps * 16 rows * kUnroll
};

constexpr int kDecWarps = 8;
constexpr int kDecUnroll = 4;   // 16-row tiles in flight per warp

__device__ __forceinline__ void mma_f16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
  __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)v, __NV_E4M3);
  return *reinterpret_cast<uint32_t*>(&hr);
}

// D = feature width (64 | 128), NT = heads / 8 (n-tiles of the MMA)
template <int D, int NT>
__global__ void __launch_bounds__(kDecWarps * 32) indexer_decode_kernel(DecodeIdxParams p) {
  constexpr int EPL = D / 4;    // features (= key bytes) per lane per row
  constexpr int KS = D / 16;    // MMA k-steps
  constexpr int VPL = EPL / 16; // 16-byte loads per lane per row
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int b = blockIdx.y;
  const int64_t count = p.row_count ? (int64_t)p.row_count[b] : p.n_rows;
  const int64_t rbase = p.row_start ? p.row_start[b] : (int64_t)b * p.n_rows;
  const int64_t cta_row0 = (int64_t)blockIdx.x * p.rows_per_cta;
  if (cta_row0 >= count) return;

  // ---- query fragments: head 8j + g, features t*EPL .. t*EPL + EPL - 1, scaled to fp16
  uint32_t bq[NT][KS][2];
  float wq[NT][2];   // weights * 2^-a of heads 8j + 2t, 8j + 2t + 1 (the accumulator's columns)
#pragma unroll
  for (int j = 0; j < NT; ++j) {
    const int h = 8 * j + g;
    float x[EPL];
    float amax = 0.f;
    const int64_t base = (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + t * EPL;
#pragma unroll
    for (int e = 0; e < EPL; ++e) {
      x[e] = p.q_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.q)[base + e])
                         : __half2float(reinterpret_cast<const __half*>(p.q)[base + e]);
      amax = fmaxf(amax, fabsf(x[e]));
    }
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    int a = 0;
    if (amax > 0.f && amax < 3.0e38f) {
      int e;
      frexpf(amax, &e);
      a = max(-100, min(100, 14 - e));
    }
#pragma unroll
    for (int s = 0; s < KS; ++s) {
      __half2 lo = __floats2half2_rn(ldexpf(x[4 * s], a), ldexpf(x[4 * s + 1], a));
      __half2 hi = __floats2half2_rn(ldexpf(x[4 * s + 2], a), ldexpf(x[4 * s + 3], a));
      bq[j][s][0] = *reinterpret_cast<uint32_t*>(&lo);
      bq[j][s][1] = *reinterpret_cast<uint32_t*>(&hi);
    }
    // the scale of head 8j + c is known to the quad g == c: fetch the two this lane's columns need
    const int a0 = __shfl_sync(0xffffffffu, a, (2 * t) * 4);
    const int a1 = __shfl_sync(0xffffffffu, a, (2 * t + 1) * 4);
    wq[j][0] = ldexpf(p.weights[(int64_t)b * p.H + 8 * j + 2 * t], -a0);
    wq[j][1] = ldexpf(p.weights[(int64_t)b * p.H + 8 * j + 2 * t + 1], -a1);
  }

  const uint8_t* kbase = p.keys + rbase * D;
  float* sbase = p.scores + (p.row_start ? p.row_start[b] : 0) + (int64_t)b * p.s_sb;
  int64_t cta_end = cta_row0 + p.rows_per_cta;
  if (cta_end > count) cta_end = count;
  const int64_t last = count - 1;

  // warps interleave groups of kDecUnroll tiles so that the CTA reads one contiguous stream
  for (int64_t r0 = cta_row0 + (int64_t)warp * (16 * kDecUnroll); r0 < cta_end;
       r0 += (int64_t)kDecWarps * 16 * kDecUnroll) {
    uint4 raw[kDecUnroll][2][VPL];
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
#pragma unroll
      for (int hrow = 0; hrow < 2; ++hrow) {
        int64_t r = r0 + u * 16 + g + 8 * hrow;
        if (r > last) r = last;   // clamped rows are computed and discarded
        const uint4* src = reinterpret_cast<const uint4*>(kbase + r * D + t * EPL);
#pragma unroll
        for (int v = 0; v < VPL; ++v) raw[u][hrow][v] = __ldg(src + v);
      }
    }
#pragma unroll
    for (int u = 0; u < kDecUnroll; ++u) {
      float acc[NT][4];
#pragma unroll
      for (int j = 0; j < NT; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.f;
      const uint16_t* lo16 = reinterpret_cast<const uint16_t*>(&raw[u][0][0]);
      const uint16_t* hi16 = reinterpret_cast<const uint16_t*>(&raw[u][1][0]);
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        uint32_t af[4];
        af[0] = e4m3x2_to_f16x2(lo16[2 * s]);       // row g,     slots 2t, 2t+1
        af[1] = e4m3x2_to_f16x2(hi16[2 * s]);       // row g + 8, slots 2t, 2t+1
        af[2] = e4m3x2_to_f16x2(lo16[2 * s + 1]);   // row g,     slots 2t+8, 2t+9
        af[3] = e4m3x2_to_f16x2(hi16[2 * s + 1]);   // row g + 8, slots 2t+8, 2t+9
#pragma unroll
        for (int j = 0; j < NT; ++j) mma_f16_16816(acc[j], af, bq[j][s][0], bq[j][s][1]);
      }
      float s_lo = 0.f, s_hi = 0.f;
#pragma unroll
      for (int j = 0; j < NT; ++j) {
        s_lo = fmaf(wq[j][0], fmaxf(acc[j][0], 0.f), s_lo);
        s_lo = fmaf(wq[j][1], fmaxf(acc[j][1], 0.f), s_lo);
        s_hi = fmaf(wq[j][0], fmaxf(acc[j][2], 0.f), s_hi);
        s_hi = fmaf(wq[j][1], fmaxf(acc[j][3], 0.f), s_hi);
      }
      s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 1);
      s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 1);
      s_lo += __shfl_xor_sync(0xffffffffu, s_lo, 2);
      s_hi += __shfl_xor_sync(0xffffffffu, s_hi, 2);
      // lane t of the quad stores: t == 0 -> row g, t == 1 -> row g + 8
      const int64_t r = r0 + u * 16 + g + 8 * t;
      if (t < 2 && r < cta_end) sbase[r] = t == 0 ? s_lo : s_hi;
    }
  }
}

template <int D>
static int launch_decode_d(DecodeIdxParams& p, cudaStream_t st) {
  // chunks of rows per CTA: a few thousand CTAs so that ragged sequences balance over the SMs
  const int64_t unit = (int64_t)kDecWarps * 16 * kDecUnroll;   // 512 rows
  int64_t per = ceil_div(p.n_rows * p.B, (int64_t)sm_count() * 16);
  per = round_up(per < unit ? unit : per, unit);
  if (per > round_up(p.n_rows, unit)) per = round_up(p.n_rows, unit);
  p.rows_per_cta = (int)per;
  dim3 grid((unsigned)ceil_div(p.n_rows, per), (unsigned)p.B);
  const int nt = p.H / 8;
#define MXB_DEC(NT)                                                        \
  if (nt == NT) {                                                          \
    indexer_decode_kernel<D, NT><<<grid, kDecWarps * 32, 0, st>>>(p);      \
    MXB_CUDA_OK(cudaGetLastError());                                       \
    return MXB_OK;                                                         \
  }
  MXB_DEC(1) MXB_DEC(2) MXB_DEC(4) MXB_DEC(8)
#undef MXB_DEC
  return fail(MXB_ERR_UNSUPPORTED, "decode indexer: head count %d is not 8, 16, 32 or 64", p.H);
}

bool indexer_decode_eligible(const mxb_indexer_scores_args* a) {
  const bool q16 = a->q_dtype == MXB_F16 || a->q_dtype == MXB_BF16;
  return a->T == 1 && a->key_dtype == MXB_F8E4M3 && q16 && (a->H == 8 || a->H == 16 || a->H == 32 || a->H == 64) &&
         !(a->flags & (MXB_INDEXER_EXACT_FP32 | MXB_INDEXER_FP8_MMA));
}

int launch_indexer_decode(const mxb_indexer_scores_args* a, cudaStream_t st) {
  DecodeIdxParams p{};
  p.keys = reinterpret_cast<const uint8_t*>(a->keys);
  p.q = a->q; p.q_is_bf16 = a->q_dtype == MXB_BF16; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
  p.weights = a->weights; p.scores = a->scores; p.s_sb = a->score_stride_b;
  p.row_start = a->row_start; p.row_count = a->row_count; p.B = a->B; p.H = a->H; p.n_rows = a->n_rows;
  if (a->D == 64) return launch_decode_d<64>(p, st);
  return launch_decode_d<128>(p, st);
}

}  // namespace mxb
