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
// Work is split evenly, not per sequence: every CTA prefix-sums the row counts of the batch
// (a few hundred bytes of shared memory), takes an equal share of the concatenated row space
// and walks the one or two sequences its share overlaps.  The grid is one resident wave, so a
// ragged batch leaves no tail and the query fragments are set up once or twice per CTA.
// Latency is hidden by the loads of several tiles in flight per warp and by occupancy.  The
// tensor work is tiny (32 flop per byte); this kernel is bound by HBM, which is why it uses
// warp-level MMA rather than the tcgen05 pipeline the prefill form needs.
#include "common.cuh"
#include "topk_common.cuh"

namespace mxb {

// 16 bytes of read-only global memory that nobody reads again soon: past L1, first in line for eviction from L2.
__device__ __forceinline__ uint64_t make_stream_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ld_stream(const uint4* src, uint64_t policy) {
  uint4 v;
  asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0, %1, %2, %3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(src), "l"(policy));
  return v;
}


struct DecodeIdxParams {
  const uint8_t* keys;
  const void* q;
  int q_is_bf16;
  int q_vec;              // q rows may be read with 16-byte loads
  int64_t q_sb, q_sh;
  const float* weights;   // [B, H]
  float* scores;
  int64_t s_sb;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t B, H;
  int64_t n_rows;
  uint32_t* hist;         // [B, 2048] first-digit histogram of the selection keys, or null
};

constexpr int kDecWarps = 8;
constexpr int kDecUnroll = 4;                               // 16-row tiles in flight per warp
constexpr int kDecGroup = 16 * kDecUnroll;                  // rows per warp per loop trip
constexpr int kDecCtaRows = kDecWarps * kDecGroup;          // rows per CTA per loop trip
constexpr int kDecMaxBatch = 4096;                          // prefix sums live in shared memory

__device__ __forceinline__ void mma_f16_16816(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t e4m3x2_to_f16x2(uint16_t v) {
  uint32_t r;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(r) : "h"(v));
  return r;
}

// 2^a as a float, a in [-126, 127]
__device__ __forceinline__ float pow2i(int a) { return __int_as_float((127 + a) << 23); }

// D = feature width (64 | 128), NT = heads / 8 (n-tiles of the MMA).  HIST: the score is still in a register when
// it is stored, so the first radix digit of the selection that follows is counted here (a shared-memory histogram
// per CTA, flushed with one global add per non-empty bin at the end of each sequence's segment).
template <int D, int NT, bool HIST>
__global__ void __launch_bounds__(kDecWarps * 32, (D == 64 && NT <= 2) ? 3 : 1) indexer_decode_kernel(DecodeIdxParams p) {
  constexpr int EPL = D / 4;    // features (= key bytes) per lane per row
  constexpr int KS = D / 16;    // MMA k-steps
  constexpr int VPL = EPL / 16; // 16-byte loads per lane per row
  extern __shared__ int64_t pre_s[];   // [B + 1] exclusive prefix sums of the row counts
  __shared__ uint32_t hist_s[HIST ? kBigBins : 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  if constexpr (HIST)
    for (int i = threadIdx.x; i < kBigBins; i += kDecWarps * 32) hist_s[i] = 0;

  if (warp == 0) {
    int64_t carry = 0;
    for (int i0 = 0; i0 < p.B; i0 += 32) {   // trip count is the same for every lane
      const int i = i0 + lane;
      int64_t x = 0;
      if (i < p.B) x = p.row_count ? (int64_t)max(p.row_count[i], 0) : p.n_rows;
      if (x > p.n_rows) x = p.n_rows;
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const int64_t y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
      }
      if (i < p.B) pre_s[i + 1] = carry + x;
      carry += __shfl_sync(0xffffffffu, x, 31);
    }
    if (lane == 0) pre_s[0] = 0;
  }
  __syncthreads();
  const int64_t total = pre_s[p.B];
  const int64_t share = round_up(ceil_div(total, (int64_t)gridDim.x), (int64_t)kDecCtaRows);
  const int64_t lo = (int64_t)blockIdx.x * share;
  const int64_t hi = lo + share < total ? lo + share : total;
  if (lo >= hi) return;
  int b = 0;
  {  // largest b with pre_s[b] <= lo
    int l = 0, r = p.B;
    while (r - l > 1) {
      const int m = (l + r) >> 1;
      if (pre_s[m] <= lo) l = m; else r = m;
    }
    b = l;
  }

  for (; b < p.B && pre_s[b] < hi; ++b) {
    const int64_t seg_lo = (lo > pre_s[b] ? lo : pre_s[b]) - pre_s[b];
    const int64_t seg_hi = (hi < pre_s[b + 1] ? hi : pre_s[b + 1]) - pre_s[b];
    if (seg_lo >= seg_hi) continue;   // empty sequence

    // ---- query fragments: head 8j + g, features t*EPL .. t*EPL + EPL - 1, scaled to fp16
    uint32_t bq[NT][KS][2];
    float wq[NT][2];   // weights * 2^-a of heads 8j + 2t, 8j + 2t + 1 (the accumulator's columns)
#pragma unroll
    for (int j = 0; j < NT; ++j) {
      const int h = 8 * j + g;
      float x[EPL];
      const int64_t base = (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + t * EPL;
      if (p.q_vec) {
        const uint4* qp = reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + base);
#pragma unroll
        for (int v = 0; v < EPL / 8; ++v) {
          const uint4 w4 = __ldg(qp + v);
          const uint32_t w[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            if (p.q_is_bf16) {
              x[8 * v + 2 * e] = __uint_as_float(w[e] << 16);
              x[8 * v + 2 * e + 1] = __uint_as_float(w[e] & 0xffff0000u);
            } else {
              const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&w[e]));
              x[8 * v + 2 * e] = f.x;
              x[8 * v + 2 * e + 1] = f.y;
            }
          }
        }
      } else {
#pragma unroll
        for (int e = 0; e < EPL; ++e)
          x[e] = p.q_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.q)[base + e])
                             : __half2float(reinterpret_cast<const __half*>(p.q)[base + e]);
      }
      float amax = 0.f;
#pragma unroll
      for (int e = 0; e < EPL; ++e) amax = fmaxf(amax, fabsf(x[e]));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
      amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
      int a = 0;
      if (amax > 0.f && amax < 3.0e38f) {
        const int e = (int)((__float_as_uint(amax) >> 23) & 0xff) - 126;   // amax = m * 2^e, m in [0.5, 1)
        a = max(-100, min(100, 14 - e));
      }
      const float up = pow2i(a);
#pragma unroll
      for (int s = 0; s < KS; ++s) {
        __half2 l2 = __floats2half2_rn(x[4 * s] * up, x[4 * s + 1] * up);
        __half2 h2 = __floats2half2_rn(x[4 * s + 2] * up, x[4 * s + 3] * up);
        bq[j][s][0] = *reinterpret_cast<uint32_t*>(&l2);
        bq[j][s][1] = *reinterpret_cast<uint32_t*>(&h2);
      }
      // the scale of head 8j + c is known to the quad g == c: fetch the two this lane's columns need
      const int a0 = __shfl_sync(0xffffffffu, a, (2 * t) * 4);
      const int a1 = __shfl_sync(0xffffffffu, a, (2 * t + 1) * 4);
      wq[j][0] = p.weights[(int64_t)b * p.H + 8 * j + 2 * t] * pow2i(-a0);
      wq[j][1] = p.weights[(int64_t)b * p.H + 8 * j + 2 * t + 1] * pow2i(-a1);
    }

    const int64_t rbase = p.row_start ? p.row_start[b] : (int64_t)b * p.n_rows;
    const uint8_t* kt = p.keys + (rbase + seg_lo) * D + t * EPL;          // row 0 of the segment, this lane's quarter
    float* st = p.scores + (p.row_start ? p.row_start[b] : 0) + (int64_t)b * p.s_sb + seg_lo + g + 8 * t;
    const int64_t n_here = seg_hi - seg_lo;

    // The keys are read once per step and are larger than L2: they are marked to be evicted first, so that they do
    // not push out what the next kernels of the step come back to (their code, the scores, the lists, the queries).
    const uint64_t stream_policy = make_stream_policy();
    // warps interleave groups of kDecUnroll tiles so that the CTA reads one contiguous stream
    for (int64_t go = (int64_t)warp * kDecGroup; go < n_here; go += kDecCtaRows) {
      const int64_t left64 = n_here - go;
      const int left = left64 < kDecGroup ? (int)left64 : kDecGroup;
      uint4 raw[kDecUnroll][2][VPL];
      if (left == kDecGroup) {
        const uint4* src = reinterpret_cast<const uint4*>(kt + (go + g) * D);
#pragma unroll
        for (int u = 0; u < kDecUnroll; ++u)
#pragma unroll
          for (int hrow = 0; hrow < 2; ++hrow)
#pragma unroll
            for (int v = 0; v < VPL; ++v) raw[u][hrow][v] = ld_stream(src + (u * 16 + hrow * 8) * (D / 16) + v, stream_policy);
      } else {
#pragma unroll
        for (int u = 0; u < kDecUnroll; ++u)
#pragma unroll
          for (int hrow = 0; hrow < 2; ++hrow) {
            const int rr = min(u * 16 + hrow * 8 + g, left - 1);   // clamped rows are computed and discarded
            const uint4* src = reinterpret_cast<const uint4*>(kt + (go + rr) * D);
#pragma unroll
            for (int v = 0; v < VPL; ++v) raw[u][hrow][v] = ld_stream(src + v, stream_policy);
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
        if (t < 2 && u * 16 + g + 8 * t < left) {
          const float sc = t == 0 ? s_lo : s_hi;
          st[go + u * 16] = sc;
          if constexpr (HIST) {
            const uint32_t key = score_key_full(sc);
            if (key) atomicAdd(&hist_s[key >> 21], 1u);
          }
        }
      }
    }
    if constexpr (HIST) {   // b and the segment bounds are the same for every thread of the CTA
      __syncthreads();
      for (int i = threadIdx.x; i < kBigBins; i += kDecWarps * 32) {
        const uint32_t v = hist_s[i];
        if (v) {
          atomicAdd(&p.hist[(int64_t)b * kBigBins + i], v);
          hist_s[i] = 0;
        }
      }
      __syncthreads();
    }
  }
}

template <int D, int NT, bool HIST>
static int launch_decode_nt(DecodeIdxParams& p, cudaStream_t st) {
  auto kern = indexer_decode_kernel<D, NT, HIST>;
  static int per_sm[64] = {0};   // resident CTAs per SM, per device
  int dev = 0;
  MXB_CUDA_OK(cudaGetDevice(&dev));
  const size_t smem = (size_t)(p.B + 1) * sizeof(int64_t);
  if (dev < 0 || dev >= 64) return fail(MXB_ERR_UNSUPPORTED, "decode indexer: device ordinal %d out of range", dev);
  if (per_sm[dev] == 0) {
    int n = 0;
    MXB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kern, kDecWarps * 32, 1024));
    per_sm[dev] = n < 1 ? 1 : n;
  }
  // one resident wave; small problems get one CTA per kDecCtaRows rows of the largest possible total
  int64_t ctas = (int64_t)sm_count() * per_sm[dev];
  const int64_t most = ceil_div(p.n_rows * p.B, (int64_t)kDecCtaRows);
  if (ctas > most) ctas = most;
  kern<<<(unsigned)ctas, kDecWarps * 32, smem, st>>>(p);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

template <int D>
static int launch_decode_d(DecodeIdxParams& p, cudaStream_t st) {
  if (p.hist) {
    switch (p.H / 8) {
      case 1: return launch_decode_nt<D, 1, true>(p, st);
      case 2: return launch_decode_nt<D, 2, true>(p, st);
      case 4: return launch_decode_nt<D, 4, true>(p, st);
      case 8: return launch_decode_nt<D, 8, true>(p, st);
    }
  }
  switch (p.H / 8) {
    case 1: return launch_decode_nt<D, 1, false>(p, st);
    case 2: return launch_decode_nt<D, 2, false>(p, st);
    case 4: return launch_decode_nt<D, 4, false>(p, st);
    case 8: return launch_decode_nt<D, 8, false>(p, st);
  }
  return fail(MXB_ERR_UNSUPPORTED, "decode indexer: head count %d is not 8, 16, 32 or 64", p.H);
}

bool indexer_decode_eligible(const mxb_indexer_scores_args* a) {
  const bool q16 = a->q_dtype == MXB_F16 || a->q_dtype == MXB_BF16;
  // the scan applies no causal row mask: a single-token call that asks for one (ratio > 0) goes to the tiled
  // kernel, which reads the per-token visibility table
  return a->T == 1 && a->ratio == 0 && a->B <= kDecMaxBatch && a->key_dtype == MXB_F8E4M3 && q16 &&
         (a->H == 8 || a->H == 16 || a->H == 32 || a->H == 64) &&
         !(a->flags & (MXB_INDEXER_EXACT_FP32 | MXB_INDEXER_FP8_MMA));
}

int launch_indexer_decode(const mxb_indexer_scores_args* a, cudaStream_t st) {
  DecodeIdxParams p{};
  p.keys = reinterpret_cast<const uint8_t*>(a->keys);
  p.q = a->q; p.q_is_bf16 = a->q_dtype == MXB_BF16; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h;
  p.q_vec = (reinterpret_cast<uintptr_t>(a->q) & 15) == 0 && a->q_stride_b % 8 == 0 && a->q_stride_h % 8 == 0;
  p.weights = a->weights; p.scores = a->scores; p.s_sb = a->score_stride_b;
  p.row_start = a->row_start; p.row_count = a->row_count; p.B = a->B; p.H = a->H; p.n_rows = a->n_rows;
  p.hist = a->digit_hist;
  if (a->D == 64) return launch_decode_d<64>(p, st);
  return launch_decode_d<128>(p, st);
}

}  // namespace mxb
