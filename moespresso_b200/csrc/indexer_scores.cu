// Indexer score:  scores[b,t,r] = sum_h w[b,t,h] * relu(q[b,h,t,:] . key[b][r,:])
//
// This file holds the entry point, its dispatch and the exact kernel:
//  * indexer_exact_kernel — fp32 FMA on CUDA cores in a fixed order, for fp32
//    operands (1e-5 agreement with a float64 evaluation) and as the explicit
//    MXB_INDEXER_EXACT_FP32 mode for any operand type.
// The tensor-core kernels live beside it: indexer_decode.cu (one token per sequence, FP8 keys,
// warp-level MMA straight from global memory) and indexer_scores_fp8.cu (token tiles, FP8 or
// 16-bit keys, warp-specialised tcgen05 pipeline).  In all of them a row's score is a fixed-order
// sum over heads, so it does not depend on how rows are partitioned over CTAs or GPUs.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace mxb {

struct IndexerParams {
  const void* q;
  int64_t q_sb, q_sh, q_st;
  const void* keys;
  const float* weights;
  float* scores;
  int64_t s_sb, s_st;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t B, T, H;
  int64_t n_rows;
  int64_t pos0;
  int32_t ratio;
  int32_t t_tile;        // tokens per CTA
  int32_t* status;
};

__device__ __forceinline__ int64_t visible_rows(int64_t pos0, int tok, int ratio, int64_t count) {
  if (ratio <= 0) return count;
  int64_t v = (pos0 + tok + 1) / ratio;
  return v < count ? v : count;
}

// --------------------------------------------------------------------------
// exact fp32 kernel
// --------------------------------------------------------------------------
template <int D, int QT, int KT>
__global__ void __launch_bounds__(128) indexer_exact_kernel(IndexerParams p) {
  extern __shared__ float q_s[];  // [t_tile][H][D]
  float* w_s = q_s + (size_t)p.t_tile * p.H * D;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * p.t_tile;
  const int64_t count = p.row_count ? (int64_t)p.row_count[b] : p.n_rows;
  const int64_t rbase = p.row_start ? p.row_start[b] : (int64_t)b * p.n_rows;
  const int64_t r = (int64_t)blockIdx.x * 128 + threadIdx.x;
  if ((int64_t)blockIdx.x * 128 >= count) return;

  const int nt = min(p.t_tile, p.T - t0);
  for (int i = threadIdx.x; i < nt * p.H * D; i += 128) {
    int d = i % D, h = (i / D) % p.H, t = i / (D * p.H);
    q_s[i] = load_elem<QT>(p.q, (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)(t0 + t) * p.q_st + d);
  }
  for (int i = threadIdx.x; i < nt * p.H; i += 128)
    w_s[i] = p.weights[((int64_t)b * p.T + t0 + i / p.H) * p.H + i % p.H];
  __syncthreads();
  if (r >= count) return;

  float kreg[D];
  {
    const char* kp = reinterpret_cast<const char*>(p.keys) + (rbase + r) * (int64_t)D * ElemBytes<KT>::v;
    constexpr int EPV = 16 / ElemBytes<KT>::v;
#pragma unroll
    for (int c = 0; c < D / EPV; ++c) {
      uint4 v = __ldg(reinterpret_cast<const uint4*>(kp) + c);
      unpack16<KT>(v, &kreg[c * EPV]);
    }
  }
  const int64_t sbase = (p.row_start ? p.row_start[b] : 0) + (int64_t)b * p.s_sb;
  for (int t = 0; t < nt; ++t) {
    float acc = 0.f;
    for (int h = 0; h < p.H; ++h) {
      const float4* qv = reinterpret_cast<const float4*>(q_s + ((size_t)t * p.H + h) * D);
      float dot = 0.f;
#pragma unroll
      for (int c = 0; c < D / 4; ++c) {
        float4 x = qv[c];
        dot = fmaf(kreg[4 * c + 0], x.x, dot);
        dot = fmaf(kreg[4 * c + 1], x.y, dot);
        dot = fmaf(kreg[4 * c + 2], x.z, dot);
        dot = fmaf(kreg[4 * c + 3], x.w, dot);
      }
      acc = fmaf(w_s[t * p.H + h], fmaxf(dot, 0.f), acc);
    }
    const int tok = t0 + t;
    const bool vis = r < visible_rows(p.pos0, tok, p.ratio, count);
    p.scores[sbase + (int64_t)tok * p.s_st + r] = vis ? acc : -INFINITY;
  }
}

// --------------------------------------------------------------------------
// host
// --------------------------------------------------------------------------
template <int D, int QT, int KT>
static int launch_exact(IndexerParams& p, cudaStream_t st) {
  int t_tile = (int)(8192 / ((int64_t)p.H * D));
  if (t_tile < 1) t_tile = 1;
  if (t_tile > p.T) t_tile = p.T;
  p.t_tile = t_tile;
  size_t smem = (size_t)t_tile * p.H * D * 4 + (size_t)t_tile * p.H * 4;
  auto kern = indexer_exact_kernel<D, QT, KT>;
  if (smem > 48 * 1024) MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid((unsigned)ceil_div(p.n_rows, 128), (unsigned)ceil_div(p.T, t_tile), (unsigned)p.B);
  kern<<<grid, 128, smem, st>>>(p);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

template <int D>
static int dispatch_exact(IndexerParams& p, int qt, int kt, cudaStream_t st) {
#define MXB_EX(QT, KT) \
  if (qt == QT && kt == KT) return launch_exact<D, QT, KT>(p, st);
  MXB_EX(MXB_F32, MXB_F32)
  MXB_EX(MXB_F32, MXB_F16)
  MXB_EX(MXB_F32, MXB_BF16)
  MXB_EX(MXB_F16, MXB_F16)
  MXB_EX(MXB_F16, MXB_F32)
  MXB_EX(MXB_F16, MXB_F8E4M3)
  MXB_EX(MXB_BF16, MXB_BF16)
  MXB_EX(MXB_BF16, MXB_F32)
  MXB_EX(MXB_BF16, MXB_F8E4M3)
  MXB_EX(MXB_F32, MXB_F8E4M3)
#undef MXB_EX
  return fail(MXB_ERR_UNSUPPORTED, "indexer scores: unsupported q/key dtype pair (%d, %d)", qt, kt);
}

int launch_indexer_fp8(const mxb_indexer_scores_args* a, cudaStream_t st);  // indexer_scores_fp8.cu
bool indexer_decode_eligible(const mxb_indexer_scores_args* a);                // indexer_decode.cu
int launch_indexer_decode(const mxb_indexer_scores_args* a, cudaStream_t st);

}  // namespace mxb

using namespace mxb;

extern "C" int mxb_indexer_scores(const mxb_indexer_scores_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "indexer scores: null args");
  MXB_REQUIRE(a->B > 0 && a->T > 0, MXB_ERR_INVALID, "q must contain at least one batch and token");
  MXB_REQUIRE(a->D == 64 || a->D == 128, MXB_ERR_INVALID, "indexer score requires head_dim=64 or head_dim=128");
  MXB_REQUIRE(a->H >= 1 && a->H <= 64, MXB_ERR_INVALID, "indexer score requires between 1 and 64 heads");
  MXB_REQUIRE(a->n_rows > 0, MXB_ERR_INVALID, "index_comp must contain at least one compressed row");
  MXB_REQUIRE(a->q && a->keys && a->weights && a->scores, MXB_ERR_INVALID, "indexer scores: null tensor");
  MXB_REQUIRE(a->ratio >= 0, MXB_ERR_INVALID, "ratio must be non-negative");
  MXB_REQUIRE((reinterpret_cast<uintptr_t>(a->keys) & 15) == 0, MXB_ERR_INVALID, "keys must be 16-byte aligned");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);

  IndexerParams p{};
  p.q = a->q; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h; p.q_st = a->q_stride_t;
  p.keys = a->keys; p.weights = a->weights; p.scores = a->scores;
  p.s_sb = a->score_stride_b; p.s_st = a->score_stride_t;
  p.row_start = a->row_start; p.row_count = a->row_count;
  p.B = a->B; p.T = a->T; p.H = a->H; p.n_rows = a->n_rows;
  p.pos0 = a->pos0; p.ratio = a->ratio; p.status = a->status;

  if (indexer_decode_eligible(a)) return launch_indexer_decode(a, st);
  MXB_REQUIRE(a->digit_hist == nullptr, MXB_ERR_UNSUPPORTED,
              "indexer scores: digit_hist needs the decode scan (one token, ratio 0, FP8 keys, 16-bit q, 8/16/32/64 heads)");
  const bool q16 = a->q_dtype == MXB_F16 || a->q_dtype == MXB_BF16;
  const bool keys_match = a->key_dtype == a->q_dtype || a->key_dtype == MXB_F8E4M3;
  const bool q_vec_ok = (reinterpret_cast<uintptr_t>(a->q) & 15) == 0 && a->q_stride_b % 8 == 0 &&
                        a->q_stride_h % 8 == 0 && a->q_stride_t % 8 == 0;
  const bool tc = !(a->flags & MXB_INDEXER_EXACT_FP32) && q16 && keys_match && q_vec_ok && (a->H % 16 == 0);
  if (tc) return launch_indexer_fp8(a, st);
  if (a->D == 64) return dispatch_exact<64>(p, a->q_dtype, a->key_dtype, st);
  return dispatch_exact<128>(p, a->q_dtype, a->key_dtype, st);
}
