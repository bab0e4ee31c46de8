// Indexer score:  scores[b,t,r] = sum_h w[b,t,h] * relu(q[b,h,t,:] . key[b][r,:])
//
// Two kernels.
//  * indexer_tc_kernel   — 16-bit keys (bf16 / fp16, same type as q).  Key rows sit on the MMA
//    M axis (128 rows per tile, streamed by TMA), the (token, head) pairs of one token tile on N,
//    D = 64/128 on K.  tcgen05.mma accumulates in TMEM; the drain applies relu, the head weights
//    and the head sum in a fixed order, so a row's score does not depend on how rows are
//    partitioned over CTAs or GPUs.  FP8 key tables are handled by indexer_decode.cu (one token)
//    and indexer_scores_fp8.cu (token tiles).
//  * indexer_exact_kernel — fp32 FMA on CUDA cores in a fixed order, for fp32
//    operands (1e-5 agreement with a float64 evaluation) and as the explicit
//    MXB_INDEXER_EXACT_FP32 mode for any operand type.
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
  int32_t N;             // MMA N = round_up(t_tile * H, 16)
  int32_t rows_per_cta;  // multiple of 128
  int32_t tmem_cols;
  int32_t acc_stride;     // TMEM columns between the two accumulators
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
// tcgen05 kernel
// --------------------------------------------------------------------------
constexpr int kStages = 4;

template <int D>
struct TcSmem {
  static constexpr int kABytes = 128 * D * 2;               // one 16-bit operand tile
  static constexpr int a_off = 0;
  static constexpr int b_off = a_off + kStages * kABytes;   // q tile, up to 256 x D x 2
  static constexpr int w_off = b_off + 256 * D * 2;
  static constexpr int bar_off = w_off + 256 * 4;
  static constexpr int total = bar_off + 128;
};

template <int D>
__global__ void __launch_bounds__(128, 1) indexer_tc_kernel(const __grid_constant__ CUtensorMap tmap,
                                                            IndexerParams p, int q_is_bf16) {
  using L = TcSmem<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* a_buf = smem + L::a_off;
  uint8_t* b_buf = smem + L::b_off;
  float* w_s = reinterpret_cast<float*>(smem + L::w_off);
  uint64_t* full_bar = reinterpret_cast<uint64_t*>(smem + L::bar_off);  // [kStages]
  uint64_t* mma_bar = full_bar + kStages;                               // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(mma_bar + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x;
  const int warp = tid >> 5;
  const int b = blockIdx.z;
  const int t0 = blockIdx.y * p.t_tile;
  const int64_t count = p.row_count ? (int64_t)p.row_count[b] : p.n_rows;
  const int64_t rbase = p.row_start ? p.row_start[b] : (int64_t)b * p.n_rows;
  const int64_t row0 = (int64_t)blockIdx.x * p.rows_per_cta;
  if (row0 >= count) return;
  int64_t span = count - row0;
  if (span > p.rows_per_cta) span = p.rows_per_cta;
  const int ntiles = (int)((span + 127) / 128);
  const int nt = min(p.t_tile, p.T - t0);
  const int N = p.N;

  if (tid == 0) {
    for (int s = 0; s < kStages; ++s) ptx::mbar_init(&full_bar[s], 1);
    ptx::mbar_init(&mma_bar[0], 1);
    ptx::mbar_init(&mma_bar[1], 1);
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tmap);
  }
  __syncwarp();
  if (warp == 0) {
    ptx::tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
    ptx::tmem_relinquish();
  }

  // q tile -> B operand (K-major, 128-byte swizzle); weights -> smem
  {
    constexpr int CPR = D / 8;  // 16-byte chunks per row
    for (int i = tid; i < N * CPR; i += 128) {
      const int n = i / CPR, c = i % CPR;
      const int t = n / p.H, h = n % p.H;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t < nt) {
        const char* src = reinterpret_cast<const char*>(p.q) +
                          ((int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)(t0 + t) * p.q_st + c * 8) * 2;
        v = __ldg(reinterpret_cast<const uint4*>(src));
      }
      const int kb = c >> 3, cc = c & 7;
      *reinterpret_cast<uint4*>(b_buf + (size_t)kb * N * 128 + (size_t)n * 128 + ((cc ^ (n & 7)) << 4)) = v;
    }
    for (int i = tid; i < N; i += 128) {
      const int t = i / p.H, h = i % p.H;
      w_s[i] = (t < nt) ? p.weights[((int64_t)b * p.T + t0 + t) * p.H + h] : 0.f;
    }
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  constexpr uint32_t kTileTx = 128 * D * 2;
  auto issue_load = [&](int tile) {
    const int s = tile % kStages;
    ptx::mbar_expect_tx(&full_bar[s], kTileTx);
    const int32_t y = (int32_t)(rbase + row0 + (int64_t)tile * 128);
#pragma unroll
    for (int kb = 0; kb < D / 64; ++kb)
      ptx::tma_load_2d(a_buf + (size_t)s * L::kABytes + (size_t)kb * 16384, &tmap, &full_bar[s], kb * 64, y);
  };

  int issued = 0;
  if (tid == 0) {
    for (; issued < kStages && issued < ntiles; ++issued) issue_load(issued);
  }

  const uint32_t idesc = ptx::idesc_f16(q_is_bf16 ? ptx::kFmtBF16 : ptx::kFmtF16,
                                        q_is_bf16 ? ptx::kFmtBF16 : ptx::kFmtF16, 128, (uint32_t)N, 0, 0);
  const int64_t sbase = (p.row_start ? p.row_start[b] : 0) + (int64_t)b * p.s_sb;

  auto epilogue = [&](int tile) {
    const int acc = tile & 1;
    ptx::mbar_wait(&mma_bar[acc], (uint32_t)((tile >> 1) & 1), abort_flag);
    ptx::tc_fence_after_sync();
    // the operand stage of `tile` is free again: refill it
    if (tid == 0 && issued < ntiles && (issued % kStages) == (tile % kStages)) {
      issue_load(issued);
      ++issued;
    }
    const int64_t r = row0 + (int64_t)tile * 128 + tid;
    const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)(acc * p.acc_stride);
    for (int t = 0; t < nt; ++t) {
      float sum = 0.f;
      for (int c0 = 0; c0 < p.H; c0 += 16) {
        uint32_t v[16];
        ptx::tmem_ld16(taddr + (uint32_t)(t * p.H + c0), v);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int j = 0; j < 16; ++j)
          sum = fmaf(w_s[t * p.H + c0 + j], fmaxf(__uint_as_float(v[j]), 0.f), sum);
      }
      if (r < count) {
        const int tok = t0 + t;
        const bool vis = r < visible_rows(p.pos0, tok, p.ratio, count);
        p.scores[sbase + (int64_t)tok * p.s_st + r] = vis ? sum : -INFINITY;
      }
    }
    ptx::tc_fence_before_sync();
  };

  for (int i = 0; i < ntiles; ++i) {
    const int s = i % kStages;
    ptx::mbar_wait(&full_bar[s], (uint32_t)((i / kStages) & 1), abort_flag);
    uint8_t* a_tile = a_buf + (size_t)s * L::kABytes;
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (tid == 0) {
      ptx::tc_fence_after_sync();
      const uint32_t d_tmem = tmem_base + (uint32_t)((i & 1) * p.acc_stride);
      const uint32_t a_addr = ptx::smem_u32(a_tile);
      const uint32_t b_addr = ptx::smem_u32(b_buf);
#pragma unroll
      for (int kb = 0; kb < D / 64; ++kb) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          const uint64_t ad = ptx::smem_desc_sw128(a_addr + kb * 16384 + ks * 32, 16, 1024);
          const uint64_t bd = ptx::smem_desc_sw128(b_addr + kb * N * 128 + ks * 32, 16, 1024);
          ptx::mma_f16_ss(d_tmem, ad, bd, idesc, (kb | ks) ? 1u : 0u);
        }
      }
      ptx::mma_commit(&mma_bar[i & 1]);
    }
    if (i > 0) epilogue(i - 1);
  }
  epilogue(ntiles - 1);

  // abort path only: let outstanding TMA writes land before the CTA's smem is released
  if (*abort_flag && tid == 0) {
    for (int s = 0; s < kStages; ++s)
      for (uint32_t it = 0; it < (1u << 16); ++it)
        if (ptx::mbar_try_wait(&full_bar[s], 0) || ptx::mbar_try_wait(&full_bar[s], 1)) break;
  }
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
  if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
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

template <int D>
static int launch_tc(IndexerParams& p, const mxb_indexer_scores_args* a, cudaStream_t st) {
  using L = TcSmem<D>;
  int t_tile = 256 / p.H;
  if (t_tile > p.T) t_tile = p.T;
  p.t_tile = t_tile;
  p.N = (int)round_up((int64_t)t_tile * p.H, 16);
  p.acc_stride = (int)round_up(p.N, 32);
  int cols = 32;
  while (cols < 2 * p.acc_stride) cols <<= 1;
  p.tmem_cols = cols;
  // rows per CTA: enough CTAs to fill the machine a few times over, at least 8 tiles each when possible
  const int64_t t_tiles = ceil_div(p.T, t_tile);
  int64_t tiles = ceil_div(p.n_rows, 128);
  int64_t want_ctas = (int64_t)sm_count() * 6;
  int64_t per = ceil_div(tiles * p.B * t_tiles, want_ctas);
  if (per < 8) per = 8;
  if (per > tiles) per = tiles;
  p.rows_per_cta = (int)(per * 128);

  CUtensorMap tmap;
  uint64_t dims[2] = {(uint64_t)D, (uint64_t)a->rows_total};
  uint64_t strides[1] = {(uint64_t)D * 2};
  uint32_t box[2] = {64u, 128u};
  int rc = make_tensor_map(&tmap,
                           a->key_dtype == MXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                           2, a->keys, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  if (rc != MXB_OK) return rc;

  auto kern = indexer_tc_kernel<D>;
  const int smem = L::total + 1024;
  MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((unsigned)ceil_div(p.n_rows, p.rows_per_cta), (unsigned)t_tiles, (unsigned)p.B);
  kern<<<grid, 128, smem, st>>>(tmap, p, a->q_dtype == MXB_BF16 ? 1 : 0);
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
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
  const bool q16 = a->q_dtype == MXB_F16 || a->q_dtype == MXB_BF16;
  const bool keys_match = a->key_dtype == a->q_dtype || a->key_dtype == MXB_F8E4M3;
  const bool q_vec_ok = (reinterpret_cast<uintptr_t>(a->q) & 15) == 0 && a->q_stride_b % 8 == 0 &&
                        a->q_stride_h % 8 == 0 && a->q_stride_t % 8 == 0;
  const bool tc = !(a->flags & MXB_INDEXER_EXACT_FP32) && q16 && keys_match && q_vec_ok && (a->H % 16 == 0);
  if (tc) {
    const bool fp8 = a->key_dtype == MXB_F8E4M3;
    if (fp8 || !(a->flags & 4)) return launch_indexer_fp8(a, st);   // flag 4 (temporary): previous in-order kernel
    if (a->D == 64) return launch_tc<64>(p, a, st);
    return launch_tc<128>(p, a, st);
  }
  if (a->D == 64) return dispatch_exact<64>(p, a->q_dtype, a->key_dtype, st);
  return dispatch_exact<128>(p, a->q_dtype, a->key_dtype, st);
}
