// Exact top-k selection on fp32 score rows (radix select on monotone keys).
//
// key(x): -0 -> +0, then bits ^ 0xFFFFFFFF for negatives, bits | 0x80000000 otherwise,
// so unsigned key order == float order.  Non-finite scores (-inf, +inf, NaN) map to key 0 =
// "never selected", as the NumPy contract keeps only finite scores.
// Selected set: every row with key > T, plus the `need` LOWEST-index rows with
// key == T, where T is the k-th largest key.  Output ids ascending, -1 padded.
//
//  * topk_row_kernel      — one CTA per row, the row's keys resident in shared memory
//    (rows up to kSmemRowMax); four 8-bit radix passes, then an ordered emission
//    through a block scan, so the output is ascending without a sort.
//  * topk_hist / filter / finish — rows longer than that (up to 2^31 - 1): an 11-bit
//    histogram pass over all CTAs, a filter pass that emits the strictly-above
//    rows and compacts the threshold bin's candidates, and a one-CTA finish that
//    resolves the remaining 21 bits, the ties by lowest index, and sorts the ids.
#include "common.cuh"

namespace mxb {

constexpr int kSmemRowMax = 45056;  // 176 KB of keys
constexpr int kBigBins = 2048;      // top 11 bits
constexpr int kBigChunk = 16384;    // elements per CTA in the multi-CTA passes

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

struct TopkParams {
  const float* scores;
  int64_t row_stride;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t* out_ids;
  int32_t rows;
  int64_t n;
  int32_t k;
  // multi-CTA path scratch
  uint32_t* hist;      // [rows][kBigBins]
  uint32_t* counters;  // [rows][4]: above count, candidate count
  uint32_t* cand_key;  // [rows][n]
  int32_t* cand_idx;   // [rows][n]
  int32_t* above_idx;  // [rows][k]
};

// --------------------------------------------------------------------------
// one CTA per row, keys in shared memory
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) topk_row_kernel(TopkParams p) {
  extern __shared__ uint32_t keys[];  // [n]
  __shared__ uint32_t hist[256];
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_digit, s_above, s_total, s_total2, s_nvalid;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t base = p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride;
  int n = (int)(p.row_count ? min((int64_t)p.row_count[row], p.n) : p.n);
  if (n < 0) n = 0;
  const float* src = p.scores + base;
  int32_t* out = p.out_ids + (int64_t)row * p.k;

  if (tid == 0) s_nvalid = 0;
  __syncthreads();
  uint32_t nv = 0;
  for (int i = tid; i < n; i += blockDim.x) {
    uint32_t key = score_key_full(src[i]);
    keys[i] = key;
    nv += key != 0;
  }
  nv = __reduce_add_sync(0xffffffffu, nv);
  if ((tid & 31) == 0 && nv) atomicAdd(&s_nvalid, nv);
  __syncthreads();
  const uint32_t k_eff = min((uint32_t)p.k, s_nvalid);
  for (int i = tid + (int)k_eff; i < p.k; i += blockDim.x) out[i] = -1;
  if (k_eff == 0) return;

  uint32_t prefix = 0, prefix_mask = 0, want = k_eff;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
      uint32_t key = keys[i];
      if (key != 0 && (key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid < 32) pick_digit_256(hist, want, &s_digit, &s_above);
    __syncthreads();
    prefix |= s_digit << shift;
    prefix_mask |= 255u << shift;
    want -= s_above;
    __syncthreads();
  }
  const uint32_t thr = prefix;
  const uint32_t need = want;  // ties to take, >= 1

  // ordered emission: thread t owns the contiguous slice [t*per, (t+1)*per)
  const int per = (n + (int)blockDim.x - 1) / (int)blockDim.x;
  const int lo = min(tid * per, n), hi = min(lo + per, n);
  uint32_t ca = 0, ct = 0;
  for (int i = lo; i < hi; ++i) {
    uint32_t key = keys[i];
    ca += key > thr;
    ct += key == thr;
  }
  uint32_t base_a = block_excl_scan(ca, warp_sums, &s_total);
  uint32_t base_t = block_excl_scan(ct, warp_sums, &s_total2);
  for (int i = lo; i < hi; ++i) {
    uint32_t key = keys[i];
    if (key > thr) {
      out[base_a + min(base_t, need)] = i;
      ++base_a;
    } else if (key == thr) {
      if (base_t < need) out[base_a + base_t] = i;
      ++base_t;
    }
  }
}

// --------------------------------------------------------------------------
// long rows: histogram -> filter -> finish
// --------------------------------------------------------------------------
__global__ void __launch_bounds__(512) topk_hist_kernel(TopkParams p) {
  __shared__ uint32_t hist[kBigBins];
  const int row = blockIdx.y;
  const int64_t n = p.row_count ? min((int64_t)p.row_count[row], p.n) : p.n;
  const int64_t lo = (int64_t)blockIdx.x * kBigChunk;
  if (lo >= n) return;
  const int64_t hi = min(lo + kBigChunk, n);
  const int64_t base = p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride;
  for (int i = threadIdx.x; i < kBigBins; i += blockDim.x) hist[i] = 0;
  __syncthreads();
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    uint32_t key = score_key_full(p.scores[base + i]);
    if (key) atomicAdd(&hist[key >> 21], 1u);
  }
  __syncthreads();
  uint32_t* g = p.hist + (int64_t)row * kBigBins;
  for (int i = threadIdx.x; i < kBigBins; i += blockDim.x)
    if (hist[i]) atomicAdd(&g[i], hist[i]);
}

// Threshold bin of a row from its global 2048-bin histogram.  Executed by the whole CTA
// (>= 256 threads).  Outputs through shared memory: k_eff, thr_bin, count above the bin.
__device__ __forceinline__ void big_threshold(const uint32_t* g, int k, uint32_t* sh /*[260]*/, uint32_t* k_eff,
                                              uint32_t* thr_bin, uint32_t* above) {
  const int tid = threadIdx.x;
  // thread t (< 256) sums bins [2047-8t-7, 2047-8t], highest first
  uint32_t loc[8];
  uint32_t s = 0;
  if (tid < 256) {
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      loc[j] = g[2047 - (tid * 8 + j)];
      s += loc[j];
    }
    sh[tid] = s;
  }
  __syncthreads();
  // inclusive scan over 256 entries (Hillis-Steele, in place with double sync)
  for (int o = 1; o < 256; o <<= 1) {
    uint32_t t = 0;
    if (tid < 256 && tid >= o) t = sh[tid - o];
    __syncthreads();
    if (tid < 256) sh[tid] += t;
    __syncthreads();
  }
  const uint32_t total = sh[255];
  const uint32_t ke = min((uint32_t)k, total);
  if (tid == 0) {
    *k_eff = ke;
    *thr_bin = 0;
    *above = 0;
  }
  __syncthreads();
  if (tid < 256 && ke > 0) {
    const uint32_t incl = sh[tid], excl = incl - s;
    if (excl < ke && incl >= ke) {
      uint32_t run = excl;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        if (run + loc[j] >= ke) {
          *thr_bin = 2047 - (tid * 8 + j);
          *above = run;
          break;
        }
        run += loc[j];
      }
    }
  }
  __syncthreads();
}

__global__ void __launch_bounds__(512) topk_filter_kernel(TopkParams p) {
  __shared__ uint32_t sh[260];
  __shared__ uint32_t s_keff, s_bin, s_above;
  const int row = blockIdx.y;
  const int64_t n = p.row_count ? min((int64_t)p.row_count[row], p.n) : p.n;
  const int64_t lo = (int64_t)blockIdx.x * kBigChunk;
  if (lo >= n) return;
  const int64_t hi = min(lo + kBigChunk, n);
  const int64_t base = p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride;
  big_threshold(p.hist + (int64_t)row * kBigBins, p.k, sh, &s_keff, &s_bin, &s_above);
  if (s_keff == 0) return;
  const uint32_t bin = s_bin;
  uint32_t* cnt = p.counters + (int64_t)row * 4;
  uint32_t* ck = p.cand_key + (int64_t)row * p.n;
  int32_t* ci = p.cand_idx + (int64_t)row * p.n;
  int32_t* ab = p.above_idx + (int64_t)row * p.k;
  for (int64_t i = lo + threadIdx.x; i < hi; i += blockDim.x) {
    uint32_t key = score_key_full(p.scores[base + i]);
    if (!key) continue;
    uint32_t kb = key >> 21;
    if (kb > bin) {
      uint32_t pos = atomicAdd(&cnt[0], 1u);
      if (pos < (uint32_t)p.k) ab[pos] = (int32_t)i;
    } else if (kb == bin) {
      uint32_t pos = atomicAdd(&cnt[1], 1u);
      ck[pos] = key;
      ci[pos] = (int32_t)i;
    }
  }
}

// One CTA per row: resolve the threshold inside the candidate bin, the ties, and sort.
__global__ void __launch_bounds__(1024) topk_finish_kernel(TopkParams p, int sort_n) {
  extern __shared__ int32_t sel[];  // [sort_n] ids to sort (padded with INT_MAX)
  __shared__ uint32_t sh[260];
  __shared__ uint32_t hist[256];
  __shared__ uint32_t s_keff, s_bin, s_above, s_digit, s_dabove, s_cnt;
  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  int32_t* out = p.out_ids + (int64_t)row * p.k;
  big_threshold(p.hist + (int64_t)row * kBigBins, p.k, sh, &s_keff, &s_bin, &s_above);
  const uint32_t k_eff = s_keff;
  for (int i = tid + (int)k_eff; i < p.k; i += blockDim.x) out[i] = -1;
  if (k_eff == 0) return;
  const uint32_t n_above = s_above;
  const uint32_t C = p.counters[(int64_t)row * 4 + 1];
  const uint32_t* ck = p.cand_key + (int64_t)row * p.n;
  const int32_t* ci = p.cand_idx + (int64_t)row * p.n;
  const int32_t* ab = p.above_idx + (int64_t)row * p.k;

  // radix select of the `want` largest among the C candidates on the low 21 bits (8+8+5)
  uint32_t want = k_eff - n_above;
  uint32_t prefix = s_bin << 21, prefix_mask = 0xFFE00000u;
  const int shifts[3] = {13, 5, 0};
  const uint32_t widths[3] = {255u, 255u, 31u};
  for (int ps = 0; ps < 3; ++ps) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < C; i += blockDim.x) {
      uint32_t key = ck[i];
      if ((key & prefix_mask) == prefix) atomicAdd(&hist[(key >> shifts[ps]) & widths[ps]], 1u);
    }
    __syncthreads();
    if (tid < 32) pick_digit_256(hist, want, &s_digit, &s_dabove);
    __syncthreads();
    prefix |= s_digit << shifts[ps];
    prefix_mask |= widths[ps] << shifts[ps];
    want -= s_dabove;
    __syncthreads();
  }
  const uint32_t thr = prefix;
  const uint32_t need = want;  // ties to take (lowest indices), >= 1

  // ties: find the need-th smallest index among candidates with key == thr (indices are unique)
  uint32_t ipre = 0, imask = 0, iwant = need;
  for (int shift = 24; shift >= 0; shift -= 8) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < C; i += blockDim.x) {
      if (ck[i] == thr) {
        uint32_t v = ~(uint32_t)ci[i];  // descending scan of ~idx == ascending idx
        if ((v & imask) == ipre) atomicAdd(&hist[(v >> shift) & 255u], 1u);
      }
    }
    __syncthreads();
    if (tid < 32) pick_digit_256(hist, iwant, &s_digit, &s_dabove);
    __syncthreads();
    ipre |= s_digit << shift;
    imask |= 255u << shift;
    iwant -= s_dabove;
    __syncthreads();
  }
  const uint32_t idx_thr = ~ipre;  // ties with idx <= idx_thr are taken

  if (tid == 0) s_cnt = 0;
  for (int i = tid; i < sort_n; i += blockDim.x) sel[i] = 0x7FFFFFFF;
  __syncthreads();
  for (uint32_t i = tid; i < n_above; i += blockDim.x) sel[i] = ab[i];
  for (uint32_t i = tid; i < C; i += blockDim.x) {
    uint32_t key = ck[i];
    int32_t id = ci[i];
    if (key > thr || (key == thr && (uint32_t)id <= idx_thr)) {
      uint32_t pos = atomicAdd(&s_cnt, 1u);
      if (n_above + pos < (uint32_t)sort_n) sel[n_above + pos] = id;
    }
  }
  __syncthreads();
  // bitonic sort ascending
  for (int size = 2; size <= sort_n; size <<= 1) {
    for (int stride = size >> 1; stride > 0; stride >>= 1) {
      for (int i = tid; i < sort_n / 2; i += blockDim.x) {
        int a = 2 * i - (i & (stride - 1));
        int b = a + stride;
        bool up = ((a & size) == 0);
        int32_t x = sel[a], y = sel[b];
        if ((x > y) == up) {
          sel[a] = y;
          sel[b] = x;
        }
      }
      __syncthreads();
    }
  }
  for (uint32_t i = tid; i < k_eff; i += blockDim.x) out[i] = sel[i];
}

static void big_layout(int32_t rows, int64_t n, int32_t k, size_t* hist_off, size_t* cnt_off, size_t* ck_off,
                       size_t* ci_off, size_t* ab_off, size_t* total) {
  size_t o = 0;
  *hist_off = o; o += (size_t)rows * kBigBins * 4;
  *cnt_off = o;  o += (size_t)rows * 4 * 4;
  o = (size_t)round_up((int64_t)o, 256);
  *ck_off = o;   o += (size_t)rows * (size_t)n * 4;
  o = (size_t)round_up((int64_t)o, 256);
  *ci_off = o;   o += (size_t)rows * (size_t)n * 4;
  o = (size_t)round_up((int64_t)o, 256);
  *ab_off = o;   o += (size_t)rows * (size_t)k * 4;
  *total = (size_t)round_up((int64_t)o, 256);
}

}  // namespace mxb

using namespace mxb;

extern "C" int64_t mxb_topk_workspace_bytes(int32_t rows, int64_t n, int32_t k) {
  if (rows <= 0 || n <= 0 || k <= 0) return 0;
  if (n <= kSmemRowMax) return 0;
  size_t a, b, c, d, e, total;
  big_layout(rows, n, k, &a, &b, &c, &d, &e, &total);
  return (int64_t)total;
}

extern "C" int mxb_topk_select(const mxb_topk_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "topk: null args");
  MXB_REQUIRE(a->rows > 0 && a->n > 0, MXB_ERR_INVALID, "topk: scores must contain at least one row and column");
  MXB_REQUIRE(a->k >= 1 && a->k <= 8192, MXB_ERR_INVALID, "topk must be between 1 and 8192");
  MXB_REQUIRE(a->n < ((int64_t)1 << 31), MXB_ERR_INVALID, "topk: row length must be below 2^31");
  MXB_REQUIRE(a->scores && a->out_ids, MXB_ERR_INVALID, "topk: null tensor");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  TopkParams p{};
  p.scores = a->scores; p.row_stride = a->row_stride; p.row_start = a->row_start; p.row_count = a->row_count;
  p.out_ids = a->out_ids; p.rows = a->rows; p.n = a->n; p.k = a->k;

  if (a->n <= kSmemRowMax) {
    size_t smem = (size_t)a->n * 4;
    if (smem > 48 * 1024)
      MXB_CUDA_OK(cudaFuncSetAttribute(topk_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    int threads = a->n >= 8192 ? 1024 : (a->n >= 2048 ? 512 : 256);
    topk_row_kernel<<<a->rows, threads, smem, st>>>(p);
    MXB_CUDA_OK(cudaGetLastError());
    return MXB_OK;
  }

  size_t ho, co, cko, cio, abo, total;
  big_layout(a->rows, a->n, a->k, &ho, &co, &cko, &cio, &abo, &total);
  MXB_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= (int64_t)total, MXB_ERR_WORKSPACE,
              "topk: workspace of %lld bytes required", (long long)total);
  char* ws = reinterpret_cast<char*>(a->workspace);
  p.hist = reinterpret_cast<uint32_t*>(ws + ho);
  p.counters = reinterpret_cast<uint32_t*>(ws + co);
  p.cand_key = reinterpret_cast<uint32_t*>(ws + cko);
  p.cand_idx = reinterpret_cast<int32_t*>(ws + cio);
  p.above_idx = reinterpret_cast<int32_t*>(ws + abo);
  MXB_CUDA_OK(cudaMemsetAsync(ws, 0, cko, st));  // histograms + counters
  dim3 grid((unsigned)ceil_div(a->n, kBigChunk), (unsigned)a->rows);
  topk_hist_kernel<<<grid, 512, 0, st>>>(p);
  MXB_CUDA_OK(cudaGetLastError());
  topk_filter_kernel<<<grid, 512, 0, st>>>(p);
  MXB_CUDA_OK(cudaGetLastError());
  int sort_n = 2;
  while (sort_n < a->k) sort_n <<= 1;
  topk_finish_kernel<<<a->rows, 1024, (size_t)sort_n * 4, st>>>(p, sort_n);
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
