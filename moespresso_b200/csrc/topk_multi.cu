// Exact top-k for long rows, several CTAs per row.
//
// A decode batch has few rows (one per sequence) but each is long, so one CTA per row leaves
// most SMs idle and is bound by the instruction rate of a single SM.  Three launches:
//   topk_mhist    grid (parts, rows): 11-bit histogram of the part in shared memory, merged
//                 into the row's global histogram;
//   topk_mfilter  grid (parts, rows): threshold bin from the global histogram, then
//                 strictly-above ids -> above_idx[row], threshold-bin candidates -> cand[row]
//                 (keys of a sweep live in registers; one block scan and one global atomic per class per sweep);
//   topk_mfinish  grid (rows): remaining 21 bits and the ties (lowest id first) among the
//                 candidates, then an id BITMAP in shared memory turns the unordered set
//                 into ascending output by a prefix scan of popcounts (no sort).
// Every loop that contains a warp-wide vote has a trip count that is uniform over the CTA.
#include "common.cuh"
#include "topk_common.cuh"

namespace mxb {

constexpr int kMThreads = 512;
constexpr int kMUnroll = 8;
constexpr int kFilterRegs = 32;                // keys per thread per sweep of the filter kernel
constexpr int kFinishCandSmem = 12288;        // candidate pairs kept in shared memory by the finish kernel
constexpr int64_t kBitmapMaxN = 1 << 20;      // 128 KB bitmap

struct TopkMultiParams {
  const float* scores;
  int64_t row_stride;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t* out_ids;
  int32_t rows;
  int64_t n;
  int32_t k;
  int64_t part;          // elements per CTA in the first two kernels (multiple of kMThreads * kMUnroll)
  uint32_t* hist;        // [rows][2048]
  uint32_t* counters;    // [rows][4]: above, candidates
  int32_t* above_idx;    // [rows][k]
  uint32_t* cand_key;    // [rows][n]
  int32_t* cand_idx;     // [rows][n]
};

__global__ void __launch_bounds__(kMThreads) topk_mhist_kernel(TopkMultiParams p) {
  __shared__ uint32_t hist[kBigBins];
  const int row = blockIdx.y, tid = threadIdx.x;
  const int64_t n = p.row_count ? min((int64_t)p.row_count[row], p.n) : p.n;
  const int64_t lo = (int64_t)blockIdx.x * p.part;
  if (lo >= n) return;
  const int64_t hi = min(lo + p.part, n);
  const float* src = p.scores + (p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride);
  for (int i = tid; i < kBigBins; i += kMThreads) hist[i] = 0;
  __syncthreads();
  for (int64_t i0 = lo; i0 < hi; i0 += kMThreads * kMUnroll) {
    float x[kMUnroll];
#pragma unroll
    for (int u = 0; u < kMUnroll; ++u) {
      const int64_t i = i0 + tid + u * kMThreads;
      x[u] = i < hi ? __ldg(src + i) : -INFINITY;
    }
#pragma unroll
    for (int u = 0; u < kMUnroll; ++u) {
      const uint32_t key = score_key_full(x[u]);
      if (key) atomicAdd(&hist[key >> 21], 1u);
    }
  }
  __syncthreads();
  uint32_t* g = p.hist + (int64_t)row * kBigBins;
  for (int i = tid; i < kBigBins; i += kMThreads)
    if (hist[i]) atomicAdd(&g[i], hist[i]);
}

#ifdef MXB_TRACE_MF
#define TRF(k) do { if (threadIdx.x == 0 && blockIdx.x == 0 && blockIdx.y == 0) reinterpret_cast<long long*>(p.cand_idx + p.n - 64)[k] = clock64(); } while (0)
#else
#define TRF(k)
#endif

__global__ void __launch_bounds__(kMThreads) topk_mfilter_kernel(TopkMultiParams p) {
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_total, s_thr[4], s_base[2];
  const int row = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  const int64_t n = p.row_count ? min((int64_t)p.row_count[row], p.n) : p.n;
  const int64_t lo = (int64_t)blockIdx.x * p.part;
  if (lo >= n) return;
  const int64_t hi = min(lo + p.part, n);
  const float* src = p.scores + (p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride);
  TRF(0);
  if (tid < 4) s_thr[tid] = 0;
  __syncthreads();
  row_threshold(p.hist + (int64_t)row * kBigBins, p.k, warp_sums, &s_total, s_thr);
  TRF(1);
  if (s_thr[0] == 0) return;
  const uint32_t bin = s_thr[1];
  uint32_t* cnt = p.counters + (int64_t)row * 4;
  int32_t* ab = p.above_idx + (int64_t)row * p.k;
  uint32_t* ck = p.cand_key + (int64_t)row * p.n;
  int32_t* ci = p.cand_idx + (int64_t)row * p.n;
  // Sweeps of kMThreads * kFilterRegs elements held in registers: count this thread's hits, one block
  // scan, ONE global atomic per class per sweep (same-address atomics serialise in L2), then write.
  (void)lane;
  for (int64_t i0 = lo; i0 < hi; i0 += (int64_t)kMThreads * kFilterRegs) {
    uint32_t key[kFilterRegs];
#pragma unroll
    for (int u = 0; u < kFilterRegs; ++u) {
      const int64_t i = i0 + tid + (int64_t)u * kMThreads;
      key[u] = i < hi ? score_key_full(__ldg(src + i)) : 0u;
    }
    TRF(2);
    uint32_t na = 0, nc = 0;
#pragma unroll
    for (int u = 0; u < kFilterRegs; ++u) {
      const uint32_t kb = key[u] >> 21;
      na += (key[u] != 0 && kb > bin);
      nc += (key[u] != 0 && kb == bin);
    }
    TRF(3);
    uint32_t pa = block_excl_scan(na, warp_sums, &s_total);
    if (tid == 0) s_base[0] = s_total ? atomicAdd(&cnt[0], s_total) : 0u;
    uint32_t pc = block_excl_scan(nc, warp_sums, &s_total);
    if (tid == 0) s_base[1] = s_total ? atomicAdd(&cnt[1], s_total) : 0u;
    __syncthreads();
    pa += s_base[0];
    pc += s_base[1];
    TRF(4);
#pragma unroll
    for (int u = 0; u < kFilterRegs; ++u) {
      const uint32_t kb = key[u] >> 21;
      const int32_t id = (int32_t)(i0 + tid + (int64_t)u * kMThreads);
      if (key[u] != 0 && kb > bin) {
        if (pa < (uint32_t)p.k) ab[pa] = id;
        ++pa;
      } else if (key[u] != 0 && kb == bin) {
        ck[pc] = key[u];
        ci[pc] = id;
        ++pc;
      }
    }
    __syncthreads();
    TRF(5);
  }
}

// One CTA (1024 threads) per row.
__global__ void __launch_bounds__(1024) topk_mfinish_kernel(TopkMultiParams p, int use_bitmap, int sort_n) {
  extern __shared__ uint32_t dyn[];
  // layout: [bitmap words or sort buffer][cand keys][cand ids]
  const int64_t n = p.row_count ? min((int64_t)p.row_count[blockIdx.x], p.n) : p.n;
  const int words = use_bitmap ? (int)((p.n + 31) / 32) : sort_n;
  uint32_t* bitmap = dyn;
  uint32_t* ck_s = dyn + words;
  int32_t* ci_s = reinterpret_cast<int32_t*>(ck_s + kFinishCandSmem);
  __shared__ uint32_t hist[256];
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_total, s_thr[4], s_digit, s_dabove, s_cnt;

  const int row = blockIdx.x, tid = threadIdx.x;
  int32_t* out = p.out_ids + (int64_t)row * p.k;
  if (tid < 4) s_thr[tid] = 0;
  if (tid == 0) s_cnt = 0;
  __syncthreads();
  row_threshold(p.hist + (int64_t)row * kBigBins, p.k, warp_sums, &s_total, s_thr);
  const uint32_t k_eff = s_thr[0];
  for (int i = tid + (int)k_eff; i < p.k; i += 1024) out[i] = -1;
  if (k_eff == 0 || n <= 0) return;
  const uint32_t bin = s_thr[1], n_above = s_thr[2], C = s_thr[3];
  const int32_t* ab = p.above_idx + (int64_t)row * p.k;
  const uint32_t* ck = p.cand_key + (int64_t)row * p.n;
  const int32_t* ci = p.cand_idx + (int64_t)row * p.n;
  if (C <= (uint32_t)kFinishCandSmem) {   // stage the candidates once
    for (uint32_t i = tid; i < C; i += 1024) {
      ck_s[i] = ck[i];
      ci_s[i] = ci[i];
    }
    ck = ck_s;
    ci = ci_s;
  }
  for (int i = tid; i < words; i += 1024) bitmap[i] = use_bitmap ? 0u : 0x7FFFFFFFu;
  __syncthreads();

  // ---- the `want` largest among the candidates on the low 21 bits (8 + 8 + 5)
  uint32_t want = k_eff - n_above;
  uint32_t prefix = bin << 21, prefix_mask = 0xFFE00000u;
  const int shifts[3] = {13, 5, 0};
  const uint32_t widths[3] = {255u, 255u, 31u};
  for (int ps = 0; ps < 3; ++ps) {
    if (tid < 256) hist[tid] = 0;
    __syncthreads();
    for (uint32_t i = tid; i < C; i += 1024) {
      const uint32_t key = ck[i];
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
  const uint32_t thr = prefix, need = want;
  // ---- ties: the need-th smallest id among candidates with key == thr
  {
    uint32_t nt = 0;
    for (uint32_t i = tid; i < C; i += 1024) nt += ck[i] == thr;
    nt = __reduce_add_sync(0xffffffffu, nt);
    if ((tid & 31) == 0 && nt) atomicAdd(&s_cnt, nt);
  }
  __syncthreads();
  uint32_t idx_thr = 0xFFFFFFFFu;
  if (s_cnt > need) {
    uint32_t ipre = 0, imask = 0, iwant = need;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (uint32_t i = tid; i < C; i += 1024) {
        if (ck[i] == thr) {
          const uint32_t v = ~(uint32_t)ci[i];
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
    idx_thr = ~ipre;
  }
  if (tid == 0) s_cnt = 0;
  __syncthreads();

  if (use_bitmap) {
    // ---- mark the selected ids, then emit them in ascending order by a scan of popcounts
    for (uint32_t i = tid; i < n_above; i += 1024) {
      const uint32_t id = (uint32_t)ab[i];
      atomicOr(&bitmap[id >> 5], 1u << (id & 31));
    }
    for (uint32_t i = tid; i < C; i += 1024) {
      const uint32_t key = ck[i];
      const uint32_t id = (uint32_t)ci[i];
      if (key > thr || (key == thr && id <= idx_thr)) atomicOr(&bitmap[id >> 5], 1u << (id & 31));
    }
    __syncthreads();
    const int per = (words + 1023) / 1024;
    const int w0 = min(tid * per, words), w1 = min(w0 + per, words);
    uint32_t cntw = 0;
    for (int w = w0; w < w1; ++w) cntw += __popc(bitmap[w]);
    uint32_t pos = block_excl_scan(cntw, warp_sums, &s_total);
    for (int w = w0; w < w1; ++w) {
      uint32_t bits = bitmap[w];
      while (bits) {
        const int bpos = __ffs(bits) - 1;
        bits &= bits - 1;
        if (pos < k_eff) out[pos] = w * 32 + bpos;
        ++pos;
      }
    }
  } else {
    // ---- rows too long for a bitmap: gather and bitonic-sort the ids
    int32_t* sel = reinterpret_cast<int32_t*>(bitmap);
    for (uint32_t i = tid; i < n_above; i += 1024) sel[i] = ab[i];
    for (uint32_t i = tid; i < C; i += 1024) {
      const uint32_t key = ck[i];
      const int32_t id = ci[i];
      if (key > thr || (key == thr && (uint32_t)id <= idx_thr)) {
        const uint32_t q = atomicAdd(&s_cnt, 1u);
        if (n_above + q < (uint32_t)sort_n) sel[n_above + q] = id;
      }
    }
    __syncthreads();
    for (int size = 2; size <= sort_n; size <<= 1) {
      for (int stride = size >> 1; stride > 0; stride >>= 1) {
        for (int i = tid; i < sort_n / 2; i += 1024) {
          const int a = 2 * i - (i & (stride - 1));
          const int b = a + stride;
          const bool up = ((a & size) == 0);
          const int32_t x = sel[a], y = sel[b];
          if ((x > y) == up) { sel[a] = y; sel[b] = x; }
        }
        __syncthreads();
      }
    }
    for (uint32_t i = tid; i < k_eff; i += 1024) out[i] = sel[i];
  }
}

static void multi_layout(int32_t rows, int64_t n, int32_t k, size_t* off /*[5]*/, size_t* zero_bytes, size_t* total) {
  size_t o = 0;
  off[0] = o; o += (size_t)rows * kBigBins * 4;                 // hist
  off[1] = o; o += (size_t)rows * 4 * 4;                        // counters
  o = (size_t)round_up((int64_t)o, 256);
  *zero_bytes = o;
  off[2] = o; o += (size_t)rows * (size_t)k * 4;                // above ids
  o = (size_t)round_up((int64_t)o, 256);
  off[3] = o; o += (size_t)rows * (size_t)n * 4;                // candidate keys
  o = (size_t)round_up((int64_t)o, 256);
  off[4] = o; o += (size_t)rows * (size_t)n * 4;                // candidate ids
  *total = (size_t)round_up((int64_t)o, 256);
}

int64_t topk_multi_workspace(int32_t rows, int64_t n, int32_t k) {
  size_t off[5], zb, total;
  multi_layout(rows, n, k, off, &zb, &total);
  return (int64_t)total;
}

int launch_topk_multi(const mxb_topk_args* a, cudaStream_t st) {
  size_t off[5], zb, total;
  multi_layout(a->rows, a->n, a->k, off, &zb, &total);
  MXB_REQUIRE(a->workspace != nullptr && a->workspace_bytes >= (int64_t)total, MXB_ERR_WORKSPACE,
              "topk: workspace of %lld bytes required", (long long)total);
  char* ws = reinterpret_cast<char*>(a->workspace);
  TopkMultiParams p{};
  p.scores = a->scores; p.row_stride = a->row_stride; p.row_start = a->row_start; p.row_count = a->row_count;
  p.out_ids = a->out_ids; p.rows = a->rows; p.n = a->n; p.k = a->k;
  p.hist = reinterpret_cast<uint32_t*>(ws + off[0]);
  p.counters = reinterpret_cast<uint32_t*>(ws + off[1]);
  p.above_idx = reinterpret_cast<int32_t*>(ws + off[2]);
  p.cand_key = reinterpret_cast<uint32_t*>(ws + off[3]);
  p.cand_idx = reinterpret_cast<int32_t*>(ws + off[4]);
  // parts per row: about two CTAs per SM in total, each at least one full unrolled sweep
  const int64_t unit = (int64_t)kMThreads * kMUnroll;
  int64_t parts = ceil_div(2 * (int64_t)sm_count(), a->rows);
  const int64_t max_parts = ceil_div(a->n, unit);
  if (parts > max_parts) parts = max_parts;
  if (parts < 1) parts = 1;
  p.part = round_up(ceil_div(a->n, parts), unit);
  parts = ceil_div(a->n, p.part);
  MXB_CUDA_OK(cudaMemsetAsync(ws, 0, zb, st));
  dim3 grid((unsigned)parts, (unsigned)a->rows);
  topk_mhist_kernel<<<grid, kMThreads, 0, st>>>(p);
  MXB_CUDA_OK(cudaGetLastError());
  topk_mfilter_kernel<<<grid, kMThreads, 0, st>>>(p);
  MXB_CUDA_OK(cudaGetLastError());
  const int use_bitmap = a->n <= kBitmapMaxN ? 1 : 0;
  int sort_n = 2;
  while (sort_n < a->k) sort_n <<= 1;
  const size_t words = use_bitmap ? (size_t)((a->n + 31) / 32) : (size_t)sort_n;
  const size_t smem = words * 4 + (size_t)kFinishCandSmem * 8;
  MXB_CUDA_OK(cudaFuncSetAttribute(topk_mfinish_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  topk_mfinish_kernel<<<a->rows, 1024, smem, st>>>(p, use_bitmap, sort_n);
  note_launch(3);
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

}  // namespace mxb
