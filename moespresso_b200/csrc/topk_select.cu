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
//  * topk_stream_kernel   — rows longer than that (up to 2^31 - 1): one CTA streams the
//    row twice from L2 (11-bit histogram, then strictly-above ids + the threshold bin's
//    candidates), resolves the remaining 21 bits and the ties by lowest index among the
//    candidates, and sorts the selected ids.
#include <mutex>

#include "common.cuh"
#include "topk_common.cuh"

namespace mxb {

struct TopkParams {
  const float* scores;
  int64_t row_stride;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t* out_ids;
  int32_t rows;
  int64_t n;
  int32_t k;
  // global scratch for a threshold bin that does not fit in shared memory
  uint32_t* cand_key;  // [rows][n]
  int32_t* cand_idx;   // [rows][n]
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
  // Scores cluster in a few exponent values, so one shared histogram would serialise almost every
  // atomic on the same address; each warp counts into its own 256 bins, merged afterwards.
  uint32_t* whist = keys + p.n;                    // [warps][256]
  const int nwarps = (int)blockDim.x >> 5;
  uint32_t* my_hist = whist + (tid >> 5) * 256;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int i = tid; i < nwarps * 256; i += blockDim.x) whist[i] = 0;
    __syncthreads();
    for (int i = tid; i < n; i += blockDim.x) {
      uint32_t key = keys[i];
      if (key != 0 && (key & prefix_mask) == prefix) atomicAdd(&my_hist[(key >> shift) & 255u], 1u);
    }
    __syncthreads();
    if (tid < 256) {
      uint32_t t = 0;
      for (int w = 0; w < nwarps; ++w) t += whist[w * 256 + tid];
      hist[tid] = t;
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
  // (odd slice length: lanes of a warp then walk different shared-memory banks)
  const int per = ((n + (int)blockDim.x - 1) / (int)blockDim.x) | 1;
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
// long rows: one CTA per row streams the row twice (the scores were just written by
// the score kernel and sit in L2): pass 1 = 11-bit histogram in shared memory, pass 2 =
// strictly-above ids and the threshold bin's candidates into shared memory (global
// scratch only if the bin holds more than kCandSmem entries, e.g. all-equal scores);
// then the remaining 21 bits, the ties by lowest id and a bitonic sort of the ids.
// --------------------------------------------------------------------------
constexpr int kCandSmem = 16384;
constexpr int kStreamUnroll = 16;   // independent loads in flight per thread in the streaming passes

#ifdef MXB_TRACE_TK
#define TRK(k) do { if (threadIdx.x == 0 && blockIdx.x == MXB_TRACE_TK) reinterpret_cast<long long*>(p.cand_key)[k] = clock64(); } while (0)
#else
#define TRK(k)
#endif

__global__ void __launch_bounds__(1024) topk_stream_kernel(TopkParams p, int sort_n) {
  extern __shared__ uint32_t dyn[];
  int32_t* sel = reinterpret_cast<int32_t*>(dyn);                 // [sort_n]
  uint32_t* ck_s = dyn + sort_n;                                  // [kCandSmem]
  int32_t* ci_s = reinterpret_cast<int32_t*>(ck_s + kCandSmem);   // [kCandSmem]
  __shared__ uint32_t hist[kBigBins];
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_total, s_keff, s_bin, s_above, s_cnt_bin, s_na, s_nc, s_digit, s_dabove;

  const int row = blockIdx.x;
  const int tid = threadIdx.x;
  const int64_t n = p.row_count ? min((int64_t)p.row_count[row], p.n) : p.n;
  const int64_t base = p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride;
  const float* src = p.scores + base;
  int32_t* out = p.out_ids + (int64_t)row * p.k;

  for (int i = tid; i < kBigBins; i += 1024) hist[i] = 0;
  if (tid == 0) { s_na = 0; s_nc = 0; s_keff = 0; s_bin = 0; s_above = 0; s_cnt_bin = 0; }
  __syncthreads();
  TRK(0);
  // ---- pass 1
  for (int64_t i0 = 0; i0 < n; i0 += 1024 * kStreamUnroll) {   // trip count uniform over the CTA (warp-wide votes inside)
    const int64_t i = i0 + tid;
    float x[kStreamUnroll];
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) x[u] = (i + 1024 * u < n) ? __ldg(src + i + 1024 * u) : -INFINITY;
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) {
      const uint32_t key = score_key_full(x[u]);
      if (key) atomicAdd(&hist[key >> 21], 1u);
    }
  }
  __syncthreads();
  TRK(1);
  // ---- threshold bin: thread t owns bins 2047-2t and 2046-2t (descending)
  {
    const uint32_t h0 = hist[2047 - 2 * tid], h1 = hist[2046 - 2 * tid];
    const uint32_t excl = block_excl_scan(h0 + h1, warp_sums, &s_total);
    const uint32_t ke = min((uint32_t)p.k, s_total);
    if (tid == 0) s_keff = ke;
    if (ke > 0 && excl < ke && excl + h0 + h1 >= ke) {
      if (excl + h0 >= ke) { s_bin = 2047 - 2 * tid; s_above = excl; s_cnt_bin = h0; }
      else { s_bin = 2046 - 2 * tid; s_above = excl + h0; s_cnt_bin = h1; }
    }
  }
  __syncthreads();
  const uint32_t k_eff = s_keff;
  for (int i = tid + (int)k_eff; i < p.k; i += 1024) out[i] = -1;
  if (k_eff == 0) return;
  const uint32_t bin = s_bin, n_above = s_above, C = s_cnt_bin;
  const bool in_smem = C <= (uint32_t)kCandSmem;
  uint32_t* ck = in_smem ? ck_s : p.cand_key + (int64_t)row * p.n;
  int32_t* ci = in_smem ? ci_s : p.cand_idx + (int64_t)row * p.n;
  for (int i = tid; i < sort_n; i += 1024) sel[i] = 0x7FFFFFFF;
  __syncthreads();
  TRK(2);
  // ---- pass 2
  for (int64_t i0 = 0; i0 < n; i0 += 1024 * kStreamUnroll) {   // trip count uniform over the CTA (warp-wide votes inside)
    const int64_t i = i0 + tid;
    float x[kStreamUnroll];
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) x[u] = (i + 1024 * u < n) ? __ldg(src + i + 1024 * u) : -INFINITY;
#pragma unroll
    for (int u = 0; u < kStreamUnroll; ++u) {
      const uint32_t key = score_key_full(x[u]);
      const uint32_t kb = key >> 21;
      const bool above = key && kb > bin, cand = key && kb == bin;
      const uint32_t lane_lt = (1u << (tid & 31)) - 1u;
      const uint32_t m_above = __ballot_sync(0xffffffffu, above), m_cand = __ballot_sync(0xffffffffu, cand);
      uint32_t base_a = 0, base_c = 0;
      if ((tid & 31) == 0) {   // one counter update per warp
        if (m_above) base_a = atomicAdd(&s_na, (uint32_t)__popc(m_above));
        if (m_cand) base_c = atomicAdd(&s_nc, (uint32_t)__popc(m_cand));
      }
      base_a = __shfl_sync(0xffffffffu, base_a, 0);
      base_c = __shfl_sync(0xffffffffu, base_c, 0);
      if (above) {
        sel[base_a + __popc(m_above & lane_lt)] = (int32_t)(i + 1024 * u);
      } else if (cand) {
        const uint32_t pos = base_c + __popc(m_cand & lane_lt);
        ck[pos] = key;
        ci[pos] = (int32_t)(i + 1024 * u);
      }
    }
  }
  __syncthreads();

  TRK(3);
  // ---- the `want` largest among the C candidates on the low 21 bits (8 + 8 + 5)
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
  const uint32_t thr = prefix;
  const uint32_t need = want;  // ties to take (lowest ids), >= 1
  TRK(4);
  // ---- ties: the need-th smallest id among candidates with key == thr (ids are unique)
  if (tid == 0) s_total = 0;
  __syncthreads();
  {
    uint32_t nt = 0;
    for (uint32_t i = tid; i < C; i += 1024) nt += ck[i] == thr;
    nt = __reduce_add_sync(0xffffffffu, nt);
    if ((tid & 31) == 0 && nt) atomicAdd(&s_total, nt);
  }
  __syncthreads();
  uint32_t idx_thr = 0xFFFFFFFFu;  // all ties taken
  if (s_total > need) {
    uint32_t ipre = 0, imask = 0, iwant = need;
    for (int shift = 24; shift >= 0; shift -= 8) {
      if (tid < 256) hist[tid] = 0;
      __syncthreads();
      for (uint32_t i = tid; i < C; i += 1024) {
        if (ck[i] == thr) {
          const uint32_t v = ~(uint32_t)ci[i];  // descending scan of ~id == ascending id
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
  for (uint32_t i = tid; i < C; i += 1024) {
    const uint32_t key = ck[i];
    const int32_t id = ci[i];
    if (key > thr || (key == thr && (uint32_t)id <= idx_thr)) sel[atomicAdd(&s_na, 1u)] = id;
  }
  __syncthreads();
  TRK(5);
  // ---- bitonic sort ascending (padding = INT_MAX)
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
  TRK(6);
  for (uint32_t i = tid; i < k_eff; i += 1024) out[i] = sel[i];
  TRK(7);
}

int64_t topk_multi_workspace(int32_t rows, int64_t n, int32_t k);   // topk_multi.cu
int launch_topk_multi(const mxb_topk_args* a, cudaStream_t st);
int topk_cluster_size(int32_t rows, int64_t n);                        // topk_cluster.cu
int launch_topk_cluster(const mxb_topk_args* a, int cs, cudaStream_t st);

}  // namespace mxb

using namespace mxb;

extern "C" int64_t mxb_topk_workspace_bytes(int32_t rows, int64_t n, int32_t k) {
  if (rows <= 0 || n <= 0 || k <= 0) return 0;
  if (topk_cluster_size(rows, n) > 0 || n <= kSmemRowMax) return 0;
  return topk_multi_workspace(rows, n, k);
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

  if (const int cs = topk_cluster_size(a->rows, a->n)) return launch_topk_cluster(a, cs, st);
  // the other kernels count their own first digit: only keep the promise that the counters end up clear
  if (a->digit_hist) MXB_CUDA_OK(cudaMemsetAsync(a->digit_hist, 0, (size_t)a->rows * kBigBins * sizeof(uint32_t), st));
  if (a->n <= kSmemRowMax) {
    int threads = a->n >= 8192 ? 1024 : (a->n >= 2048 ? 512 : 256);
    size_t smem = (size_t)a->n * 4 + (size_t)(threads / 32) * 256 * 4;   // keys + per-warp histograms
    if (smem > 48 * 1024)
      MXB_CUDA_OK(cudaFuncSetAttribute(topk_row_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    topk_row_kernel<<<a->rows, threads, smem, st>>>(p);
    note_launch();
    MXB_CUDA_OK(cudaGetLastError());
    return MXB_OK;
  }

  return launch_topk_multi(a, st);
}

// --------------------------------------------------------------------------
// Top-k for callers that must not allocate device memory.
//
// Some hosts of this library cannot hand over a workspace: a serving process that froze
// its memory pool after start-up, or code running inside another framework's allocator
// callback, where cudaMalloc (or any allocating library call) is off limits.  This entry
// point gives them the long-row selection with its candidate scratch in a fixed array
// that is part of the library image: kStaticCandEntries (key, id) pairs = 8 MiB, held by
// every GPU that loads the library until the process exits.
//
// The array's name is only a host-side handle here; the kernel needs the device address,
// which cudaGetSymbolAddress returns for the CURRENT device.  It is looked up once per
// device, on the first call made with that device current — make that first call before
// any stream capture — and kept for the life of that device's primary context (a
// cudaDeviceReset inside the process invalidates it).  Every call shares the array (it keeps the previous call's
// candidates; nothing in it has to start at zero because the kernel's counters live in
// shared memory), so two calls whose kernels overlap on the GPU race on it: keep calls on
// one stream, or otherwise ordered.  rows * n above kStaticCandEntries is rejected.
// --------------------------------------------------------------------------
namespace mxb {
constexpr int64_t kStaticCandEntries = (int64_t)1 << 20;
static __device__ __align__(256) uint32_t g_static_cand[2 * kStaticCandEntries];

static int static_cand_address(uint32_t** out) {
  static std::mutex mu;
  static uint32_t* per_device[64] = {nullptr};
  int dev = -1;
  MXB_CUDA_OK(cudaGetDevice(&dev));
  MXB_REQUIRE(dev >= 0 && dev < 64, MXB_ERR_UNSUPPORTED, "topk (static scratch): device index %d out of range", dev);
  std::lock_guard<std::mutex> lock(mu);
  if (!per_device[dev]) {
    void* ptr = nullptr;
    MXB_CUDA_OK(cudaGetSymbolAddress(&ptr, g_static_cand));
    per_device[dev] = reinterpret_cast<uint32_t*>(ptr);
  }
  *out = per_device[dev];
  return MXB_OK;
}
}  // namespace mxb

extern "C" int mxb_topk_select_static(const mxb_topk_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "topk: null args");
  MXB_REQUIRE(a->rows > 0 && a->n > 0, MXB_ERR_INVALID, "topk: scores must contain at least one row and column");
  MXB_REQUIRE(a->k >= 1 && a->k <= 8192, MXB_ERR_INVALID, "topk must be between 1 and 8192");
  MXB_REQUIRE(a->scores && a->out_ids, MXB_ERR_INVALID, "topk: null tensor");
  MXB_REQUIRE(a->digit_hist == nullptr, MXB_ERR_INVALID, "topk (static): digit_hist is not taken by this entry point");
  MXB_REQUIRE((int64_t)a->rows * a->n <= kStaticCandEntries, MXB_ERR_INVALID,
              "topk (static scratch): rows * n = %lld exceeds the built-in scratch of %lld entries; "
              "use mxb_topk_select with a workspace",
              (long long)((int64_t)a->rows * a->n), (long long)kStaticCandEntries);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  uint32_t* scratch = nullptr;
  int rc = static_cand_address(&scratch);
  if (rc != MXB_OK) return rc;
  TopkParams p{};
  p.scores = a->scores; p.row_stride = a->row_stride; p.row_start = a->row_start; p.row_count = a->row_count;
  p.out_ids = a->out_ids; p.rows = a->rows; p.n = a->n; p.k = a->k;
  p.cand_key = scratch;
  p.cand_idx = reinterpret_cast<int32_t*>(scratch + kStaticCandEntries);
  int sort_n = 2;
  while (sort_n < a->k) sort_n <<= 1;
  const size_t smem = (size_t)sort_n * 4 + (size_t)kCandSmem * 8;
  MXB_CUDA_OK(cudaFuncSetAttribute(topk_stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  topk_stream_kernel<<<a->rows, 1024, smem, st>>>(p, sort_n);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
