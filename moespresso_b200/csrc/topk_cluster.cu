// Exact top-k for long rows: one thread-block CLUSTER per row, keys resident in shared memory.
//
// A decode batch has few rows (one per sequence) but each is long.  The CTAs of a cluster split
// a row into contiguous parts, read their part of the scores ONCE into shared memory as
// monotone 32-bit keys, and run a three-digit radix select (11 + 11 + 10 bits) together:
//
//   * every CTA histograms its part in shared memory and adds its non-zero bins to the copy of
//     the row histogram that EVERY CTA of the cluster keeps (remote shared-memory atomics), so
//     after one cluster barrier each CTA finds the threshold bin on its own, from local memory;
//   * after the third digit the threshold key is exact; ties on it go to the LOWEST ids: the
//     CTAs exchange their counts of (greater, equal) keys, and because parts, warp chunks and
//     lanes are all in ascending id order, the output slot of a selected id is
//         (greater keys before it) + min(equal keys before it, ties still needed),
//     which every lane gets from two ballots.  Ids come out ascending without a sort and with
//     no scratch in global memory.
//
// Cluster barriers are the hardware's (barrier.cluster): the CTAs of a cluster are scheduled
// together, nothing here spins on memory.  No CTA leaves before the last remote access to
// its shared memory has been made.
#include <cooperative_groups.h>

#include "common.cuh"
#include "topk_common.cuh"

namespace cg = cooperative_groups;

namespace mxb {

constexpr int kCThreads = 512;
constexpr int kCWarps = kCThreads / 32;
constexpr int kCMaxCluster = 8;                 // portable cluster size
constexpr int kCPartUnit = kCThreads * 4;       // parts are multiples of 16 warps x 32 lanes x 4 keys
constexpr int kCPartMax = 45056;                // keys per CTA (176 KB)

struct TopkClusterParams {
  const float* scores;
  int64_t row_stride;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t* out_ids;
  int32_t rows;
  int64_t n;
  int32_t k;
};

#ifdef MXB_TRACE_TC
__device__ long long g_tc_trace[32];
#define TRC(k) do { if (threadIdx.x == 0 && blockIdx.x == 0) g_tc_trace[k] = clock64(); } while (0)
#else
#define TRC(k)
#endif

// Adds the non-zero bins of `local` into `remote` of every CTA of the cluster and clears `local`.
__device__ __forceinline__ void push_hist(cg::cluster_group& cluster, uint32_t* local, uint32_t* remote, int cs) {
  for (int b = threadIdx.x; b < kBigBins; b += kCThreads) {
    const uint32_t v = local[b];
    if (v) {
      local[b] = 0;
      for (int r = 0; r < cs; ++r) atomicAdd(cluster.map_shared_rank(remote + b, r), v);
    }
  }
}

__global__ void __launch_bounds__(kCThreads) topk_cluster_kernel(TopkClusterParams p) {
  extern __shared__ uint32_t keys[];              // this CTA's part of the row
  __shared__ uint32_t lhist[kBigBins];            // histogram of the part, one digit at a time
  __shared__ uint32_t ghist[3][kBigBins];         // histogram of the row, one per digit (summed by all CTAs)
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_total, s_thr[3][4];
  __shared__ uint32_t cl_cnt[2][kCMaxCluster];    // (greater, equal) counts of every CTA of the cluster
  __shared__ uint32_t w_cnt[2][kCWarps];

  cg::cluster_group cluster = cg::this_cluster();
  const int cs = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int row = blockIdx.x / cs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  TRC(0);
  for (int i = tid; i < kBigBins; i += kCThreads) {
    lhist[i] = 0;
    ghist[0][i] = 0;
    ghist[1][i] = 0;
    ghist[2][i] = 0;
  }
  if (tid < 12) (&s_thr[0][0])[tid] = 0;
  __syncthreads();
  cluster.barrier_arrive();   // my row histograms are clear; waited for before the first push

  int64_t n_row = p.row_count ? (int64_t)p.row_count[row] : p.n;
  n_row = n_row < 0 ? 0 : (n_row > p.n ? p.n : n_row);
  const int part = (int)round_up(ceil_div(n_row, (int64_t)cs), (int64_t)kCPartUnit);   // <= kCPartMax (host)
  const int64_t lo = (int64_t)rank * part;
  const int cnt = (int)(n_row - lo < 0 ? 0 : (n_row - lo > part ? part : n_row - lo));
  const int wchunk = part / kCWarps;          // ids of one warp: [wbase, wbase + wchunk)
  const int iters = wchunk / 128;             // same for every thread of the cluster; a lane owns 4 consecutive ids
  const int wbase = warp * wchunk + lane * 4;
  const float* src = p.scores + (p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride) + lo;
  const bool src_vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  int32_t* out = p.out_ids + (int64_t)row * p.k;

  TRC(1);
  // ---- digit 1 (top 11 bits) while loading
  for (int it0 = 0; it0 < iters; it0 += 2) {
    float x[2][4];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int e = wbase + (it0 + u) * 128;
#pragma unroll
      for (int j = 0; j < 4; ++j) x[u][j] = -INFINITY;
      if (it0 + u < iters) {
        if (src_vec && e + 3 < cnt) {
          const float4 v = __ldg(reinterpret_cast<const float4*>(src + e));
          x[u][0] = v.x; x[u][1] = v.y; x[u][2] = v.z; x[u][3] = v.w;
        } else {
#pragma unroll
          for (int j = 0; j < 4; ++j)
            if (e + j < cnt) x[u][j] = __ldg(src + e + j);
        }
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      if (it0 + u < iters) {
        uint32_t k4[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          k4[j] = score_key_full(x[u][j]);
          if (k4[j]) atomicAdd(&lhist[k4[j] >> 21], 1u);
        }
        *reinterpret_cast<uint4*>(&keys[wbase + (it0 + u) * 128]) = make_uint4(k4[0], k4[1], k4[2], k4[3]);
      }
    }
  }
  __syncthreads();
  TRC(2);
  cluster.barrier_wait();
  TRC(3);
  push_hist(cluster, lhist, ghist[0], cs);
  TRC(4);
  cluster.sync();
  TRC(5);
  row_threshold(ghist[0], p.k, warp_sums, &s_total, s_thr[0]);
  TRC(6);
  const uint32_t k_eff = s_thr[0][0];
  if (rank == 0)
    for (int i = tid + (int)k_eff; i < p.k; i += kCThreads) out[i] = -1;
  if (k_eff == 0) return;   // the same in every CTA of the cluster; all remote traffic so far is complete
  const uint32_t bin1 = s_thr[0][1];
  uint32_t want = k_eff - s_thr[0][2];

  // ---- digit 2 (next 11 bits) among keys in the threshold bin
  for (int it = 0; it < iters; ++it) {
    const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[wbase + it * 128]);
    const uint32_t kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)   // valid keys are >= 0x00800000, so bin1 >= 4 and key 0 never matches
      if ((kk[j] >> 21) == bin1) atomicAdd(&lhist[(kk[j] >> 10) & 2047u], 1u);
  }
  __syncthreads();
  TRC(7);
  push_hist(cluster, lhist, ghist[1], cs);
  cluster.sync();
  TRC(8);
  row_threshold(ghist[1], (int)want, warp_sums, &s_total, s_thr[1]);
  const uint32_t prefix22 = (bin1 << 11) | s_thr[1][1];
  want -= s_thr[1][2];

  // ---- digit 3 (last 10 bits)
  for (int it = 0; it < iters; ++it) {
    const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[wbase + it * 128]);
    const uint32_t kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
    for (int j = 0; j < 4; ++j)
      if ((kk[j] >> 10) == prefix22) atomicAdd(&lhist[kk[j] & 1023u], 1u);
  }
  __syncthreads();
  TRC(9);
  push_hist(cluster, lhist, ghist[2], cs);
  cluster.sync();
  TRC(10);
  row_threshold(ghist[2], (int)want, warp_sums, &s_total, s_thr[2]);
  const uint32_t thr = (prefix22 << 10) | s_thr[2][1];
  const uint32_t need = want - s_thr[2][2];   // ties on thr to take, lowest ids first (1 <= need <= count of thr)

  TRC(11);
  // ---- counts of (greater, equal) keys per warp chunk, per CTA, per cluster
  uint32_t c_gt = 0, c_eq = 0;
  for (int it = 0; it < iters; ++it) {
    const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[wbase + it * 128]);
    c_gt += (k4.x > thr) + (k4.y > thr) + (k4.z > thr) + (k4.w > thr);
    c_eq += (k4.x == thr) + (k4.y == thr) + (k4.z == thr) + (k4.w == thr);
  }
  c_gt = __reduce_add_sync(0xffffffffu, c_gt);
  c_eq = __reduce_add_sync(0xffffffffu, c_eq);
  if (lane == 0) {
    w_cnt[0][warp] = c_gt;
    w_cnt[1][warp] = c_eq;
  }
  __syncthreads();
  uint32_t gt_run = 0, eq_run = 0, cta_gt = 0, cta_eq = 0;
#pragma unroll
  for (int w = 0; w < kCWarps; ++w) {
    const uint32_t a = w_cnt[0][w], b = w_cnt[1][w];
    if (w < warp) {
      gt_run += a;
      eq_run += b;
    }
    cta_gt += a;
    cta_eq += b;
  }
  if (tid < cs) {
    *cluster.map_shared_rank(&cl_cnt[0][rank], tid) = cta_gt;
    *cluster.map_shared_rank(&cl_cnt[1][rank], tid) = cta_eq;
  }
  TRC(12);
  cluster.sync();   // last remote access to anyone's shared memory
  for (int r = 0; r < rank; ++r) {
    gt_run += cl_cnt[0][r];
    eq_run += cl_cnt[1][r];
  }

  TRC(13);
  // ---- ordered emission: ids ascend with (iteration, lane, slot), so the output slot of a selected id is
  // (greater keys before it) + min(equal keys before it, need)
  if (c_gt == 0 && (c_eq == 0 || eq_run >= need)) return;   // nothing of this warp's chunk is selected
  const uint32_t lt = (1u << lane) - 1u;
  for (int it = 0; it < iters; ++it) {
    const int e = wbase + it * 128;
    const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[e]);
    const uint32_t kk[4] = {k4.x, k4.y, k4.z, k4.w};
    uint32_t gt_below = 0, eq_below = 0, gt_all = 0, eq_all = 0;   // over lower lanes / over the whole warp
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t m_gt = __ballot_sync(0xffffffffu, kk[j] > thr);
      const uint32_t m_eq = __ballot_sync(0xffffffffu, kk[j] == thr);
      gt_below += __popc(m_gt & lt);
      eq_below += __popc(m_eq & lt);
      gt_all += __popc(m_gt);
      eq_all += __popc(m_eq);
    }
    uint32_t g = gt_run + gt_below, q = eq_run + eq_below;   // counts before this lane's first key
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const bool gt = kk[j] > thr, eq = kk[j] == thr;
      if (gt || (eq && q < need)) out[g + min(q, need)] = (int32_t)(lo + e + j);
      g += gt;
      q += eq;
    }
    gt_run += gt_all;
    eq_run += eq_all;
  }
  TRC(14);
}

#ifdef MXB_TRACE_TC
extern "C" int mxb_tc_trace_read(long long* host) {
  return (int)cudaMemcpyFromSymbol(host, g_tc_trace, sizeof(long long) * 32);
}
#endif

// cluster size for a shape, 0 = this kernel does not apply
int topk_cluster_size(int32_t rows, int64_t n) {
#ifdef MXB_TOPK_CS
  return (MXB_TOPK_CS) > 0 && n <= (int64_t)(MXB_TOPK_CS) * kCPartMax ? (MXB_TOPK_CS) : 0;
#else
  if (n > (int64_t)kCMaxCluster * kCPartMax) return 0;
  if (n > kSmemRowMax) return kCMaxCluster;
  // shorter rows: clusters only while single CTAs would leave most of the machine idle
  if (n >= 16384 && (int64_t)rows * 2 <= sm_count()) return kCMaxCluster;
  return 0;
#endif
}

int launch_topk_cluster(const mxb_topk_args* a, int cs, cudaStream_t st) {
  TopkClusterParams p{};
  p.scores = a->scores; p.row_stride = a->row_stride; p.row_start = a->row_start; p.row_count = a->row_count;
  p.out_ids = a->out_ids; p.rows = a->rows; p.n = a->n; p.k = a->k;
  const int64_t part_cap = round_up(ceil_div(a->n, (int64_t)cs), (int64_t)kCPartUnit);
  MXB_REQUIRE(part_cap <= kCPartMax, MXB_ERR_INVALID, "topk: row length %lld exceeds the cluster kernel's capacity",
              (long long)a->n);
  const size_t smem = (size_t)part_cap * 4;
  MXB_CUDA_OK(cudaFuncSetAttribute(topk_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)((int64_t)a->rows * cs));
  cfg.blockDim = dim3(kCThreads);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeClusterDimension;
  at[0].val.clusterDim.x = (unsigned)cs;
  at[0].val.clusterDim.y = 1;
  at[0].val.clusterDim.z = 1;
  cfg.attrs = at;
  cfg.numAttrs = 1;
  MXB_CUDA_OK(cudaLaunchKernelEx(&cfg, topk_cluster_kernel, p));
  note_launch();
  return MXB_OK;
}

}  // namespace mxb
