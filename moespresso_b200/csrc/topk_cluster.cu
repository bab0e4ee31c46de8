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
constexpr int kCListCap = 128;                  // entries per warp in each of the four 16-bit lists (16 KB per CTA)

struct TopkClusterParams {
  const float* scores;
  int64_t row_stride;
  const int64_t* row_start;
  const int32_t* row_count;
  int32_t* out_ids;
  int32_t rows;
  int64_t n;
  int32_t k;
  int32_t part_cap;   // keys per CTA the launch reserved shared memory for
  uint32_t* hist;     // [rows, 2048] digit-1 histogram of every row, counted by the producer of the scores, or null
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

// Adds the non-zero bins of a 256-bin `local` into `remote` of every CTA of the cluster and clears `local`.
__device__ __forceinline__ void push_hist256(cg::cluster_group& cluster, uint32_t* local, uint32_t* remote, int cs) {
  if (threadIdx.x < 256) {
    const uint32_t v = local[threadIdx.x];
    if (v) {
      local[threadIdx.x] = 0;
      for (int r = 0; r < cs; ++r) atomicAdd(cluster.map_shared_rank(remote + threadIdx.x, r), v);
    }
  }
}

// number of entries of the ascending list `a[0..n)` that are < x
__device__ __forceinline__ int lower_rank(const uint16_t* a, int n, uint32_t x) {
  int lo = 0, hi = n;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (a[mid] < x) lo = mid + 1; else hi = mid;
  }
  return lo;
}

__global__ void __launch_bounds__(kCThreads) topk_cluster_kernel(TopkClusterParams p) {
  extern __shared__ uint32_t keys[];              // this CTA's part of the row, then the per-warp lists
  __shared__ uint32_t lhist[kBigBins];            // histogram of the part, one digit at a time
  __shared__ uint32_t ghist[kBigBins];            // digit 1 of the whole row (summed by all CTAs)
  __shared__ uint32_t ghs[3][256];                // digits 2-4 of the whole row
  __shared__ uint32_t warp_sums[32];
  __shared__ uint32_t s_total, s_thr[4], s_digit, s_dabove;
  __shared__ uint32_t cl_cnt[2][kCMaxCluster];    // (greater, equal) counts of every CTA of the cluster
  __shared__ uint32_t w_cnt[2][kCWarps];
  __shared__ int s_overflow;

  cg::cluster_group cluster = cg::this_cluster();
  const int cs = (int)cluster.num_blocks();
  const int rank = (int)cluster.block_rank();
  const int row = blockIdx.x / cs;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  TRC(0);
  for (int i = tid; i < kBigBins; i += kCThreads) {
    lhist[i] = 0;
    ghist[i] = 0;
  }
  for (int i = tid; i < 3 * 256; i += kCThreads) (&ghs[0][0])[i] = 0;
  if (tid < 4) s_thr[tid] = 0;
  if (tid == 0) s_overflow = 0;
  __syncthreads();
  cluster.barrier_arrive();   // my row histograms are clear; waited for before the first push

  int64_t n_row = p.row_count ? (int64_t)p.row_count[row] : p.n;
  n_row = n_row < 0 ? 0 : (n_row > p.n ? p.n : n_row);
  const int part = (int)round_up(ceil_div(n_row, (int64_t)cs), (int64_t)kCPartUnit);   // <= part_cap (host)
  const int64_t lo = (int64_t)rank * part;
  const int cnt = (int)(n_row - lo < 0 ? 0 : (n_row - lo > part ? part : n_row - lo));
  const int wchunk = part / kCWarps;          // ids of one warp: [warp * wchunk, + wchunk)
  const int iters = wchunk / 128;             // same for every thread of the cluster; a lane owns 4 consecutive ids
  const int wbase = warp * wchunk + lane * 4;
  const float* src = p.scores + (p.row_start ? p.row_start[row] : (int64_t)row * p.row_stride) + lo;
  const bool src_vec = (reinterpret_cast<uintptr_t>(src) & 15) == 0;
  int32_t* out = p.out_ids + (int64_t)row * p.k;
  // per-warp lists behind the keys (offsets are relative to the warp's chunk, ascending):
  //   above: keys whose digit 1 is above the threshold bin (selected for sure)
  //   cand : keys in the threshold bin, with exclusive prefix counts of (greater, equal) filled in at the end
  uint16_t* lists = reinterpret_cast<uint16_t*>(keys + p.part_cap);
  uint16_t* above_off = lists + (0 * kCWarps + warp) * kCListCap;
  uint16_t* cand_off = lists + (1 * kCWarps + warp) * kCListCap;
  uint16_t* cand_gt = lists + (2 * kCWarps + warp) * kCListCap;
  uint16_t* cand_eq = lists + (3 * kCWarps + warp) * kCListCap;
  const uint32_t* wkeys = keys + warp * wchunk;
  const uint32_t lt = (1u << lane) - 1u;

  // With the row's digit-1 histogram already counted (by the kernel that wrote the scores), the load only fills
  // shared memory and the threshold bin comes straight from that histogram: no counting, no push, one cluster
  // barrier less.
  const bool pre = p.hist != nullptr;
  const uint32_t* row_hist = pre ? p.hist + (int64_t)row * kBigBins : ghist;
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
          if (!pre && k4[j]) atomicAdd(&lhist[k4[j] >> 21], 1u);
        }
        *reinterpret_cast<uint4*>(&keys[wbase + (it0 + u) * 128]) = make_uint4(k4[0], k4[1], k4[2], k4[3]);
      }
    }
  }
  __syncthreads();
  TRC(2);
  cluster.barrier_wait();
  TRC(3);
  if (!pre) {
    push_hist(cluster, lhist, ghist, cs);
    TRC(4);
    cluster.sync();
  }
  TRC(5);
  row_threshold(row_hist, p.k, warp_sums, &s_total, s_thr);
  TRC(6);
  const uint32_t k_eff = s_thr[0];
  if (rank == 0)
    for (int i = tid + (int)k_eff; i < p.k; i += kCThreads) out[i] = -1;
  if (k_eff == 0) return;   // the same in every CTA of the cluster; all remote traffic so far is complete
  const uint32_t bin1 = s_thr[1];   // valid keys are >= 0x00800000, so bin1 >= 4 and key 0 is in no list
  uint32_t want = k_eff - s_thr[2];

  // ---- one pass over the keys: ordered lists of the "above" and "candidate" keys of every warp chunk,
  //      digit 2 (bits 20..13) of the candidates
  int n_a = 0, n_c = 0;   // warp-uniform list lengths (may exceed the capacity: then the CTA falls back)
  for (int it = 0; it < iters; ++it) {
    const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[wbase + it * 128]);
    const uint32_t kk[4] = {k4.x, k4.y, k4.z, k4.w};
    bool isa[4], isc[4];
    uint32_t mine = 0;   // this lane's counts: above in bits 0..15, candidates in bits 16..31
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint32_t bin = kk[j] >> 21;
      isa[j] = bin > bin1;
      isc[j] = bin == bin1;
      mine += (isa[j] ? 1u : 0u) + (isc[j] ? 0x10000u : 0u);
    }
    uint32_t incl = mine;   // one warp scan carries both counts
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t y = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += y;
    }
    const uint32_t all = __shfl_sync(0xffffffffu, incl, 31);
    const uint32_t a_below = (incl - mine) & 0xffffu, c_below = (incl - mine) >> 16;
    const uint32_t a_all = all & 0xffffu, c_all = all >> 16;
    int pa = n_a + (int)a_below, pc = n_c + (int)c_below;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const uint16_t off = (uint16_t)(it * 128 + lane * 4 + j);
      if (isa[j]) {
        if (pa < kCListCap) above_off[pa] = off;
        ++pa;
      }
      if (isc[j]) {
        if (pc < kCListCap) cand_off[pc] = off;
        ++pc;
        atomicAdd(&lhist[(kk[j] >> 13) & 255u], 1u);
      }
    }
    n_a += (int)a_all;
    n_c += (int)c_all;
  }
  if (lane == 0 && (n_a > kCListCap || n_c > kCListCap)) s_overflow = 1;
  __syncthreads();
  TRC(7);
  const bool listed = s_overflow == 0;   // per CTA: otherwise the later steps scan all keys of the part
  push_hist256(cluster, lhist, ghs[0], cs);
  cluster.sync();
  if (pre && rank == 0)   // every CTA of the cluster has read the row's histogram: leave it clear for the next step
    for (int i = tid; i < kBigBins; i += kCThreads) p.hist[(int64_t)row * kBigBins + i] = 0;
  TRC(8);
  if (tid < 32) pick_digit_256(ghs[0], want, &s_digit, &s_dabove);
  __syncthreads();
  TRC(9);
  uint32_t prefix = (bin1 << 21) | (s_digit << 13), pmask = 0xFFFFE000u;
  want -= s_dabove;

  // ---- digits 3 (bits 12..5) and 4 (bits 4..0)
#pragma unroll 1
  for (int dg = 0; dg < 2; ++dg) {
    const int shift = dg == 0 ? 5 : 0;
    const uint32_t width = dg == 0 ? 255u : 31u;
    if (listed) {
      for (int i0 = 0; i0 < n_c; i0 += 32) {
        const int i = i0 + lane;
        if (i < n_c) {
          const uint32_t key = wkeys[cand_off[i]];
          if ((key & pmask) == prefix) atomicAdd(&lhist[(key >> shift) & width], 1u);
        }
      }
    } else {
      for (int it = 0; it < iters; ++it) {
        const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[wbase + it * 128]);
        const uint32_t kk[4] = {k4.x, k4.y, k4.z, k4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if ((kk[j] & pmask) == prefix) atomicAdd(&lhist[(kk[j] >> shift) & width], 1u);
      }
    }
    __syncthreads();
    push_hist256(cluster, lhist, ghs[1 + dg], cs);
    cluster.sync();
    if (tid < 32) pick_digit_256(ghs[1 + dg], want, &s_digit, &s_dabove);
    __syncthreads();
    prefix |= s_digit << shift;
    pmask |= width << shift;
    want -= s_dabove;
    __syncthreads();   // s_digit / s_dabove are rewritten by the next digit
  }
  TRC(10);
  const uint32_t thr = prefix;
  const uint32_t need = want;   // ties on thr to take, lowest ids first (1 <= need <= count of thr)

  TRC(11);
  // ---- counts of (greater, equal) keys per warp chunk, per CTA, per cluster
  uint32_t c_gt = 0, c_eq = 0;
  if (listed) {
    // candidates in list order; leave the exclusive prefix counts behind for the emission
    uint32_t run_gt = 0, run_eq = 0;
    for (int i0 = 0; i0 < n_c; i0 += 32) {
      const int i = i0 + lane;
      const uint32_t key = i < n_c ? wkeys[cand_off[i]] : 0u;
      const uint32_t m_gt = __ballot_sync(0xffffffffu, key > thr);
      const uint32_t m_eq = __ballot_sync(0xffffffffu, key == thr);
      if (i < n_c) {
        cand_gt[i] = (uint16_t)(run_gt + __popc(m_gt & lt));
        cand_eq[i] = (uint16_t)(run_eq + __popc(m_eq & lt));
      }
      run_gt += __popc(m_gt);
      run_eq += __popc(m_eq);
    }
    c_gt = (uint32_t)n_a + run_gt;   // warp-uniform already
    c_eq = run_eq;
  } else {
    for (int it = 0; it < iters; ++it) {
      const uint4 k4 = *reinterpret_cast<const uint4*>(&keys[wbase + it * 128]);
      c_gt += (k4.x > thr) + (k4.y > thr) + (k4.z > thr) + (k4.w > thr);
      c_eq += (k4.x == thr) + (k4.y == thr) + (k4.z == thr) + (k4.w == thr);
    }
    c_gt = __reduce_add_sync(0xffffffffu, c_gt);
    c_eq = __reduce_add_sync(0xffffffffu, c_eq);
  }
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
  // ---- ordered emission: ids ascend with the position in the row, so the output slot of a selected id is
  // (greater keys before it) + min(equal keys before it, need)
  if (c_gt == 0 && (c_eq == 0 || eq_run >= need)) return;   // nothing of this warp's chunk is selected
  const int64_t id0 = lo + (int64_t)warp * wchunk;
  if (listed) {
    // candidates: before a candidate lie the above-keys with a smaller offset and the candidates before it
    for (int i0 = 0; i0 < n_c; i0 += 32) {
      const int i = i0 + lane;
      if (i < n_c) {
        const uint32_t off = cand_off[i];
        const uint32_t key = wkeys[off];
        const uint32_t q = eq_run + cand_eq[i];
        if (key > thr || (key == thr && q < need)) {
          const uint32_t g = gt_run + (uint32_t)lower_rank(above_off, n_a, off) + cand_gt[i];
          out[g + min(q, need)] = (int32_t)(id0 + off);
        }
      }
    }
    // above-keys: before one lie the above-keys before it and the candidates with a smaller offset
    for (int i0 = 0; i0 < n_a; i0 += 32) {
      const int i = i0 + lane;
      if (i < n_a) {
        const uint32_t off = above_off[i];
        const int rc = lower_rank(cand_off, n_c, off);   // candidates before this key
        uint32_t g_c, q_c;   // (greater, equal) among those: prefix counts of entry rc, or the totals at the end
        if (rc < n_c) {
          g_c = cand_gt[rc];
          q_c = cand_eq[rc];
        } else {
          g_c = c_gt - (uint32_t)n_a;
          q_c = c_eq;
        }
        out[gt_run + (uint32_t)i + g_c + min(eq_run + q_c, need)] = (int32_t)(id0 + off);
      }
    }
  } else {
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
  // Rows that one CTA could hold.  Few rows: wide clusters, or most of the machine idles.  Many rows of 24 K
  // keys and more (prefill): pairs of CTAs, each with half a row, finish a batch of rows sooner than one full-row
  // CTA per SM (256 x 32768: 43 us against 61; 1024 x 32768: 142 against 254); below that the one-CTA kernel wins.
  const int64_t sms = sm_count();
  if (n >= 16384 && (int64_t)rows * 4 <= sms) return kCMaxCluster;
  if (n >= 24576) return (int64_t)rows * 2 <= sms ? 4 : 2;
  if (n >= 16384 && (int64_t)rows * 2 <= sms) return kCMaxCluster;
  return 0;
#endif
}

int launch_topk_cluster(const mxb_topk_args* a, int cs, cudaStream_t st) {
  TopkClusterParams p{};
  p.scores = a->scores; p.row_stride = a->row_stride; p.row_start = a->row_start; p.row_count = a->row_count;
  p.out_ids = a->out_ids; p.rows = a->rows; p.n = a->n; p.k = a->k;
  p.hist = a->digit_hist;
  const int64_t part_cap = round_up(ceil_div(a->n, (int64_t)cs), (int64_t)kCPartUnit);
  MXB_REQUIRE(part_cap <= kCPartMax, MXB_ERR_INVALID, "topk: row length %lld exceeds the cluster kernel's capacity",
              (long long)a->n);
  p.part_cap = (int32_t)part_cap;
  const size_t smem = (size_t)part_cap * 4 + (size_t)4 * kCWarps * kCListCap * sizeof(uint16_t);
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
