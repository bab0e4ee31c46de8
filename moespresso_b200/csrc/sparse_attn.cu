// Indexed mixed (sparse) attention: per (sequence, token, head) an online softmax over
// the raw-window rows visible to the token followed by the selected rows of the
// compressed table, K = the whole row, V = its first Dv features.
//
// sparse_attn_kernel: one CTA = one (split, group of 8 heads, (sequence, token)).
// A tile of 32 gathered rows is staged in shared memory as fp32 by 16-byte vector
// loads (int8 rows are multiplied by their per-row fp16 scale while staging, fp16 /
// bf16 rows are widened), then every warp (= one head) scores the 32 rows (lane = row),
// updates its running (max, sum) and accumulates P.V with lane = feature.  Splits over
// the row list write (o, m, l) partials that merge_kernel combines by log-sum-exp; the
// sink joins once, in the merge (or in the single-split epilogue).
#include "common.cuh"
#include "sparse_attn.cuh"

namespace mxb {

constexpr int kTileRows = 32;
constexpr int kHeadsPerCta = 8;
constexpr int kMaxDvRegs = 16;  // Dv <= 512


// Two rows of a tile at once, four 16-byte chunks of each per trip: eight loads are in flight before the first
// is unpacked (a decode step of one sequence is a latency problem, not a bandwidth one).  A null row is zeros.
template <int KVT>
__device__ __forceinline__ void stage_row_pair(float* dst0, float* dst1, const void* src0, const void* src1, int Dqk,
                                               float rs0, float rs1, int lane) {
  constexpr int EPV = 16 / ElemBytes<KVT>::v;
  const int nchunks = Dqk / EPV;
  const uint4* s0 = reinterpret_cast<const uint4*>(src0);
  const uint4* s1 = reinterpret_cast<const uint4*>(src1);
  for (int c0 = lane; c0 < nchunks; c0 += 128) {
    uint4 v[2][4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + 32 * u;
      v[0][u] = (s0 && c < nchunks) ? __ldg(s0 + c) : make_uint4(0, 0, 0, 0);
      v[1][u] = (s1 && c < nchunks) ? __ldg(s1 + c) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int c = c0 + 32 * u;
      if (c < nchunks) {
        float f[EPV];
        unpack16<KVT>(v[0][u], f);
#pragma unroll
        for (int j = 0; j < EPV; ++j) dst0[c * EPV + j] = (KVT == MXB_I8) ? f[j] * rs0 : f[j];
        unpack16<KVT>(v[1][u], f);
#pragma unroll
        for (int j = 0; j < EPV; ++j) dst1[c * EPV + j] = (KVT == MXB_I8) ? f[j] * rs1 : f[j];
      }
    }
  }
}

template <int KVT, int QT, int OT>
__global__ void __launch_bounds__(256) sparse_attn_kernel(SparseParams p) {
  extern __shared__ float smem_f[];
  const int ld = p.Dqk + 4;   // rows stay 16-byte aligned; a quarter warp of 16-byte reads covers all 32 banks
  float* rows_s = smem_f;                                  // [32][Dqk+4]
  float* q_s = rows_s + kTileRows * ld;                    // [8][Dqk]
  float* p_s = q_s + kHeadsPerCta * p.Dqk;                 // [8][32]
  int* valid_s = reinterpret_cast<int*>(p_s + kHeadsPerCta * kTileRows);  // [32]
  __shared__ int s_keff;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int split = blockIdx.x;
  const int h = blockIdx.y * kHeadsPerCta + warp;
  const int bt = blockIdx.z;
  const int b = bt / p.T, t = bt % p.T;
  const bool head_ok = h < p.H;

  const int64_t pos_b = p.pos0_dev ? p.pos0_dev[b] : p.pos0;
  const int64_t qpos = pos_b + t;
  const int64_t last_pos = pos_b + p.T - 1;
  const int64_t count = p.comp_row_count ? (int64_t)p.comp_row_count[b] : p.n_comp;
  const int64_t cbase = p.comp_row_start ? p.comp_row_start[b] : (int64_t)b * p.n_comp;
  int64_t visible = count;
  if (p.ratio > 0) {
    visible = (qpos + 1) / p.ratio;
    if (visible > count) visible = count;
  }
  // raw window
  int64_t first_raw_pos = 0, first = 0;
  int n_raw = 0;
  if (p.raw_cap > 0) {
    first_raw_pos = last_pos + 1 - p.raw_cap;
    const int64_t window_first = (p.window != 0 && qpos + 1 > p.window) ? qpos + 1 - p.window : 0;
    first = first_raw_pos > window_first ? first_raw_pos : window_first;
    if (first < 0) first = 0;
    const int64_t last = qpos < last_pos ? qpos : last_pos;
    n_raw = last >= first ? (int)(last - first + 1) : 0;
  }
  // first list entry that ends the walk
  const int32_t* ids = p.topk + (int64_t)bt * p.k;
  if (tid == 0) s_keff = p.k;
  __syncthreads();
  {
    int mine = p.k;
    for (int j = tid; j < p.k; j += blockDim.x)
      if ((int64_t)ids[j] >= visible) { mine = j; break; }
    if (mine < p.k) atomicMin(&s_keff, mine);
  }
  // q -> smem (fp32)
  for (int hl = 0; hl < kHeadsPerCta; ++hl) {
    const int hh = blockIdx.y * kHeadsPerCta + hl;
    const int64_t qbase = (int64_t)b * p.q_sb + (int64_t)hh * p.q_sh + (int64_t)t * p.q_st;
    for (int d = tid; d < p.Dqk; d += blockDim.x) q_s[hl * p.Dqk + d] = hh < p.H ? load_elem<QT>(p.q, qbase + d) : 0.f;
  }
  __syncthreads();
  const int total = n_raw + s_keff;
  int per = (total + p.nsplit - 1) / p.nsplit;
  per = ((per + kTileRows - 1) / kTileRows) * kTileRows;
  const int e_lo = min(split * per, total), e_hi = min(e_lo + per, total);

  float M = -INFINITY, S = 0.f;
  // lane owns the features 4 (lane + 32 i) + e, i < 4, e < 4: one 16-byte shared-memory read per (row, i)
  float o[kMaxDvRegs];
#pragma unroll
  for (int i = 0; i < kMaxDvRegs; ++i) o[i] = 0.f;
  const int nq4 = (p.Dv + 127) / 128;         // groups of 128 features in use
  const bool dv4 = (p.Dv & 3) == 0;

  for (int e0 = e_lo; e0 < e_hi; e0 += kTileRows) {
    // stage up to 32 rows: warp w takes rows w, w + 8 and w + 16, w + 24, a pair at a time
    for (int pr = 0; pr < 2; ++pr) {
      const void* src[2] = {nullptr, nullptr};
      float rs[2] = {1.f, 1.f};
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int e = e0 + warp + 8 * (2 * pr + u);
        if (e < e_hi) {
          if (e < n_raw) {
            const int64_t pabs = first + e;
            const int64_t phys = ((int64_t)p.raw_start + (pabs - first_raw_pos)) % p.raw_cap;
            const int64_t ridx = (int64_t)b * p.raw_cap + phys;
            src[u] = reinterpret_cast<const char*>(p.raw_kv) + ridx * p.Dqk * ElemBytes<KVT>::v;
            if (KVT == MXB_I8) rs[u] = __half2float(p.raw_scales[ridx]);
          } else {
            const int32_t id = ids[e - n_raw];
            if (id >= 0) {
              const int64_t ridx = cbase + id;
              src[u] = reinterpret_cast<const char*>(p.comp_kv) + ridx * p.Dqk * ElemBytes<KVT>::v;
              if (KVT == MXB_I8) rs[u] = __half2float(p.comp_scales[ridx]);
            }
          }
        }
      }
      const int r0 = warp + 8 * (2 * pr), r1 = r0 + 8;
      stage_row_pair<KVT>(rows_s + r0 * ld, rows_s + r1 * ld, src[0], src[1], p.Dqk, rs[0], rs[1], lane);
      if (lane == 0) {
        valid_s[r0] = src[0] != nullptr;
        valid_s[r1] = src[1] != nullptr;
      }
    }
    __syncthreads();

    if (head_ok) {
      const float4* qh = reinterpret_cast<const float4*>(q_s + warp * p.Dqk);
      const float4* rj = reinterpret_cast<const float4*>(rows_s + lane * ld);
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;   // four partial sums, combined in a fixed order
      for (int d = 0; d < p.Dqk / 4; ++d) {
        const float4 a = qh[d], r = rj[d];
        d0 = fmaf(a.x, r.x, d0);
        d1 = fmaf(a.y, r.y, d1);
        d2 = fmaf(a.z, r.z, d2);
        d3 = fmaf(a.w, r.w, d3);
      }
      const float dot = (d0 + d1) + (d2 + d3);
      const bool ok = valid_s[lane] != 0;
      const float s = ok ? dot * p.scale : -INFINITY;
      const float tmax = warp_max(s);
      if (tmax > -INFINITY) {
        const float m_new = fmaxf(M, tmax);
        const float pj = ok ? expf(s - m_new) : 0.f;
        const float corr = (M == -INFINITY) ? 0.f : expf(M - m_new);
        S = S * corr + warp_sum(pj);
        M = m_new;
        p_s[warp * kTileRows + lane] = pj;
        __syncwarp();
#pragma unroll
        for (int i = 0; i < kMaxDvRegs; ++i) o[i] *= corr;
        for (int j = 0; j < kTileRows; ++j) {
          const float pw = p_s[warp * kTileRows + j];
          const float* r = rows_s + j * ld + 4 * lane;
#pragma unroll
          for (int i = 0; i < kMaxDvRegs / 4; ++i) {
            if (i < nq4) {
              const int f0 = 4 * (lane + 32 * i);
              float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
              if (dv4) {
                if (f0 < p.Dv) v = *reinterpret_cast<const float4*>(r + 128 * i);
              } else {
                if (f0 < p.Dv) v.x = r[128 * i];
                if (f0 + 1 < p.Dv) v.y = r[128 * i + 1];
                if (f0 + 2 < p.Dv) v.z = r[128 * i + 2];
                if (f0 + 3 < p.Dv) v.w = r[128 * i + 3];
              }
              o[4 * i] = fmaf(pw, v.x, o[4 * i]);
              o[4 * i + 1] = fmaf(pw, v.y, o[4 * i + 1]);
              o[4 * i + 2] = fmaf(pw, v.z, o[4 * i + 2]);
              o[4 * i + 3] = fmaf(pw, v.w, o[4 * i + 3]);
            }
          }
        }
        __syncwarp();
      }
    }
    __syncthreads();
  }

  if (!head_ok) return;
  const int64_t n_idx = (int64_t)bt * p.H + h;
  if (p.nsplit == 1) {
    if (p.partial_ml) {
      float* outp = reinterpret_cast<float*>(p.out) + (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)t * p.o_st;
#pragma unroll
      for (int i = 0; i < kMaxDvRegs; ++i) {
        const int f = 4 * (lane + 32 * (i >> 2)) + (i & 3);
        if (f < p.Dv) outp[f] = o[i];
      }
      if (lane == 0) {
        p.partial_ml[n_idx * 2 + 0] = M;
        p.partial_ml[n_idx * 2 + 1] = S;
      }
    } else {
      const float sink = p.sinks ? p.sinks[h] : -INFINITY;
      const float m2 = fmaxf(M, sink);
      float den = 0.f, w = 0.f;
      if (m2 > -INFINITY) {
        w = (M == -INFINITY) ? 0.f : expf(M - m2);
        den = S * w + ((sink == -INFINITY) ? 0.f : expf(sink - m2));
      }
      const float inv = den > 0.f ? w / den : 0.f;
      const int64_t ob = (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)t * p.o_st;
#pragma unroll
      for (int i = 0; i < kMaxDvRegs; ++i) {
        const int f = 4 * (lane + 32 * (i >> 2)) + (i & 3);
        if (f < p.Dv) store_elem<OT>(p.out, ob + f, o[i] * inv);
      }
    }
  } else {
    const int64_t N = (int64_t)p.B * p.T * p.H;
    float* wo = p.ws_o + ((int64_t)split * N + n_idx) * p.Dv;
#pragma unroll
    if (dv4) {
#pragma unroll
      for (int i = 0; i < kMaxDvRegs / 4; ++i) {
        const int f0 = 4 * (lane + 32 * i);
        if (f0 < p.Dv) *reinterpret_cast<float4*>(wo + f0) = make_float4(o[4 * i], o[4 * i + 1], o[4 * i + 2], o[4 * i + 3]);
      }
    } else {
#pragma unroll
      for (int i = 0; i < kMaxDvRegs; ++i) {
        const int f = 4 * (lane + 32 * (i >> 2)) + (i & 3);
        if (f < p.Dv) wo[f] = o[i];
      }
    }
    if (lane == 0) {
      p.ws_ml[((int64_t)split * N + n_idx) * 2 + 0] = M;
      p.ws_ml[((int64_t)split * N + n_idx) * 2 + 1] = S;
    }
  }
}

// Merge P partials per (b,t,h) row in a fixed order.  finalize != 0: join the sink, normalise,
// store in the output dtype; finalize == 0: store the merged un-normalised sum (fp32) and (m, l).
struct MergeParams {
  const float* o_parts;
  const float* ml_parts;
  const float* sinks;
  void* out;
  float* out_ml;
  int64_t o_sb, o_sh, o_st;
  int32_t P, B, T, H, Dv;
  int32_t finalize;
};

template <int OT, int VEC>
__global__ void __launch_bounds__(256) merge_kernel(MergeParams p) {
  // one thread = one (row, VEC consecutive features); partial loads are independent, so many are in flight
  const int64_t N = (int64_t)p.B * p.T * p.H;
  const int per_row = p.Dv / VEC;
  const int64_t idx = (int64_t)blockIdx.x * 256 + threadIdx.x;
  if (idx >= N * per_row) return;
  const int64_t n = idx / per_row;
  const int d0 = (int)(idx % per_row) * VEC;
  const int h = (int)(n % p.H);
  const int t = (int)((n / p.H) % p.T);
  const int b = (int)(n / ((int64_t)p.H * p.T));
  const float sink = (p.finalize && p.sinks) ? p.sinks[h] : -INFINITY;
  float m = -INFINITY, l = 0.f;
  float acc[VEC];
#pragma unroll
  for (int j = 0; j < VEC; ++j) acc[j] = 0.f;
  constexpr int kFast = 8;
  if (VEC == 4 && p.P <= kFast) {
    // every load of the row is issued before anything depends on one: a single round trip to L2
    float4 v[kFast];
    float ms[kFast], ls[kFast];
#pragma unroll
    for (int s = 0; s < kFast; ++s) {
      ms[s] = -INFINITY;
      ls[s] = 0.f;
      v[s] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (s < p.P) {
        const float2 ml = __ldg(reinterpret_cast<const float2*>(p.ml_parts + ((int64_t)s * N + n) * 2));
        ms[s] = ml.x;
        ls[s] = ml.y;
        v[s] = __ldg(reinterpret_cast<const float4*>(p.o_parts + ((int64_t)s * N + n) * p.Dv + d0));
      }
    }
#pragma unroll
    for (int s = 0; s < kFast; ++s) m = fmaxf(m, ms[s]);
    m = fmaxf(m, sink);
    if (m > -INFINITY) {
#pragma unroll
      for (int s = 0; s < kFast; ++s) {   // split order: the same sum on every run
        if (s < p.P && ms[s] > -INFINITY) {
          const float w = expf(ms[s] - m);
          l = fmaf(ls[s], w, l);
          acc[0] = fmaf(v[s].x, w, acc[0]);
          if constexpr (VEC == 4) {
            acc[1] = fmaf(v[s].y, w, acc[1]); acc[2] = fmaf(v[s].z, w, acc[2]); acc[3] = fmaf(v[s].w, w, acc[3]);
          }
        }
      }
      if (sink > -INFINITY) l += expf(sink - m);
    }
  } else {
    // many splits: sixteen at a time, every load of a batch issued before anything depends on one (a thread's
    // loads are otherwise a chain of L2 round trips: 128 splits took 80 us); the sum stays in split order
    constexpr int kBatch = 16;
    for (int s0 = 0; s0 < p.P; s0 += kBatch) {
      float ms[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u)
        ms[u] = s0 + u < p.P ? __ldg(p.ml_parts + ((int64_t)(s0 + u) * N + n) * 2) : -INFINITY;
#pragma unroll
      for (int u = 0; u < kBatch; ++u) m = fmaxf(m, ms[u]);
    }
    m = fmaxf(m, sink);
    if (m > -INFINITY) {
      for (int s0 = 0; s0 < p.P; s0 += kBatch) {
        float2 ml[kBatch];
        float4 v[kBatch];
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          ml[u] = make_float2(-INFINITY, 0.f);
          v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          if (s0 + u < p.P) {
            const int64_t row = (int64_t)(s0 + u) * N + n;
            ml[u].x = __ldg(p.ml_parts + row * 2);
            ml[u].y = __ldg(p.ml_parts + row * 2 + 1);
            const float* src = p.o_parts + row * p.Dv + d0;
            if constexpr (VEC == 4) v[u] = __ldg(reinterpret_cast<const float4*>(src));
            else v[u].x = __ldg(src);
          }
        }
#pragma unroll
        for (int u = 0; u < kBatch; ++u) {
          if (ml[u].x > -INFINITY) {
            const float w = expf(ml[u].x - m);
            l = fmaf(ml[u].y, w, l);
            acc[0] = fmaf(v[u].x, w, acc[0]);
            if constexpr (VEC == 4) {
              acc[1] = fmaf(v[u].y, w, acc[1]); acc[2] = fmaf(v[u].z, w, acc[2]); acc[3] = fmaf(v[u].w, w, acc[3]);
            }
          }
        }
      }
      if (sink > -INFINITY) l += expf(sink - m);
    }
  }
  const int64_t ob = (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)t * p.o_st + d0;
  const float inv = (p.finalize ? (l > 0.f ? 1.f / l : 0.f) : 1.f);
#pragma unroll
  for (int j = 0; j < VEC; ++j) {
    if (p.finalize) store_elem<OT>(p.out, ob + j, acc[j] * inv);
    else reinterpret_cast<float*>(p.out)[ob + j] = acc[j];
  }
  if (!p.finalize && d0 == 0) {
    p.out_ml[n * 2 + 0] = m;
    p.out_ml[n * 2 + 1] = l;
  }
}

// Many splits of few rows (a decode token split 128 ways): one CTA per row, the splits spread over the CTA so that a
// thread's chain of dependent loads is P / lanes long instead of P.  Weights exp(m_s - m) are computed once into
// shared memory; thread (lane, vec) sums the splits lane, lane + L, ... in ascending order and the L partial sums
// are added in lane order: the same order on every run.
constexpr int kMergeRowsMaxP = 1024;
template <int OT>
__global__ void __launch_bounds__(256) merge_rows_kernel(MergeParams p) {
  __shared__ float w_s[kMergeRowsMaxP];
  __shared__ float red[256];
  __shared__ float4 part[256];
  const int64_t N = (int64_t)p.B * p.T * p.H;
  const int64_t n = blockIdx.x;
  const int tid = threadIdx.x;
  const int h = (int)(n % p.H);
  const int t = (int)((n / p.H) % p.T);
  const int b = (int)(n / ((int64_t)p.H * p.T));
  const float sink = (p.finalize && p.sinks) ? p.sinks[h] : -INFINITY;
  // global maximum
  float m = -INFINITY;
  for (int s = tid; s < p.P; s += 256) m = fmaxf(m, __ldg(p.ml_parts + ((int64_t)s * N + n) * 2));
  red[tid] = m;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) red[tid] = fmaxf(red[tid], red[tid + o]);
    __syncthreads();
  }
  m = fmaxf(red[0], sink);
  __syncthreads();
  // weights and the denominator (fixed tree order)
  float lp = 0.f;
  for (int s = tid; s < p.P; s += 256) {
    const float ms = __ldg(p.ml_parts + ((int64_t)s * N + n) * 2);
    const float w = (ms > -INFINITY && m > -INFINITY) ? expf(ms - m) : 0.f;
    w_s[s] = w;
    lp = fmaf(__ldg(p.ml_parts + ((int64_t)s * N + n) * 2 + 1), w, lp);
  }
  red[tid] = lp;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (tid < o) red[tid] += red[tid + o];
    __syncthreads();
  }
  float l = red[0];
  if (m > -INFINITY && sink > -INFINITY) l += expf(sink - m);
  // features: nvec = Dv / 4 vectors, L = 256 / nvec lanes of splits
  const int nvec = p.Dv / 4, L = 256 / nvec;
  const int vec = tid % nvec, lane = tid / nvec;
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  if (lane < L) {
    constexpr int kBatch = 16;   // loads in flight per thread: the splits' rows come from L2, one round trip per batch
    for (int s0 = lane; s0 < p.P; s0 += L * kBatch) {
      float4 v[kBatch];
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int s = s0 + u * L;
        v[u] = s < p.P ? __ldg(reinterpret_cast<const float4*>(p.o_parts + ((int64_t)s * N + n) * p.Dv) + vec)
                       : make_float4(0.f, 0.f, 0.f, 0.f);
      }
#pragma unroll
      for (int u = 0; u < kBatch; ++u) {
        const int s = s0 + u * L;
        const float w = s < p.P ? w_s[s] : 0.f;
        acc.x = fmaf(v[u].x, w, acc.x); acc.y = fmaf(v[u].y, w, acc.y);
        acc.z = fmaf(v[u].z, w, acc.z); acc.w = fmaf(v[u].w, w, acc.w);
      }
    }
  }
  part[tid] = acc;
  __syncthreads();
  if (tid < nvec) {
    float4 r = part[tid];
    for (int q = 1; q < L; ++q) {
      const float4 x = part[q * nvec + tid];
      r.x += x.x; r.y += x.y; r.z += x.z; r.w += x.w;
    }
    const int64_t ob = (int64_t)b * p.o_sb + (int64_t)h * p.o_sh + (int64_t)t * p.o_st + 4 * tid;
    const float inv = (p.finalize ? (l > 0.f ? 1.f / l : 0.f) : 1.f);
    const float o4[4] = {r.x, r.y, r.z, r.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      if (p.finalize) store_elem<OT>(p.out, ob + j, o4[j] * inv);
      else reinterpret_cast<float*>(p.out)[ob + j] = o4[j];
    }
    if (!p.finalize && tid == 0) {
      p.out_ml[n * 2 + 0] = m;
      p.out_ml[n * 2 + 1] = l;
    }
  }
}

static int launch_merge(const MergeParams& mp, int out_dtype, cudaStream_t st) {
  const int64_t N = (int64_t)mp.B * mp.T * mp.H;
  const bool vec = (mp.Dv % 4 == 0) && ((reinterpret_cast<uintptr_t>(mp.o_parts) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(mp.ml_parts) & 7) == 0);
  const int64_t items = N * (vec ? mp.Dv / 4 : mp.Dv);
  // few rows, many splits: spread the splits over a CTA per row instead of one thread walking them all
  if (vec && mp.P > 16 && mp.P <= kMergeRowsMaxP && mp.Dv / 4 <= 256 && 256 % (mp.Dv / 4) == 0 && items < 148 * 2 * 256) {
    if (out_dtype == MXB_F32) merge_rows_kernel<MXB_F32><<<(unsigned)N, 256, 0, st>>>(mp);
    else if (out_dtype == MXB_BF16) merge_rows_kernel<MXB_BF16><<<(unsigned)N, 256, 0, st>>>(mp);
    else merge_rows_kernel<MXB_F16><<<(unsigned)N, 256, 0, st>>>(mp);
    note_launch();
    MXB_CUDA_OK(cudaGetLastError());
    return MXB_OK;
  }
  dim3 grid((unsigned)ceil_div(items, 256));
#define MXB_MG(OT)                                             \
  if (vec) merge_kernel<OT, 4><<<grid, 256, 0, st>>>(mp);      \
  else merge_kernel<OT, 1><<<grid, 256, 0, st>>>(mp);
  if (out_dtype == MXB_F32) { MXB_MG(MXB_F32) }
  else if (out_dtype == MXB_BF16) { MXB_MG(MXB_BF16) }
  else { MXB_MG(MXB_F16) }
#undef MXB_MG
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

static bool use_tc(const mxb_sparse_attn_args* a) {
  return !(a->flags & MXB_SPARSE_EXACT_FP32) && sparse_tc_eligible(a->kv_dtype, a->q_dtype, a->H, a->Dqk, a->Dv);
}

static int choose_splits(const mxb_sparse_attn_args* a) {
  if (use_tc(a)) return sparse_tc_splits(a->B, a->T, a->H, a->k, a->raw_cap, a->n_splits);
  if (a->n_splits > 0) return a->n_splits > 64 ? 64 : a->n_splits;
  const int64_t base = (int64_t)a->B * a->T * ceil_div(a->H, kHeadsPerCta);
  const int64_t max_rows = (int64_t)a->k + a->raw_cap;
  int64_t want = ceil_div(2 * (int64_t)sm_count(), base);
  int64_t cap = ceil_div(max_rows, (int64_t)kTileRows);   // down to one 32-row tile per split
  if (cap < 1) cap = 1;
  if (want > cap) want = cap;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return (int)want;
}

template <int KVT, int QT>
static int launch_sparse(SparseParams& p, int out_dtype, size_t smem, dim3 grid, cudaStream_t st) {
#define MXB_SP(OT)                                                                                         \
  {                                                                                                        \
    auto kern = sparse_attn_kernel<KVT, QT, OT>;                                                           \
    MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));       \
    kern<<<grid, 256, smem, st>>>(p);                                                                      \
  }
  if (out_dtype == MXB_F32 || p.nsplit > 1 || p.partial_ml) MXB_SP(MXB_F32)
  else if (out_dtype == MXB_BF16) MXB_SP(MXB_BF16)
  else MXB_SP(MXB_F16)
#undef MXB_SP
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

static int validate_sparse(const mxb_sparse_attn_args* a) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "sparse attention: null args");
  MXB_REQUIRE(a->B > 0 && a->T > 0, MXB_ERR_INVALID, "q must contain at least one batch and token");
  MXB_REQUIRE(a->H >= 1, MXB_ERR_INVALID, "q must contain at least one head");
  MXB_REQUIRE(a->Dqk >= 32 && a->Dqk <= 1024 && a->Dqk % 16 == 0, MXB_ERR_INVALID,
              "head width must be a multiple of 16 between 32 and 1024");
  MXB_REQUIRE(a->Dv >= 1 && a->Dv <= a->Dqk && a->Dv <= 32 * kMaxDvRegs, MXB_ERR_INVALID,
              "value width must be between 1 and min(head width, 512)");
  MXB_REQUIRE(a->k >= 0, MXB_ERR_INVALID, "topk must have a non-negative width");
  MXB_REQUIRE(a->raw_cap >= 0, MXB_ERR_INVALID, "raw_cap must be non-negative");
  MXB_REQUIRE(a->raw_cap == 0 || (a->raw_start >= 0 && a->raw_start < a->raw_cap), MXB_ERR_INVALID,
              "raw_start must be inside raw_kv");
  MXB_REQUIRE(a->window >= 0 && a->ratio >= 0, MXB_ERR_INVALID, "window and ratio must be non-negative");
  MXB_REQUIRE(a->q && a->out && (a->k == 0 || (a->topk && a->comp_kv)), MXB_ERR_INVALID,
              "sparse attention: null tensor");
  MXB_REQUIRE(a->raw_cap == 0 || a->raw_kv, MXB_ERR_INVALID, "raw_kv is null but raw_cap > 0");
  MXB_REQUIRE(a->kv_dtype != MXB_I8 || (a->comp_scales && (a->raw_cap == 0 || a->raw_scales)), MXB_ERR_INVALID,
              "int8 KV needs per-row scales");
  MXB_REQUIRE((reinterpret_cast<uintptr_t>(a->comp_kv) & 15) == 0 && (reinterpret_cast<uintptr_t>(a->raw_kv) & 15) == 0,
              MXB_ERR_INVALID, "KV tables must be 16-byte aligned");
  MXB_REQUIRE(!a->partial_ml || a->out_dtype == MXB_F32, MXB_ERR_INVALID, "partial output must be float32");
  return MXB_OK;
}

}  // namespace mxb

using namespace mxb;

extern "C" int64_t mxb_sparse_attn_workspace_bytes(const mxb_sparse_attn_args* a) {
  if (!a || a->B <= 0 || a->T <= 0 || a->H <= 0) return 0;
  const int ns = choose_splits(a);
  if (ns <= 1) return 0;
  const int64_t N = (int64_t)a->B * a->T * a->H;
  return ns * N * ((int64_t)a->Dv + 2) * 4;
}

extern "C" int mxb_sparse_attn(const mxb_sparse_attn_args* a, void* stream) {
  int rc = validate_sparse(a);
  if (rc != MXB_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  SparseParams p{};
  p.q = a->q; p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h; p.q_st = a->q_stride_t;
  p.comp_kv = a->comp_kv; p.comp_scales = reinterpret_cast<const __half*>(a->comp_scales);
  p.comp_row_start = a->comp_row_start; p.comp_row_count = a->comp_row_count; p.n_comp = a->n_comp;
  p.raw_kv = a->raw_kv; p.raw_scales = reinterpret_cast<const __half*>(a->raw_scales);
  p.raw_cap = a->raw_cap; p.raw_start = a->raw_start;
  p.topk = a->topk; p.k = a->k; p.sinks = a->sinks;
  p.out = a->out; p.o_sb = a->out_stride_b; p.o_sh = a->out_stride_h; p.o_st = a->out_stride_t;
  p.partial_ml = a->partial_ml;
  p.B = a->B; p.T = a->T; p.H = a->H; p.Dqk = a->Dqk; p.Dv = a->Dv; p.scale = a->scale;
  p.pos0 = a->pos0; p.pos0_dev = a->pos0_dev; p.window = a->window; p.ratio = a->ratio;
  p.nsplit = choose_splits(a);
  p.status = a->status;

  const int64_t N = (int64_t)a->B * a->T * a->H;
  if (p.nsplit > 1) {
    const int64_t need = p.nsplit * N * ((int64_t)a->Dv + 2) * 4;
    MXB_REQUIRE(a->workspace && a->workspace_bytes >= need, MXB_ERR_WORKSPACE,
                "sparse attention: workspace of %lld bytes required", (long long)need);
    p.ws_o = reinterpret_cast<float*>(a->workspace);
    p.ws_ml = p.ws_o + (int64_t)p.nsplit * N * a->Dv;
  }
  const size_t smem = ((size_t)kTileRows * (a->Dqk + 4) + (size_t)kHeadsPerCta * a->Dqk +
                       (size_t)kHeadsPerCta * kTileRows + kTileRows) * 4;
  dim3 grid((unsigned)p.nsplit, (unsigned)ceil_div(a->H, kHeadsPerCta), (unsigned)(a->B * a->T));

  const int kt = a->kv_dtype, qt = a->q_dtype;
  if (use_tc(a)) {
    rc = launch_sparse_tc(p, kt, qt, a->out_dtype, st);
  } else
#define MXB_PAIR(QT, KT) \
  if (qt == QT && kt == KT) rc = launch_sparse<KT, QT>(p, a->out_dtype, smem, grid, st); else
  MXB_PAIR(MXB_F32, MXB_F32)
  MXB_PAIR(MXB_F32, MXB_F16)
  MXB_PAIR(MXB_F32, MXB_BF16)
  MXB_PAIR(MXB_F32, MXB_I8)
  MXB_PAIR(MXB_F16, MXB_F16)
  MXB_PAIR(MXB_F16, MXB_I8)
  MXB_PAIR(MXB_BF16, MXB_BF16)
  MXB_PAIR(MXB_BF16, MXB_I8)
  return fail(MXB_ERR_UNSUPPORTED, "sparse attention: unsupported q/kv dtype pair (%d, %d)", qt, kt);
#undef MXB_PAIR
  if (rc != MXB_OK) return rc;

  if (p.nsplit > 1 && !p.cluster_merge) {
    MergeParams mp{};
    mp.o_parts = p.ws_o; mp.ml_parts = p.ws_ml; mp.sinks = a->sinks;
    mp.out = a->out; mp.out_ml = a->partial_ml;
    mp.o_sb = a->out_stride_b; mp.o_sh = a->out_stride_h; mp.o_st = a->out_stride_t;
    mp.P = p.nsplit; mp.B = a->B; mp.T = a->T; mp.H = a->H; mp.Dv = a->Dv;
    mp.finalize = a->partial_ml ? 0 : 1;
    return launch_merge(mp, a->partial_ml ? MXB_F32 : a->out_dtype, st);
  }
  return MXB_OK;
}

extern "C" int mxb_merge_partials(const mxb_merge_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "merge: null args");
  MXB_REQUIRE(a->P >= 1 && a->B > 0 && a->T > 0 && a->H > 0 && a->Dv > 0, MXB_ERR_INVALID,
              "merge: sizes must be positive");
  MXB_REQUIRE(a->o_parts && a->ml_parts && a->out, MXB_ERR_INVALID, "merge: null tensor");
  MergeParams mp{};
  mp.o_parts = a->o_parts; mp.ml_parts = a->ml_parts; mp.sinks = a->sinks; mp.out = a->out; mp.out_ml = nullptr;
  mp.o_sb = a->out_stride_b; mp.o_sh = a->out_stride_h; mp.o_st = a->out_stride_t;
  mp.P = a->P; mp.B = a->B; mp.T = a->T; mp.H = a->H; mp.Dv = a->Dv; mp.finalize = 1;
  return launch_merge(mp, a->out_dtype, reinterpret_cast<cudaStream_t>(stream));
}
