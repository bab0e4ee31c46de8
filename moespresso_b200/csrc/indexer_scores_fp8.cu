// Indexer score over FP8-E4M3 key tables: a warp-specialised streaming pipeline.
//
//   warp roles      drain warps (2 sets x 4, thread = key row = TMEM lane)
//                   1 MMA-issue warp, 1 TMA-producer warp, [NA widening warps]
//
// Two operand modes.
//  * WIDEN (default): TMA streams raw 128-row FP8 tiles; each widening warp owns one
//    16-bit operand buffer and turns a tile into fp16 (cvt.f16x2.e4m3x2, exact) in the
//    128-byte-swizzled K-major layout; tcgen05.mma kind::f16 multiplies it with the
//    query held as fp16.  The 16-bit query (bf16 or fp16) is scaled per head by a power
//    of two, q * 2^a with max |q| * 2^a in [2^13, 2^14), so that every element within 2^-27
//    of the head's maximum is an exact fp16 value (bf16 has 8 significant bits, fp16 11);
//    the head weight carries 2^-a.  Products are exact, accumulation is fp32.
//  * DIRECT (MXB_INDEXER_FP8_MMA): no widening — raw tiles are the A operand of
//    tcgen05.mma kind::f8f6f4 and the query is split exactly into two E4M3 pieces
//    (q * 2^a = q1 + q2 / 16) that sit side by side on N.  The FP8 tensor-core path
//    accumulates with reduced precision (scores agree with a float64 evaluation to
//    about 1e-3 relative instead of 1e-6), so this mode is opt-in.
//
// No CTA-wide barrier inside the tile loop: stages, operand buffers and TMEM accumulators
// are handed over with mbarriers.  The head sum runs in a fixed order, so a row's score
// does not depend on the partition of rows over CTAs or GPUs.
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace mxb {

#if defined(MXB_TRACE_MMA)
#define TR(role, i)
#define TRM(role, i) do { if (tr_on && (i) < 64) tr[(role) * 64 + (i)] = clock64(); } while (0)
#elif defined(MXB_TRACE)
#define TR(role, i) do { if (tr_on && (i) < 64) tr[(role) * 64 + (i)] = clock64(); } while (0)
#define TRM(role, i)
#else
#define TR(role, i)
#define TRM(role, i)
#endif

struct Fp8Params {
  const uint8_t* keys;
  int64_t rows_total;
  const void* q;
  int q_is_bf16;
  int64_t q_sb, q_sh, q_st;
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
  int32_t N;             // MMA N
  int32_t acc_stride;    // TMEM columns per accumulator (N rounded up to 32)
  int32_t n_acc;         // accumulators in the TMEM ring
  int32_t tmem_cols;
  int32_t rows_per_cta;  // multiple of 128
  int32_t b_bytes;       // bytes of the query operand region (multiple of 1024)
  int32_t* status;
};

constexpr int kWiden = 0, kDirect = 1, kKeys16 = 2;   // operand modes
constexpr int kMmaWarps = 2;               // two issuing threads: tile i belongs to issuer i % 2

template <int D, int MODE>
struct Fp8Cfg {
  static constexpr int kStages = MODE == kDirect ? 8 : (MODE == kWiden ? 4 : 0);   // raw FP8 tiles in flight
  // 16-bit operand buffers (WIDEN: one per widening warp; KEYS16: the TMA ring itself)
  static constexpr int kNA = MODE == kDirect ? 0 : (MODE == kWiden ? (D == 64 ? 4 : 2) : (D == 64 ? 4 : 3));
  static constexpr int kConv = MODE == kWiden ? kNA : 0;                            // widening warps
  // drain warps: kTileGroups tiles drained concurrently, each by kColSplit groups of 4 warps that share
  // the tile's columns (the wide prefill tiles of KEYS16 need more drain threads per tile)
  static constexpr int kTileGroups = 2;
  static constexpr int kColSplit = MODE == kKeys16 ? 2 : 1;
  static constexpr int kDrainWarps = 4 * kTileGroups * kColSplit;
  static constexpr int kMmaWarp = kDrainWarps;
  static constexpr int kTmaWarp = kDrainWarps + kMmaWarps;
  static constexpr int kConvWarp0 = kTmaWarp + 1;
  static constexpr int kRaw = 128 * D;
  static constexpr int kA16 = 128 * D * 2;
  static constexpr int raw_off = 0;
  static constexpr int a16_off = raw_off + kStages * kRaw;
  static constexpr int b_off = a16_off + kNA * kA16;        // + b_bytes, then weights and barriers
  static constexpr int kThreads = 32 * (kConvWarp0 + kConv);
};

__device__ __forceinline__ float e4m3_round(float x, uint8_t* bits) {
  const __nv_fp8_storage_t b = __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3);
  *bits = (uint8_t)b;
  return __half2float(__half(__nv_cvt_fp8_to_halfraw(b, __NV_E4M3)));
}

template <int D, int MODE>
__global__ void __launch_bounds__(Fp8Cfg<D, MODE>::kThreads, 1)
indexer_fp8_kernel(const __grid_constant__ CUtensorMap tmap, Fp8Params p) {
  using C = Fp8Cfg<D, MODE>;
  constexpr bool DIRECT = MODE == kDirect;
  constexpr bool K16 = MODE == kKeys16;
  constexpr int kMmaWarp = C::kMmaWarp, kTmaWarp = C::kTmaWarp, kConvWarp0 = C::kConvWarp0;
  constexpr int S = C::kStages;
  constexpr int NA = C::kNA;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* raw_buf = smem + C::raw_off;
  uint8_t* a16_buf = smem + C::a16_off;
  uint8_t* b_buf = smem + C::b_off;
  float* w_s = reinterpret_cast<float*>(b_buf + p.b_bytes);              // [<= 256]
  int32_t* vis_s = reinterpret_cast<int32_t*>(w_s + 256);                // [<= 256] rows visible to each token
  uint64_t* raw_full = reinterpret_cast<uint64_t*>(vis_s + 256);         // [8]
  uint64_t* raw_empty = raw_full + 8;                                    // [8]
  uint64_t* a_full = raw_empty + 8;                                      // [4]
  uint64_t* a_empty = a_full + 4;                                        // [4]
  uint64_t* acc_full = a_empty + 4;                                      // [16]
  uint64_t* acc_empty = acc_full + 16;                                   // [16]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 16);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
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
  const int N = p.N, H = p.H, n_acc = p.n_acc;
#if defined(MXB_TRACE) || defined(MXB_TRACE_MMA)
  long long* tr = reinterpret_cast<long long*>(p.status);
  const bool tr_on = p.status && blockIdx.x == 1 && blockIdx.z == 0 && lane == 0;
  if (tr_on && tid == 0) tr[6 * 64] = clock64();
#endif

  if (tid == 0) {
    for (int s = 0; s < S; ++s) {
      ptx::mbar_init(&raw_full[s], 1);
      ptx::mbar_init(&raw_empty[s], DIRECT ? 1 : 32);
    }
    for (int a = 0; a < NA; ++a) {
      ptx::mbar_init(&a_full[a], K16 ? 1 : 32);
      ptx::mbar_init(&a_empty[a], 1);
    }
    for (int a = 0; a < n_acc; ++a) {
      ptx::mbar_init(&acc_full[a], 1);
      ptx::mbar_init(&acc_empty[a], 128 * C::kColSplit);
    }
    *abort_flag = 0;
    ptx::mbar_fence_init();
    ptx::tma_prefetch_desc(&tmap);
  }
  __syncwarp();
  if (warp == 0) {
    ptx::tmem_alloc(tmem_slot, (uint32_t)p.tmem_cols);
    ptx::tmem_relinquish();
  }

  // ---- query -> B operand.
  // 16-bit keys: q has the keys' type and is used as it is, so the operand is a plain copy, one 16-byte chunk
  // (8 features of one (token, head) column) per thread and step, all loads independent.
  const bool q_copy = K16 && ((reinterpret_cast<uintptr_t>(p.q) & 15) == 0) && p.q_sb % 8 == 0 && p.q_sh % 8 == 0 &&
                      p.q_st % 8 == 0;
  if (q_copy) {
    constexpr int CPRq = D / 8;   // chunks per column
    for (int i = tid; i < p.t_tile * H * CPRq; i += C::kThreads) {
      const int n = i / CPRq, cq = i % CPRq;   // column = t * H + h
      const int t = n / H, h = n % H;
      uint4 v = make_uint4(0, 0, 0, 0);
      if (t < nt)
        v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + (int64_t)b * p.q_sb +
                                                 (int64_t)h * p.q_sh + (int64_t)(t0 + t) * p.q_st) + cq);
      const int kb = cq >> 3, c = cq & 7;
      *reinterpret_cast<uint4*>(b_buf + (size_t)kb * N * 128 + (size_t)n * 128 + ((c ^ (n & 7)) << 4)) = v;
    }
    for (int n = tid; n < p.t_tile * H; n += C::kThreads) {
      const int t = n / H, h = n % H;
      w_s[n] = (t < nt) ? p.weights[((int64_t)b * p.T + t0 + t) * H + h] : 0.f;
    }
  }
  // Otherwise one warp per (token, head) row; lane owns D/32 features.
  for (int r = warp; !q_copy && r < p.t_tile * H; r += C::kThreads / 32) {
    const int t = r / H, h = r % H;
    constexpr int EPL = D / 32;
    float x[EPL];
    float amax = 0.f;
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      float v = 0.f;
      if (t < nt) {
        const int64_t idx = (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)(t0 + t) * p.q_st + lane * EPL + j;
        v = p.q_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.q)[idx])
                        : __half2float(reinterpret_cast<const __half*>(p.q)[idx]);
      }
      x[j] = v;
      amax = fmaxf(amax, fabsf(v));
    }
    amax = warp_max(amax);
    int a = 0;
    if (!K16 && amax > 0.f && amax < 3.0e38f) {   // 16-bit keys: the query is used as it is
      int e;
      frexpf(amax, &e);                       // amax = m * 2^e, m in [0.5, 1)
      a = (DIRECT ? 8 : 14) - e;              // amax * 2^a in [128, 256) resp. [2^13, 2^14)
      a = max(-100, min(100, a));
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
      const int d = lane * EPL + j;
      const float xs = ldexpf(x[j], a);
      if constexpr (DIRECT) {
        const int n1 = t * 2 * H + h, n2 = n1 + H;
        uint8_t b1, b2;
        const float q1 = e4m3_round(xs, &b1);
        e4m3_round((xs - q1) * 16.f, &b2);
        const int c = d >> 4, within = d & 15;
        if constexpr (D == 64) {
          b_buf[n1 * 64 + ((c ^ ((n1 >> 1) & 3)) << 4) + within] = b1;
          b_buf[n2 * 64 + ((c ^ ((n2 >> 1) & 3)) << 4) + within] = b2;
        } else {
          b_buf[n1 * 128 + ((c ^ (n1 & 7)) << 4) + within] = b1;
          b_buf[n2 * 128 + ((c ^ (n2 & 7)) << 4) + within] = b2;
        }
      } else {
        const int n = r;                      // column = t * H + h
        const int kb = d >> 6, c = (d & 63) >> 3, within = d & 7;
        uint16_t bits;
        if (K16 && p.q_is_bf16) {
          __nv_bfloat16 v = __float2bfloat16_rn(xs);
          bits = *reinterpret_cast<uint16_t*>(&v);
        } else {
          __half v = __float2half_rn(xs);
          bits = *reinterpret_cast<uint16_t*>(&v);
        }
        reinterpret_cast<uint16_t*>(b_buf + (size_t)kb * N * 128 + (size_t)n * 128 + ((c ^ (n & 7)) << 4))[within] = bits;
      }
    }
    if (lane == 0) w_s[r] = (t < nt) ? ldexpf(p.weights[((int64_t)b * p.T + t0 + t) * H + h], -a) : 0.f;
  }
  // rows a token may see (causal mask over compressed rows), once per token instead of once per score
  for (int t = tid; t < nt; t += C::kThreads) {
    int64_t v = count;
    if (p.ratio > 0) {
      v = (p.pos0 + t0 + t + 1) / p.ratio;
      if (v > count) v = count;
    }
    vis_s[t] = (int32_t)v;
  }
  ptx::fence_proxy_async_smem();
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == kTmaWarp) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      for (int i = 0; i < ntiles; ++i) {
        int s = 0;
        if constexpr (!K16) {
          s = i % S;
          if (i >= S) ptx::mbar_wait(&raw_empty[s], (uint32_t)((i / S - 1) & 1), abort_flag);
        }
        const int64_t grow = rbase + row0 + (int64_t)i * 128;
        TR(0, i);
        if constexpr (K16) {
          // 16-bit keys go straight into the swizzled operand ring
          constexpr int NAk = C::kNA;
          const int ab = i % NAk;
          if (i >= NAk) ptx::mbar_wait(&a_empty[ab], (uint32_t)((i / NAk - 1) & 1), abort_flag);
          ptx::mbar_expect_tx(&a_full[ab], (uint32_t)C::kA16);
#pragma unroll
          for (int kb = 0; kb < D / 64; ++kb)
            ptx::tma_load_2d(a16_buf + (size_t)ab * C::kA16 + (size_t)kb * 16384, &tmap, &a_full[ab], kb * 64,
                             (int32_t)grow);
        } else if constexpr (DIRECT) {
          ptx::mbar_expect_tx(&raw_full[s], (uint32_t)C::kRaw);
          ptx::tma_load_2d(raw_buf + (size_t)s * C::kRaw, &tmap, &raw_full[s], 0, (int32_t)grow);
        } else {
          // the 128 rows of a tile are contiguous in the table: one untiled bulk copy, clamped at the table end
          int64_t rows = p.rows_total - grow;
          if (rows > 128) rows = 128;
          const uint32_t bytes = (uint32_t)(rows * D);
          ptx::mbar_expect_tx(&raw_full[s], bytes);
          ptx::bulk_load_1d(raw_buf + (size_t)s * C::kRaw, p.keys + grow * D, bytes, &raw_full[s]);
        }
      }
    }
  } else if (warp >= kMmaWarp && warp < kMmaWarp + kMmaWarps) {
    // ------------------------------------------------------------ MMA issuers
    // A single thread needs ~1000 cycles per tile for its waits, four MMAs and two commits, more than
    // the 700 cycles a tile may take at HBM speed with two CTAs per SM; two issuers alternate tiles.
    if (lane == 0) {
      const int mw = warp - kMmaWarp;
      const uint32_t b_addr = ptx::smem_u32(b_buf);
      const uint64_t a_desc0 = ptx::smem_desc_sw128(ptx::smem_u32(a16_buf), 16, 1024);
      const uint64_t b_desc0 = ptx::smem_desc_sw128(b_addr, 16, 1024);
      const uint32_t fmt16 = (K16 && p.q_is_bf16) ? ptx::kFmtBF16 : ptx::kFmtF16;
      const uint32_t idesc16 = ptx::idesc_f16(fmt16, fmt16, 128, (uint32_t)N, 0, 0);
      int a = mw % n_acc, ab = NA > 0 ? mw % (NA > 0 ? NA : 1) : 0;   // ring positions of this issuer's first tile
      uint32_t a_ph = 1, ab_ph = 0;      // parity to wait for: acc_empty of the previous use, a_full of this use
      for (int i = mw; i < ntiles; i += kMmaWarps) {
        const uint32_t d_tmem = tmem_base + (uint32_t)(a * p.acc_stride);
        if constexpr (DIRECT) {
          constexpr uint32_t kMode = (D == 64) ? 4u : 2u;   // 64-byte / 128-byte swizzle
          constexpr uint32_t kSbo = 8 * D;
          const int s = i % S;
          ptx::mbar_wait(&raw_full[s], (uint32_t)((i / S) & 1), abort_flag);
          if (i >= n_acc) ptx::mbar_wait(&acc_empty[a], (uint32_t)((i / n_acc - 1) & 1), abort_flag);
          ptx::tc_fence_after_sync();
          const uint32_t idesc = ptx::idesc_e4m3(128, (uint32_t)N);
          const uint32_t a_addr = ptx::smem_u32(raw_buf) + s * C::kRaw;
#pragma unroll
          for (int ks = 0; ks < D / 32; ++ks) {
            const uint64_t ad = ptx::smem_desc(a_addr + ks * 32, 16, kSbo, kMode);
            const uint64_t bd = ptx::smem_desc(b_addr + ks * 32, 16, kSbo, kMode);
            ptx::mma_f8_ss(d_tmem, ad, bd, idesc, ks ? 1u : 0u);
          }
          ptx::mma_commit(&raw_empty[s]);
        } else {
          // descriptors differ from the precomputed bases only in their start-address field
          TRM(0, i);
          ptx::mbar_wait(&a_full[ab], ab_ph, abort_flag);
          TRM(1, i);
          if (i >= n_acc) ptx::mbar_wait(&acc_empty[a], a_ph, abort_flag);
          TRM(2, i);
          ptx::tc_fence_after_sync();
          const uint64_t ad0 = ptx::desc_advance(a_desc0, (uint32_t)(ab * C::kA16));
#pragma unroll
          for (int kb = 0; kb < D / 64; ++kb)
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              ptx::mma_f16_ss(d_tmem, ptx::desc_advance(ad0, kb * 16384 + ks * 32),
                              ptx::desc_advance(b_desc0, kb * N * 128 + ks * 32), idesc16, (kb | ks) ? 1u : 0u);
          TRM(3, i);
          ptx::mma_commit(&a_empty[ab]);
          TRM(4, i);
          TR(3, i);
        }
        ptx::mma_commit(&acc_full[a]);
        TRM(5, i);
        a += kMmaWarps;
        if (a >= n_acc) { a -= n_acc; a_ph ^= 1u; }
        if (NA > 0) {
          ab += kMmaWarps;
          if (ab >= NA) { ab -= NA; ab_ph ^= 1u; }
        }
      }
    }
  } else if (warp >= kConvWarp0) {
    // ------------------------------------------------------------ widening warps (WIDEN only)
    if constexpr (MODE == kWiden) {
      const int cw = warp - kConvWarp0;   // owns operand buffer cw, handles tiles cw, cw + NA, ...
      uint8_t* a_tile = a16_buf + (size_t)cw * C::kA16;
      constexpr int CPR = D / 16;         // 16-byte FP8 chunks per row
      for (int i = cw; i < ntiles; i += NA) {
        const int s = i % S;
        ptx::mbar_wait(&raw_full[s], (uint32_t)((i / S) & 1), abort_flag);
        if (i >= NA) ptx::mbar_wait(&a_empty[cw], (uint32_t)((i / NA - 1) & 1), abort_flag);
        TR(1, i);
        const uint8_t* raw = raw_buf + (size_t)s * C::kRaw;
#pragma unroll 4
        for (int ci = lane; ci < 128 * CPR; ci += 32) {
          const int row = ci / CPR, cc = ci % CPR;
          const uint4 in = *reinterpret_cast<const uint4*>(raw + (size_t)ci * 16);
          const uint16_t* pr = reinterpret_cast<const uint16_t*>(&in);
          uint32_t o[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)pr[j], __NV_E4M3);
            o[j] = *reinterpret_cast<uint32_t*>(&hr);
          }
          const int kb = cc >> 2, c = (cc & 3) * 2;
          uint8_t* dst = a_tile + (size_t)kb * 16384 + (size_t)row * 128;
          *reinterpret_cast<uint4*>(dst + ((c ^ (row & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          *reinterpret_cast<uint4*>(dst + (((c + 1) ^ (row & 7)) << 4)) = make_uint4(o[4], o[5], o[6], o[7]);
        }
        ptx::fence_proxy_async_smem();
        ptx::mbar_arrive(&a_full[cw]);
        ptx::mbar_arrive(&raw_empty[s]);
        TR(2, i);
      }
    }
  } else {
    // ------------------------------------------------------------ drain: thread = key row
    const int set = warp >> 2, quad = warp & 3;
    const int tg = set / C::kColSplit, ch = set % C::kColSplit;   // tile group, share of the tile's tokens
    const int t_per = (p.t_tile + C::kColSplit - 1) / C::kColSplit;
    const int t_lo = min(ch * t_per, nt), t_hi = min(t_lo + t_per, nt);
    const int rloc = quad * 32 + lane;
    const int64_t sbase = (p.row_start ? p.row_start[b] : 0) + (int64_t)b * p.s_sb;
    for (int i = tg; i < ntiles; i += C::kTileGroups) {
      const int a = i % n_acc;
      ptx::mbar_wait(&acc_full[a], (uint32_t)((i / n_acc) & 1), abort_flag);
      ptx::tc_fence_after_sync();
      if (quad == 0) TR(4, i);
      const int64_t r = row0 + (int64_t)i * 128 + rloc;
      const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)(a * p.acc_stride);
      const bool r_ok = r < count;
      float* sp = p.scores + sbase + (int64_t)(t0 + t_lo) * p.s_st + r;
      // two tokens per step: their TMEM loads travel together and their two head sums (each in head order) are
      // independent chains, so the loop is no longer one load latency plus one dependent chain per token
      auto load_tok = [&](int t, int c0, uint32_t* v) {
        if constexpr (DIRECT) {
          uint32_t v2[16];
          ptx::tmem_ld16(taddr + (uint32_t)(t * 2 * H + c0), v);
          ptx::tmem_ld16(taddr + (uint32_t)(t * 2 * H + H + c0), v2);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int j = 0; j < 16; ++j) v[j] = __float_as_uint(fmaf(__uint_as_float(v2[j]), 0.0625f, __uint_as_float(v[j])));
        } else {
          ptx::tmem_ld16(taddr + (uint32_t)(t * H + c0), v);
        }
      };
      int t = t_lo;
      for (; t + 1 < t_hi; t += 2, sp += 2 * p.s_st) {
        float sum0 = 0.f, sum1 = 0.f;
        for (int c0 = 0; c0 < H; c0 += 16) {
          uint32_t va[16], vb[16];
          load_tok(t, c0, va);
          load_tok(t + 1, c0, vb);
          ptx::tmem_ld_wait();
          const float4* wa = reinterpret_cast<const float4*>(w_s + t * H + c0);   // H is a multiple of 16
          const float4* wb = reinterpret_cast<const float4*>(w_s + (t + 1) * H + c0);
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const float4 x = wa[j4], y = wb[j4];
            sum0 = fmaf(x.x, fmaxf(__uint_as_float(va[4 * j4 + 0]), 0.f), sum0);
            sum1 = fmaf(y.x, fmaxf(__uint_as_float(vb[4 * j4 + 0]), 0.f), sum1);
            sum0 = fmaf(x.y, fmaxf(__uint_as_float(va[4 * j4 + 1]), 0.f), sum0);
            sum1 = fmaf(y.y, fmaxf(__uint_as_float(vb[4 * j4 + 1]), 0.f), sum1);
            sum0 = fmaf(x.z, fmaxf(__uint_as_float(va[4 * j4 + 2]), 0.f), sum0);
            sum1 = fmaf(y.z, fmaxf(__uint_as_float(vb[4 * j4 + 2]), 0.f), sum1);
            sum0 = fmaf(x.w, fmaxf(__uint_as_float(va[4 * j4 + 3]), 0.f), sum0);
            sum1 = fmaf(y.w, fmaxf(__uint_as_float(vb[4 * j4 + 3]), 0.f), sum1);
          }
        }
        if (r_ok) {
          sp[0] = r < (int64_t)vis_s[t] ? sum0 : -INFINITY;
          sp[p.s_st] = r < (int64_t)vis_s[t + 1] ? sum1 : -INFINITY;
        }
      }
      if (t < t_hi) {
        float sum = 0.f;
        for (int c0 = 0; c0 < H; c0 += 16) {
          uint32_t v1[16];
          load_tok(t, c0, v1);
          ptx::tmem_ld_wait();
          const float4* w4 = reinterpret_cast<const float4*>(w_s + t * H + c0);
#pragma unroll
          for (int j4 = 0; j4 < 4; ++j4) {
            const float4 w = w4[j4];
            sum = fmaf(w.x, fmaxf(__uint_as_float(v1[4 * j4 + 0]), 0.f), sum);
            sum = fmaf(w.y, fmaxf(__uint_as_float(v1[4 * j4 + 1]), 0.f), sum);
            sum = fmaf(w.z, fmaxf(__uint_as_float(v1[4 * j4 + 2]), 0.f), sum);
            sum = fmaf(w.w, fmaxf(__uint_as_float(v1[4 * j4 + 3]), 0.f), sum);
          }
        }
        if (r_ok) *sp = r < (int64_t)vis_s[t] ? sum : -INFINITY;
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&acc_empty[a]);
      if (quad == 0) TR(5, i);
    }
  }

  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_base, (uint32_t)p.tmem_cols);
#if !defined(MXB_TRACE) && !defined(MXB_TRACE_MMA)
  if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
#endif
}

template <int D, int MODE>
static int launch_fp8_d(Fp8Params& p, const mxb_indexer_scores_args* a, cudaStream_t st) {
  using C = Fp8Cfg<D, MODE>;
  constexpr bool DIRECT = MODE == kDirect;
  constexpr bool K16 = MODE == kKeys16;
  const int cols_per_token = (DIRECT ? 2 : 1) * p.H;
  int t_tile = 256 / cols_per_token;
  if (t_tile > p.T) t_tile = p.T;
  p.t_tile = t_tile;
  p.N = t_tile * cols_per_token;
  p.acc_stride = (int)round_up(p.N, 32);
  int n_acc = 512 / p.acc_stride;
  if (n_acc > 8) n_acc = 8;
  n_acc &= ~1;   // even: the two MMA issuers stride the ring by two
  p.n_acc = n_acc;
  int cols = 32;
  while (cols < n_acc * p.acc_stride) cols <<= 1;
  p.tmem_cols = cols;
  p.b_bytes = (int)round_up((int64_t)p.N * D * (DIRECT ? 1 : 2), 1024);
  const int64_t t_tiles = ceil_div(p.T, t_tile);
  const int64_t tiles = ceil_div(p.n_rows, 128);
  const int smem = C::b_off + p.b_bytes + 256 * 4 + 256 * 4 + 56 * 8 + 64 + 1024;
  const int ctas_per_sm = smem <= 113 * 1024 ? 2 : 1;
  // static chunks of rows per CTA, several per resident slot so that ragged sequences balance
  int64_t want_ctas = (int64_t)sm_count() * ctas_per_sm * 6;
  int64_t per = ceil_div(tiles * p.B * t_tiles, want_ctas);
  if (per < 16) per = 16;
  if (per > tiles) per = tiles;
  // Equal-length sequences (one prefill chunk): all CTAs cost the same, so a grid of 1.7 waves wastes the
  // difference to 2.  Cut the rows so that one wave holds everything when that leaves enough tiles per CTA.
  const int64_t slots = (int64_t)sm_count() * (p.tmem_cols > 256 ? 1 : ctas_per_sm);   // 512 TMEM columns: one CTA per SM
  if (!p.row_count && p.B * t_tiles <= slots) {
    const int64_t gx = slots / (p.B * t_tiles);
    const int64_t one_wave = ceil_div(tiles, gx);
    if (one_wave >= 8) per = one_wave;
  }
  p.rows_per_cta = (int)(per * 128);

  CUtensorMap tmap;
  int rc;
  if (K16) {
    uint64_t dims[2] = {(uint64_t)D, (uint64_t)a->rows_total};
    uint64_t strides[1] = {(uint64_t)D * 2};
    uint32_t box[2] = {64u, 128u};
    rc = make_tensor_map(&tmap,
                         a->key_dtype == MXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16,
                         2, a->keys, dims, strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
  } else {
    uint64_t dims[2] = {(uint64_t)D, (uint64_t)a->rows_total};
    uint64_t strides[1] = {(uint64_t)D};
    uint32_t box[2] = {(uint32_t)D, 128u};
    const CUtensorMapSwizzle sw = !DIRECT ? CU_TENSOR_MAP_SWIZZLE_NONE
                                          : (D == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B);
    rc = make_tensor_map(&tmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, a->keys, dims, strides, box, sw);
  }
  if (rc != MXB_OK) return rc;
  auto kern = indexer_fp8_kernel<D, MODE>;
  MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((unsigned)ceil_div(p.n_rows, p.rows_per_cta), (unsigned)t_tiles, (unsigned)p.B);
  kern<<<grid, C::kThreads, smem, st>>>(tmap, p);
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

// FP8 key tables (widened or fed to the FP8 tensor path) and 16-bit key tables (bf16 / fp16, same type as q).
int launch_indexer_fp8(const mxb_indexer_scores_args* a, cudaStream_t st) {
  Fp8Params p{};
  p.keys = reinterpret_cast<const uint8_t*>(a->keys); p.rows_total = a->rows_total;
  p.q = a->q; p.q_is_bf16 = a->q_dtype == MXB_BF16;
  p.q_sb = a->q_stride_b; p.q_sh = a->q_stride_h; p.q_st = a->q_stride_t;
  p.weights = a->weights; p.scores = a->scores; p.s_sb = a->score_stride_b; p.s_st = a->score_stride_t;
  p.row_start = a->row_start; p.row_count = a->row_count;
  p.B = a->B; p.T = a->T; p.H = a->H; p.n_rows = a->n_rows; p.pos0 = a->pos0; p.ratio = a->ratio;
  p.status = a->status;
  if (a->key_dtype != MXB_F8E4M3)
    return a->D == 64 ? launch_fp8_d<64, kKeys16>(p, a, st) : launch_fp8_d<128, kKeys16>(p, a, st);
  const bool direct = (a->flags & MXB_INDEXER_FP8_MMA) != 0;
  if (a->D == 64) return direct ? launch_fp8_d<64, kDirect>(p, a, st) : launch_fp8_d<64, kWiden>(p, a, st);
  return direct ? launch_fp8_d<128, kDirect>(p, a, st) : launch_fp8_d<128, kWiden>(p, a, st);
}

}  // namespace mxb
