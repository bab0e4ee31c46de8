// Indexed mixed (sparse) attention on tcgen05 / TMEM for 16-bit and int8 KV tables, warp-specialised.
//
// One CTA = one (sequence, token, split of its row list): all heads (<= 64) of that token share every
// gathered row.  The row list (raw window rows, then the selected compressed rows) is cut into UNITS of 64
// rows.  The gathered rows sit on the MMA M axis:
//
//   S^T[64 rows  x 64 heads]  = Kunit[64 x Dqk] . Q^T             (M = 64)
//   O^T[Dv dims  x 64 heads] += Vunit^T[Dv x 64] . P^T            (M = 128, A read MN-major)
//
// Twenty warps:
//   warps 0-7    softmax, one unit at a time.  An M = 64 accumulator occupies lanes 0-15 of each 32-lane
//                quarter of TMEM; thread = (row, 16 heads)
//   warps 8, 9   issue S^T (measured: a thread issues one tcgen05.mma per ~105 cycles whatever its shape; four
//                threads together reach one per ~37 cycles for M = 64, ~53 for M = 128)
//   warps 10, 11 issue O^T += V^T P^T for the value blocks 0-1 / 2-3; every 128-feature block has a barrier of its
//                own, so that its two slabs can be refilled while the other blocks are still being multiplied
//   warps 12-19  (int8 tables: 12-15) resolve list entries to rows ahead of time and bring the rows in by TMA row
//                gathers (tile::gather4: four rows x one slab per instruction, swizzled on the way in, row -1 =
//                zeros).  Loads through registers are not used for rows: measured, an SM sustains ~5 bytes per
//                clock of gathered row pieces that way whatever their source, several times that through TMA.
//   warps 16-19  int8 tables only: widen the value features of a landed unit
//
// 16-bit tables: two operand buffers (64-feature slabs of [64 rows x 128 B]) alternate; one staged copy of a
// unit feeds both contractions (K-major for the logits, MN-major for the values) and nothing is transposed.  The
// two logit issuers split the slabs, each into an accumulator of its own that the softmax adds, and multiply a
// slab as soon as it has landed.
//
// int8 tables: the logits run on the int8 tensor-core path (kind::i8, int32 accumulation) straight from the rows as
// they are stored.  The gathers land the int8 rows in operand layout (128-feature slabs, two buffers); q is held
// as two int8 digit planes of a per-head 15-bit fixed-point number, q = (256 hi + lo) step_h, stacked on the MMA N
// axis (N = 128), so S^T = step_h (256 S_hi + S_lo) is exact integer arithmetic and q is never rounded to fp16.
// Only the values need 16-bit operands: the producers widen the first Dv features of a landed unit to exact fp16
// integers into ONE value buffer, block by block behind the previous unit's P V and in parallel with the softmax
// of this one; the per-row scale is folded into the logit and into P.
// Operand type of the 16-bit contractions: bf16 for bf16 tables, fp16 otherwise (16-bit tables: q rounded to the
// table's type, as the reference kernels round it to fp16).
//
// The softmax keeps one per-head reference maximum m_ref in shared memory, moved only when a logit exceeds it by
// more than a gap (2^15 for fp16 operands, 2^60 for bf16); O^T in TMEM is rescaled only then, after the previous
// unit's P V has completed.  The row sum uses the ROUNDED 16-bit P values, so out = sum(p~ v) / sum(p~) is an
// exactly normalised average.  Splits over the row list emit (o, m, l) partials for the log-sum-exp merge kernel.
//
// TMEM columns: S^T of even units [0,128), of odd units [128,256) (two accumulators of 64 columns, or the hi and
// lo planes), O^T at [256, 256 + Dv/2).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "sparse_attn.cuh"

namespace mxb {

#ifdef MXB_TRACE_SP   // development aid: cycle stamps of CTA 0's roles for its first 16 units, written behind `status`
#define TRS(k, i) do { if (tr_on && (i) < 16) tr[(k) * 16 + (i)] = clock64(); } while (0)   // needs 16 x 16 slots
#else
#define TRS(k, i)
#endif

constexpr int WS_UNIT = 64;       // gathered rows per unit
constexpr int WS_HEADS = 64;      // heads per CTA (MMA N; two planes of 64 for int8 tables)
constexpr int WS_MAX_SLABS = 9;   // Dqk <= 576
constexpr int WS_SLAB = 8192;     // [64 rows or heads] x 128 B
constexpr int WS_THREADS = 640;   // 20 warps
constexpr int kWsMiscBytes = 10240;
constexpr int kRing = 8;          // units of row metadata kept in shared memory (a slot is rewritten six units later)
constexpr int kMaxClusterMerge = 4;   // splits of a token that can merge through shared memory
// An operand weight 2^(s - m_ref) may be as large as 2^gap.  bf16 operands have fp32's range; fp16 operands top out
// at 65504.  (The int8 path folds the row's dequantisation scale into the weight: there s = logit + log2(scale).)
constexpr float kRescaleGapF16 = 15.f;
constexpr float kRescaleGapBF16 = 60.f;
// A reference that moves is put this far above the unit's maximum (fp16 operands): moving it costs a wait for the
// previous P V and a pass over O^T, and the maxima of the first units of a list are still far from the list's.  The
// largest weight of a head is then at least 2^-kRescaleHeadroom, 10 bits above fp16's smallest normal number: weights
// below a thousandth of the largest one are the first to lose precision.
constexpr float kRescaleHeadroom = 4.f;
constexpr uint32_t kNoRow = 0xFFFFFFFFu;

struct WsLayout {
  int nslab;        // Dqk / 64: 64-feature slabs of 16-bit operands
  int n128, tail;   // int8 operands: full 128-feature slabs, and 64 tail features (0 or 64) in a 64-byte-swizzled slab
  int q_off;        // q operand.  16-bit: nslab slabs of [64 heads x 128 B]; int8: [128 rows x 128 B] slabs (+ [128 x 64 B])
  int ub_off[2];    // 16-bit operand buffers of a unit (int8 tables: one value buffer of Dv / 64 slabs)
  int pt_off[2];    // P^T of the unit in buffer b: [64 heads x 128 B] (64 rows of 16 bits)
  int kb_off[2];    // int8 tables: the two int8 row buffers, n128 slabs of [64 rows x 128 B] (+ [64 x 64 B])
  int qtmp_off;     // int8 tables: where a 16-bit q lands before it is turned into digit planes (-1: no room)
  int misc_off;
  int total;
};

__host__ __device__ inline WsLayout ws_layout(int Dqk, int Dv, bool i8) {
  WsLayout L;
  L.nslab = Dqk / 64;
  L.n128 = Dqk / 128;
  L.tail = Dqk % 128;
  L.q_off = 0;
  L.qtmp_off = -1;
  L.kb_off[0] = L.kb_off[1] = 0;
  int end;
  if (i8) {
    const int q_bytes = L.n128 * 2 * WS_SLAB + (L.tail ? WS_SLAB : 0);
    const int k_bytes = WS_UNIT * Dqk;
    L.kb_off[0] = q_bytes;
    L.kb_off[1] = q_bytes + k_bytes;
    L.ub_off[0] = L.ub_off[1] = (q_bytes + 2 * k_bytes + 1023) & ~1023;
    L.pt_off[0] = L.pt_off[1] = L.ub_off[0] + (Dv / 64) * WS_SLAB;
    end = L.pt_off[0] + WS_SLAB;
    if (end - L.ub_off[0] >= L.nslab * WS_SLAB) L.qtmp_off = L.ub_off[0];   // value buffer + P^T hold a 16-bit q
  } else {
    L.ub_off[0] = L.nslab * WS_SLAB;
    L.ub_off[1] = 2 * L.nslab * WS_SLAB;
    end = 3 * L.nslab * WS_SLAB;
    if (Dqk - Dv >= 64) {
      // the last slab feeds only the logits: it is free once S^T of its unit is complete
      L.pt_off[0] = L.ub_off[0] + (L.nslab - 1) * WS_SLAB;
      L.pt_off[1] = L.ub_off[1] + (L.nslab - 1) * WS_SLAB;
    } else {
      L.pt_off[0] = end;
      L.pt_off[1] = end + WS_SLAB;
      end += 2 * WS_SLAB;
    }
  }
  L.misc_off = (end + 15) & ~15;
  L.total = L.misc_off + kWsMiscBytes;
  return L;
}

struct WsMisc {
  float m_ref[WS_HEADS];
  float factor[WS_HEADS];          // of the latest move of m_ref; the output factors at the end
  float l_tot[WS_HEADS];
  float colmax[4][WS_HEADS];       // per row quarter; reused for the row sums at the end
  float q_step[WS_HEADS];          // int8 tables: q[h, :] = (256 hi + lo) * q_step[h]
  float v_bias[WS_HEADS];          // int8 tables: kValueBias x (sum of the fp16 weights), taken off O^T at the end
  float xm[kMaxClusterMerge][WS_HEADS];   // cluster merge: every split's reference maximum (log2 units) and
  float xl[kMaxClusterMerge][WS_HEADS];   //   denominator, written here by the splits themselves (remote stores)
  uint32_t q_amax[WS_HEADS];       // bits of max |q[h, :]|
  uint32_t row_ref[kRing][WS_UNIT];   // kNoRow, or row index within its table (< 2^31), bit 31 set for the raw table
  float row_scale[kRing][WS_UNIT];
  uint64_t q_full, q_ready;
  uint64_t full[2][WS_MAX_SLABS];  // a slab of the unit in row buffer b has landed
  uint64_t v_full[4];              // int8 tables: a 128-feature block of the value buffer has been widened
  uint64_t k_free[2];              // int8 tables: the widening warps have read row buffer b
  uint64_t meta_ready;             // int8 tables: the scales of units 0 and 1 have been published
  uint64_t s_ready[2], s_free[2], p_ready[2];
  uint64_t p_summed;               // int8 tables: the widening warps have added a unit's P^T to the row sums
  float row_inv[2][WS_UNIT];       // int8 tables: 1 / row scale of the unit whose P^T is in the buffer (by unit parity)
  int grew[2];                     // int8 tables: the reference maxima moved before this unit's P^T (by unit parity)
  uint64_t pv_blk[2][4];           // P V of one 128-feature block of the unit in buffer b has completed: its two slabs are free
  uint32_t tmem_slot;
  int abort_flag;
  int keff;
};
static_assert(sizeof(WsMisc) <= kWsMiscBytes, "WsMisc must fit the bytes the layout reserves for it");

// 16 int8 -> 16 fp16 values v + kValueBias (exact): the byte, biased by 128, is dropped into the mantissa of
// 1024.0.  The bias stays in the operand: O^T accumulates sum P (v + bias), and bias x sum P (the sum of the very
// fp16 weights the MMA reads) is taken off once, in the epilogue.  The products are exact in fp32 and the bias
// term is at most ~9 x the value term, so the cancellation costs about three of the accumulator's 24 bits.
constexpr float kValueBias = 1152.f;
__device__ __forceinline__ void widen_i8x16_f16(const uint4& in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x ^ 0x80808080u, in.y ^ 0x80808080u, in.z ^ 0x80808080u, in.w ^ 0x80808080u};
  lo = make_uint4(__byte_perm(w[0], 0x64646464u, 0x4140), __byte_perm(w[0], 0x64646464u, 0x4342),
                  __byte_perm(w[1], 0x64646464u, 0x4140), __byte_perm(w[1], 0x64646464u, 0x4342));
  hi = make_uint4(__byte_perm(w[2], 0x64646464u, 0x4140), __byte_perm(w[2], 0x64646464u, 0x4342),
                  __byte_perm(w[3], 0x64646464u, 0x4140), __byte_perm(w[3], 0x64646464u, 0x4342));
}

// Sums a[c] over the 16 lanes of a half warp: at each step a lane keeps half of its columns and hands the other
// half to its partner, so 15 shuffles leave lane li with column li in a[0].
__device__ __forceinline__ float half_warp_column_sum(float (&a)[16], int li) {
#pragma unroll
  for (int step = 8; step >= 1; step >>= 1) {
    const bool upper = (li & step) != 0;
#pragma unroll
    for (int c = 0; c < step; ++c) {
      const float send = upper ? a[c] : a[c + step];
      const float keep = upper ? a[c + step] : a[c];
      a[c] = keep + __shfl_xor_sync(0xffffffffu, send, step);
    }
  }
  return a[0];
}

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Two floats -> two operand-type values in one register (low half = a), and what they round back to.
template <bool BF16>
__device__ __forceinline__ uint32_t pack_op16x2(float a, float b, float& back_a, float& back_b) {
  if constexpr (BF16) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    const float2 f = __bfloat1622float2(v);
    back_a = f.x;
    back_b = f.y;
    return *reinterpret_cast<const uint32_t*>(&v);
  } else {
    const __half2 v = __floats2half2_rn(a, b);
    const float2 f = __half22float2(v);
    back_a = f.x;
    back_b = f.y;
    return *reinterpret_cast<const uint32_t*>(&v);
  }
}

// order-preserving map between floats (no NaN) and signed integers
__device__ __forceinline__ int float_order(float x) {
  const int i = __float_as_int(x);
  return i ^ ((i >> 31) & 0x7fffffff);
}
__device__ __forceinline__ float order_float(int i) { return __int_as_float(i ^ ((i >> 31) & 0x7fffffff)); }

__device__ __forceinline__ void group_sync(int id, int nthreads) {
  asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(nthreads) : "memory");
}
// barrier 4 over the 256 softmax threads with an OR reduction of `pred`
__device__ __forceinline__ bool __syncthreads_or_256(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n\t"
      ".reg .pred p, q;\n\t"
      "setp.ne.b32 p, %1, 0;\n\t"
      "bar.red.or.pred q, 4, 256, p;\n\t"
      "selp.b32 %0, 1, 0, q;\n\t"
      "}"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

template <int KVT, int QT, int OT>
__global__ void __launch_bounds__(WS_THREADS, 1)
sparse_attn_tc_kernel(SparseParams p, const __grid_constant__ CUtensorMap tm_comp,
                      const __grid_constant__ CUtensorMap tm_raw, const __grid_constant__ CUtensorMap tm_comp_tail,
                      const __grid_constant__ CUtensorMap tm_raw_tail, const __grid_constant__ CUtensorMap tm_q) {
  constexpr bool I8 = (KVT == MXB_I8);
  constexpr bool BF16 = (KVT == MXB_BF16);       // type of the 16-bit operands: bf16 for bf16 tables, fp16 otherwise
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const WsLayout L = ws_layout(p.Dqk, p.Dv, I8);
  uint8_t* q_s = smem + L.q_off;
  // buffer b of a pair sits at first + b * stride (no run-time index into L: that would push it to local memory)
  const int ub0 = L.ub_off[0], ub_st = L.ub_off[1] - L.ub_off[0];
  const int pt0 = L.pt_off[0], pt_st = L.pt_off[1] - L.pt_off[0];
  const int kb0 = L.kb_off[0], kb_st = L.kb_off[1] - L.kb_off[0];
  WsMisc* mi = reinterpret_cast<WsMisc*>(smem + L.misc_off);
  volatile int* abort_flag = &mi->abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const unsigned cta = blockIdx.x + (unsigned)p.cta_base;
  const int bt = (int)(cta / (unsigned)p.nsplit);
  const int split = (int)(cta - (unsigned)bt * (unsigned)p.nsplit);
  const int b = bt / p.T, t = bt % p.T;
  const int nslab = L.nslab;
  const int n_mt = p.Dv / 128;
  // Row buffers and S^T alternate with the unit's parity.  The value operand (and P^T) of a unit: 16-bit tables
  // read it from the unit's own row buffer, int8 tables have one value buffer.
  auto sbuf = [](int u) { return u & 1; };
  auto sphase = [](int u) { return (uint32_t)((u >> 1) & 1); };
  auto pbuf = [](int u) { return I8 ? 0 : (u & 1); };
  auto pphase = [](int u) { return (uint32_t)((I8 ? u : (u >> 1)) & 1); };
  // slabs of a row buffer: 16-bit tables nslab slabs of 64 features, int8 tables n128 slabs of 128 features and
  // the 64-feature tail; [slab_lo(j), slab_lo(j + 1)) go to logit issuer j of the 16-bit path
  const int nrs = I8 ? L.n128 + (L.tail ? 1 : 0) : nslab;
  auto slab_lo = [&](int j) { return (nslab * j + 1) / 2; };
  // P V of unit u: one barrier per 128-feature block.  The slabs beyond the value width (the rotary slab of a
  // 16-bit unit, where P^T lives) are free when every block is done.
  auto wait_pv_block = [&](int u, int mt) { ptx::mbar_wait(&mi->pv_blk[pbuf(u)][mt], pphase(u), abort_flag); };
  auto wait_pv_all = [&](int u) {
    for (int mt = 0; mt < n_mt; ++mt) wait_pv_block(u, mt);
  };
  auto wait_pv_slab = [&](int u, int slab) {   // before 16-bit slab `slab` of the buffer that unit u used is overwritten
    if (slab < 2 * n_mt) wait_pv_block(u, slab >> 1);
    else wait_pv_all(u);
  };

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
  // The list of entries: raw rows, padding up to a multiple of four (a TMA gather fetches four rows of ONE
  // table), then the selected compressed rows.
  const int n_raw_pad = (n_raw + 3) & ~3;
  const int32_t* ids = p.topk + (int64_t)bt * p.k;
#ifdef MXB_TRACE_SP
  long long* tr = reinterpret_cast<long long*>(p.status);
  const bool tr_on = p.status && blockIdx.x == 0 && (lane == 0);
  if (tid == 0) TRS(11, 0);
#endif

  if (tid == 0) {
    ptx::mbar_init(&mi->q_full, 1);
    ptx::mbar_init(&mi->q_ready, I8 ? (uint32_t)(WS_THREADS - 128) : 256u);
    for (int i = 0; i < 2; ++i) {
      for (int kb = 0; kb < WS_MAX_SLABS; ++kb) ptx::mbar_init(&mi->full[i][kb], 1);
      ptx::mbar_init(&mi->s_ready[i], I8 ? 1u : 2u);
      ptx::mbar_init(&mi->s_free[i], 256);
      ptx::mbar_init(&mi->p_ready[i], 256);
      for (int mt = 0; mt < 4; ++mt) ptx::mbar_init(&mi->pv_blk[i][mt], 1);
    }
    for (int mt = 0; mt < 4; ++mt) ptx::mbar_init(&mi->v_full[mt], 4);
    ptx::mbar_init(&mi->k_free[0], 4);
    ptx::mbar_init(&mi->k_free[1], 4);
    ptx::mbar_init(&mi->meta_ready, (uint32_t)WS_UNIT);
    ptx::mbar_init(&mi->p_summed, 4);
    mi->abort_flag = 0;
    mi->keff = p.k;
    ptx::mbar_fence_init();
  }
  if (tid == 384) {   // the row tables' descriptors are on their way while the barriers and TMEM are set up
    ptx::tma_prefetch_desc(&tm_comp);
    if (p.raw_cap > 0) ptx::tma_prefetch_desc(&tm_raw);
    if (I8 && (p.Dqk & 127) != 0) {   // the 64-feature tail slab has maps of its own
      ptx::tma_prefetch_desc(&tm_comp_tail);
      if (p.raw_cap > 0) ptx::tma_prefetch_desc(&tm_raw_tail);
    }
  }
  if (tid < WS_HEADS) {
    mi->m_ref[tid] = -INFINITY;
    mi->factor[tid] = 1.f;
    mi->l_tot[tid] = 0.f;
    mi->q_amax[tid] = 0u;
  }
  __syncwarp();
  if (warp == 0) {
    ptx::tmem_alloc(&mi->tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = mi->tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;

  // ------------------------------------------------------------------ q on its way, and the list scan
  // A 16-bit q that a tensor map can describe lands by TMA as 64-feature slabs of [64 heads x 128 B] (heads beyond
  // H arrive as zeros): in place as the B operand for 16-bit tables, in a scratch region (the value buffer) for
  // int8 tables, where it is turned into digit planes.  Otherwise q goes through registers.
  uint8_t* q_land = I8 ? smem + (L.qtmp_off >= 0 ? L.qtmp_off : 0) : q_s;
  if (p.q_tma) {
    if (tid == 256) {
      ptx::tma_prefetch_desc(&tm_q);
      ptx::mbar_expect_tx(&mi->q_full, (uint32_t)(nslab * WS_SLAB));
      int32_t c[3];
#pragma unroll
      for (int i = 0; i < 3; ++i) c[i] = p.q_axis[i] == 0 ? 0 : (p.q_axis[i] == 1 ? t : b);
      for (int kb = 0; kb < nslab; ++kb) ptx::tma_load_4d(q_land + kb * WS_SLAB, &tm_q, &mi->q_full, kb * 64, c[0], c[1], c[2]);
    }
  }
  const bool q_vec = ((reinterpret_cast<uintptr_t>(p.q) & 15) == 0) && (p.q_sb % 8 == 0) && (p.q_sh % 8 == 0) &&
                     (p.q_st % 8 == 0);
  const int n_items = WS_HEADS * (p.Dqk / 8);   // item i = (head i % 64, 8 features i / 64)
  // eight consecutive features of q as floats: from the landed copy, or from global memory
  auto load_q_item = [&](int i, float* f) {
    const int h = i & (WS_HEADS - 1), c = i >> 6;
#pragma unroll
    for (int e = 0; e < 8; ++e) f[e] = 0.f;
    if (p.q_tma) {
      if constexpr (QT != MXB_F32) {
        const uint4 u4 = *reinterpret_cast<const uint4*>(q_land + (size_t)(c >> 3) * WS_SLAB + (size_t)h * 128 +
                                                         (((c & 7) ^ (h & 7)) << 4));
        unpack16<QT>(u4, f);
      }
    } else if (h < p.H) {
      const int64_t base = (int64_t)b * p.q_sb + (int64_t)h * p.q_sh + (int64_t)t * p.q_st + c * 8;
      if (q_vec) {
        if constexpr (QT == MXB_F32) {
          const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.q) + base));
          const float4 bq = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.q) + base) + 1);
          f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = bq.x; f[5] = bq.y; f[6] = bq.z; f[7] = bq.w;
        } else {
          const uint4 u4 = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + base));
          unpack16<QT>(u4, f);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = load_elem<QT>(p.q, base + e);
      }
    }
  };
  {  // first list entry that ends the walk
    int mine = p.k;
#pragma unroll 4
    for (int j = tid; j < p.k; j += WS_THREADS) {   // no early exit: the loads stay independent
      const int64_t v = ids[j];
      if (v >= visible && j < mine) mine = j;
    }
    if (mine < p.k) atomicMin(&mi->keff, mine);
  }
  __syncthreads();

  const int total = n_raw_pad + mi->keff;
  int per = (total + p.nsplit - 1) / p.nsplit;
  per = ((per + WS_UNIT - 1) / WS_UNIT) * WS_UNIT;
  const int e_lo = min(split * per, total), e_hi = min(e_lo + per, total);
  const int nunits = (e_hi - e_lo + WS_UNIT - 1) / WS_UNIT;
  if (tid == 0) TRS(11, 1);

  constexpr uint32_t fmt = BF16 ? ptx::kFmtBF16 : ptx::kFmtF16;
  const float scale_log2 = p.scale * 1.4426950408889634f;

  if constexpr (I8) {
    // ---- q as two int8 digit planes, by every warp but the four that are already gathering rows
    // Per head h: step_h = 2^(e - 13) with 2^e <= max |q[h, :]| < 2^(e + 1); Q = round(q / step_h), |Q| <= 2^14;
    // Q = 256 hi + lo with lo in [-128, 127]: lo is the low byte of Q and hi the second byte of Q + 128.  Rows h (hi)
    // and 64 + h (lo) of the B operand: 128-feature slabs of [128 rows x 128 B] with the 128-byte swizzle, the 64
    // tail features in [128 rows x 64 B] with the 64-byte one.
    if (warp < 12 || warp >= 16) {
      constexpr int NST = WS_THREADS - 128;
      const int st = warp < 12 ? tid : tid - 128;
      if (p.q_tma) ptx::mbar_wait(&mi->q_full, 0, abort_flag);
      float amax = 0.f;
      for (int i = st; i < n_items; i += NST) {   // i % 64 = st % 64: one head per thread
        float f[8];
        load_q_item(i, f);
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
      }
      atomicMax(&mi->q_amax[st & (WS_HEADS - 1)], __float_as_uint(amax));
      group_sync(6, NST);
      const uint32_t abits = mi->q_amax[st & (WS_HEADS - 1)];
      const int ex = (int)(abits >> 23) - 127;   // floor(log2(max)); zeros and denormals: a harmless tiny step
      const float step = abits == 0u ? 1.f : __uint_as_float((uint32_t)(max(ex - 13, -126) + 127) << 23);
      const float inv_step = 1.f / step;
      if (st < WS_HEADS) mi->q_step[st] = step;
      for (int i = st; i < n_items; i += NST) {
        const int h = i & (WS_HEADS - 1), c = i >> 6;
        float f[8];
        load_q_item(i, f);
        uint32_t hi_w[2], lo_w[2];
#pragma unroll
        for (int w = 0; w < 2; ++w) {
          // round(q / step) by one fused multiply-add: adding 1.5 * 2^23 leaves the integer (|Q| <= 2^14 by the choice
          // of the step, rounded to nearest even like a conversion) in the low mantissa bits, in two's complement
          uint32_t Q[4];
#pragma unroll
          for (int e = 0; e < 4; ++e) Q[e] = __float_as_uint(fmaf(f[4 * w + e], inv_step, 12582912.f));
          lo_w[w] = __byte_perm(__byte_perm(Q[0], Q[1], 0x0040), __byte_perm(Q[2], Q[3], 0x0040), 0x5410);
          hi_w[w] = __byte_perm(__byte_perm(Q[0] + 128u, Q[1] + 128u, 0x0051), __byte_perm(Q[2] + 128u, Q[3] + 128u, 0x0051), 0x5410);
        }
        const int f0 = c * 8;
        if (f0 < L.n128 * 128) {
          uint8_t* base = q_s + (size_t)(f0 >> 7) * 2 * WS_SLAB + (f0 & 8);
          const int ck = (f0 & 127) >> 4;
          *reinterpret_cast<uint2*>(base + (size_t)h * 128 + ((ck ^ (h & 7)) << 4)) = make_uint2(hi_w[0], hi_w[1]);
          *reinterpret_cast<uint2*>(base + (size_t)(64 + h) * 128 + ((ck ^ (h & 7)) << 4)) = make_uint2(lo_w[0], lo_w[1]);
        } else {
          const int bb = f0 - L.n128 * 128;
          uint8_t* base = q_s + (size_t)L.n128 * 2 * WS_SLAB + (bb & 8);
          const int ck = bb >> 4;
          *reinterpret_cast<uint2*>(base + (size_t)h * 64 + ((ck ^ ((h >> 1) & 3)) << 4)) = make_uint2(hi_w[0], hi_w[1]);
          *reinterpret_cast<uint2*>(base + (size_t)(64 + h) * 64 + ((ck ^ (((64 + h) >> 1) & 3)) << 4)) =
              make_uint2(lo_w[0], lo_w[1]);
        }
      }
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(&mi->q_ready);
    }
  }

  constexpr int NG = I8 ? 4 : 8;   // gather warps (int8 tables: the other four producer warps widen the values)
  if (warp >= 12 && warp < 12 + NG) {
    // ================================================================ row gathers
    const int pt = tid - 384;             // threads 0-63 resolve entry pt of every unit
    const bool resolver = pt < WS_UNIT;
    // Row metadata (list id -> row -> dequantisation scale) is a chain of dependent global loads, run as a
    // pipeline, one stage per unit, so that nobody waits on it: stage A fetches the list id, stage B turns it
    // into the row and fetches the scale; the last stage publishes both in shared memory two units before they
    // are needed.
    auto fetch_id = [&](int U) -> int32_t {   // -1: no compressed row behind this slot
      if (!resolver || U >= nunits) return -1;
      const int e = e_lo + U * WS_UNIT + pt;
      return (e < e_hi && e >= n_raw_pad) ? ids[e - n_raw_pad] : -1;
    };
    auto fetch_row = [&](int U, int32_t id, uint32_t& ref, float& rs) {
      ref = kNoRow;
      rs = 1.f;
      if (!resolver || U >= nunits) return;
      const int e = e_lo + U * WS_UNIT + pt;
      if (e >= e_hi) return;
      int64_t ridx;
      bool raw;
      if (e < n_raw) {
        const int64_t pabs = first + e;
        const int64_t phys = ((int64_t)p.raw_start + (pabs - first_raw_pos)) % p.raw_cap;
        ridx = (int64_t)b * p.raw_cap + phys;
        raw = true;
      } else if (e >= n_raw_pad && id >= 0) {
        ridx = cbase + id;
        raw = false;
      } else {
        return;
      }
      ref = (uint32_t)ridx | (raw ? 0x80000000u : 0u);
      // (a zero scale, i.e. an all-zero row, still counts in the denominator: it is taken as fp16's smallest number)
      if (I8) rs = fmaxf(__half2float(raw ? p.raw_scales[ridx] : p.comp_scales[ridx]), 5.9604645e-8f);
    };
    auto publish_ref = [&](int U, uint32_t ref) {
      if (resolver && U < nunits) mi->row_ref[U & (kRing - 1)][pt] = ref;
    };
    auto publish_scale = [&](int U, float rs) {
      if (I8 && resolver && U < nunits) mi->row_scale[U & (kRing - 1)][pt] = rs;
    };
    int32_t id_a = -1;          // stage A result: list id of this thread's entry of unit v + 3
    uint32_t src_b = kNoRow;    // stage B result: row and scale of this thread's entry of unit v + 2
    float rs_b = 1.f;
    float rs0 = 1.f, rs1 = 1.f;   // scales of units 0 and 1: published behind the first gathers
    if (pt == 0) TRS(14, 0);
    if (nunits > 0) {
      const int32_t i0 = fetch_id(0), i1 = fetch_id(1), i2 = fetch_id(2);
      id_a = fetch_id(3);
      uint32_t s0, s1;
      fetch_row(0, i0, s0, rs0);
      fetch_row(1, i1, s1, rs1);
      fetch_row(2, i2, src_b, rs_b);
      publish_ref(0, s0);
      publish_ref(1, s1);
    }
    group_sync(5, NG * 32);
    if (pt == 0) TRS(14, 3);
    for (int v = 0; v < nunits; ++v) {
      const int buf = v & 1, slot = v & (kRing - 1);
      if (pt == 0) TRS(0, v);
      if (I8 && v >= 2) {
        // row buffer `buf` is free once the widening warps and the logit MMAs of unit v - 2 have read it
        ptx::mbar_wait(&mi->k_free[buf], sphase(v - 2), abort_flag);
        ptx::mbar_wait(&mi->s_ready[buf], sphase(v - 2), abort_flag);
      }
      if (pt == 0) TRS(1, v);
      // Unit v into row buffer v & 1, slab by slab (so that the logit MMAs of the first slabs can start while the
      // later ones travel); a thread owns (slab, group of four rows) pairs; rows without data are fetched from
      // row -1 (zeros).
      uint8_t* rb = smem + (I8 ? (kb0 + (buf) * kb_st) : (ub0 + (buf) * ub_st));
      if (pt == 0)
        for (int sl = 0; sl < nrs; ++sl)
          ptx::mbar_expect_tx(&mi->full[buf][sl], (uint32_t)((I8 && sl == L.n128) ? WS_UNIT * 64 : WS_SLAB));
      // (One TMA operation per instruction, a lane at a time, was measured three times slower: the operations of
      // one warp-wide instruction pipeline, separate instructions of a warp do not.)
      for (int i = pt; i < 16 * nrs; i += NG * 32) {
        const int sl = i >> 4, r0 = (i & 15) * 4;
        if (!I8 && v >= 2) wait_pv_slab(v - 2, sl);   // this slab has been multiplied by P V of unit v - 2
        uint32_t ref[4];
        bool from_raw = false;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          ref[j] = mi->row_ref[slot][r0 + j];
          if (ref[j] != kNoRow && (ref[j] >> 31)) from_raw = true;
        }
        int32_t y[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) y[j] = ref[j] != kNoRow ? (int32_t)(ref[j] & 0x7FFFFFFFu) : -1;
        if (I8 && sl == L.n128)
          ptx::tma_gather4_2d(rb + (size_t)sl * WS_SLAB + (size_t)r0 * 64, from_raw ? &tm_raw_tail : &tm_comp_tail,
                              &mi->full[buf][sl], sl * 128, y[0], y[1], y[2], y[3]);
        else
          ptx::tma_gather4_2d(rb + (size_t)sl * WS_SLAB + (size_t)r0 * 128, from_raw ? &tm_raw : &tm_comp,
                              &mi->full[buf][sl], I8 ? sl * 128 : sl * 64, y[0], y[1], y[2], y[3]);
      }
      if (pt == 0) TRS(2, v);
      if (I8 && v == 0 && resolver) {
        publish_scale(0, rs0);
        publish_scale(1, rs1);
        ptx::mbar_arrive(&mi->meta_ready);
      }
      // a metadata slot is rewritten six units after its unit: that unit's softmax is long over, because the
      // buffer wait above implies that the softmax of unit v - 4 has started
      publish_ref(v + 2, src_b);
      publish_scale(v + 2, rs_b);
      fetch_row(v + 3, id_a, src_b, rs_b);
      id_a = fetch_id(v + 4);
      group_sync(5, NG * 32);
    }
  } else if (warp >= 12 + NG) {
    // ================================================================ widening (warps 16-19, int8 tables)
    // The int8 rows land in operand layout and feed the logit MMAs as they are; only the values need 16-bit
    // operands.  An item = 8 rows x the 64 features of one fp16 slab = one warp instruction of 16-byte chunks
    // (lane = row % 8 + 8 * chunk): the rows have 8 different swizzle phases, so the 128-bit shared-memory loads
    // and stores are conflict-free.  Warp cw takes the row groups cw and cw + 4 of every slab, four slabs (two
    // 128-feature blocks) at a time; a block is announced as soon as every warp has stored its items of it, and
    // may be overwritten as soon as the previous unit's P V has multiplied it.  Every address is a per-lane base
    // plus a compile-time offset.
    if constexpr (I8) {
      const int cw = warp - (12 + NG);
      const int r8 = lane & 7, cl = lane >> 3;
      const int nsl = p.Dv / 64;   // fp16 slabs of the value buffer
      const uint32_t row_off = (uint32_t)(cw * 8 + r8) * 128;
      const uint32_t src_lo = row_off + (uint32_t)((cl ^ r8) << 4), src_hi = src_lo ^ 64u;   // features 0-63 / 64-127 of an int8 slab
      const uint32_t dst0 = row_off + (uint32_t)(((2 * cl) ^ r8) << 4), dst1 = dst0 ^ 16u;
      // These warps also keep the row sums of P^T, so that the softmax warps do not have to: thread = (head, half
      // of the unit's rows) reads its 32 fp16 weights of a finished P^T from shared memory and adds them up, once
      // as they are (for the value bias) and once divided by the row scale (the softmax denominator).  When the
      // reference maxima moved before a unit, the sums so far are rescaled first, as O^T was.
      const int sh = (cw * 32 + lane) & (WS_HEADS - 1), shalf = (cw * 32 + lane) >> 6;
      float l_run = 0.f, w_run = 0.f;
      auto add_unit = [&](int v) {
        ptx::mbar_wait(&mi->p_ready[0], pphase(v), abort_flag);
        if (mi->grew[v & 1]) {
          const float f = mi->factor[sh];
          l_run *= f;
          w_run *= f;
        }
        const uint8_t* prow = smem + pt0 + (size_t)sh * 128;
        float ls = 0.f, ws = 0.f;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int c = 4 * shalf + i;   // rows 8 c .. 8 c + 7
          const uint4 x = *reinterpret_cast<const uint4*>(prow + ((c ^ (sh & 7)) << 4));
          const float4 i0 = *reinterpret_cast<const float4*>(&mi->row_inv[v & 1][8 * c]);
          const float4 i1 = *reinterpret_cast<const float4*>(&mi->row_inv[v & 1][8 * c + 4]);
          const __half2* hx = reinterpret_cast<const __half2*>(&x);
          const float2 a = __half22float2(hx[0]), b2 = __half22float2(hx[1]), c2 = __half22float2(hx[2]), d = __half22float2(hx[3]);
          ws += ((a.x + a.y) + (b2.x + b2.y)) + ((c2.x + c2.y) + (d.x + d.y));
          ls = fmaf(a.x, i0.x, ls); ls = fmaf(a.y, i0.y, ls); ls = fmaf(b2.x, i0.z, ls); ls = fmaf(b2.y, i0.w, ls);
          ls = fmaf(c2.x, i1.x, ls); ls = fmaf(c2.y, i1.y, ls); ls = fmaf(d.x, i1.z, ls); ls = fmaf(d.y, i1.w, ls);
        }
        l_run += ls;
        w_run += ws;
        if (v == nunits - 1) {   // the totals, for the epilogue (the column maxima are not needed any more)
          mi->colmax[shalf][sh] = l_run;
          mi->colmax[2 + shalf][sh] = w_run;
        }
        __syncwarp();
        if (lane == 0) ptx::mbar_arrive(&mi->p_summed);
      };
      ptx::mbar_wait(&mi->q_ready, 0, abort_flag);   // q's scratch copy (in the value buffer) has been consumed
      for (int u = 0; u < nunits; ++u) {
        const int buf = u & 1;
        if (u >= 1) add_unit(u - 1);
        for (int sl = 0; sl < n_mt; ++sl) ptx::mbar_wait(&mi->full[buf][sl], sphase(u), abort_flag);   // the value features have landed
        if (cw == 0) TRS(13, u);
        const uint8_t* src = smem + (kb0 + buf * kb_st);
        uint8_t* dst = smem + ub0;
        for (int hb = 0; hb * 4 < nsl; ++hb) {
          uint4 v[8];
          if (cw == 0) TRS(16 + hb * 4, u);
#pragma unroll
          for (int j = 0; j < 8; ++j) {   // item j: slab 4 hb + j / 2, row group cw + 4 (j % 2)
            const int i = hb * 4 + (j >> 1);
            v[j] = make_uint4(0, 0, 0, 0);
            if (i < nsl) v[j] = *reinterpret_cast<const uint4*>(src + (i >> 1) * WS_SLAB + ((i & 1) ? src_hi : src_lo) + (j & 1) * 4096);
          }
          if ((hb + 1) * 4 >= nsl) {
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(&mi->k_free[buf]);   // this warp has read what it needs of the row buffer
          }
          if (cw == 0) TRS(17 + hb * 4, u);
#pragma unroll
          for (int jb = 0; jb < 2; ++jb) {
            const int blk = hb * 2 + jb;
            if (blk * 2 < nsl) {
              if (u >= 1) wait_pv_block(u - 1, blk);   // the previous unit's P V has read this block
#pragma unroll
              for (int jj = 0; jj < 4; ++jj) {
                const int j = jb * 4 + jj, i = hb * 4 + (j >> 1);
                uint4 lo, hi;
                widen_i8x16_f16(v[j], lo, hi);
                uint8_t* d = dst + i * WS_SLAB + (j & 1) * 4096;
                *reinterpret_cast<uint4*>(d + dst0) = lo;
                *reinterpret_cast<uint4*>(d + dst1) = hi;
              }
              if (cw == 0) TRS(24 + blk, u);
              ptx::fence_proxy_async_smem();
              __syncwarp();
              if (lane == 0) ptx::mbar_arrive(&mi->v_full[blk]);
              if (cw == 0) TRS(18 + (blk & 1) + (blk >> 1) * 4, u);
            }
          }
        }
        if (cw == 0) TRS(15, u);
      }
      if (nunits >= 1) add_unit(nunits - 1);
    }
  } else if (warp == 8 || warp == 9) {
    // ================================================================ S^T = Kunit . Q^T issuers
    if (lane == 0) {
      const int j = warp - 8;
      ptx::mbar_wait(&mi->q_ready, 0, abort_flag);   // also when there is no unit: q has landed before the CTA exits
      if constexpr (I8) {
        // int8 x int8 -> int32, K = 32 per instruction, N = 128 = the hi and lo planes of q.  Issuer j takes the
        // units of parity j, whole.
        const uint32_t idesc_s = ptx::idesc_i8(WS_UNIT, 2 * WS_HEADS, 1, 1);
        const uint32_t q_addr = ptx::smem_u32(q_s), k_addr = ptx::smem_u32(smem + (kb0 + (j) * kb_st));
        const uint32_t d = tmem_base + (uint32_t)(j * 128);
        for (int u = j; u < nunits; u += 2) {
          if (u >= 2) ptx::mbar_wait(&mi->s_free[j], sphase(u - 2), abort_flag);   // S^T(u - 2) has been read
          for (int sl = 0; sl < nrs; ++sl) {
            ptx::mbar_wait(&mi->full[j][sl], sphase(u), abort_flag);   // each slab as soon as it has landed
            ptx::tc_fence_after_sync();
            if (sl == 0) TRS(3, u);
            const bool tail = sl == L.n128;
            const uint64_t ka = tail ? ptx::smem_desc(k_addr + sl * WS_SLAB, 16, 512, 4)
                                     : ptx::smem_desc_sw128(k_addr + sl * WS_SLAB, 16, 1024);
            const uint64_t qb = tail ? ptx::smem_desc(q_addr + sl * 2 * WS_SLAB, 16, 512, 4)
                                     : ptx::smem_desc_sw128(q_addr + sl * 2 * WS_SLAB, 16, 1024);
            for (int ks = 0; ks < (tail ? 2 : 4); ++ks)
              ptx::mma_i8_ss(d, ptx::desc_advance(ka, ks * 32), ptx::desc_advance(qb, ks * 32), idesc_s,
                             (sl | ks) ? 1u : 0u);
          }
          ptx::mma_commit(&mi->s_ready[j]);
          TRS(4, u);
        }
      } else {
        // Issuer j accumulates its half of the feature slabs of every unit into an accumulator of its own.
        const int kb_lo = slab_lo(j), kb_hi = slab_lo(j + 1);
        const uint32_t idesc_s = ptx::idesc_f16(fmt, fmt, WS_UNIT, WS_HEADS, 0, 0);
        const uint64_t q_desc = ptx::smem_desc_sw128(ptx::smem_u32(q_s), 16, 1024);
        for (int u = 0; u < nunits; ++u) {
          const int buf = sbuf(u);
          const uint64_t k_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + (ub0 + (buf) * ub_st)), 16, 1024);
          const uint32_t d = tmem_base + (uint32_t)(buf * 128 + j * WS_HEADS);
          if (u >= 2) ptx::mbar_wait(&mi->s_free[buf], sphase(u - 2), abort_flag);   // S^T(u - 2) has been read
          for (int kb = kb_lo; kb < kb_hi; ++kb) {
            ptx::mbar_wait(&mi->full[buf][kb], sphase(u), abort_flag);   // each slab as soon as it has landed
            ptx::tc_fence_after_sync();
            if (kb == kb_lo && j == 0) TRS(3, u);
#pragma unroll
            for (int ks = 0; ks < 4; ++ks)
              ptx::mma_f16_ss(d, ptx::desc_advance(k_desc, kb * WS_SLAB + ks * 32),
                              ptx::desc_advance(q_desc, kb * WS_SLAB + ks * 32), idesc_s, (kb > kb_lo || ks) ? 1u : 0u);
          }
          ptx::mma_commit(&mi->s_ready[buf]);
          if (j == 0) TRS(4, u);
        }
      }
    }
  } else if (warp == 10 || warp == 11) {
    // ================================================================ O^T += Vunit^T . P^T issuers
    const int mt0 = (warp - 10) * 2;
    if (lane == 0 && mt0 < n_mt) {
      const uint32_t idesc_o = ptx::idesc_f16(fmt, fmt, 128, WS_HEADS, 1, 0);   // A read MN-major
      for (int u = 0; u < nunits; ++u) {
        const int buf = pbuf(u);
        // A, MN-major: 64-feature blocks 8 KB apart (LBO), 8-row groups 1 KB apart (SBO); 16 rows per K step
        const uint64_t v_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + (ub0 + (buf) * ub_st)), WS_SLAB, 1024);
        const uint64_t pt_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + (pt0 + (buf) * pt_st)), 16, 1024);
        ptx::mbar_wait(&mi->p_ready[buf], pphase(u), abort_flag);
        ptx::tc_fence_after_sync();
        if (warp == 10) TRS(9, u);
        for (int mt = mt0; mt < mt0 + 2 && mt < n_mt; ++mt) {
          if (I8) {
            ptx::mbar_wait(&mi->v_full[mt], (uint32_t)(u & 1), abort_flag);   // this block has been widened
            ptx::tc_fence_after_sync();
          }
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::mma_f16_ss(tmem_o + (uint32_t)(mt * WS_HEADS), ptx::desc_advance(v_desc, (2 * mt) * WS_SLAB + ks * 2048),
                            ptx::desc_advance(pt_desc, ks * 32), idesc_o, (u > 0 || ks > 0) ? 1u : 0u);
          ptx::mma_commit(&mi->pv_blk[buf][mt]);
        }
        if (warp == 10) TRS(10, u);
      }
    }
  } else {
    // ================================================================ softmax (warps 0-7), one unit at a time
    // Warp w reaches the TMEM lanes 32 (w % 4) .., where an M = 64 accumulator keeps rows 16 (w % 4) .. + 15 in
    // the first 16 lanes.  Warps 0-3 take heads 0-31, warps 4-7 heads 32-63; inside a warp lanes 0-15 take the
    // first 16 of those heads and lanes 16-31 the other 16: thread = (row, 16 heads).
    const int wq = warp & 3, cset = warp >> 2;
    const int li = lane & 15, ch = lane >> 4;
    const int row = wq * 16 + li;              // row of the unit
    const int col0 = cset * 32 + ch * 16;      // first head of this thread
    const uint32_t lane_off = (uint32_t)(wq * 32) << 16;

    // ---- q: finish the operand
    if (p.q_tma) ptx::mbar_wait(&mi->q_full, 0, abort_flag);
    if constexpr (I8) {
      // the digit planes were written before the roles parted
    } else if (!p.q_tma) {
      // [64 heads x Dqk] K-major, 128-byte swizzle, rounded to the operand type; a warp writes 32 different rows
      for (int i = tid; i < n_items; i += 256) {
        const int h = i & (WS_HEADS - 1), c = i >> 6;
        float f[8];
        load_q_item(i, f);
        uint32_t w[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          float b0, b1;
          w[e] = pack_op16x2<BF16>(f[2 * e], f[2 * e + 1], b0, b1);
        }
        *reinterpret_cast<uint4*>(q_s + (size_t)(c >> 3) * WS_SLAB + (size_t)h * 128 + (((c & 7) ^ (h & 7)) << 4)) =
            make_uint4(w[0], w[1], w[2], w[3]);
      }
    }
    if constexpr (!I8) {
      ptx::fence_proxy_async_smem();
      ptx::mbar_arrive(&mi->q_ready);
    } else {
      ptx::mbar_wait(&mi->q_ready, 0, abort_flag);   // every fixed-point step has been written
    }

    // 16-bit tables: l1 = the sum of the softmax weights of head col0 + li over this warp's rows of all units (the
    // denominator).  Int8 tables: the widening warps keep both sums (see add_unit).
    float l1 = 0.f;
    for (int u = 0; u < nunits; ++u) {
      const int sb_i = sbuf(u), pb_i = pbuf(u), slot = u & (kRing - 1);
      ptx::mbar_wait(&mi->s_ready[sb_i], sphase(u), abort_flag);
      ptx::tc_fence_after_sync();
      if (warp == 0) TRS(5, u);
      uint32_t sv[16];
      {
        // two accumulators per unit: the halves of the feature slabs (16-bit tables), or the digit planes of q
        const uint32_t sa = tmem_base + lane_off + (uint32_t)(sb_i * 128 + cset * 32);
        uint32_t sb[16];
        ptx::tmem_ld_16x32bx2_x16(sa, sv);
        ptx::tmem_ld_16x32bx2_x16(sa + (uint32_t)WS_HEADS, sb);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 16; c += 4) {
          if constexpr (I8) {
            const float4 qs = *reinterpret_cast<const float4*>(&mi->q_step[col0 + c]);   // the heads' fixed-point steps
            sv[c] = __float_as_uint(fmaf((float)(int)sv[c], 256.f, (float)(int)sb[c]) * qs.x);
            sv[c + 1] = __float_as_uint(fmaf((float)(int)sv[c + 1], 256.f, (float)(int)sb[c + 1]) * qs.y);
            sv[c + 2] = __float_as_uint(fmaf((float)(int)sv[c + 2], 256.f, (float)(int)sb[c + 2]) * qs.z);
            sv[c + 3] = __float_as_uint(fmaf((float)(int)sv[c + 3], 256.f, (float)(int)sb[c + 3]) * qs.w);
          } else {
#pragma unroll
            for (int e = 0; e < 4; ++e) sv[c + e] = __float_as_uint(__uint_as_float(sv[c + e]) + __uint_as_float(sb[c + e]));
          }
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&mi->s_free[sb_i]);
      if (I8 && u == 0) ptx::mbar_wait(&mi->meta_ready, 0, abort_flag);   // the first scales are published behind the gathers
      const bool ok = mi->row_ref[slot][row] != kNoRow;
      const float rs = I8 ? mi->row_scale[slot][row] : 1.f;
      const float mul = scale_log2 * rs;
      // Int8 tables: the operand weight of a row is its softmax weight times the row's dequantisation scale, and
      // that product is what has to fit fp16.  So the references follow the maxima of logit + log2(scale): the
      // largest operand weight of a head is 1 (2^-headroom) when its reference moves, whatever the scales are.
      const float lrs = (I8 && ok) ? log2f(rs) : 0.f;
      const float gap = BF16 ? kRescaleGapBF16 : kRescaleGapF16;
      bool grow = false;
#pragma unroll
      for (int c = 0; c < 16; c += 4) {
        const float4 mr = *reinterpret_cast<const float4*>(&mi->m_ref[col0 + c]);   // the heads' reference maxima
        const float mrv[4] = {mr.x, mr.y, mr.z, mr.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float x = ok ? fmaf(__uint_as_float(sv[c + e]), mul, lrs) : -INFINITY;
          sv[c + e] = __float_as_uint(x);
          grow |= x > mrv[e] + gap;
        }
      }
      if (warp == 0) TRS(6, u);
      bool grown = false;
      if (__syncthreads_or_256(grow)) {
        // exact column maxima of this unit (xor shuffles of 8, 4, 2, 1 stay inside a half warp = one head range)
#pragma unroll
        for (int c = 0; c < 16; ++c) {
          int o = float_order(__uint_as_float(sv[c]));
          o = max(o, __shfl_xor_sync(0xffffffffu, o, 8));
          o = max(o, __shfl_xor_sync(0xffffffffu, o, 4));
          o = max(o, __shfl_xor_sync(0xffffffffu, o, 2));
          o = max(o, __shfl_xor_sync(0xffffffffu, o, 1));
          if (li == c) mi->colmax[wq][col0 + c] = order_float(o);
        }
        // O^T belongs to the old reference: it is final for the units so far once the previous P V is done (and
        // the row sums have taken the previous factor, if any, before this one replaces it)
        if (warp == 0) TRS(29, u);
        if (u >= 1) wait_pv_all(u - 1);
        if (I8 && u >= 1) ptx::mbar_wait(&mi->p_summed, (uint32_t)((u - 1) & 1), abort_flag);
        if (warp == 0) TRS(30, u);
        group_sync(4, 256);
        if (tid < WS_HEADS) {
          const float old = mi->m_ref[tid];
          float mx = fmaxf(fmaxf(mi->colmax[0][tid], mi->colmax[1][tid]), fmaxf(mi->colmax[2][tid], mi->colmax[3][tid]));
          mx = mx > old ? mx + (BF16 ? 0.f : kRescaleHeadroom) : old;
          mi->factor[tid] = (old == -INFINITY) ? 0.f : exp2f(old - mx);
          mi->m_ref[tid] = mx;
        }
        group_sync(4, 256);
        ptx::tc_fence_after_sync();
        if constexpr (!I8) l1 *= mi->factor[col0 + li];
        grown = true;
        if (u >= 1) {
          // warp -> (lane quarter of TMEM = 32 features, two of the four 128-feature blocks); columns = heads
          for (int m2 = 0; m2 < 2; ++m2) {
            const int mt = cset * 2 + m2;
            if (mt < n_mt) {
#pragma unroll 1
              for (int hh = 0; hh < 2; ++hh) {
                uint32_t ov[32];
                const uint32_t ta = tmem_o + lane_off + (uint32_t)(mt * WS_HEADS + hh * 32);
                ptx::tmem_ld32(ta, ov);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * mi->factor[hh * 32 + c]);
                ptx::tmem_st32(ta, ov);
              }
            }
          }
          ptx::tmem_st_wait();
        }
        if (warp == 0) TRS(28, u);
      }
      // ---- P^T (16-bit, K-major, swizzled); the weights join this thread's sums as the operand holds them
      uint32_t prw[8];
      {
#pragma unroll
        for (int c = 0; c < 16; c += 2) {   // two heads per step: one packed conversion each way
          const float2 mr = *reinterpret_cast<const float2*>(&mi->m_ref[col0 + c]);   // (moves only in the branch above)
          const float s0 = __uint_as_float(sv[c]), s1 = __uint_as_float(sv[c + 1]);
          float p0 = (s0 == -INFINITY) ? 0.f : fast_exp2(s0 - mr.x);
          float p1 = (s1 == -INFINITY) ? 0.f : fast_exp2(s1 - mr.y);
          float b0, b1;
          prw[c >> 1] = pack_op16x2<BF16>(p0, p1, b0, b1);
          sv[c] = __float_as_uint(b0);   // the weights as the operand holds them
          sv[c + 1] = __float_as_uint(b1);
        }
      }
      if (warp == 0) TRS(7, u);
      if (I8 && u >= 1) {   // the one P^T buffer has been read by the previous unit's P V and by the row sums
        wait_pv_all(u - 1);
        ptx::mbar_wait(&mi->p_summed, (uint32_t)((u - 1) & 1), abort_flag);
      }
      if constexpr (I8) {
        if (cset == 0 && ch == 0) mi->row_inv[u & 1][row] = ok ? __frcp_rn(rs) : 0.f;
        if (tid == 0) mi->grew[u & 1] = grown ? 1 : 0;
      }
      {
        uint8_t* pbase = smem + (pt0 + (pb_i) * pt_st) + (row & 7) * 2;
        const int cj = row >> 3;
#pragma unroll
        for (int c = 0; c < 16; c += 2) {
          const int h = col0 + c;
          *reinterpret_cast<uint16_t*>(pbase + (size_t)h * 128 + ((cj ^ (h & 7)) << 4)) = (uint16_t)(prw[c >> 1] & 0xffffu);
          *reinterpret_cast<uint16_t*>(pbase + (size_t)(h + 1) * 128 + ((cj ^ ((h + 1) & 7)) << 4)) = (uint16_t)(prw[c >> 1] >> 16);
        }
      }
      if (warp == 0) TRS(12, u);
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&mi->p_ready[pb_i]);
      if (warp == 0) TRS(8, u);
      // 16-bit tables: the sums over the 16 rows of this half warp, behind the hand-off (int8 tables: the widening
      // warps sum P^T from shared memory)
      if constexpr (!I8) {
        float a[16];
#pragma unroll
        for (int c = 0; c < 16; ++c) a[c] = __uint_as_float(sv[c]);
        l1 += half_warp_column_sum(a, li);
      }
    }

    // ------------------------------------------------------------------ row sums over all units
    if (tid == 0) TRS(11, 2);
    group_sync(4, 256);   // nobody reads the column maxima or the row ring any more
    if constexpr (!I8) mi->colmax[wq][col0 + li] = l1;
    if (I8 && nunits >= 1) ptx::mbar_wait(&mi->p_summed, (uint32_t)((nunits - 1) & 1), abort_flag);   // the totals are in
    if (nunits >= 1) wait_pv_all(nunits - 1);
    if (!I8 && nunits >= 2) wait_pv_all(nunits - 2);
    ptx::tc_fence_after_sync();
    group_sync(4, 256);
    if (tid == 0) TRS(11, 3);

    // ------------------------------------------------------------------ per-head sums of this split
    if (tid < WS_HEADS) {
      float l, vb = 0.f;
      if constexpr (I8) {   // rows 0-1: the denominator's two halves, rows 2-3: the operand weights' (widening warps)
        l = nunits >= 1 ? mi->colmax[0][tid] + mi->colmax[1][tid] : 0.f;
        vb = nunits >= 1 ? kValueBias * (mi->colmax[2][tid] + mi->colmax[3][tid]) : 0.f;
      } else {
        l = (mi->colmax[0][tid] + mi->colmax[1][tid]) + (mi->colmax[2][tid] + mi->colmax[3][tid]);
      }
      mi->l_tot[tid] = l;
      mi->v_bias[tid] = vb;
      if (p.cluster_merge) {   // tell every split of this token (this one included) where this one stands
        const uint32_t am = ptx::smem_u32(&mi->xm[split][tid]), al = ptx::smem_u32(&mi->xl[split][tid]);
        for (int r = 0; r < p.nsplit; ++r) {
          ptx::st_cluster_f32(ptx::cluster_map(am, (uint32_t)r), mi->m_ref[tid]);
          ptx::st_cluster_f32(ptx::cluster_map(al, (uint32_t)r), l);
        }
      }
    }
  }

  // ====================================================================== output
  // Every role is done with this CTA's operand buffers (the softmax warps arrive here only after the last P V).
  // Three ways out: one split -> final or external-partial output straight from TMEM; splits in a cluster ->
  // merged through shared memory below; otherwise (o, m, l) partials for the merge kernel.
  const bool cmerge = p.cluster_merge != 0;
  if (cmerge) {
    __syncwarp();
    ptx::cluster_arrive();   // (1) every split's (m, l) is in place and every CTA's buffers are idle
    ptx::cluster_wait();
    if (tid == 0) TRS(11, 5);
  }
  const int n_slots = cmerge ? (n_mt + p.nsplit - 1) / p.nsplit : 0;   // value blocks a CTA merges: mt = rank + slot * nsplit
  float* recv = reinterpret_cast<float*>(smem);   // cluster merge: [slot][source split][16 head groups][128 features][4 heads]
  if (warp < 8) {
    const int wq = warp & 3, cset = warp >> 2;
    const uint32_t lane_off = (uint32_t)(wq * 32) << 16;
    const int64_t N = (int64_t)p.B * p.T * p.H;
    const bool direct = p.nsplit == 1;
    const bool finalize = direct && !p.partial_ml;
    const bool have_o = nunits > 0;
    if (tid < WS_HEADS) {
      // per-head factor applied to O^T: 1 for partial output; otherwise this split's weight over the denominator
      // of the whole token, exp2(m - m*) / (sum over splits of l exp2(m_s - m*) + sink), the sink joining once
      float fac = 1.f;
      if (finalize || cmerge) {
        const float m = mi->m_ref[tid];
        const float sink2 = (p.sinks && tid < p.H) ? p.sinks[tid] * 1.4426950408889634f : -INFINITY;
        float m2v = fmaxf(m, sink2);
        if (cmerge)
          for (int r = 0; r < p.nsplit; ++r) m2v = fmaxf(m2v, mi->xm[r][tid]);
        float w = 0.f, den = 0.f;
        if (m2v > -INFINITY) {
          w = (m == -INFINITY) ? 0.f : exp2f(m - m2v);
          if (cmerge) {
            for (int r = 0; r < p.nsplit; ++r)   // split order: the same sum in every CTA and on every run
              if (mi->xm[r][tid] > -INFINITY) den = fmaf(mi->xl[r][tid], exp2f(mi->xm[r][tid] - m2v), den);
          } else {
            den = mi->l_tot[tid] * w;
          }
          den += (sink2 == -INFINITY) ? 0.f : exp2f(sink2 - m2v);
        }
        fac = den > 0.f ? w / den : 0.f;
      }
      mi->factor[tid] = fac;
    }
    group_sync(4, 256);
    // warp -> (lane quarter of TMEM = 32 features, two of the four 128-feature blocks); columns = heads
    const int64_t gbase = direct ? (int64_t)b * p.o_sb + (int64_t)t * p.o_st : ((int64_t)split * N + (int64_t)bt * p.H) * p.Dv;
    const int64_t ostep = direct ? p.o_sh : (int64_t)p.Dv;
    for (int m2 = 0; m2 < 2; ++m2) {
      const int mt = cset * 2 + m2;
      if (mt >= n_mt) continue;
      const int d = mt * 128 + wq * 32 + lane;
      // cluster merge: block mt belongs to split mt % nsplit; this thread's feature row of it goes there, four
      // heads per 16-byte store, consecutive features in consecutive lanes
      const uint32_t owner = (uint32_t)(mt % p.nsplit);
      const uint32_t dst0 = cmerge ? ptx::cluster_map(ptx::smem_u32(recv) + (uint32_t)((((mt / p.nsplit) * p.nsplit + split) * 16) * 128 + wq * 32 + lane) * 16u, owner) : 0u;
#pragma unroll 1
      for (int hh = 0; hh < 2; ++hh) {
        uint32_t ov[32];
        if (have_o) {
          ptx::tmem_ld32(tmem_o + lane_off + (uint32_t)(mt * WS_HEADS + hh * 32), ov);
          ptx::tmem_ld_wait();
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) ov[c] = 0u;
        }
        if (cmerge) {
#pragma unroll
          for (int c = 0; c < 32; c += 4) {
            float o4[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int h = hh * 32 + c + e;
              o4[e] = have_o ? (__uint_as_float(ov[c + e]) - mi->v_bias[h]) * mi->factor[h] : 0.f;
            }
            ptx::st_cluster_v4(dst0 + (uint32_t)((hh * 8 + (c >> 2)) * 128) * 16u, o4[0], o4[1], o4[2], o4[3]);
          }
          continue;
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int h = hh * 32 + c;
          if (h >= p.H) continue;
          const float o = (__uint_as_float(ov[c]) - mi->v_bias[h]) * mi->factor[h];
          if (finalize) store_elem<OT>(p.out, gbase + d + h * ostep, o);
          else if (direct) reinterpret_cast<float*>(p.out)[gbase + d + h * ostep] = o;
          else p.ws_o[gbase + d + h * ostep] = o;
        }
      }
    }
    if (!cmerge && tid < p.H && (!direct || p.partial_ml)) {
      // (m, l) in natural-log units for the merge kernel
      const float m_nat = mi->m_ref[tid] == -INFINITY ? -INFINITY : mi->m_ref[tid] * 0.6931471805599453f;
      float* ml = direct ? p.partial_ml + ((int64_t)bt * p.H + tid) * 2
                         : p.ws_ml + ((int64_t)split * N + (int64_t)bt * p.H + tid) * 2;
      ml[0] = m_nat;
      ml[1] = mi->l_tot[tid];
    }
  }
  if (cmerge) {
    if (tid == 0) TRS(11, 6);
    __syncwarp();
    ptx::cluster_arrive();   // (2) every split's weighted blocks have arrived; nothing remote is touched after this
    ptx::cluster_wait();
    if (tid == 0) TRS(11, 7);
    if (warp < 8) {
      // thread = (feature of the block, half of the head groups): sum the splits in split order, store the output
      const int f = tid & 127, hg0 = (tid >> 7) * 8;
      for (int slot = 0; slot < n_slots; ++slot) {
        const int mt = split + slot * p.nsplit;
        if (mt >= n_mt) break;
        const int d = mt * 128 + f;
        const float4* src = reinterpret_cast<const float4*>(recv) + (size_t)(slot * p.nsplit) * 16 * 128 + f;
#pragma unroll 4
        for (int hg = hg0; hg < hg0 + 8; ++hg) {   // (several head groups' loads in flight)
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
          for (int r = 0; r < kMaxClusterMerge; ++r) {
            if (r < p.nsplit) {
              const float4 v = src[(size_t)(r * 16 + hg) * 128];
              acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
            }
          }
          const float o4[4] = {acc.x, acc.y, acc.z, acc.w};
          const int64_t ob = (int64_t)b * p.o_sb + (int64_t)t * p.o_st + d;
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const int h = hg * 4 + e;
            if (h < p.H) store_elem<OT>(p.out, ob + h * p.o_sh, o4[e]);
          }
        }
      }
    }
  }

  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_base, 512);
  if (tid == 0) TRS(11, 4);
#ifndef MXB_TRACE_SP
  if (tid == 0 && *abort_flag) {
    // a wait gave up: leave a visibly wrong marker for the caller
    if (p.status) atomicExch(p.status, 2);
  }
#endif
}

bool sparse_tc_eligible(int kv_dtype, int q_dtype, int H, int Dqk, int Dv) {
  if (!(kv_dtype == MXB_F16 || kv_dtype == MXB_BF16 || kv_dtype == MXB_I8)) return false;
  if (kv_dtype == MXB_BF16 && q_dtype == MXB_F16) return false;
  if (kv_dtype == MXB_F16 && q_dtype == MXB_BF16) return false;
  if (H < 1 || H > WS_HEADS) return false;
  if (Dqk % 64 != 0 || Dqk < 128 || Dqk > 576) return false;
  if (Dv % 128 != 0 || Dv < 128 || Dv > 512 || Dv > Dqk) return false;
  return ws_layout(Dqk, Dv, kv_dtype == MXB_I8).total + 1024 <= 227 * 1024;
}

int sparse_tc_splits(int B, int T, int H, int k, int raw_cap, int requested) {
  const int64_t max_parts = ceil_div((int64_t)k + raw_cap, 2 * WS_UNIT);   // at least two units per split
  const int64_t base = (int64_t)B * T > 0 ? (int64_t)B * T : 1;
  // Splits exist to fill idle SMs, so a split launch never has more CTAs than the device has SMs (one CTA per SM):
  // a request beyond that is cut down.  (One launch of 40 tokens x 4 splits = 160 CTAs ended in "unspecified launch
  // failure"; the cause was not found by reading and that shape is not launched again.)
  const int64_t one_wave = (int64_t)sm_count() / base;
  int64_t want = requested > 0 ? (int64_t)requested : one_wave;
  if (want > one_wave) want = one_wave;
  if (want > max_parts) want = max_parts;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return (int)want;
}

// Tensor map over a [rows, Dqk] table for row gathers: box = `box_elems` features of one row (one shared-memory
// slab row).  The row extent is left open (the caller's ids are what bounds the reads); row -1 is the zero row.
static int row_gather_map(CUtensorMap* out, const void* table, int Dqk, int kv_dtype, int box_elems) {
  const int esz = kv_dtype == MXB_I8 ? 1 : 2;
  const uint64_t dims[2] = {(uint64_t)Dqk, (uint64_t)0x7FFFFFFF};
  const uint64_t strides[1] = {(uint64_t)Dqk * esz};
  const uint32_t box[2] = {(uint32_t)box_elems, 1};
  const CUtensorMapDataType dt = kv_dtype == MXB_I8     ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                 : kv_dtype == MXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                                                        : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  return make_tensor_map(out, dt, 2, table, dims, strides, box,
                         box_elems * esz == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B);
}

// Tensor map over q [B, H, T, Dqk] (any strides on the first three axes) whose box is the 64 heads x 64 features
// of one (batch, token): the three outer axes go into the map in ascending stride order; axes of extent 1 carry
// no address and go last with a stride of their own.  Returns false when q's layout cannot be described (then
// the kernel stages q through registers).
static bool q_tile_map(CUtensorMap* out, SparseParams& p, bool bf16) {
  if ((reinterpret_cast<uintptr_t>(p.q) & 15) != 0) return false;
  const int64_t extent[3] = {p.H, p.T, p.B};
  const int64_t stride[3] = {p.q_sh, p.q_st, p.q_sb};
  int order[3], n = 0;
  for (int pass = 0; pass < 2; ++pass)
    for (int a = 0; a < 3; ++a)
      if ((extent[a] > 1) == (pass == 0)) order[n++] = a;
  int real = 0;
  for (int a = 0; a < 3; ++a) real += extent[a] > 1;
  for (int i = 0; i < real; ++i)
    for (int j = i + 1; j < real; ++j)
      if (stride[order[j]] < stride[order[i]]) { int tmp = order[i]; order[i] = order[j]; order[j] = tmp; }
  uint64_t dims[4] = {(uint64_t)p.Dqk, 0, 0, 0}, str[3];
  uint32_t box[4] = {64, 1, 1, 1};
  uint64_t prev = (uint64_t)p.Dqk * 2;   // bytes covered so far
  for (int i = 0; i < 3; ++i) {
    const int a = order[i];
    uint64_t sb;
    if (extent[a] > 1) {
      if (stride[a] <= 0 || stride[a] % 8 != 0) return false;
      sb = (uint64_t)stride[a] * 2;
      if (sb < prev) return false;   // overlapping axes: not a plain nested layout
    } else {
      sb = prev;
    }
    dims[i + 1] = (uint64_t)extent[a];
    str[i] = sb;
    box[i + 1] = a == 0 ? (uint32_t)WS_HEADS : 1u;
    p.q_axis[i] = a;
    prev = sb * (uint64_t)extent[a];
  }
  return make_tensor_map(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 4, p.q, dims, str,
                         box, CU_TENSOR_MAP_SWIZZLE_128B) == MXB_OK;
}

template <int KVT, int QT>
static int launch_tc_typed(SparseParams& p, int out_dtype, cudaStream_t st) {
  constexpr bool I8 = (KVT == MXB_I8);
  const WsLayout L = ws_layout(p.Dqk, p.Dv, I8);
  const int smem = L.total + 1024;
  CUtensorMap tm_comp, tm_raw, tm_comp_tail, tm_raw_tail, tm_q;
  memset(&tm_comp, 0, sizeof(tm_comp));
  memset(&tm_raw, 0, sizeof(tm_raw));
  memset(&tm_comp_tail, 0, sizeof(tm_comp_tail));
  memset(&tm_raw_tail, 0, sizeof(tm_raw_tail));
  memset(&tm_q, 0, sizeof(tm_q));
  const void* comp = p.comp_kv ? p.comp_kv : p.raw_kv;
  const void* raw = p.raw_kv ? p.raw_kv : comp;
  MXB_REQUIRE(comp != nullptr || p.k + p.raw_cap == 0, MXB_ERR_INVALID, "sparse attention: no KV table");
  if (comp) {
    const int box = I8 ? 128 : 64;   // one 128-byte slab row
    int rc = row_gather_map(&tm_comp, comp, p.Dqk, KVT, I8 && p.Dqk < 128 ? 64 : box);
    if (rc != MXB_OK) return rc;
    rc = row_gather_map(&tm_raw, raw, p.Dqk, KVT, I8 && p.Dqk < 128 ? 64 : box);
    if (rc != MXB_OK) return rc;
    if (I8 && L.tail) {
      rc = row_gather_map(&tm_comp_tail, comp, p.Dqk, KVT, 64);
      if (rc != MXB_OK) return rc;
      rc = row_gather_map(&tm_raw_tail, raw, p.Dqk, KVT, 64);
      if (rc != MXB_OK) return rc;
    }
  }
  // a 16-bit q lands by TMA (int8 tables: into the value buffer, when that is large enough to hold it)
  p.q_tma = 0;
  if ((QT == MXB_BF16 || QT == MXB_F16) && (!I8 || L.qtmp_off >= 0)) p.q_tma = q_tile_map(&tm_q, p, QT == MXB_BF16) ? 1 : 0;
  const int64_t ctas = (int64_t)p.B * p.T * p.nsplit;
  MXB_REQUIRE(ctas <= 0x7FFFFFFFll, MXB_ERR_INVALID, "sparse attention: too many (batch, token, split) items");
  dim3 grid((unsigned)ctas);
  // The splits of a token as one thread-block cluster that merges through shared memory: when a final output is
  // wanted, the blocks to merge fit the (then idle) operand buffers, and every cluster is resident at once (a
  // cluster needs nsplit whole SMs of one GPC; a second wave of clusters would cost more than the merge kernel).
  p.cluster_merge = 0;
  const int n_mt = p.Dv / 128;
  const int n_slots = p.nsplit > 0 ? (n_mt + p.nsplit - 1) / p.nsplit : 0;
  const bool merge_fits = (size_t)n_slots * p.nsplit * 32768 <= (size_t)L.misc_off;
#define MXB_TC(OT, CLUSTER)                                                                          \
  {                                                                                                  \
    auto kern = sparse_attn_tc_kernel<KVT, QT, OT>;                                                  \
    MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));      \
    cudaLaunchConfig_t cfg = {};                                                                     \
    cfg.gridDim = grid;                                                                              \
    cfg.blockDim = dim3(WS_THREADS);                                                                 \
    cfg.dynamicSmemBytes = (size_t)smem;                                                             \
    cfg.stream = st;                                                                                 \
    cudaLaunchAttribute at[1];                                                                       \
    at[0].id = cudaLaunchAttributeClusterDimension;                                                  \
    at[0].val.clusterDim.x = (unsigned)p.nsplit;                                                     \
    at[0].val.clusterDim.y = 1;                                                                      \
    at[0].val.clusterDim.z = 1;                                                                      \
    cfg.attrs = at;                                                                                  \
    cfg.numAttrs = 1;                                                                                \
    bool as_cluster = false;                                                                         \
    if (CLUSTER) {                                                                                   \
      static int resident_cache[16][kMaxClusterMerge + 1]; /* per device and cluster size; 0 = not asked yet */ \
      int dev = 0;                                                                                   \
      MXB_CUDA_OK(cudaGetDevice(&dev));                                                              \
      int resident = (dev >= 0 && dev < 16) ? resident_cache[dev][p.nsplit] : 0;                     \
      if (resident == 0) {                                                                           \
        if (cudaOccupancyMaxActiveClusters(&resident, kern, &cfg) != cudaSuccess) {                  \
          (void)cudaGetLastError();                                                                  \
          resident = -1;                                                                             \
        }                                                                                            \
        if (resident == 0) resident = -1;                                                            \
        if (dev >= 0 && dev < 16) resident_cache[dev][p.nsplit] = resident;                          \
      }                                                                                              \
      as_cluster = (int64_t)resident >= (int64_t)p.B * p.T;                                          \
    }                                                                                                \
    if (as_cluster) {                                                                                \
      p.cluster_merge = 1;                                                                           \
      p.cta_base = 0;                                                                                \
      MXB_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, p, tm_comp, tm_raw, tm_comp_tail, tm_raw_tail, tm_q)); \
    } else if (CLUSTER) {                                                                            \
      return MXB_ERR_UNSUPPORTED; /* the caller retries with fp32 partials */                         \
    } else {                                                                                         \
      /* One wave per launch.  Launches of this kernel that put a second CTA on an SM which a CTA of  \
         the same launch had just left have failed ("unspecified launch failure": always for 160    \
         split CTAs, rarely for 4,096 one-split CTAs) and launches of at most one CTA per SM never   \
         have; the cause is not known.  Between launches nothing of the previous wave is in flight. */ \
      const int64_t wave = (int64_t)(sm_count() / p.nsplit) * p.nsplit > 0                           \
                               ? (int64_t)(sm_count() / p.nsplit) * p.nsplit : p.nsplit;             \
      for (int64_t base = 0; base < ctas; base += wave) {                                            \
        p.cta_base = (int32_t)base;                                                                  \
        const unsigned n = (unsigned)(ctas - base < wave ? ctas - base : wave);                      \
        kern<<<dim3(n), WS_THREADS, smem, st>>>(p, tm_comp, tm_raw, tm_comp_tail, tm_raw_tail, tm_q); \
        if (base > 0) note_launch(); /* the first launch is counted below */                          \
      }                                                                                              \
      p.cta_base = 0;                                                                                \
    }                                                                                                \
  }
  const bool try_cluster = p.nsplit >= 2 && p.nsplit <= kMaxClusterMerge && !p.partial_ml && merge_fits;
  int rc_cluster = MXB_ERR_UNSUPPORTED;
  if (try_cluster) {
    auto attempt = [&]() -> int {
      if (out_dtype == MXB_F32) MXB_TC(MXB_F32, true)
      else if (out_dtype == MXB_BF16) MXB_TC(MXB_BF16, true)
      else MXB_TC(MXB_F16, true)
      return MXB_OK;
    };
    rc_cluster = attempt();
    if (rc_cluster != MXB_OK && rc_cluster != MXB_ERR_UNSUPPORTED) return rc_cluster;
  }
  if (rc_cluster != MXB_OK) {
    p.cluster_merge = 0;
    auto plain = [&]() -> int {
      if (out_dtype == MXB_F32 || p.nsplit > 1 || p.partial_ml) MXB_TC(MXB_F32, false)
      else if (out_dtype == MXB_BF16) MXB_TC(MXB_BF16, false)
      else MXB_TC(MXB_F16, false)
      return MXB_OK;
    };
    const int rc = plain();
    if (rc != MXB_OK) return rc;
  }
#undef MXB_TC
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

int launch_sparse_tc(SparseParams& p, int kv_dtype, int q_dtype, int out_dtype, cudaStream_t st) {
#define MXB_TCP(QT, KT) \
  if (q_dtype == QT && kv_dtype == KT) return launch_tc_typed<KT, QT>(p, out_dtype, st);
  MXB_TCP(MXB_F32, MXB_F16)
  MXB_TCP(MXB_F16, MXB_F16)
  MXB_TCP(MXB_F32, MXB_BF16)
  MXB_TCP(MXB_BF16, MXB_BF16)
  MXB_TCP(MXB_F32, MXB_I8)
  MXB_TCP(MXB_F16, MXB_I8)
  MXB_TCP(MXB_BF16, MXB_I8)
#undef MXB_TCP
  return fail(MXB_ERR_UNSUPPORTED, "sparse attention (tensor-core path): unsupported q/kv dtype pair (%d, %d)",
              q_dtype, kv_dtype);
}

}  // namespace mxb
