// Indexed mixed (sparse) attention on tcgen05 / TMEM for 16-bit and int8 KV tables, warp-specialised.
//
// One CTA = one (sequence, token, split of its row list): all heads (<= 64) of that token share every
// gathered row.  The row list (raw window rows, then the selected compressed rows) is cut into UNITS of 64
// rows.  The gathered rows sit on the MMA M axis:
//
//   S^T[64 rows  x 64 heads]  = Kunit[64 x Dqk] . Q^T             (M = 64:  A = operand buffer, K-major)
//   O^T[Dv dims  x 64 heads] += Vunit^T[Dv x 64] . P^T            (M = 128: A = the SAME buffer read MN-major)
//
// so one staged copy of the rows (128-byte-swizzled 64-feature slabs of [64 rows x 128 B]) feeds both
// contractions and nothing is transposed.  Warp roles:
//   warps 0-7    softmax, one unit at a time.  An M = 64 accumulator occupies lanes 0-15 of each 32-lane
//                quarter of TMEM; thread = (row, 16 heads)
//   next 2 or 4  issue S^T, each into an accumulator of its own for its share of the feature slabs (measured: a
//                thread issues one tcgen05.mma per ~105 cycles whatever its shape, four threads together one per
//                ~37 (M = 64) or ~53 (M = 128) cycles); the softmax adds the accumulators
//   next 4       issue O^T += V^T P^T, one 128-feature value block each
//   last 8       producers: resolve list entries to rows ahead of time and bring the rows in.
// 16-bit tables: two operand buffers alternate; TMA row gathers (tile::gather4: four rows x one 128-byte slab per
// instruction, swizzled on the way in, row -1 = zeros) fill one while the other is multiplied, slab by slab, and
// the logit MMAs of a slab start as soon as it has landed.
// int8 tables: the rows of units u + 1 and u + 2 travel by bulk copies (one 576-byte copy per row) into a ring of
// two int8 staging buffers while unit u is processed; the producers widen a landed unit to exact 16-bit integers
// into the ONE operand buffer (shared memory cannot hold two beside the staging ring) and the per-row scale is
// folded into the logit and into P, so the tensor core multiplies exact values.  Loads through registers are not
// used for rows: measured, an SM sustains ~5 bytes per clock of gathered row pieces that way whatever their
// source, against 16-19 through its bulk-copy engine.
// Operand type: bf16 for bf16 tables, fp16 otherwise (q is rounded to fp16, as the reference kernels do; a bf16
// q over int8 rows lands by TMA and is converted in place).
//
// The softmax keeps one per-head reference maximum m_ref in shared memory, moved only when a logit exceeds it by
// more than a gap (2^15 for fp16 operands, 2^60 for bf16); O^T in TMEM is rescaled only then, after the previous
// unit's P V has completed.  The row sum uses the ROUNDED 16-bit P values, so out = sum(p~ v) / sum(p~) is an
// exactly normalised average.  Splits over the row list emit (o, m, l) partials for the log-sum-exp merge kernel.
//
// TMEM columns: four S^T accumulators of 64 columns at [0,256) (16-bit tables: two per operand buffer; int8:
// four issuers on the one buffer), O^T at [256, 256 + Dv/2).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "sparse_attn.cuh"

namespace mxb {

#ifdef MXB_TRACE_SP   // development aid: cycle stamps of CTA 0's roles for its first 16 units, written behind `status`
#define TRS(k, i) do { if (tr_on && (i) < 16) tr[(k) * 16 + (i)] = clock64(); } while (0)
#else
#define TRS(k, i)
#endif

constexpr int WS_UNIT = 64;       // gathered rows per unit
constexpr int WS_HEADS = 64;      // MMA N
constexpr int WS_MAX_SLABS = 9;   // Dqk <= 576
constexpr int WS_SLAB = 8192;     // [64 rows or heads] x 128 B
constexpr int kWsMiscBytes = 5120;
constexpr int kRing = 4;          // units of row metadata kept in shared memory
// warps: 8 softmax, NQK logit issuers, 4 value issuers (one per 128-feature block), 8 producers
__host__ __device__ constexpr int ws_nqk(bool i8) { return i8 ? 4 : 2; }
__host__ __device__ constexpr int ws_threads(bool i8) { return (8 + ws_nqk(i8) + 4 + 8) * 32; }
// P = 2^(s - m_ref) may be as large as 2^gap.  bf16 operands have fp32's range; fp16 operands top out at 65504,
// and the int8 path folds the row's dequantisation scale into P, so its gap shrinks by log2(scale) when positive.
constexpr float kRescaleGapF16 = 15.f;
constexpr float kRescaleGapBF16 = 60.f;
constexpr uint32_t kNoRow = 0xFFFFFFFFu;

struct WsLayout {
  int nslab;        // Dqk / 64
  int q_off;        // q operand: nslab slabs of [64 heads x 128 B]
  int ub_off[2];    // operand buffers: nslab slabs of [64 rows x 128 B] each (int8 tables: only the first)
  int pt_off[2];    // P^T of the unit in buffer b: [64 heads x 128 B] (64 rows of 16 bits)
  int st_off[2];    // int8 tables: staging ring, 64 rows of st_stride bytes each
  int st_stride;    // Dqk + 16: consecutive rows start in different 16-byte bank groups
  int misc_off;
  int total;
};

__host__ __device__ inline WsLayout ws_layout(int Dqk, int Dv, bool i8) {
  WsLayout L;
  L.nslab = Dqk / 64;
  L.q_off = 0;
  L.ub_off[0] = L.nslab * WS_SLAB;
  L.ub_off[1] = 2 * L.nslab * WS_SLAB;
  L.st_stride = Dqk + 16;
  L.st_off[0] = L.st_off[1] = 0;
  int end;
  if (i8) {
    L.ub_off[1] = L.ub_off[0];
    L.st_off[0] = 2 * L.nslab * WS_SLAB;
    L.st_off[1] = L.st_off[0] + WS_UNIT * L.st_stride;
    end = L.st_off[1] + WS_UNIT * L.st_stride;
  } else {
    end = 3 * L.nslab * WS_SLAB;
  }
  if (Dqk - Dv >= 64) {
    // the last slab feeds only the logits: it is free once S^T of its unit is complete
    L.pt_off[0] = L.ub_off[0] + (L.nslab - 1) * WS_SLAB;
    L.pt_off[1] = L.ub_off[1] + (L.nslab - 1) * WS_SLAB;
  } else {
    end = (end + 1023) & ~1023;
    L.pt_off[0] = end;
    L.pt_off[1] = i8 ? end : end + WS_SLAB;
    end += i8 ? WS_SLAB : 2 * WS_SLAB;
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
  uint32_t row_ref[kRing][WS_UNIT];   // kNoRow, or row index within its table (< 2^31), bit 31 set for the raw table
  float row_scale[kRing][WS_UNIT];
  // full: operand slabs ready for the logit MMAs (16-bit tables: [buffer][slab], completed by the row gathers;
  // int8 tables: [0][issuer], completed by the widening warps); st_full: an int8 staging buffer has landed
  uint64_t q_full, q_ready, full[2][WS_MAX_SLABS], st_full[2], s_ready[2], s_free[2], p_ready[2];
  uint64_t pv_blk[2][4];           // P V of one 128-feature block of the unit in buffer b has completed: its two slabs are free
  uint32_t tmem_slot;
  int abort_flag;
  int keff;
};
static_assert(sizeof(WsMisc) <= kWsMiscBytes, "WsMisc must fit the bytes the layout reserves for it");

// 16 int8 -> 16 fp16 integers (exact): bytes biased by 128 are dropped into the mantissa of 1024.0
__device__ __forceinline__ void widen_i8x16_f16(const uint4& in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x ^ 0x80808080u, in.y ^ 0x80808080u, in.z ^ 0x80808080u, in.w ^ 0x80808080u};
  uint32_t o[8];
  const __half2 bias = __floats2half2_rn(1152.f, 1152.f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint32_t a = __byte_perm(w[i], 0x64646464u, 0x4140);
    uint32_t b = __byte_perm(w[i], 0x64646464u, 0x4342);
    __half2 ha = __hsub2(*reinterpret_cast<__half2*>(&a), bias);
    __half2 hb = __hsub2(*reinterpret_cast<__half2*>(&b), bias);
    o[2 * i] = *reinterpret_cast<uint32_t*>(&ha);
    o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&hb);
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
}

// 16 int8 -> 16 bf16 integers (exact).  bf16 carries 7 mantissa bits: the low 7 bits u7 of the biased byte go into
// the mantissa of 128.0 (giving 128 + u7), and 128 (byte >= 128, value >= 0) or 256 (value < 0) is subtracted.
__device__ __forceinline__ uint32_t i8pair_to_bf16x2(uint32_t a) {   // a = [u0][0x43][u1][0x43]
  uint32_t hi = a & 0xFF7FFF7Fu;
  uint32_t sub = 0x43804380u ^ (a & 0x00800080u);
  __nv_bfloat162 r = __hsub2(*reinterpret_cast<__nv_bfloat162*>(&hi), *reinterpret_cast<__nv_bfloat162*>(&sub));
  return *reinterpret_cast<uint32_t*>(&r);
}
__device__ __forceinline__ void widen_i8x16_bf16(const uint4& in, uint4& lo, uint4& hi) {
  const uint32_t w[4] = {in.x ^ 0x80808080u, in.y ^ 0x80808080u, in.z ^ 0x80808080u, in.w ^ 0x80808080u};
  uint32_t o[8];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    o[2 * i] = i8pair_to_bf16x2(__byte_perm(w[i], 0x43434343u, 0x4140));
    o[2 * i + 1] = i8pair_to_bf16x2(__byte_perm(w[i], 0x43434343u, 0x4342));
  }
  lo = make_uint4(o[0], o[1], o[2], o[3]);
  hi = make_uint4(o[4], o[5], o[6], o[7]);
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
__global__ void __launch_bounds__(ws_threads(KVT == MXB_I8), 1)
sparse_attn_tc_kernel(SparseParams p, const __grid_constant__ CUtensorMap tm_comp,
                      const __grid_constant__ CUtensorMap tm_raw, const __grid_constant__ CUtensorMap tm_q) {
  constexpr bool I8 = (KVT == MXB_I8);
  constexpr bool BF16 = (KVT == MXB_BF16);       // operand type: bf16 for bf16 tables, fp16 otherwise
  constexpr bool Q_CONVERT = I8 && QT == MXB_BF16;   // q lands by TMA as bf16 and is turned into fp16 in place
  constexpr int NQK = ws_nqk(I8);
  constexpr int THREADS = ws_threads(I8);
  constexpr int W_PV = 8 + NQK, W_PROD = W_PV + 4;   // first warp of the value issuers / of the producers
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const WsLayout L = ws_layout(p.Dqk, p.Dv, I8);
  uint8_t* q_s = smem + L.q_off;
  WsMisc* mi = reinterpret_cast<WsMisc*>(smem + L.misc_off);
  volatile int* abort_flag = &mi->abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bt = (int)(blockIdx.x / (unsigned)p.nsplit);
  const int split = (int)(blockIdx.x - (unsigned)bt * (unsigned)p.nsplit);
  const int b = bt / p.T, t = bt % p.T;
  const int nslab = L.nslab;
  const int n_mt = p.Dv / 128;
  // Operand / S^T / P^T buffer of unit u and the parity of that buffer's barriers for it: 16-bit tables alternate
  // two buffers, int8 tables reuse the one.  `prev_use(u)` is the unit that had the buffer before (< 0: none).
  auto xbuf = [](int u) { return I8 ? 0 : (u & 1); };
  auto xphase = [](int u) { return (uint32_t)((I8 ? u : (u >> 1)) & 1); };
  auto prev_use = [](int u) { return I8 ? u - 1 : u - 2; };
  // slabs [slab_lo(j), slab_lo(j + 1)) go to logit issuer j.  16-bit tables: two halves (9 slabs: 5 + 4).  int8
  // tables: the last issuer gets one slab, so that little is left to multiply when the widening ends (9: 3 + 3 + 2 + 1)
  auto slab_lo = [&](int j) {
    if (!I8 || nslab < 5) return (nslab * j + NQK - 1) / NQK;
    return j >= NQK ? nslab : ((nslab - 1) * j + NQK - 2) / (NQK - 1);
  };
  // P V of unit u: one barrier per 128-feature block, so that the two slabs of a block can be refilled as soon
  // as that block has been multiplied.  The slabs beyond the value width (the rotary slab, where P^T lives) are
  // free when every block is done.
  auto wait_pv_block = [&](int u, int mt) { ptx::mbar_wait(&mi->pv_blk[xbuf(u)][mt], xphase(u), abort_flag); };
  auto wait_pv_all = [&](int u) {
    for (int mt = 0; mt < n_mt; ++mt) wait_pv_block(u, mt);
  };
  auto wait_pv_slab = [&](int u, int slab) {   // before slab `slab` of the buffer that unit u used is overwritten
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
    ptx::mbar_init(&mi->q_ready, 256);
    for (int i = 0; i < 2; ++i) {
      for (int kb = 0; kb < WS_MAX_SLABS; ++kb) ptx::mbar_init(&mi->full[i][kb], I8 ? 8u : 1u);
      ptx::mbar_init(&mi->st_full[i], (uint32_t)WS_UNIT);
      ptx::mbar_init(&mi->s_ready[i], (uint32_t)NQK);
      ptx::mbar_init(&mi->s_free[i], 256);
      ptx::mbar_init(&mi->p_ready[i], 256);
      for (int mt = 0; mt < 4; ++mt) ptx::mbar_init(&mi->pv_blk[i][mt], 1);
    }
    mi->abort_flag = 0;
    mi->keff = p.k;
    ptx::mbar_fence_init();
  }
  if (tid < WS_HEADS) {
    mi->m_ref[tid] = -INFINITY;
    mi->factor[tid] = 1.f;
    mi->l_tot[tid] = 0.f;
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

  // ------------------------------------------------------------------ q -> B operand of S^T, and the list scan
  // [64 heads x Dqk] K-major, 128-byte swizzle, in the operand type.  By TMA when q is a 16-bit tensor that a
  // tensor map can describe (heads beyond H arrive as zeros); through registers (rounded) otherwise.
  if (p.q_tma) {
    if (tid == 256) {
      ptx::tma_prefetch_desc(&tm_q);
      ptx::mbar_expect_tx(&mi->q_full, (uint32_t)(nslab * WS_SLAB));
      int32_t c[3];
#pragma unroll
      for (int i = 0; i < 3; ++i) c[i] = p.q_axis[i] == 0 ? 0 : (p.q_axis[i] == 1 ? t : b);
      for (int kb = 0; kb < nslab; ++kb) ptx::tma_load_4d(q_s + kb * WS_SLAB, &tm_q, &mi->q_full, kb * 64, c[0], c[1], c[2]);
    }
  }
  const bool q_vec = ((reinterpret_cast<uintptr_t>(p.q) & 15) == 0) && (p.q_sb % 8 == 0) && (p.q_sh % 8 == 0) &&
                     (p.q_st % 8 == 0);
  const int n_items = WS_HEADS * (p.Dqk / 8);
  auto store_q_item = [&](int i, const float* f) {
    // item i = (head i % 64, 16-byte chunk i / 64): a warp writes 32 different rows, conflict-free stores
    const int h = i & (WS_HEADS - 1), c = i >> 6;
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float b0, b1;
      w[e] = pack_op16x2<BF16>(f[2 * e], f[2 * e + 1], b0, b1);
    }
    const int kb = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(q_s + (size_t)kb * WS_SLAB + (size_t)h * 128 + ((cc ^ (h & 7)) << 4)) =
        make_uint4(w[0], w[1], w[2], w[3]);
  };
  constexpr int kQB = 9;   // 16-bit q, vector path: this many 16-byte loads in flight per thread and pass
  const bool q_regs = !p.q_tma && warp < 8;
  const bool q_fast = q_regs && q_vec && QT != MXB_F32;
  uint4 qraw[kQB];
  auto load_q_pass = [&](int pass) {
#pragma unroll
    for (int j = 0; j < kQB; ++j) {
      const int i = tid + (pass * kQB + j) * 256;
      const int h = i & (WS_HEADS - 1), c = i >> 6;
      qraw[j] = make_uint4(0, 0, 0, 0);
      if (i < n_items && h < p.H)
        qraw[j] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + (int64_t)b * p.q_sb +
                                                       (int64_t)h * p.q_sh + (int64_t)t * p.q_st + c * 8));
    }
  };
  auto store_q_pass = [&](int pass) {
#pragma unroll
    for (int j = 0; j < kQB; ++j) {
      const int i = tid + (pass * kQB + j) * 256;
      if (i < n_items) {
        float f[8];
        if constexpr (QT != MXB_F32) unpack16<QT>(qraw[j], f);
        store_q_item(i, f);
      }
    }
  };
  if (q_fast) load_q_pass(0);
  {  // first list entry that ends the walk (its loads overlap the q loads above)
    int mine = p.k;
#pragma unroll 4
    for (int j = tid; j < p.k; j += THREADS) {   // no early exit: the loads stay independent
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

  if (warp >= W_PROD) {
    // ================================================================ producers (8 warps)
    const int pt = tid - W_PROD * 32, pw = warp - W_PROD;
    const bool resolver = pt < WS_UNIT;   // thread pt resolves entry pt of every unit
    // Row metadata (list id -> row -> dequantisation scale) is a chain of dependent global loads, run as a
    // pipeline, one stage per unit, so that nobody waits on it: stage A fetches the list id, stage B turns it
    // into the row and fetches the scale; the last stage publishes both in shared memory two units before they
    // are needed (and, for int8 tables, starts the row's copy).
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
      if (I8) rs = __half2float(raw ? p.raw_scales[ridx] : p.comp_scales[ridx]);
    };
    auto publish_ref = [&](int U, uint32_t ref) {
      if (resolver && U < nunits) mi->row_ref[U & (kRing - 1)][pt] = ref;
    };
    auto publish_scale = [&](int U, float rs) {
      if (resolver && U < nunits) mi->row_scale[U & (kRing - 1)][pt] = rs;
    };
    // int8 tables: one bulk copy brings this thread's row of unit U into the staging ring (nothing to bring:
    // a plain arrival, and the widening warps write zeros)
    auto start_copy = [&](int U, uint32_t ref) {
      if (!resolver || U >= nunits) return;
      uint64_t* bar = &mi->st_full[U & 1];
      if (ref != kNoRow) {
        const uint8_t* src = reinterpret_cast<const uint8_t*>((ref >> 31) ? p.raw_kv : p.comp_kv) +
                             (int64_t)(ref & 0x7FFFFFFFu) * p.Dqk;
        ptx::mbar_expect_tx(bar, (uint32_t)p.Dqk);
        ptx::bulk_load_1d(smem + L.st_off[U & 1] + (size_t)pt * L.st_stride, src, (uint32_t)p.Dqk, bar);
      } else {
        ptx::mbar_arrive(bar);
      }
    };
    int32_t id_a = -1;          // stage A result: list id of this thread's entry of unit u + 3
    uint32_t src_b = kNoRow;    // stage B result: row and scale of this thread's entry of unit u + 2
    float rs_b = 1.f;
    float rs0 = 1.f, rs1 = 1.f;   // scales of units 0 and 1: published inside the first step, behind the row traffic
    if (pt == 0) TRS(14, 0);
    if (nunits > 0) {
      const int32_t i0 = fetch_id(0), i1 = fetch_id(1), i2 = fetch_id(2);
      id_a = fetch_id(3);
      uint32_t s0, s1;
      fetch_row(0, i0, s0, rs0);
      fetch_row(1, i1, s1, rs1);
      if (I8) {
        start_copy(0, s0);
        start_copy(1, s1);
      }
      if (pt == 0) TRS(14, 1);
      fetch_row(2, i2, src_b, rs_b);
      publish_ref(0, s0);
      publish_ref(1, s1);
    }
    if (pt == 0) TRS(14, 2);
    group_sync(3, 256);
    if (pt == 0) TRS(14, 3);

    if constexpr (I8) {
      // Widening, staging ring -> operand buffer.  One warp instruction covers 8 rows x 4 consecutive 16-byte
      // chunks (lane = row % 8 + 8 * chunk) = the 64 features of one operand slab: the staging rows are
      // Dqk + 16 bytes apart and the operand rows have 8 different swizzle phases, so the 128-bit shared-memory
      // loads and stores are conflict-free.  Warp pw takes rows 8 pw .. 8 pw + 7, nine chunks per lane for a
      // 576-byte row.  The slabs of a logit issuer are announced as soon as every warp has stored them.
      const int nch = p.Dqk / 16;
      const int r8 = lane & 7, cl = lane >> 3;
      const int rr = pw * 8 + r8;
      uint8_t* drow = smem + L.ub_off[0] + (size_t)rr * 128;
      for (int u = 0; u < nunits; ++u) {
        const int slot = u & 1;
        if (pt == 0) TRS(0, u);
        ptx::mbar_wait(&mi->st_full[slot], (uint32_t)((u >> 1) & 1), abort_flag);      // the rows have landed
        if (pt == 0) TRS(1, u);
        if (u == 0) {
          publish_scale(0, rs0);
          publish_scale(1, rs1);
        }
        const bool valid = mi->row_ref[u & (kRing - 1)][rr] != kNoRow;
        const uint8_t* srow = smem + L.st_off[slot] + (size_t)rr * L.st_stride;
        uint4 v[WS_MAX_SLABS];   // this lane's chunks, read while the previous unit's P V still owns the operand buffer
#pragma unroll
        for (int i = 0; i < WS_MAX_SLABS; ++i) {
          const int c = i * 4 + cl;
          v[i] = make_uint4(0, 0, 0, 0);
          if (valid && c < nch) v[i] = *reinterpret_cast<const uint4*>(srow + c * 16);
        }
        int grp = 0;
#pragma unroll
        for (int i = 0; i < WS_MAX_SLABS; ++i) {
          if (i < nslab) {
            if (u >= 1 && (i == 2 * n_mt || (i < 2 * n_mt && (i & 1) == 0))) wait_pv_slab(u - 1, i);   // slab pair free
            if (pt == 0 && i == 0) TRS(13, u);
            uint4 lo, hi;
            widen_i8x16_f16(v[i], lo, hi);   // zero bytes (no row) widen to 0.0
            uint8_t* d = drow + (size_t)i * WS_SLAB;
            *reinterpret_cast<uint4*>(d + (((2 * cl) ^ r8) << 4)) = lo;
            *reinterpret_cast<uint4*>(d + (((2 * cl + 1) ^ r8) << 4)) = hi;
            while (grp < NQK && i + 1 == slab_lo(grp + 1)) {   // the last slab of issuer grp (empty shares pass through)
              if (slab_lo(grp + 1) > slab_lo(grp)) {
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive(&mi->full[0][grp]);
              }
              ++grp;
            }
          }
        }
        if (pt == 0) TRS(2, u);
        group_sync(3, 256);   // every warp is done with the staging buffer: the rows of unit u + 2 may land in it
        publish_ref(u + 2, src_b);
        publish_scale(u + 2, rs_b);
        start_copy(u + 2, src_b);
        fetch_row(u + 3, id_a, src_b, rs_b);
        id_a = fetch_id(u + 4);
      }
    } else {
      // 16-bit tables need no widening: TMA row gathers write the operand layout directly.  A thread owns
      // (slab, group of four rows) pairs, slab by slab, so that the logit MMAs of the first slabs can start
      // while the later ones travel; rows without data are fetched from row -1 (zeros).
      for (int u = 0; u < nunits; ++u) {
        const int buf = u & 1, slot = u & (kRing - 1);
        uint8_t* ub = smem + L.ub_off[buf];
        if (pt == 0) TRS(0, u);
        // the row metadata slot written below was last read for unit u - 2, whose softmax is over once its first
        // value block has been multiplied
        if (u >= 2) wait_pv_block(u - 2, 0);
        if (pt == 0) TRS(1, u);
        publish_ref(u + 2, src_b);
        fetch_row(u + 3, id_a, src_b, rs_b);
        id_a = fetch_id(u + 4);
        if (pt == 0)
          for (int kb = 0; kb < nslab; ++kb) ptx::mbar_expect_tx(&mi->full[buf][kb], (uint32_t)WS_SLAB);
        for (int i = pt; i < 16 * nslab; i += 256) {
          const int sl = i >> 4, r0 = (i & 15) * 4;
          if (u >= 2) wait_pv_slab(u - 2, sl);   // this slab of the buffer has been multiplied by P V of unit u - 2
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
          ptx::tma_gather4_2d(ub + (size_t)sl * WS_SLAB + (size_t)r0 * 128, from_raw ? &tm_raw : &tm_comp,
                              &mi->full[buf][sl], sl * 64, y[0], y[1], y[2], y[3]);
        }
        if (pt == 0) TRS(2, u);
        group_sync(3, 256);
      }
    }
  } else if (warp >= 8 && warp < W_PV) {
    // ================================================================ S^T = Kunit . Q^T issuers
    // Issuer j accumulates its share of the feature slabs into an accumulator of its own; the softmax adds them.
    if (lane == 0) {
      const int j = warp - 8;
      const int kb_lo = slab_lo(j), kb_hi = slab_lo(j + 1);
      const uint32_t idesc_s = ptx::idesc_f16(fmt, fmt, WS_UNIT, WS_HEADS, 0, 0);
      const uint64_t q_desc = ptx::smem_desc_sw128(ptx::smem_u32(q_s), 16, 1024);
      ptx::mbar_wait(&mi->q_ready, 0, abort_flag);   // also when there is no unit: q has landed before the CTA exits
      for (int u = 0; u < nunits; ++u) {
        const int buf = xbuf(u);
        const uint64_t k_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + L.ub_off[buf]), 16, 1024);
        const uint32_t d = tmem_base + (uint32_t)((I8 ? 0 : buf * 128) + j * WS_HEADS);
        if (prev_use(u) >= 0) ptx::mbar_wait(&mi->s_free[buf], xphase(prev_use(u)), abort_flag);   // S^T has been read
        if (I8 && kb_hi > kb_lo) ptx::mbar_wait(&mi->full[0][j], xphase(u), abort_flag);
        for (int kb = kb_lo; kb < kb_hi; ++kb) {
          if (!I8) ptx::mbar_wait(&mi->full[buf][kb], xphase(u), abort_flag);   // each slab as soon as it has landed
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
  } else if (warp >= W_PV && warp < W_PROD) {
    // ================================================================ O^T += Vunit^T . P^T issuers
    const int mt = warp - W_PV;
    if (lane == 0 && mt < n_mt) {
      const uint32_t idesc_o = ptx::idesc_f16(fmt, fmt, 128, WS_HEADS, 1, 0);   // A read MN-major
      for (int u = 0; u < nunits; ++u) {
        const int buf = xbuf(u);
        // A, MN-major: 64-feature blocks 8 KB apart (LBO), 8-row groups 1 KB apart (SBO); 16 rows per K step
        const uint64_t v_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + L.ub_off[buf]), WS_SLAB, 1024);
        const uint64_t pt_desc = ptx::smem_desc_sw128(ptx::smem_u32(smem + L.pt_off[buf]), 16, 1024);
        ptx::mbar_wait(&mi->p_ready[buf], xphase(u), abort_flag);
        ptx::tc_fence_after_sync();
        if (warp == W_PV) TRS(9, u);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ptx::mma_f16_ss(tmem_o + (uint32_t)(mt * WS_HEADS), ptx::desc_advance(v_desc, (2 * mt) * WS_SLAB + ks * 2048),
                          ptx::desc_advance(pt_desc, ks * 32), idesc_o, (u > 0 || ks > 0) ? 1u : 0u);
        ptx::mma_commit(&mi->pv_blk[buf][mt]);
        if (warp == W_PV) TRS(10, u);
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

    // q: finish the operand (register path: convert and store; TMA path: wait, convert in place if needed)
    if (q_regs) {
      if (q_fast) {
        store_q_pass(0);
        for (int pass = 1; pass * kQB * 256 < n_items; ++pass) {
          load_q_pass(pass);
          store_q_pass(pass);
        }
      } else {
        for (int i = tid; i < n_items; i += 256) {   // fp32 q, unaligned q
          const int h = i & (WS_HEADS - 1), c = i >> 6;
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = 0.f;
          if (h < p.H) {
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
          store_q_item(i, f);
        }
      }
    } else {
      ptx::mbar_wait(&mi->q_full, 0, abort_flag);
      if constexpr (Q_CONVERT) {
        // bf16 -> fp16 in place, element by element (the swizzled position of a chunk does not change);
        // exact for magnitudes in [2^-14, 65504], which is where the reference's fp16 q lives as well
        for (int i = tid; i < nslab * (WS_SLAB / 16); i += 256) {
          uint4* cell = reinterpret_cast<uint4*>(q_s) + i;
          uint4 x = *cell;
          uint32_t* w = reinterpret_cast<uint32_t*>(&x);
#pragma unroll
          for (int e = 0; e < 4; ++e) {
            const float2 f = __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&w[e]));
            const __half2 h2 = __floats2half2_rn(f.x, f.y);
            w[e] = *reinterpret_cast<const uint32_t*>(&h2);
          }
          *cell = x;
        }
      }
    }
    ptx::fence_proxy_async_smem();
    ptx::mbar_arrive(&mi->q_ready);

    float l1 = 0.f;   // row sum of head col0 + li over this warp's rows of all units
    for (int u = 0; u < nunits; ++u) {
      const int buf = xbuf(u), slot = u & (kRing - 1);
      ptx::mbar_wait(&mi->s_ready[buf], xphase(u), abort_flag);
      ptx::tc_fence_after_sync();
      if (warp == 0) TRS(5, u);
      uint32_t sv[16];
      {
        // add the issuers' accumulators, two loads in flight at a time (issuers without a slab leave theirs untouched)
        const uint32_t sa = tmem_base + lane_off + (uint32_t)((I8 ? 0 : buf * 128) + cset * 32);
        uint32_t sb[16];
        const bool has1 = slab_lo(2) > slab_lo(1);
        ptx::tmem_ld_16x32bx2_x16(sa, sv);
        if (has1) ptx::tmem_ld_16x32bx2_x16(sa + (uint32_t)WS_HEADS, sb);
        ptx::tmem_ld_wait();
        if (has1) {
#pragma unroll
          for (int c = 0; c < 16; ++c) sv[c] = __float_as_uint(__uint_as_float(sv[c]) + __uint_as_float(sb[c]));
        }
        if constexpr (NQK == 4) {
          const bool has2 = slab_lo(3) > slab_lo(2), has3 = slab_lo(4) > slab_lo(3);
          uint32_t sc[16];
          if (has2) ptx::tmem_ld_16x32bx2_x16(sa + (uint32_t)(2 * WS_HEADS), sb);
          if (has3) ptx::tmem_ld_16x32bx2_x16(sa + (uint32_t)(3 * WS_HEADS), sc);
          ptx::tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 16; ++c) {
            float x = __uint_as_float(sv[c]);
            if (has2) x += __uint_as_float(sb[c]);
            if (has3) x += __uint_as_float(sc[c]);
            sv[c] = __float_as_uint(x);
          }
        }
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&mi->s_free[buf]);
      const bool ok = mi->row_ref[slot][row] != kNoRow;
      const float rs = I8 ? mi->row_scale[slot][row] : 1.f;
      const float mul = scale_log2 * rs;
      float gap = BF16 ? kRescaleGapBF16 : kRescaleGapF16;
      if (I8 && rs > 1.f) gap -= log2f(rs);
      float mr[16];   // this thread's 16 reference maxima (they move only in the branch below)
#pragma unroll
      for (int c = 0; c < 16; c += 4)
        *reinterpret_cast<float4*>(&mr[c]) = *reinterpret_cast<const float4*>(&mi->m_ref[col0 + c]);
      bool grow = false;
#pragma unroll
      for (int c = 0; c < 16; ++c) {
        const float x = ok ? __uint_as_float(sv[c]) * mul : -INFINITY;
        sv[c] = __float_as_uint(x);
        grow |= x > mr[c] + gap;
      }
      if (warp == 0) TRS(6, u);
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
        // O^T belongs to the old reference: it is final for the units so far once the previous P V is done
        if (u >= 1) wait_pv_all(u - 1);
        group_sync(4, 256);
        if (tid < WS_HEADS) {
          const float old = mi->m_ref[tid];
          float mx = fmaxf(fmaxf(mi->colmax[0][tid], mi->colmax[1][tid]), fmaxf(mi->colmax[2][tid], mi->colmax[3][tid]));
          mx = fmaxf(mx, old);
          mi->factor[tid] = (old == -INFINITY) ? 0.f : exp2f(old - mx);
          mi->m_ref[tid] = mx;
        }
        group_sync(4, 256);
        ptx::tc_fence_after_sync();
        l1 *= mi->factor[col0 + li];
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
#pragma unroll
        for (int c = 0; c < 16; c += 4)
          *reinterpret_cast<float4*>(&mr[c]) = *reinterpret_cast<const float4*>(&mi->m_ref[col0 + c]);
      }
      if (warp == 0) TRS(7, u);
      // ---- P^T (16-bit, K-major, swizzled) and the row sums
      {
        const float inv = I8 ? __frcp_rn(rs) : 1.f;
        uint8_t* pbase = smem + L.pt_off[buf] + (row & 7) * 2;
        const int cj = row >> 3;
#pragma unroll
        for (int c = 0; c < 16; c += 2) {   // two heads per step: one packed conversion each way
          const int h = col0 + c;
          const float s0 = __uint_as_float(sv[c]), s1 = __uint_as_float(sv[c + 1]);
          float p0 = (s0 == -INFINITY) ? 0.f : fast_exp2(s0 - mr[c]);
          float p1 = (s1 == -INFINITY) ? 0.f : fast_exp2(s1 - mr[c + 1]);
          if (I8) {
            p0 *= rs;
            p1 *= rs;
          }
          float b0, b1;
          const uint32_t pr = pack_op16x2<BF16>(p0, p1, b0, b1);
          sv[c] = __float_as_uint(I8 ? b0 * inv : b0);
          sv[c + 1] = __float_as_uint(I8 ? b1 * inv : b1);
          *reinterpret_cast<uint16_t*>(pbase + (size_t)h * 128 + ((cj ^ (h & 7)) << 4)) = (uint16_t)(pr & 0xffffu);
          *reinterpret_cast<uint16_t*>(pbase + (size_t)(h + 1) * 128 + ((cj ^ ((h + 1) & 7)) << 4)) = (uint16_t)(pr >> 16);
        }
      }
      if (warp == 0) TRS(12, u);
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&mi->p_ready[buf]);
      if (warp == 0) TRS(8, u);
      // Sum over the 16 rows of this half warp, behind the hand-off: at each step a lane keeps half of its
      // columns and hands the other half to its partner, so 15 shuffles leave lane li with column li.
#pragma unroll
      for (int step = 8; step >= 1; step >>= 1) {
        const bool upper = (li & step) != 0;
#pragma unroll
        for (int c = 0; c < step; ++c) {
          const float send = upper ? __uint_as_float(sv[c]) : __uint_as_float(sv[c + step]);
          const float keep = upper ? __uint_as_float(sv[c + step]) : __uint_as_float(sv[c]);
          sv[c] = __float_as_uint(keep + __shfl_xor_sync(0xffffffffu, send, step));
        }
      }
      l1 += __uint_as_float(sv[0]);
    }

    // ------------------------------------------------------------------ row sums over all units
    if (tid == 0) TRS(11, 2);
    group_sync(4, 256);   // nobody reads the column maxima any more
    mi->colmax[wq][col0 + li] = l1;
    if (nunits >= 1) wait_pv_all(nunits - 1);
    if (!I8 && nunits >= 2) wait_pv_all(nunits - 2);
    ptx::tc_fence_after_sync();
    group_sync(4, 256);
    if (tid == 0) TRS(11, 3);

    // ------------------------------------------------------------------ output
    const int64_t N = (int64_t)p.B * p.T * p.H;
    const bool direct = p.nsplit == 1;
    const bool finalize = direct && !p.partial_ml;
    const bool have_o = nunits > 0;
    if (tid < WS_HEADS) {
      const float l = (mi->colmax[0][tid] + mi->colmax[1][tid]) + (mi->colmax[2][tid] + mi->colmax[3][tid]);
      mi->l_tot[tid] = l;
      // per-head factor applied to O^T: 1 for partial output, exp(m - m') / denominator with the sink joined otherwise
      float fac = 1.f;
      if (finalize) {
        const float m = mi->m_ref[tid];
        const float sink2 = (p.sinks && tid < p.H) ? p.sinks[tid] * 1.4426950408889634f : -INFINITY;
        const float m2v = fmaxf(m, sink2);
        float w = 0.f, den = 0.f;
        if (m2v > -INFINITY) {
          w = (m == -INFINITY) ? 0.f : exp2f(m - m2v);
          den = l * w + ((sink2 == -INFINITY) ? 0.f : exp2f(sink2 - m2v));
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
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          const int h = hh * 32 + c;
          if (h >= p.H) continue;
          const float o = __uint_as_float(ov[c]) * mi->factor[h];
          if (finalize) store_elem<OT>(p.out, gbase + d + h * ostep, o);
          else if (direct) reinterpret_cast<float*>(p.out)[gbase + d + h * ostep] = o;
          else p.ws_o[gbase + d + h * ostep] = o;
        }
      }
    }
    if (tid < p.H && (!direct || p.partial_ml)) {
      // (m, l) in natural-log units for the merge kernel
      const float m_nat = mi->m_ref[tid] == -INFINITY ? -INFINITY : mi->m_ref[tid] * 0.6931471805599453f;
      float* ml = direct ? p.partial_ml + ((int64_t)bt * p.H + tid) * 2
                         : p.ws_ml + ((int64_t)split * N + (int64_t)bt * p.H + tid) * 2;
      ml[0] = m_nat;
      ml[1] = mi->l_tot[tid];
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
  int64_t want;
  if (requested > 0) {
    want = requested;
  } else {
    const int64_t base = (int64_t)B * T;
    want = (int64_t)sm_count() / (base > 0 ? base : 1);  // one wave of CTAs
  }
  if (want > max_parts) want = max_parts;
  if (want > 64) want = 64;
  if (want < 1) want = 1;
  return (int)want;
}

// Tensor map over a [rows, Dqk] table of 16-bit values for row gathers: box = one 128-byte slab of one row.  The
// row extent is left open (the caller's ids are what bounds the reads); row -1 is the zero row.
static int row_gather_map(CUtensorMap* out, const void* table, int Dqk, bool bf16) {
  const uint64_t dims[2] = {(uint64_t)Dqk, (uint64_t)0x7FFFFFFF};
  const uint64_t strides[1] = {(uint64_t)Dqk * 2};
  const uint32_t box[2] = {64, 1};
  return make_tensor_map(out, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, table, dims,
                         strides, box, CU_TENSOR_MAP_SWIZZLE_128B);
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
  const int smem = ws_layout(p.Dqk, p.Dv, I8).total + 1024;
  CUtensorMap tm_comp, tm_raw, tm_q;
  memset(&tm_comp, 0, sizeof(tm_comp));
  memset(&tm_raw, 0, sizeof(tm_raw));
  memset(&tm_q, 0, sizeof(tm_q));
  if (!I8) {
    const void* comp = p.comp_kv ? p.comp_kv : p.raw_kv;
    MXB_REQUIRE(comp != nullptr || p.k + p.raw_cap == 0, MXB_ERR_INVALID, "sparse attention: no KV table");
    if (comp) {
      int rc = row_gather_map(&tm_comp, comp, p.Dqk, KVT == MXB_BF16);
      if (rc != MXB_OK) return rc;
      rc = row_gather_map(&tm_raw, p.raw_kv ? p.raw_kv : comp, p.Dqk, KVT == MXB_BF16);
      if (rc != MXB_OK) return rc;
    }
  }
  // a 16-bit q lands by TMA: as it is when it has the operand type, converted in place for a bf16 q over int8 rows
  p.q_tma = 0;
  if (QT == MXB_BF16 || QT == MXB_F16) p.q_tma = q_tile_map(&tm_q, p, QT == MXB_BF16) ? 1 : 0;
  const int64_t ctas = (int64_t)p.B * p.T * p.nsplit;
  MXB_REQUIRE(ctas <= 0x7FFFFFFFll, MXB_ERR_INVALID, "sparse attention: too many (batch, token, split) items");
  dim3 grid((unsigned)ctas);
#define MXB_TC(OT)                                                                                   \
  {                                                                                                  \
    auto kern = sparse_attn_tc_kernel<KVT, QT, OT>;                                                  \
    MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));      \
    kern<<<grid, ws_threads(I8), smem, st>>>(p, tm_comp, tm_raw, tm_q);                                  \
  }
  if (out_dtype == MXB_F32 || p.nsplit > 1 || p.partial_ml) MXB_TC(MXB_F32)
  else if (out_dtype == MXB_BF16) MXB_TC(MXB_BF16)
  else MXB_TC(MXB_F16)
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
