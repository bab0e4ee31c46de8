// Indexed mixed (sparse) attention on tcgen05 / TMEM for 16-bit and int8 KV tables.
//
// One CTA = one (split, sequence, token): all heads (<= 64) of that token share every
// gathered row.  The gathered rows sit on the MMA M axis:
//
//   S^T[128 rows x 64 heads]  = Ktile[128 x Dqk] . Q^T          (A = row tile, K-major)
//   O^T[Dv dims  x 64 heads] += Vtile^T[Dv x 128] . P^T          (A = the SAME row tile, read
//                                                                 MN-major: dims contiguous)
//
// so one staged copy of the rows (128-byte-swizzled 64-feature slabs) feeds both
// contractions and nothing is transposed.  16-bit rows are gathered by TMA (tile::gather4: four rows x one slab
// per instruction, swizzled on the way in, row -1 = zeros for padding).  int8 rows are gathered with 16-byte
// vector loads through registers, widened to fp16 integers (exact) while staging, and their per-row scale is
// folded into the logit (s = scale_j * q.int_j) and into P (p_j * scale_j), so the tensor
// core multiplies exact values.  Thread = row for the softmax (TMEM lane), with a lazily
// updated per-head reference maximum held in shared memory: the cross-row maximum is
// reduced only when some logit exceeds the reference by more than a gap (2^15 for fp16 operands, 2^60 for bf16),
// the O accumulator in TMEM is rescaled only then.  The row sum uses the ROUNDED 16-bit P
// values, so out = sum(p~ v) / sum(p~) is an exactly normalised average.  Splits over the
// row list emit (o, m, l) partials for the log-sum-exp merge kernel.
//
// Operand type: fp16 for fp16 and int8 tables (q is rounded to fp16 on load, as the
// reference kernels do), bf16 for bf16 tables.  TMEM: S^T at columns [0,64), O^T at
// [64, 64 + Dv/2).
#include "common.cuh"
#include "ptx_sm100.cuh"
#include "sparse_attn.cuh"


namespace mxb {

#ifdef MXB_TRACE_SP
#define TRS(k, i) do { if (tr_on && (i) < 16) tr[(k) * 16 + (i)] = clock64(); } while (0)
#else
#define TRS(k, i)
#endif

constexpr int TC_ROWS = 128;
constexpr int TC_HEADS = 64;
// The running reference m_ref of a head moves only when a score exceeds it by more than a gap (log2 units):
// P = 2^(s - m_ref) may then be as large as 2^gap.  bf16 operands have fp32's range; fp16 operands top out at
// 65504, and the int8 path folds the row's dequantisation scale into P, so its gap shrinks by log2(scale) when
// that is positive.
constexpr float kRescaleGapF16 = 15.f;
constexpr float kRescaleGapBF16 = 60.f;

constexpr int kTcMiscBytes = 8192;   // reserved for TcMisc

struct TcLayout {
  int nslab;       // Dqk / 64
  int tile_off;    // rows tile: nslab slabs of [128 x 128 B]
  int q_off;       // q operand: nslab slabs of [64 x 128 B]
  int pt_off;      // P^T: 2 slabs of [64 heads x 128 B]
  int misc_off;
  int total;
};

__host__ __device__ inline TcLayout tc_layout(int Dqk, int Dv) {
  TcLayout L;
  L.nslab = Dqk / 64;
  L.tile_off = 0;
  L.q_off = L.nslab * 16384;
  int end = L.q_off + L.nslab * 8192;
  if (Dqk - Dv >= 64) {
    L.pt_off = (Dv / 64) * 16384;  // the slab that only the logits need is free once S^T is done
  } else {
    L.pt_off = end;
    end += 16384;
  }
  L.misc_off = end;
  L.total = end + kTcMiscBytes;
  return L;
}

struct TcMisc {
  float m_ref[TC_HEADS];
  float factor[TC_HEADS];
  float colmax[4][TC_HEADS];
  float l_tot[TC_HEADS];
  float row_scale[3][TC_ROWS];   // per-tile row metadata, three deep: rows are resolved (ids -> addresses -> scales)
  uint32_t row_ref[3][TC_ROWS];  // two tiles ahead, so that the loads of the next tile can be issued as soon as the
                                 // registers that carry them are free.  row_ref: kNoRow, or row index within its
                                 // table (< 2^31) with bit 31 set for the raw table
  uint64_t bar_s, bar_o, bar_t;
  uint32_t tmem_slot;
  int abort_flag;
  int keff;
};

constexpr uint32_t kNoRow = 0xFFFFFFFFu;
static_assert(sizeof(TcMisc) <= kTcMiscBytes, "TcMisc must fit the bytes the layout reserves for it");

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

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool BF16>
__device__ __forceinline__ uint16_t to_op16(float x) {
  if constexpr (BF16) {
    __nv_bfloat16 v = __float2bfloat16_rn(x);
    return *reinterpret_cast<uint16_t*>(&v);
  } else {
    __half v = __float2half_rn(x);
    return *reinterpret_cast<uint16_t*>(&v);
  }
}
template <bool BF16>
__device__ __forceinline__ float from_op16(uint16_t u) {
  if constexpr (BF16) return __bfloat162float(*reinterpret_cast<__nv_bfloat16*>(&u));
  else return __half2float(*reinterpret_cast<__half*>(&u));
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

template <int KVT, int QT, int OT>
__global__ void __launch_bounds__(256, 1) sparse_attn_tc_kernel(SparseParams p, const __grid_constant__ CUtensorMap tm_comp,
                                                                const __grid_constant__ CUtensorMap tm_raw) {
  constexpr bool BF16 = (KVT == MXB_BF16);
  constexpr int EB = ElemBytes<KVT>::v;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  const TcLayout L = tc_layout(p.Dqk, p.Dv);
  uint8_t* tile = smem + L.tile_off;
  uint8_t* q_s = smem + L.q_off;
  uint8_t* pt = smem + L.pt_off;
  TcMisc* mi = reinterpret_cast<TcMisc*>(smem + L.misc_off);
  volatile int* abort_flag = &mi->abort_flag;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int quad = warp & 3, half_id = warp >> 2;
  const int split = blockIdx.x;
  const int bt = blockIdx.z;
  const int b = bt / p.T, t = bt % p.T;
  const int nslab = L.nslab;
  const int n_mt = p.Dv / 128;

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
  const int32_t* ids = p.topk + (int64_t)bt * p.k;
#ifdef MXB_TRACE_SP
  long long* tr = reinterpret_cast<long long*>(p.status);
  const bool tr_on = p.status && blockIdx.x == 0 && blockIdx.z == 0 && tid == 0;
  TRS(7, 0);
#endif

  if (tid == 0) {
    ptx::mbar_init(&mi->bar_s, 1);
    ptx::mbar_init(&mi->bar_o, (uint32_t)(p.Dv / 128));
    ptx::mbar_init(&mi->bar_t, 1);
    mi->abort_flag = 0;
    mi->keff = p.k;
    ptx::mbar_fence_init();
  }
  if (tid < TC_HEADS) {
    mi->m_ref[tid] = -INFINITY;
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
  const uint32_t tmem_o = tmem_base + 64;
  TRS(12, 0);

  // q -> B operand of S^T: [64 heads x Dqk] K-major, 128-byte swizzle, rounded to the operand type.
  // Item i = (head i % 64, 16-byte chunk i / 64): a warp writes 32 different rows, conflict-free stores.
  const bool q_vec = ((reinterpret_cast<uintptr_t>(p.q) & 15) == 0) && (p.q_sb % 8 == 0) && (p.q_sh % 8 == 0) &&
                     (p.q_st % 8 == 0);
  const int n_items = TC_HEADS * (p.Dqk / 8);
  auto store_q_item = [&](int i, const float* f) {
    const int h = i & (TC_HEADS - 1), c = i >> 6;
    uint32_t w[4];
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float b0, b1;
      w[e] = pack_op16x2<BF16>(f[2 * e], f[2 * e + 1], b0, b1);
    }
    const int kb = c >> 3, cc = c & 7;
    *reinterpret_cast<uint4*>(q_s + (size_t)kb * 8192 + (size_t)h * 128 + ((cc ^ (h & 7)) << 4)) =
        make_uint4(w[0], w[1], w[2], w[3]);
  };
  constexpr int kQB = 18;   // 16-bit q, vector path: this many 16-byte loads in flight per thread
  uint4 qraw[kQB];
  const bool q_fast = q_vec && QT != MXB_F32;
  if (q_fast) {
#pragma unroll
    for (int j = 0; j < kQB; ++j) {
      const int i = tid + j * 256;
      const int h = i & (TC_HEADS - 1), c = i >> 6;
      qraw[j] = make_uint4(0, 0, 0, 0);
      if (i < n_items && h < p.H)
        qraw[j] = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + (int64_t)b * p.q_sb +
                                                       (int64_t)h * p.q_sh + (int64_t)t * p.q_st + c * 8));
    }
  }
  {  // first list entry that ends the walk (its loads overlap the q loads above)
    int mine = p.k;
#pragma unroll 4
    for (int j = tid; j < p.k; j += 256) {   // no early exit: the loads stay independent
      const int64_t v = ids[j];
      if (v >= visible && j < mine) mine = j;
    }
    if (mine < p.k) atomicMin(&mi->keff, mine);
  }
  TRS(12, 1);
  if (q_fast) {
#pragma unroll
    for (int j = 0; j < kQB; ++j) {
      const int i = tid + j * 256;
      if (i < n_items) {
        float f[8];
        if constexpr (QT != MXB_F32) unpack16<QT>(qraw[j], f);
        store_q_item(i, f);
      }
    }
  }
  for (int i = tid + (q_fast ? kQB * 256 : 0); i < n_items; i += 256) {   // wide rows, fp32 q, unaligned q
    const int h = i & (TC_HEADS - 1), c = i >> 6;
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
          const uint4 u = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(p.q) + base));
          unpack16<QT>(u, f);
        }
      } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = load_elem<QT>(p.q, base + e);
      }
    }
    store_q_item(i, f);
  }
  TRS(12, 2);
  __syncthreads();
  TRS(12, 3);
  const int total = n_raw + mi->keff;
  int per = (total + p.nsplit - 1) / p.nsplit;
  per = ((per + TC_ROWS - 1) / TC_ROWS) * TC_ROWS;
  const int e_lo = min(split * per, total), e_hi = min(e_lo + per, total);
  const int ntiles = (e_hi - e_lo + TC_ROWS - 1) / TC_ROWS;

  constexpr uint32_t fmt = BF16 ? ptx::kFmtBF16 : ptx::kFmtF16;
  const uint32_t idesc_s = ptx::idesc_f16(fmt, fmt, 128, TC_HEADS, 0, 0);
  const uint32_t idesc_o = ptx::idesc_f16(fmt, fmt, 128, TC_HEADS, 1, 0);  // A read MN-major
  const uint32_t tile_addr = ptx::smem_u32(tile), q_addr = ptx::smem_u32(q_s), pt_addr = ptx::smem_u32(pt);
  const float scale_log2 = p.scale * 1.4426950408889634f;
  const uint64_t tile_desc_k = ptx::smem_desc_sw128(tile_addr, 16, 1024);
  const uint64_t tile_desc_mn = ptx::smem_desc_sw128(tile_addr, 16384, 1024);
  const uint64_t q_desc = ptx::smem_desc_sw128(q_addr, 16, 1024);
  const uint64_t pt_desc = ptx::smem_desc_sw128(pt_addr, 16, 1024);

  float l_thr[32];
#pragma unroll
  for (int c = 0; c < 32; ++c) l_thr[c] = 0.f;
  bool have_o = false;

  // gather plan: one warp instruction covers 8 rows x 4 consecutive 16-byte chunks (lane = row%8 + 8*chunk):
  // the 8 rows have 8 different swizzle phases, so the 128-bit shared-memory stores are conflict-free, and
  // the 4 chunks of a row are 64 contiguous bytes in global memory.
  const int nch = p.Dqk * EB / 16;
  const int ncg = (nch + 3) / 4;   // groups of 4 chunks per row
  const int r8 = lane & 7, cl = lane >> 3;

  // Row metadata (list id -> row address -> dequantisation scale) is a chain of dependent global loads.  Warps
  // 1-7 (warp 0 issues the QK MMAs) run it as a pipeline, one stage per tile iteration, so that nobody ever
  // waits on it: stage A fetches the list id, stage B turns it into the address, fetches the scale and pulls
  // the row towards L2, and the last stage publishes both in shared memory, two tiles before they are needed.
  const int rr_res = (warp - 1) + 7 * lane;
  const bool resolver = warp >= 1 && rr_res < TC_ROWS;
  auto fetch_id = [&](int T) -> int32_t {   // -1: no compressed row behind this slot
    if (!resolver || T >= ntiles) return -1;
    const int e = e_lo + T * TC_ROWS + rr_res;
    return (e < e_hi && e >= n_raw) ? ids[e - n_raw] : -1;
  };
  auto fetch_row = [&](int T, int32_t id, uint32_t& ref, float& rs) {
    const uint8_t* src = nullptr;
    ref = kNoRow;
    rs = 1.f;
    if (!resolver || T >= ntiles) return;
    const int e = e_lo + T * TC_ROWS + rr_res;
    if (e >= e_hi) return;
    if (e < n_raw) {
      const int64_t pabs = first + e;
      const int64_t phys = ((int64_t)p.raw_start + (pabs - first_raw_pos)) % p.raw_cap;
      const int64_t ridx = (int64_t)b * p.raw_cap + phys;
      src = reinterpret_cast<const uint8_t*>(p.raw_kv) + ridx * p.Dqk * EB;
      ref = (uint32_t)ridx | 0x80000000u;
      if (KVT == MXB_I8) rs = __half2float(p.raw_scales[ridx]);
    } else if (id >= 0) {
      const int64_t ridx = cbase + id;
      src = reinterpret_cast<const uint8_t*>(p.comp_kv) + ridx * p.Dqk * EB;
      ref = (uint32_t)ridx;
      if (KVT == MXB_I8) rs = __half2float(p.comp_scales[ridx]);
    }
    if (src) {
      const int row_bytes = p.Dqk * EB;
      for (int off = 0; off < row_bytes; off += 128) asm volatile("prefetch.global.L2 [%0];" ::"l"(src + off));
      asm volatile("prefetch.global.L2 [%0];" ::"l"(src + row_bytes - 1));
    }
  };
  auto publish_row = [&](int T, uint32_t ref, float rs) {
    if (resolver && T < ntiles) {
      mi->row_ref[T % 3][rr_res] = ref;
      mi->row_scale[T % 3][rr_res] = rs;
    }
  };
  auto row_address = [&](uint32_t ref) -> const uint8_t* {
    if (ref == kNoRow) return nullptr;
    const uint8_t* base = reinterpret_cast<const uint8_t*>((ref >> 31) ? p.raw_kv : p.comp_kv);
    return base + (int64_t)(ref & 0x7FFFFFFFu) * (p.Dqk * EB);
  };
  int32_t id_a = -1;          // stage A result: list id of this lane's row of tile it + 3
  uint32_t src_b = kNoRow;    // stage B result: row and scale of this lane's row of tile it + 2
  float rs_b = 1.f;
  // Raw rows travel through registers: 18 independent 16-byte loads per lane (9 groups of 4 chunks for
  // each of the lane's two rows).  The loads of the NEXT tile are issued right after this tile's QK MMAs
  // and land during its softmax and PV; only the widening and the shared-memory stores stay on the
  // critical path.
  uint4 v[18];
  auto issue_loads = [&](int mbuf, int cg0) {
    const uint8_t* src_lo = row_address(mi->row_ref[mbuf][warp * 16 + r8]);
    const uint8_t* src_hi = row_address(mi->row_ref[mbuf][warp * 16 + 8 + r8]);
#pragma unroll
    for (int i = 0; i < 18; ++i) {
      const int c = (cg0 + (i >> 1)) * 4 + cl;
      const uint8_t* src = (i & 1) ? src_hi : src_lo;
      v[i] = make_uint4(0, 0, 0, 0);
      if (src && c < nch) v[i] = __ldg(reinterpret_cast<const uint4*>(src) + c);
    }
  };
  auto store_loaded = [&](int cg0) {
#pragma unroll
    for (int i = 0; i < 18; ++i) {
      const int c = (cg0 + (i >> 1)) * 4 + cl;
      if (c < nch) {
        const int rr = warp * 16 + (i & 1) * 8 + r8;
        uint8_t* drow = tile + (size_t)rr * 128;
        if constexpr (KVT == MXB_I8) {
          uint4 lo, hi;
          widen_i8x16_f16(v[i], lo, hi);   // zero bytes (invalid row) widen to 0.0
          const int kb = c >> 2, cc = (c & 3) * 2;
          uint8_t* d = drow + (size_t)kb * 16384;
          *reinterpret_cast<uint4*>(d + ((cc ^ r8) << 4)) = lo;
          *reinterpret_cast<uint4*>(d + (((cc + 1) ^ r8) << 4)) = hi;
        } else {
          const int kb = c >> 3, cc = c & 7;
          *reinterpret_cast<uint4*>(drow + (size_t)kb * 16384 + ((cc ^ r8) << 4)) = v[i];
        }
      }
    }
  };
  // 16-bit tables need no widening, so their rows can bypass the registers: TMA row gathers (four rows x one
  // 128-byte slab per instruction, swizzled on the way in) write the operand layout directly.  Warp w fetches rows
  // 16w .. 16w+15; a lane owns (group of four rows, slab) pairs.  Rows without data are fetched from row -1 (zeros).
  // A group of four that holds rows of BOTH tables (at most one per token, where the raw window ends) is fetched
  // from the compressed table and its raw rows are patched in with plain loads once the tile has landed.
  const bool tma_rows = KVT != MXB_I8 && p.tma_rows != 0;
  auto group_refs = [&](int mbuf, int r0, uint32_t* ref, bool& any_raw, bool& any_comp) {
    any_raw = any_comp = false;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      ref[j] = mi->row_ref[mbuf][r0 + j];
      if (ref[j] != kNoRow) {
        if (ref[j] >> 31) any_raw = true;
        else any_comp = true;
      }
    }
  };
  auto issue_tma = [&](int T) {
    const int mbuf = T % 3;
    if (tid == 0) ptx::mbar_expect_tx(&mi->bar_t, (uint32_t)(TC_ROWS * p.Dqk * 2));
    for (int i = lane; i < 4 * nslab; i += 32) {
      const int g = i / nslab, sl = i % nslab;
      const int r0 = warp * 16 + g * 4;
      uint32_t ref[4];
      bool any_raw, any_comp;
      group_refs(mbuf, r0, ref, any_raw, any_comp);
      const bool from_raw = any_raw && !any_comp;
      int32_t y[4];
#pragma unroll
      for (int j = 0; j < 4; ++j)
        y[j] = (ref[j] != kNoRow && (ref[j] >> 31) == (from_raw ? 1u : 0u)) ? (int32_t)(ref[j] & 0x7FFFFFFFu) : -1;
      ptx::tma_gather4_2d(tile + (size_t)sl * 16384 + (size_t)r0 * 128, from_raw ? &tm_raw : &tm_comp, &mi->bar_t,
                          sl * 64, y[0], y[1], y[2], y[3]);
    }
  };
  auto patch_mixed = [&](int T) {
    const int mbuf = T % 3;
    for (int i = lane; i < 4 * nslab; i += 32) {
      const int g = i / nslab, sl = i % nslab;
      const int r0 = warp * 16 + g * 4;
      uint32_t ref[4];
      bool any_raw, any_comp;
      group_refs(mbuf, r0, ref, any_raw, any_comp);
      if (!(any_raw && any_comp)) continue;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (ref[j] == kNoRow || !(ref[j] >> 31)) continue;
        const int rr = r0 + j;
        const uint4* src = reinterpret_cast<const uint4*>(row_address(ref[j]) + (size_t)sl * 128);
        uint8_t* drow = tile + (size_t)sl * 16384 + (size_t)rr * 128;
#pragma unroll
        for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(drow + ((c ^ (rr & 7)) << 4)) = __ldg(src + c);
      }
    }
  };
  if (ntiles > 0) {
    // prime the pipeline: tiles 0 and 1 published, tile 2 through stage B, tile 3 through stage A
    const int32_t i0 = fetch_id(0), i1 = fetch_id(1), i2 = fetch_id(2);
    id_a = fetch_id(3);
    uint32_t s0, s1;
    float r0, r1;
    fetch_row(0, i0, s0, r0);
    fetch_row(1, i1, s1, r1);
    fetch_row(2, i2, src_b, rs_b);
    publish_row(0, s0, r0);
    publish_row(1, s1, r1);
    TRS(12, 4);
    __syncthreads();
    TRS(12, 5);
    if (tma_rows) issue_tma(0);
    else issue_loads(0, 0);
    TRS(12, 6);
  }

  for (int it = 0; it < ntiles; ++it) {
    TRS(0, it);
    // ---------------------------------------------------------------- rows of this tile -> operand layout
    const int mb = it % 3;   // metadata buffer of this tile (filled two tiles ago, or before the loop)
    if (tma_rows) {
      ptx::mbar_wait(&mi->bar_t, (uint32_t)(it & 1), abort_flag);
      patch_mixed(it);
    } else {
      store_loaded(0);
      for (int cg0 = 9; cg0 < ncg; cg0 += 9) {   // rows wider than 9 chunk groups (16-bit tables): the rest, in place
        issue_loads(mb, cg0);
        store_loaded(cg0);
      }
    }
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();

    // ---------------------------------------------------------------- S^T = Ktile . Q^T
    TRS(1, it);
    // While the MMAs are issued and run: one step of the metadata pipeline (nothing in it waits), then the next
    // tile's rows start travelling into registers; the threads sit in that while the load queue drains, which
    // is dead time anyway.  The issuing thread takes its own branch so that the other 31 lanes of its warp can
    // queue their loads while it feeds the tensor core.
    publish_row(it + 2, src_b, rs_b);
    fetch_row(it + 3, id_a, src_b, rs_b);
    id_a = fetch_id(it + 4);
    if (tid == 0) {
      ptx::tc_fence_after_sync();
      for (int kb = 0; kb < nslab; ++kb) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks) {
          ptx::mma_f16_ss(tmem_base, ptx::desc_advance(tile_desc_k, kb * 16384 + ks * 32),
                          ptx::desc_advance(q_desc, kb * 8192 + ks * 32), idesc_s, (kb | ks) ? 1u : 0u);
        }
      }
      ptx::mma_commit(&mi->bar_s);
      TRS(2, it);
      if (!tma_rows && it + 1 < ntiles) issue_loads((it + 1) % 3, 0);
    } else {
      if (!tma_rows && it + 1 < ntiles) issue_loads((it + 1) % 3, 0);
    }
    ptx::mbar_wait(&mi->bar_s, (uint32_t)(it & 1), abort_flag);
    ptx::tc_fence_after_sync();

    // ---------------------------------------------------------------- softmax, thread = row
    TRS(3, it);
    const int row = quad * 32 + lane;
    const int col0 = half_id * 32;
    uint32_t sv[32];
    ptx::tmem_ld32(tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)col0, sv);
    ptx::tmem_ld_wait();
    TRS(8, it);
    const bool ok = mi->row_ref[mb][row] != kNoRow;
    const float rs = mi->row_scale[mb][row];
    const float mul = scale_log2 * rs;
    float gap = BF16 ? kRescaleGapBF16 : kRescaleGapF16;
    if (KVT == MXB_I8 && rs > 1.f) gap -= log2f(rs);
    bool grow = false;
#pragma unroll
    for (int c = 0; c < 32; ++c) {
      const float x = ok ? __uint_as_float(sv[c]) * mul : -INFINITY;
      sv[c] = __float_as_uint(x);
      grow |= x > mi->m_ref[col0 + c] + gap;
    }
    TRS(9, it);
    if (__syncthreads_or(grow ? 1 : 0)) {
      // exact column maxima of this tile, new reference, rescale of what has been accumulated
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        // one integer warp reduction per column on an order-preserving image of the float
        const int o = __reduce_max_sync(0xffffffffu, float_order(__uint_as_float(sv[c])));
        if (lane == c) mi->colmax[quad][col0 + c] = order_float(o);
      }
      __syncthreads();
      if (tid < TC_HEADS) {
        const float old = mi->m_ref[tid];
        float mx = fmaxf(fmaxf(mi->colmax[0][tid], mi->colmax[1][tid]), fmaxf(mi->colmax[2][tid], mi->colmax[3][tid]));
        mx = fmaxf(mx, old);
        mi->factor[tid] = (old == -INFINITY) ? 0.f : exp2f(old - mx);
        mi->m_ref[tid] = mx;
      }
      __syncthreads();
#pragma unroll
      for (int c = 0; c < 32; ++c) l_thr[c] *= mi->factor[col0 + c];
      if (have_o) {
        // warp -> (lane quadrant, two of the four 128-dim blocks); columns = heads
        for (int m2 = 0; m2 < 2; ++m2) {
          const int mt = half_id * 2 + m2;
          if (mt < n_mt) {
#pragma unroll 1
            for (int ch = 0; ch < 2; ++ch) {
              uint32_t ov[32];
              const uint32_t ta = tmem_o + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * 64 + ch * 32);
              ptx::tmem_ld32(ta, ov);
              ptx::tmem_ld_wait();
#pragma unroll
              for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * mi->factor[ch * 32 + c]);
              ptx::tmem_st32(ta, ov);
            }
          }
        }
        ptx::tmem_st_wait();
      }
    }
    TRS(10, it);
    {
      const float inv = 1.f / rs;
      const int slab = row >> 6, rj = row & 63;
      uint8_t* pbase = pt + (size_t)slab * 8192 + (rj & 7) * 2;
      const int cj = rj >> 3;
#pragma unroll
      for (int c = 0; c < 32; c += 2) {   // two heads per step: one packed conversion each way
        const int h = col0 + c;
        const float s0 = __uint_as_float(sv[c]), s1 = __uint_as_float(sv[c + 1]);
        float p0 = (s0 == -INFINITY) ? 0.f : fast_exp2(s0 - mi->m_ref[h]);
        float p1 = (s1 == -INFINITY) ? 0.f : fast_exp2(s1 - mi->m_ref[h + 1]);
        if (KVT == MXB_I8) {
          p0 *= rs;
          p1 *= rs;
        }
        float b0, b1;
        const uint32_t pr = pack_op16x2<BF16>(p0, p1, b0, b1);
        l_thr[c] += (KVT == MXB_I8) ? b0 * inv : b0;
        l_thr[c + 1] += (KVT == MXB_I8) ? b1 * inv : b1;
        *reinterpret_cast<uint16_t*>(pbase + (size_t)h * 128 + ((cj ^ (h & 7)) << 4)) = (uint16_t)(pr & 0xffffu);
        *reinterpret_cast<uint16_t*>(pbase + (size_t)(h + 1) * 128 + ((cj ^ ((h + 1) & 7)) << 4)) = (uint16_t)(pr >> 16);
      }
    }
    TRS(11, it);
    ptx::fence_proxy_async_smem();
    ptx::tc_fence_before_sync();
    __syncthreads();

    // ---------------------------------------------------------------- O^T += Vtile^T . P^T
    TRS(4, it);
    if (lane == 0 && warp < n_mt) {
      // one issuing thread per 128-feature block of O^T (separate TMEM columns, so no ordering between them)
      const int mt = warp;
      ptx::tc_fence_after_sync();
#pragma unroll
      for (int ks = 0; ks < 8; ++ks) {
        // A, MN-major: 64-feature blocks 16 KB apart (LBO), 8-row groups 1 KB apart (SBO); 16 rows per K step
        ptx::mma_f16_ss(tmem_o + (uint32_t)(mt * 64), ptx::desc_advance(tile_desc_mn, (2 * mt) * 16384 + ks * 2048),
                        ptx::desc_advance(pt_desc, (ks >> 2) * 8192 + (ks & 3) * 32), idesc_o,
                        (have_o || ks > 0) ? 1u : 0u);
      }
      ptx::mma_commit(&mi->bar_o);
      TRS(5, it);
    }
    have_o = true;
    ptx::mbar_wait(&mi->bar_o, (uint32_t)(it & 1), abort_flag);  // the single row tile is rewritten next
    ptx::tc_fence_after_sync();
    TRS(6, it);
    if (tma_rows && it + 1 < ntiles) issue_tma(it + 1);   // the tile is free: the next rows start travelling
  }

  // ------------------------------------------------------------------ reduce l over the 128 rows
  // Butterfly over the warp: at each step a lane keeps half of its columns and hands the other half to its
  // partner, so 31 shuffles (not 32 x 5) leave lane L with the warp's sum of column L.
  {
#pragma unroll
    for (int step = 16; step >= 1; step >>= 1) {
      const bool upper = (lane & step) != 0;
#pragma unroll
      for (int c = 0; c < step; ++c) {
        const float send = upper ? l_thr[c] : l_thr[c + step];
        const float keep = upper ? l_thr[c + step] : l_thr[c];
        l_thr[c] = keep + __shfl_xor_sync(0xffffffffu, send, step);
      }
    }
    mi->colmax[quad][half_id * 32 + lane] = l_thr[0];
  }
  __syncthreads();
  if (tid < TC_HEADS) mi->l_tot[tid] = (mi->colmax[0][tid] + mi->colmax[1][tid]) + (mi->colmax[2][tid] + mi->colmax[3][tid]);
  __syncthreads();

  TRS(13, 0);
  // ------------------------------------------------------------------ output
  const int64_t N = (int64_t)p.B * p.T * p.H;
  const bool direct = p.nsplit == 1;
  const bool finalize = direct && !p.partial_ml;
  if (tid < TC_HEADS) {
    // per-head factor applied to O^T: 1 for partial output, exp(m - m') / denominator with the sink joined otherwise
    float fac = 1.f;
    if (finalize) {
      const float m = mi->m_ref[tid], l = mi->l_tot[tid];
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
  __syncthreads();
  for (int m2 = 0; m2 < 2; ++m2) {
    const int mt = half_id * 2 + m2;
    if (mt >= n_mt) continue;
    const int d = mt * 128 + quad * 32 + lane;
    const int64_t obase = direct ? (int64_t)b * p.o_sb + (int64_t)t * p.o_st + d
                                 : ((int64_t)split * N + (int64_t)bt * p.H) * p.Dv + d;
    const int64_t ostep = direct ? p.o_sh : (int64_t)p.Dv;
#pragma unroll 1
    for (int ch = 0; ch < 2; ++ch) {
      uint32_t ov[32];
      if (have_o) {
        ptx::tmem_ld32(tmem_o + ((uint32_t)(quad * 32) << 16) + (uint32_t)(mt * 64 + ch * 32), ov);
        ptx::tmem_ld_wait();
      } else {
#pragma unroll
        for (int c = 0; c < 32; ++c) ov[c] = 0u;
      }
#pragma unroll
      for (int c = 0; c < 32; ++c) {
        const int h = ch * 32 + c;
        if (h >= p.H) continue;
        const float o = __uint_as_float(ov[c]) * mi->factor[h];
        if (finalize) store_elem<OT>(p.out, obase + h * ostep, o);
        else if (direct) reinterpret_cast<float*>(p.out)[obase + h * ostep] = o;
        else p.ws_o[obase + h * ostep] = o;
      }
    }
  }
  TRS(13, 1);
  if (tid < p.H && (!direct || p.partial_ml)) {
    // (m, l) in natural-log units for the merge kernel
    const float m_nat = mi->m_ref[tid] == -INFINITY ? -INFINITY : mi->m_ref[tid] * 0.6931471805599453f;
    float* ml = direct ? p.partial_ml + ((int64_t)bt * p.H + tid) * 2
                       : p.ws_ml + ((int64_t)split * N + (int64_t)bt * p.H + tid) * 2;
    ml[0] = m_nat;
    ml[1] = mi->l_tot[tid];
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_base, 512);
  TRS(7, 1);
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
  if (H < 1 || H > TC_HEADS) return false;
  if (Dqk % 64 != 0 || Dqk < 128 || Dqk > 576) return false;
  if (Dv % 128 != 0 || Dv < 128 || Dv > 512 || Dv > Dqk) return false;
  return tc_layout(Dqk, Dv).total + 1024 <= 227 * 1024;
}

int sparse_tc_splits(int B, int T, int H, int k, int raw_cap, int requested) {
  const int64_t max_tiles = ceil_div((int64_t)k + raw_cap, TC_ROWS);
  int64_t want;
  if (requested > 0) {
    want = requested;
  } else {
    const int64_t base = (int64_t)B * T;
    want = (int64_t)sm_count() / (base > 0 ? base : 1);  // one wave of CTAs
  }
  if (want > max_tiles) want = max_tiles;
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

template <int KVT, int QT>
static int launch_tc_typed(SparseParams& p, int out_dtype, cudaStream_t st) {
  const int smem = tc_layout(p.Dqk, p.Dv).total + 1024;
  CUtensorMap tm_comp, tm_raw;
  memset(&tm_comp, 0, sizeof(tm_comp));
  memset(&tm_raw, 0, sizeof(tm_raw));
  p.tma_rows = 0;
  if (KVT != MXB_I8 && p.comp_kv && (reinterpret_cast<uintptr_t>(p.comp_kv) & 15) == 0 &&
      (!p.raw_kv || (reinterpret_cast<uintptr_t>(p.raw_kv) & 15) == 0)) {
    int rc = row_gather_map(&tm_comp, p.comp_kv, p.Dqk, KVT == MXB_BF16);
    if (rc != MXB_OK) return rc;
    rc = row_gather_map(&tm_raw, p.raw_kv ? p.raw_kv : p.comp_kv, p.Dqk, KVT == MXB_BF16);
    if (rc != MXB_OK) return rc;
    p.tma_rows = 1;
  }
  dim3 grid((unsigned)p.nsplit, 1, (unsigned)(p.B * p.T));
#define MXB_TC(OT)                                                                                   \
  {                                                                                                  \
    auto kern = sparse_attn_tc_kernel<KVT, QT, OT>;                                                  \
    MXB_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));      \
    kern<<<grid, 256, smem, st>>>(p, tm_comp, tm_raw);                                                \
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
