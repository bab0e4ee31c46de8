// Causal GQA flash prefill, head_dim 256, 16-bit operands, fp32 accumulation, with the
// sigmoid-gate epilogue fused:  out = softmax(scale * Q K^T + causal) V * sigmoid(gate).
//
// One CTA = 128 query rows of one query head; the grid is one-dimensional in longest-first order (every head's
// latest query tile first), because causal tiles differ 64-fold in length.  Twelve warps:
//   warps 0-7  softmax + drain; warp w owns query rows 32 * (w % 4) .. (= its TMEM lanes) and keys
//              32 * (w / 4) .. of every 64-key tile; the two halves of a row swap maxima and sums through
//              shared memory behind a 64-thread barrier
//   warp  8    issues the first half of the S = Q K^T MMAs (feature slabs 0-1, one lane)
//   warp  9    TMA producer for Q and K (one lane)
//   warp 10    issues the O += P V MMAs and fetches the next V tile behind them (one lane)
//   warp 11    issues the second half of the S MMAs (feature slabs 2-3) into a second accumulator
// Per 64-key tile:  S = Q K^T (M128 x N64 x K256) into one of two TMEM buffers, each made of two
// accumulators that the softmax adds (one thread sustains only one tcgen05.mma per ~85 cycles, so
// the 16 MMAs of a tile are split between two issuers);
// the softmax warps read S from TMEM, keep a running maximum with lazy rescaling of
// the TMEM-resident O (only when the maximum grew by more than 2^8), write P as a
// 16-bit K-major swizzled tile to one of two shared-memory buffers; O += P V (M128 x N256 x K64)
// with V read in place as an MN-major B operand (no transposed copy).
// S of tile j+1 is issued before P of tile j is consumed and P of tile j+1 is written while P V of
// tile j runs, so the tensor pipe overlaps the softmax.
// Drain: the gate tile arrives by TMA in the Q buffer during the last tile; each thread normalises its half row,
// applies the sigmoid and writes the output chunks in place; TMA stores write the tile.
// TMEM: S0a [0,64) S0b [64,128) S1a [128,192) S1b [192,256) O [256,512).
#include "common.cuh"
#include "ptx_sm100.cuh"

namespace mxb {

constexpr int FB_M = 128, FB_N = 64, FB_D = 256;
#ifndef MXB_FLASH_POLY
#define MXB_FLASH_POLY 1
#endif
constexpr int kPolyOf8 = MXB_FLASH_POLY;   // of every eight exponentials, this many (0 .. 4) run on the FMA pipe

#ifdef MXB_TRACE_FL   // development aid: cycle stamps of one CTA's roles over 16 tiles, written behind `status`
#define TRF(k, j) do { if (tr_cta && (j) >= 32 && (j) < 48) tr[(k) * 16 + (j) - 32] = clock64(); } while (0)
#define TRX(i) do { if (tr_cta && warp == 0) tr[18 * 16 + (i)] = clock64() - c_begin; } while (0)
#else
#define TRF(k, j)
#define TRX(i)
#endif

struct FlashSmem {
  static constexpr int q_off = 0;                       // 4 slabs x [128 x 128 B]
  static constexpr int k_off = q_off + 4 * 16384;       // 2 stages x 4 slabs x [64 x 128 B]
  static constexpr int v_off = k_off + 2 * 32768;       // 2 stages x 4 slabs x [64 keys x 128 B]
  static constexpr int p_off = v_off + 2 * 32768;       // 2 buffers x [128 x 128 B]
  static constexpr int bar_off = p_off + 2 * 16384;
  static constexpr int rowmax_off = bar_off + 256;      // [2 tiles][2 halves][128 rows] bf16 (1 KB); reused for the row sums
  static constexpr int total = rowmax_off + 1024;
};

struct FlashParams {
  const void* gate;
  int64_t g_ss, g_sh;
  void* out;
  int64_t o_ss, o_sh;
  int32_t S, Skv, Hq, Hkv;
  float scale_log2;  // scale * log2(e)
  int32_t q_head_inner, k_head_inner;  // tensor-map dimension order: (D, head, row) instead of (D, row, head)
  int32_t g_head_inner, o_head_inner, v_head_inner;
  int32_t tma_drain;   // gate tile in and output tile out by TMA through the (then idle) Q buffer
  int32_t* status;
};

template <bool BF16>
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  if constexpr (BF16) {
    __nv_bfloat162 v = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  } else {
    __half2 v = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&v);
  }
}
__device__ __forceinline__ float fast_ex2(float x) {   // 2^x, x <= 0 here; -inf -> 0
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the FMA pipe for x <= ~8: round-to-nearest split x = n + f with the 1.5 * 2^23 trick, a cubic for 2^f on
// [-0.5, 0.5] (relative error 7.5e-5, below the rounding of a 16-bit P), n added into the exponent field.  One in
// eight of a tile's exponentials goes this way (measured best among 0 to 4 in eight): it takes the edge off the
// special-function unit's 16 results per clock per SM.  Inputs below -126 (masked keys) give 2^-126 instead of 0.
__device__ __forceinline__ float poly_ex2(float x) {
  x = fmaxf(x, -126.f);
  const float kMagic = 12582912.f;
  const float xr = x + kMagic;
  const float f = x - (xr - kMagic);
  float r = fmaf(0.0551716685295105f, f, 0.2426111251115799f);
  r = fmaf(r, f, 0.6932609677314758f);
  r = fmaf(r, f, 0.9999280571937561f);
  return __int_as_float(__float_as_int(r) + (__float_as_int(xr) << 23));
}

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

template <bool BF16>
__device__ __forceinline__ float2 unpack2(uint32_t u) {
  if constexpr (BF16) return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
  else return __half22float2(*reinterpret_cast<__half2*>(&u));
}

template <bool BF16>
__global__ void __launch_bounds__(384, 1) flash_prefill_kernel(const __grid_constant__ CUtensorMap tm_q,
                                                               const __grid_constant__ CUtensorMap tm_k,
                                                               const __grid_constant__ CUtensorMap tm_vt,
                                                               const __grid_constant__ CUtensorMap tm_g,
                                                               const __grid_constant__ CUtensorMap tm_o,
                                                               FlashParams p) {
  using L = FlashSmem;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* q_s = smem + L::q_off;
  uint8_t* k_s = smem + L::k_off;
  uint8_t* v_s = smem + L::v_off;
  uint8_t* p_s = smem + L::p_off;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::bar_off);
  uint16_t* rowmax_s = reinterpret_cast<uint16_t*>(smem + L::rowmax_off);
  uint64_t* q_full = bars + 0;
  uint64_t* k_full = bars + 1;   // [2]
  uint64_t* k_empty = bars + 3;  // [2]
  uint64_t* v_full = bars + 5;   // [2]
  uint64_t* s_ready = bars + 9;  // [2]
  uint64_t* p_ready = bars + 11;  // [2], one per P buffer (the softmax warps may be a tile apart)
  uint64_t* pv_done = bars + 13;  // [2], one per P buffer
  uint64_t* s_free = bars + 15;   // [2]
  uint64_t* g_full = bars + 17;   // gate tile landed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 18);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  // One-dimensional grid in longest-first order: every head's latest (heaviest) query tile, then the next tile of
  // every head, ..., so that the CTAs that start last are the 2-tile ones and the SMs finish together.  CTAs that
  // run at the same time share their K/V stream across the query heads of a KV head.
  const int n_qt = (p.S + FB_M - 1) / FB_M;
  const int qt = n_qt - 1 - (int)blockIdx.x / p.Hq;
  const int head = (int)blockIdx.x % p.Hq;
  const int kvh = head / (p.Hq / p.Hkv);
  const int m0 = qt * FB_M;
  const int past = p.Skv - p.S;
  int kv_end = m0 + FB_M + past;
  if (kv_end > p.Skv) kv_end = p.Skv;
  const int ntiles = (kv_end + FB_N - 1) / FB_N;
#ifdef MXB_TRACE_FL
  long long* tr = reinterpret_cast<long long*>(p.status);
  const bool tr_cta = p.status && blockIdx.x == 0 && (tid & 31) == 0;
  long long* tr_all = tr + 24 * 16 + (head * n_qt + (n_qt - 1 - qt)) * 4;   // per CTA: start ns, end ns, cycles, SM
  const long long c_begin = clock64();
  if (p.status && tid == 0) {
    unsigned long long ns; unsigned sm;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    asm volatile("mov.u32 %0, %%smid;" : "=r"(sm));
    tr_all[0] = (long long)ns; tr_all[3] = sm;
  }
#endif

  if (tid == 0) {
    ptx::mbar_init(q_full, 1);
    for (int i = 0; i < 2; ++i) {
      ptx::mbar_init(&k_full[i], 1);
      ptx::mbar_init(&k_empty[i], 2);   // both S issuers release a K stage
      ptx::mbar_init(&v_full[i], 1);
      ptx::mbar_init(&s_ready[i], 2);   // both halves of S
      ptx::mbar_init(&pv_done[i], 1);
      ptx::mbar_init(&p_ready[i], 256);
    }
    ptx::mbar_init(g_full, 1);
    ptx::mbar_init(&s_free[0], 256);
    ptx::mbar_init(&s_free[1], 256);
    *abort_flag = 0;
    ptx::mbar_fence_init();
  }
  __syncwarp();
  if (warp == 0) {
    ptx::tmem_alloc(tmem_slot, 512);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before_sync();
  __syncthreads();
  ptx::tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_o = tmem_base + 256;
  TRX(0);

  if (warp == 9) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      ptx::tma_prefetch_desc(&tm_q);
      ptx::tma_prefetch_desc(&tm_k);
      ptx::mbar_expect_tx(q_full, 4 * 16384);
      for (int kb = 0; kb < 4; ++kb)
        ptx::tma_load_3d(q_s + kb * 16384, &tm_q, q_full, kb * 64, p.q_head_inner ? head : m0,
                         p.q_head_inner ? m0 : head);
      for (int j = 0; j < ntiles; ++j) {   // K tiles only: V is fetched by the P V issuer, behind its own MMAs
        const int s = j & 1, u = j >> 1;
        if (j >= 2) ptx::mbar_wait(&k_empty[s], (uint32_t)((u - 1) & 1), abort_flag);
        ptx::mbar_expect_tx(&k_full[s], 32768);
        for (int kb = 0; kb < 4; ++kb)
          ptx::tma_load_3d(k_s + s * 32768 + kb * 8192, &tm_k, &k_full[s], kb * 64, p.k_head_inner ? kvh : j * FB_N,
                           p.k_head_inner ? j * FB_N : kvh);
      }
    }
  } else if (warp == 8 || warp == 11) {
    // ------------------------------------------------------------ S = Q K^T issuers
    // Warp 4 accumulates feature slabs 0-1 into S(s)a, warp 7 slabs 2-3 into S(s)b; P V (4 MMAs) is a third
    // issuer.  All write different TMEM columns, so none waits for another.
    if (lane == 0) {
      const int half = warp == 8 ? 0 : 1;
      constexpr uint32_t fmt = BF16 ? ptx::kFmtBF16 : ptx::kFmtF16;
      const uint32_t idesc_s = ptx::idesc_f16(fmt, fmt, FB_M, FB_N, 0, 0);
      const uint64_t q_desc = ptx::smem_desc_sw128(ptx::smem_u32(q_s), 16, 1024);
      const uint64_t k_desc = ptx::smem_desc_sw128(ptx::smem_u32(k_s), 16, 1024);
      ptx::mbar_wait(q_full, 0, abort_flag);
      for (int j = 0; j < ntiles; ++j) {
        const int s = j & 1;
        ptx::mbar_wait(&k_full[s], (uint32_t)((j >> 1) & 1), abort_flag);
        if (j >= 2) ptx::mbar_wait(&s_free[s], (uint32_t)(((j >> 1) - 1) & 1), abort_flag);  // softmax read S(j-2)
        ptx::tc_fence_after_sync();
        TRF(half ? 2 : 0, j);
        const uint32_t d = tmem_base + (uint32_t)(s * 2 * FB_N + half * FB_N);
        const uint64_t kd = ptx::desc_advance(k_desc, s * 32768);
#pragma unroll
        for (int kb2 = 0; kb2 < 2; ++kb2) {
          const int kb = half * 2 + kb2;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            ptx::mma_f16_ss(d, ptx::desc_advance(q_desc, kb * 16384 + ks * 32),
                            ptx::desc_advance(kd, kb * 8192 + ks * 32), idesc_s, (kb2 | ks) ? 1u : 0u);
        }
        ptx::mma_commit(&s_ready[s]);
        ptx::mma_commit(&k_empty[s]);
        TRF(half ? 3 : 1, j);
      }
    }
  } else if (warp == 10) {
    // ------------------------------------------------------------ O += P V issuer
    if (lane == 0) {
      constexpr uint32_t fmt = BF16 ? ptx::kFmtBF16 : ptx::kFmtF16;
      // V is read as it lies in memory ([key][feature]): as the B operand that is MN-major, four 64-feature slabs of
      // [64 keys x 128 B] (8 KB apart = LBO), groups of 8 keys 1 KB apart (SBO), 16 keys per K step
      const uint32_t idesc_o = ptx::idesc_f16(fmt, fmt, FB_M, FB_D, 0, 1);
      const uint64_t v_desc = ptx::smem_desc_sw128(ptx::smem_u32(v_s), 8192, 1024);
      const uint64_t p_desc = ptx::smem_desc_sw128(ptx::smem_u32(p_s), 16, 1024);
      ptx::tma_prefetch_desc(&tm_vt);
      auto load_v = [&](int j) {
        const int s = j & 1;
        ptx::mbar_expect_tx(&v_full[s], 32768);
        for (int kb = 0; kb < 4; ++kb)
          ptx::tma_load_3d(v_s + s * 32768 + kb * 8192, &tm_vt, &v_full[s], kb * 64, p.v_head_inner ? kvh : j * FB_N,
                           p.v_head_inner ? j * FB_N : kvh);
      };
      load_v(0);
      if (ntiles > 1) load_v(1);
      for (int j = 0; j < ntiles; ++j) {
        const int s = j & 1;
        ptx::mbar_wait(&p_ready[s], (uint32_t)((j >> 1) & 1), abort_flag);
        ptx::mbar_wait(&v_full[s], (uint32_t)((j >> 1) & 1), abort_flag);
        ptx::tc_fence_after_sync();
        TRF(4, j);
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          ptx::mma_f16_ss(tmem_o, ptx::desc_advance(p_desc, s * 16384 + ks * 32),
                          ptx::desc_advance(v_desc, s * 32768 + ks * 2048), idesc_o, (j > 0 || ks > 0) ? 1u : 0u);
        ptx::mma_commit(&pv_done[s]);
        TRF(5, j);
        // V of the next tile goes where P V of the previous tile read; that one was issued a whole tile ago
        if (j >= 1 && j + 1 < ntiles) {
          ptx::mbar_wait(&pv_done[s ^ 1], (uint32_t)(((j - 1) >> 1) & 1), abort_flag);
          load_v(j + 1);
        }
      }
    }
  } else {
    // ------------------------------------------------------------ softmax + epilogue (warps 0-7)
    // Thread = (query row, half of the tile's 64 keys): warps 0-3 take keys 0-31, warps 4-7 keys 32-63 of the
    // same 128 rows (a warp reaches the TMEM lanes 32 * (warp % 4) ..).  The two halves of a row swap their
    // maxima through shared memory, so both keep the same running reference; each rescales and writes out its
    // half of the 256 output features.
    const int quad = warp & 3, half = warp >> 2;
    const int row = quad * 32 + lane;   // 0..127
    const int qi = m0 + row;            // query row
    const uint32_t lane_off = (uint32_t)(quad * 32) << 16;
    float m_used = -INFINITY, l = 0.f;
    for (int j = 0; j < ntiles; ++j) {
      const int s = j & 1;
#ifdef MXB_TRACE_FL
      const int tk = warp == 0 ? 6 : (warp == 4 ? 12 : 18);
#endif
      TRF(tk + 0, j);
      ptx::mbar_wait(&s_ready[s], (uint32_t)((j >> 1) & 1), abort_flag);
      ptx::tc_fence_after_sync();
      TRF(tk + 1, j);
      if (j == 0) TRX(1);
      if (j == 1) TRX(2);
      if (j == ntiles - 1) TRX(3);
      if (j == ntiles - 1 && p.tma_drain && p.gate && tid == 0) {
        // the last S has been computed, so nothing reads Q any more: its buffer receives the gate tile
        // ([128 rows x 256] as four 64-feature slabs, swizzled like an operand) while the last tile is finished
        ptx::mbar_expect_tx(g_full, 4 * 16384);
        for (int kb = 0; kb < 4; ++kb)
          ptx::tma_load_3d(q_s + kb * 16384, &tm_g, g_full, kb * 64, p.g_head_inner ? head : m0,
                           p.g_head_inner ? m0 : head);
      }
      uint32_t sv[32];
      {
        uint32_t sb[32];
        const uint32_t sa = tmem_base + lane_off + (uint32_t)(s * 2 * FB_N + half * 32);
        ptx::tmem_ld32(sa, sv);
        ptx::tmem_ld32(sa + FB_N, sb);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int c = 0; c < 32; ++c) sv[c] = __float_as_uint(__uint_as_float(sv[c]) + __uint_as_float(sb[c]));
      }
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&s_free[s]);
      TRF(tk + 2, j);
      const int key0 = j * FB_N + half * 32;
      const bool need_mask = j * FB_N + FB_N - 1 > m0 + past;  // tile reaches past the first row's diagonal
      // sv keeps the raw dot products; the (positive) scale is applied once to the maximum here and inside the
      // exponent's fused multiply-add below
      if (need_mask) {
#pragma unroll
        for (int c = 0; c < 32; ++c)
          if (key0 + c > qi + past) sv[c] = 0xff800000u;   // -inf
      }
      float tm4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};   // four independent chains
#pragma unroll
      for (int c = 0; c < 32; c += 4) {
#pragma unroll
        for (int i = 0; i < 4; ++i) tm4[i] = fmaxf(tm4[i], __uint_as_float(sv[c + i]));
      }
      float tmax = fmaxf(fmaxf(tm4[0], tm4[1]), fmaxf(tm4[2], tm4[3])) * p.scale_log2;
      // Both halves of a row must use the SAME reference, and any upper bound of the tile's maximum will do:
      // each half publishes its maximum rounded UP to bfloat16 and both take the larger of the two rounded values.
      {
        const uint32_t tb = __float_as_uint(tmax);
        const uint16_t up = (uint16_t)(((tb >> 31) ? tb : tb + 0xFFFFu) >> 16);   // toward +inf; -inf stays -inf
        rowmax_s[(s * 2 + half) * FB_M + row] = up;
        asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");   // the two warps that share these rows
        TRF(tk + 3, j);
        const uint16_t other = rowmax_s[(s * 2 + (half ^ 1)) * FB_M + row];
        tmax = fmaxf(__uint_as_float((uint32_t)up << 16), __uint_as_float((uint32_t)other << 16));
      }
      float factor = 1.f;
      bool grow = false;
      if (j == 0) {
        m_used = tmax;  // row 0's key 0 is always visible, so tmax is finite for valid rows
      } else {
        grow = tmax > m_used + 8.f;
      }
      // P buffer s is free once P V of tile j-2 has read it
      if (j >= 2) ptx::mbar_wait(&pv_done[s], (uint32_t)(((j >> 1) - 1) & 1), abort_flag);
      if (j > 0) {
        if (__any_sync(0xffffffffu, grow)) {   // the same answer in both warps of a row quarter
          // O is final only after the previous P V finished
          ptx::mbar_wait(&pv_done[(j - 1) & 1], (uint32_t)(((j - 1) >> 1) & 1), abort_flag);
          ptx::tc_fence_after_sync();
          if (grow) {
            factor = exp2f(m_used - tmax);
            m_used = tmax;
          }
#pragma unroll 1
          for (int c0 = half * (FB_D / 2); c0 < (half + 1) * (FB_D / 2); c0 += 32) {
            uint32_t ov[32];
            ptx::tmem_ld32(tmem_o + lane_off + (uint32_t)c0, ov);
            ptx::tmem_ld_wait();
#pragma unroll
            for (int c = 0; c < 32; ++c) ov[c] = __float_as_uint(__uint_as_float(ov[c]) * factor);
            ptx::tmem_st32(tmem_o + lane_off + (uint32_t)c0, ov);
          }
          ptx::tmem_st_wait();
          l *= factor;
        }
      }
      TRF(tk + 4, j);
      float psum = 0.f;
      uint8_t* prow = p_s + s * 16384 + row * 128;
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float xa = fmaf(__uint_as_float(sv[c8 * 8 + 2 * i]), p.scale_log2, -m_used);
          const float xb = fmaf(__uint_as_float(sv[c8 * 8 + 2 * i + 1]), p.scale_log2, -m_used);
          const float a = fast_ex2(xa);
          const bool on_fma = kPolyOf8 == 1 ? i == 0 : kPolyOf8 == 2 ? (i & 1) == 0 : kPolyOf8 == 3 ? i < 3 : kPolyOf8 >= 4;
          const float b = on_fma ? poly_ex2(xb) : fast_ex2(xb);
          psum += a + b;
          w[i] = pack2<BF16>(a, b);
        }
        *reinterpret_cast<uint4*>(prow + (((half * 4 + c8) ^ (row & 7)) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
      }
      l += psum;
      ptx::fence_proxy_async_smem();
      ptx::tc_fence_before_sync();
      ptx::mbar_arrive(&p_ready[s]);
      TRF(tk + 5, j);
    }
    // epilogue: the row sum over both halves, then each half writes its 128 output features
    TRX(4);
    if (p.tma_drain) {
      // Drain through shared memory so that global memory sees whole tiles: the gate tile arrived by TMA in the Q
      // buffer; each thread turns the 16-byte chunks of its half row into output chunks in place; one TMA store
      // per slab writes the tile (rows past the end of the sequence are clipped by the tensor map).
      float* rowsum_s = reinterpret_cast<float*>(rowmax_s);   // [2 halves][128 rows]
      asm volatile("bar.sync 5, 256;" ::: "memory");   // all eight warps: every maximum of the last tile has been read
      rowsum_s[half * FB_M + row] = l;
      asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");
      l += rowsum_s[(half ^ 1) * FB_M + row];
      ptx::mbar_wait(&pv_done[(ntiles - 1) & 1], (uint32_t)(((ntiles - 1) >> 1) & 1), abort_flag);
      if (p.gate) ptx::mbar_wait(g_full, 0, abort_flag);
      ptx::tc_fence_after_sync();
      TRX(5);
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
#pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t ov[32];
        ptx::tmem_ld32(tmem_o + lane_off + (uint32_t)(half * (FB_D / 2) + cc * 32), ov);
        ptx::tmem_ld_wait();
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          const int chunk = half * 16 + cc * 4 + c8;   // 16-byte chunk of the 512-byte row
          uint4* cell = reinterpret_cast<uint4*>(q_s + (chunk >> 3) * 16384 + row * 128 + (((chunk & 7) ^ (row & 7)) << 4));
          uint32_t w[4];
          if (p.gate) {
            const uint4 g = *cell;
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float2 gg = unpack2<BF16>(gw[i]);
              // sigmoid(g) = 0.5 + 0.5 * tanh(g / 2): one special-function result per element
              const float sa = fmaf(0.5f, fast_tanh(0.5f * gg.x), 0.5f), sb = fmaf(0.5f, fast_tanh(0.5f * gg.y), 0.5f);
              w[i] = pack2<BF16>(__uint_as_float(ov[c8 * 8 + 2 * i]) * inv_l * sa,
                                 __uint_as_float(ov[c8 * 8 + 2 * i + 1]) * inv_l * sb);
            }
          } else {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              w[i] = pack2<BF16>(__uint_as_float(ov[c8 * 8 + 2 * i]) * inv_l, __uint_as_float(ov[c8 * 8 + 2 * i + 1]) * inv_l);
          }
          *cell = make_uint4(w[0], w[1], w[2], w[3]);
        }
      }
      ptx::fence_proxy_async_smem();
      asm volatile("bar.sync 5, 256;" ::: "memory");
      if (tid == 0) {
        for (int kb = 0; kb < 4; ++kb)
          ptx::tma_store_3d(&tm_o, q_s + kb * 16384, kb * 64, p.o_head_inner ? head : m0, p.o_head_inner ? m0 : head);
        ptx::tma_store_commit();
        ptx::tma_store_wait_read();
      }
    } else {
    // The gate values of this thread's half row (16 x 16 bytes) are requested first, all at once: they travel
      // while the last P V finishes and the row sums are exchanged (one load per use would put 16 round trips
      // to L2 on the drain's critical path).
      const bool row_ok = qi < p.S;
      const uint16_t* gptr = (p.gate && row_ok) ? reinterpret_cast<const uint16_t*>(p.gate) + (int64_t)qi * p.g_ss +
                                                      (int64_t)head * p.g_sh + half * (FB_D / 2)
                                                : nullptr;
      uint4 gv[16];
  #pragma unroll
      for (int i = 0; i < 16; ++i) gv[i] = gptr ? __ldg(reinterpret_cast<const uint4*>(gptr) + i) : make_uint4(0, 0, 0, 0);
      float* rowsum_s = reinterpret_cast<float*>(rowmax_s);   // [2 halves][128 rows]
      asm volatile("bar.sync 5, 256;" ::: "memory");   // all eight warps: every maximum of the last tile has been read
      rowsum_s[half * FB_M + row] = l;
      asm volatile("bar.sync %0, 64;" ::"r"(quad + 1) : "memory");
      l += rowsum_s[(half ^ 1) * FB_M + row];
      ptx::mbar_wait(&pv_done[(ntiles - 1) & 1], (uint32_t)(((ntiles - 1) >> 1) & 1), abort_flag);
      ptx::tc_fence_after_sync();
      TRX(5);
      const float inv_l = l > 0.f ? 1.f / l : 0.f;
      uint16_t* optr = reinterpret_cast<uint16_t*>(p.out) + (int64_t)qi * p.o_ss + (int64_t)head * p.o_sh + half * (FB_D / 2);
  #pragma unroll
      for (int cc = 0; cc < 4; ++cc) {
        uint32_t ov[32];
        ptx::tmem_ld32(tmem_o + lane_off + (uint32_t)(half * (FB_D / 2) + cc * 32), ov);
        ptx::tmem_ld_wait();
        if (row_ok) {
  #pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            const uint4 g = gv[cc * 4 + c8];
            const uint32_t gw[4] = {g.x, g.y, g.z, g.w};
            uint32_t w[4];
  #pragma unroll
            for (int i = 0; i < 4; ++i) {
              float a = __uint_as_float(ov[c8 * 8 + 2 * i]) * inv_l;
              float b = __uint_as_float(ov[c8 * 8 + 2 * i + 1]) * inv_l;
              if (p.gate) {
                const float2 gg = unpack2<BF16>(gw[i]);
                a = __fdividef(a, 1.f + __expf(-gg.x));
                b = __fdividef(b, 1.f + __expf(-gg.y));
              }
              w[i] = pack2<BF16>(a, b);
            }
            *reinterpret_cast<uint4*>(optr + cc * 32 + c8 * 8) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
    }
    TRX(6);
    ptx::tc_fence_before_sync();
  }

  __syncthreads();
  TRX(7);
  if (warp == 0) ptx::tmem_dealloc(tmem_base, 512);
#ifdef MXB_TRACE_FL
  if (p.status && tid == 0) {
    unsigned long long ns;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(ns));
    tr_all[1] = (long long)ns; tr_all[2] = clock64() - c_begin;
  }
#else
  if (tid == 0 && *abort_flag && p.status) atomicExch(p.status, 1);
#endif
}

}  // namespace mxb

using namespace mxb;

static int flash_validate(const mxb_flash_prefill_args* a) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "flash prefill: null args");
  MXB_REQUIRE(a->D == 256, MXB_ERR_INVALID, "flash prefill requires head_dim=256");
  MXB_REQUIRE(a->dtype == MXB_BF16 || a->dtype == MXB_F16, MXB_ERR_INVALID,
              "flash prefill requires bfloat16 or float16 operands");
  MXB_REQUIRE(a->S > 0 && a->Skv >= a->S, MXB_ERR_INVALID, "flash prefill requires 1 <= S <= Skv");
  MXB_REQUIRE(a->Hq > 0 && a->Hkv > 0 && a->Hq % a->Hkv == 0, MXB_ERR_INVALID,
              "query heads must be a multiple of kv heads");
  MXB_REQUIRE(a->q && a->k && a->v && a->out, MXB_ERR_INVALID, "flash prefill: null tensor");
  return MXB_OK;
}

extern "C" int64_t mxb_flash_prefill_workspace_bytes(const mxb_flash_prefill_args* a) {
  (void)a;
  return 0;   // V is read in place (MN-major operand): no scratch
}

extern "C" int mxb_flash_prefill(const mxb_flash_prefill_args* a, void* stream) {
  int rc = flash_validate(a);
  if (rc != MXB_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  MXB_REQUIRE((reinterpret_cast<uintptr_t>(a->out) & 15) == 0 && a->out_stride_s % 8 == 0 && a->out_stride_h % 8 == 0,
              MXB_ERR_INVALID, "out must be 16-byte aligned with strides that are multiples of 8 elements");
  MXB_REQUIRE(!a->gate || ((reinterpret_cast<uintptr_t>(a->gate) & 15) == 0 && a->gate_stride_s % 8 == 0 &&
                           a->gate_stride_h % 8 == 0),
              MXB_ERR_INVALID, "gate must be 16-byte aligned with strides that are multiples of 8 elements");
  const CUtensorMapDataType dt = a->dtype == MXB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16;
  CUtensorMap tq, tk, tv;
  // cuTensorMapEncodeTiled wants ascending strides: put the head axis before the row axis when its
  // stride is the smaller one ([rows, heads, D] layouts); the box is one head wide either way.
  const bool q_hin = a->q_stride_h < a->q_stride_s, k_hin = a->k_stride_h < a->k_stride_s;
  {
    uint64_t dims[3] = {(uint64_t)a->D, (uint64_t)(q_hin ? a->Hq : a->S), (uint64_t)(q_hin ? a->S : a->Hq)};
    uint64_t str[2] = {(uint64_t)(q_hin ? a->q_stride_h : a->q_stride_s) * 2,
                       (uint64_t)(q_hin ? a->q_stride_s : a->q_stride_h) * 2};
    uint32_t box[3] = {64, q_hin ? 1u : (uint32_t)FB_M, q_hin ? (uint32_t)FB_M : 1u};
    rc = make_tensor_map(&tq, dt, 3, a->q, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != MXB_OK) return rc;
  }
  {
    uint64_t dims[3] = {(uint64_t)a->D, (uint64_t)(k_hin ? a->Hkv : a->Skv), (uint64_t)(k_hin ? a->Skv : a->Hkv)};
    uint64_t str[2] = {(uint64_t)(k_hin ? a->k_stride_h : a->k_stride_s) * 2,
                       (uint64_t)(k_hin ? a->k_stride_s : a->k_stride_h) * 2};
    uint32_t box[3] = {64, k_hin ? 1u : (uint32_t)FB_N, k_hin ? (uint32_t)FB_N : 1u};
    rc = make_tensor_map(&tk, dt, 3, a->k, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != MXB_OK) return rc;
  }
  const bool v_hin = a->v_stride_h < a->v_stride_s;
  {
    uint64_t dims[3] = {(uint64_t)a->D, (uint64_t)(v_hin ? a->Hkv : a->Skv), (uint64_t)(v_hin ? a->Skv : a->Hkv)};
    uint64_t str[2] = {(uint64_t)(v_hin ? a->v_stride_h : a->v_stride_s) * 2,
                       (uint64_t)(v_hin ? a->v_stride_s : a->v_stride_h) * 2};
    uint32_t box[3] = {64, v_hin ? 1u : (uint32_t)FB_N, v_hin ? (uint32_t)FB_N : 1u};
    rc = make_tensor_map(&tv, dt, 3, a->v, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B);
    if (rc != MXB_OK) return rc;
  }

  // gate and output tiles travel by TMA when their layouts allow a tensor map (rows and heads at distinct,
  // 16-byte aligned strides); otherwise the kernel reads and writes them with per-thread accesses
  CUtensorMap tg, to;
  memset(&tg, 0, sizeof(tg));
  memset(&to, 0, sizeof(to));
  const bool g_hin = a->gate_stride_h < a->gate_stride_s, o_hin = a->out_stride_h < a->out_stride_s;
  auto tile_map = [&](CUtensorMap* m, const void* base, int64_t ss, int64_t sh, bool hin) -> bool {
    if (ss <= 0 || sh <= 0 || ss == sh) return false;
    uint64_t dims[3] = {(uint64_t)a->D, (uint64_t)(hin ? a->Hq : a->S), (uint64_t)(hin ? a->S : a->Hq)};
    uint64_t str[2] = {(uint64_t)(hin ? sh : ss) * 2, (uint64_t)(hin ? ss : sh) * 2};
    uint32_t box[3] = {64, hin ? 1u : (uint32_t)FB_M, hin ? (uint32_t)FB_M : 1u};
    if (str[0] > str[1] || str[1] % str[0] != 0) return false;   // plain nested layouts only
    return make_tensor_map(m, dt, 3, base, dims, str, box, CU_TENSOR_MAP_SWIZZLE_128B) == MXB_OK;
  };
  bool tma_drain = tile_map(&to, a->out, a->out_stride_s, a->out_stride_h, o_hin);
  if (tma_drain && a->gate) tma_drain = tile_map(&tg, a->gate, a->gate_stride_s, a->gate_stride_h, g_hin);

  MXB_REQUIRE(a->scale > 0.f, MXB_ERR_INVALID, "flash prefill: scale must be positive");
  FlashParams p{};
  p.g_head_inner = g_hin ? 1 : 0; p.o_head_inner = o_hin ? 1 : 0; p.tma_drain = tma_drain ? 1 : 0;
  p.v_head_inner = v_hin ? 1 : 0;
  p.gate = a->gate; p.g_ss = a->gate_stride_s; p.g_sh = a->gate_stride_h;
  p.out = a->out; p.o_ss = a->out_stride_s; p.o_sh = a->out_stride_h;
  p.S = a->S; p.Skv = a->Skv; p.Hq = a->Hq; p.Hkv = a->Hkv;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.status = a->status;
  p.q_head_inner = q_hin ? 1 : 0;
  p.k_head_inner = k_hin ? 1 : 0;
  const int smem = FlashSmem::total + 1024;
  dim3 grid((unsigned)(ceil_div(a->S, FB_M) * a->Hq));
  if (a->dtype == MXB_BF16) {
    MXB_CUDA_OK(cudaFuncSetAttribute(flash_prefill_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    flash_prefill_kernel<true><<<grid, 384, smem, st>>>(tq, tk, tv, tg, to, p);
    note_launch();
  } else {
    MXB_CUDA_OK(cudaFuncSetAttribute(flash_prefill_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    flash_prefill_kernel<false><<<grid, 384, smem, st>>>(tq, tk, tv, tg, to, p);
    note_launch();
  }
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
