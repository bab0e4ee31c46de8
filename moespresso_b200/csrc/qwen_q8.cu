// Affine 8-bit KV format of the Qwen full-attention cache (group 64) and the long-context decode attention
// over it.
//
// The reference keeps the Qwen KV cache in MLX's affine quantised form (mlx-lm QuantizedKVCache, bits 8, group
// size 64: src/moespresso/runtime/qwen/full_attention.py:200-236) and hands it to two third-party kernels:
// sdpa_fa_prefill_q8 (:372-382) and sdpa_decode_q8 (:323-335).  The format as MLX documents it for mx.quantize:
// every group of 64 consecutive features of a row has beta = min, alpha = max, scale = (alpha - beta) / 255,
// bias = beta; element = round((w - bias) / scale) in [0, 255]; w ~= element * scale + bias.  Four elements per
// uint32 word, lowest byte first; scales and biases in the row's floating type.
//
//  * affine_q8_quantize_kernel / affine_q8_dequantize_kernel — the format, one warp per row (any width that is
//    a multiple of 64); the dequantiser writes with a caller-chosen row stride so that a past can be expanded
//    straight into the front of a [past + chunk] operand of the flash prefill kernel.
//  * q8_decode_kernel — one query token over a q8 cache, split over the keys: a CTA owns (split, KV head), its four
//    warps take 16 keys at a time and run both contractions on the warp-level tensor cores straight from the packed
//    rows (see the comment at the kernel); every split writes (o, m, l) partials for the log-sum-exp merge kernel
//    (mxb_merge_partials).  HBM-bound: 2 x (256 + 16) bytes per key and KV head are read once.
#include "common.cuh"

namespace mxb {

constexpr int Q8_GROUP = 64;

template <int XT>
__global__ void __launch_bounds__(128) affine_q8_quantize_kernel(const void* __restrict__ x, int64_t x_row_stride,
                                                                 uint32_t* __restrict__ packed, void* __restrict__ scales,
                                                                 void* __restrict__ biases, int64_t n_rows, int width) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  // 8 lanes share a group of 64 features: lane l of a 256-feature span holds features 8 l .. 8 l + 7
  for (int f0 = 0; f0 < width; f0 += 256) {
    const int f = f0 + lane * 8;
    float v[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) v[e] = f < width ? load_elem<XT>(x, row * x_row_stride + f + e) : 0.f;
    float lo = v[0], hi = v[0];
#pragma unroll
    for (int e = 1; e < 8; ++e) {
      lo = fminf(lo, v[e]);
      hi = fmaxf(hi, v[e]);
    }
#pragma unroll
    for (int m = 4; m >= 1; m >>= 1) {
      lo = fminf(lo, __shfl_xor_sync(0xffffffffu, lo, m));
      hi = fmaxf(hi, __shfl_xor_sync(0xffffffffu, hi, m));
    }
    if (f >= width) continue;
    // scale and bias are stored in the row's type; the elements are taken against the STORED values
    // (every step is a single correctly rounded float32 operation, no contraction: the packed words are compared
    // bit for bit with the CPU restatement)
    float scale = __fdiv_rn(__fsub_rn(hi, lo), 255.f), bias = lo;
    if constexpr (XT == MXB_F16) {
      scale = __half2float(__float2half_rn(scale));
      bias = __half2float(__float2half_rn(bias));
    } else if constexpr (XT == MXB_BF16) {
      scale = __bfloat162float(__float2bfloat16_rn(scale));
      bias = __bfloat162float(__float2bfloat16_rn(bias));
    }
    const float inv = scale > 0.f ? __fdiv_rn(1.f, scale) : 0.f;
    uint32_t w[2] = {0u, 0u};
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float q = fminf(fmaxf(floorf(__fadd_rn(__fmul_rn(__fsub_rn(v[e], bias), inv), 0.5f)), 0.f), 255.f);
      w[e >> 2] |= (uint32_t)q << (8 * (e & 3));
    }
    *reinterpret_cast<uint2*>(packed + row * (width / 4) + f / 4) = make_uint2(w[0], w[1]);
    if ((lane & 7) == 0) {
      const int64_t g = row * (width / Q8_GROUP) + f / Q8_GROUP;
      store_elem<XT>(scales, g, scale);
      store_elem<XT>(biases, g, bias);
    }
  }
}

template <int ST, int OT>
__global__ void __launch_bounds__(128) affine_q8_dequantize_kernel(const uint32_t* __restrict__ packed,
                                                                   const void* __restrict__ scales,
                                                                   const void* __restrict__ biases, void* __restrict__ out,
                                                                   int64_t out_row_stride, int64_t n_rows, int width) {
  const int lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= n_rows) return;
  for (int f = lane * 8; f < width; f += 256) {
    const uint2 w = *reinterpret_cast<const uint2*>(packed + row * (width / 4) + f / 4);
    const int64_t g = row * (width / Q8_GROUP) + f / Q8_GROUP;
    const float scale = load_elem<ST>(scales, g), bias = load_elem<ST>(biases, g);
    const uint32_t ww[2] = {w.x, w.y};
#pragma unroll
    for (int e = 0; e < 8; ++e)
      store_elem<OT>(out, row * out_row_stride + f + e, fmaf((float)((ww[e >> 2] >> (8 * (e & 3))) & 0xffu), scale, bias));
  }
}

// ---------------------------------------------------------------------------------------------
// decode: one query token, head_dim 256, GQA group of up to 8 query heads per KV head
// ---------------------------------------------------------------------------------------------
// Warp-level tensor-core flash decoding (mma.sync m16n8k16, fp16 operands, fp32 accumulation) straight from the
// packed rows: a warp takes 16 keys at a time, and the bytes enter both contractions as they are stored.
// A byte becomes an fp16 operand exactly by one byte-permute (0x6400 | u is 1024 + u); since
// w = u * scale + bias = (1024 + u) * scale + (bias - 1024 scale) and scale and bias are constant over a group of 64
// features, the affine part is applied per GROUP, outside the MMAs: every k-step (keys) and every 16-dim block (values)
// lies inside one quantisation group.  Lane (g, t) loads the bytes [16 t, 16 t + 16) of each of the four groups of
// key rows g and g + 8.
//   S [16 keys x 8 heads] = K . q^T : k-step i = 4 grp + w takes bytes 4 w .. 4 w + 3 of the lane's piece of group
//     grp (q is loaded under the same permutation of the feature axis); after the four k-steps of a group,
//     S += scale[key, grp] * (bytes . q) + (bias - 1024 scale)[key, grp] * (sum of q over the group), the sums of q
//     coming from four MMAs against a matrix of ones in the prologue (already in the accumulator layout).
//   O^T [256 dims x 8 heads] += V^T . P : the byte pairs of a lane are 8 x 8 blocks in the layout of `movmatrix`;
//     transposed, they are A fragments whose 16 rows are dims of one group.  The key's scale for that group is
//     multiplied into P (rounded to fp16, two more transposes bring it to the B layout), and
//     sum over keys of P * bias - 1024 * (P * scale as rounded) is kept per group and head beside the accumulators
//     and added to every dim of the group at the end: the 1024s cancel against exactly the weights the MMA used.
// Online softmax per head with a lazy rescale of O^T (only when a maximum moved).  A warp's loads run one tile ahead
// of its arithmetic through shared memory (`cp.async`, see the kernel), the q fragments live in shared memory too,
// and three CTAs fit an SM.  Measured on a B200 (131,072 keys, 2 KV heads, 128 splits): 45 us with the merge
// (~41 us for this kernel = 3.6 TB/s of DRAM traffic, 0.49 of the HBM rate over the algorithmic bytes with the merge;
// 55 us before the staging and with a slower merge; 69 us when every byte pair was dequantised by three half2 operations before the MMA;
// 433 us as a scalar kernel).  What is left: 72 `movmatrix` and 36 MMAs per 16 keys on the warp-level tensor path
// (0.36 instructions per clock per scheduler; stalls spread over long scoreboard, short scoreboard and fixed
// latency).  The CTA's four warps are merged in shared memory and every split writes (o, m, l) partials for
// mxb_merge_partials.  HBM-bound: 2 x (256 + 16) bytes per key and KV head are read once.
constexpr int QD_D = 256, QD_WARPS = 4, QD_MAXG = 8, QD_TILE = 16;
constexpr int QD_STAGES = 2;   // tiles of a warp in shared memory: one in use, one on its way

struct Q8DecodeParams {
  const void* q;           // [Hq, 256]
  int32_t q_dtype;
  const uint32_t* kp; const void* ks; const void* kb;   // keys   [Hkv, P, 64] u32, [Hkv, P, 4], [Hkv, P, 4]
  const uint32_t* vp; const void* vs; const void* vb;   // values, same
  int64_t head_stride_rows;   // rows between consecutive KV heads (the cache capacity)
  int32_t sb_dtype;        // type of the scales and biases
  int32_t P, Hq, Hkv, nsplit;
  float scale_log2;
  float* o_parts;          // [nsplit, Hq, 256]
  float* ml_parts;         // [nsplit, Hq, 2]
};

__device__ __forceinline__ void mma_f16_16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                              uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// Transpose of an 8 x 8 matrix of 16-bit elements held one row per four lanes (lane 4 r + c holds columns 2 c, 2 c + 1).
__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}
// Asynchronous copies of 16 or 8 bytes from global to shared memory; groups of them are waited for in order.
__device__ __forceinline__ void stage16(void* smem_dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void stage8(void* smem_dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(src) : "memory");
}
// four consecutive scales or biases out of a lane's staging slot
template <int ST>
__device__ __forceinline__ void staged_group4(const uint8_t* slot, float (&f)[4]) {
  if constexpr (ST == MXB_F32) {
    const float4 v = *reinterpret_cast<const float4*>(slot);
    f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
  } else {
    const uint2 v = *reinterpret_cast<const uint2*>(slot);
    if constexpr (ST == MXB_F16) {
      const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), c = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      f[0] = a.x; f[1] = a.y; f[2] = c.x; f[3] = c.y;
    } else {
      f[0] = __uint_as_float(v.x << 16); f[1] = __uint_as_float(v.x & 0xFFFF0000u);
      f[2] = __uint_as_float(v.y << 16); f[3] = __uint_as_float(v.y & 0xFFFF0000u);
    }
  }
}
// bytes (2 which, 2 which + 1) of w as the fp16 pair (1024 + u0, 1024 + u1), exactly: 0x6400 | u
__device__ __forceinline__ uint32_t byte_pair_f16(uint32_t w, int which) {
  return __byte_perm(w, 0x64646464u, which == 0 ? 0x4140 : 0x4342);
}

template <int ST>
__global__ void __launch_bounds__(QD_WARPS * 32, 3) q8_decode_kernel(Q8DecodeParams p) {
  // Every lane stages its own pieces of the next tile in shared memory (16 x 16 bytes of packed rows, piece j of
  // lane l at (j * 32 + l): it reads back only what it copied itself) and two of the eight (scales | biases) x
  // (keys | values) x (row g | row g + 8) slots of its key rows, which the four lanes of a quad share (hence the
  // warp-wide wait below).  Loads run a tile ahead of the arithmetic without holding registers, which together
  // with the q fragments in shared memory leaves room for three CTAs per SM.  The staging memory takes the warps'
  // accumulators at the end.
  extern __shared__ __align__(16) uint8_t q8_smem[];
  float (*o_s)[QD_MAXG][QD_D] = reinterpret_cast<float (*)[QD_MAXG][QD_D]>(q8_smem);
  __shared__ float m_s[QD_WARPS][QD_MAXG], l_s[QD_WARPS][QD_MAXG];
  constexpr int SB = ST == MXB_F32 ? 16 : 8;               // bytes of four scales
  constexpr int STAGE_BYTES = 16 * 512 + 8 * 8 * SB;        // per warp and tile: packed pieces, then [slot][g]
  uint32_t* qb_s = reinterpret_cast<uint32_t*>(q8_smem + (size_t)QD_WARPS * QD_STAGES * STAGE_BYTES);   // [16][2][32 lanes]

  const int split = blockIdx.x, kvh = blockIdx.y;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int G = p.Hq / p.Hkv;
  uint8_t* my_stage = q8_smem + (size_t)warp * QD_STAGES * STAGE_BYTES;

  // q as B fragments of k-step i = 4 grp + w: head g, features 64 grp + 16 t + 4 w + {0, 1} and + {2, 3}, times
  // scale * log2(e), fp16.  The sixteen features of a k-step lie in ONE quantisation group.
  if (warp == 0) {
#pragma unroll 1
  for (int i = 0; i < 16; ++i) {
    float f[4] = {0.f, 0.f, 0.f, 0.f};
    if (g < G) {
      const int64_t off = (int64_t)(kvh * G + g) * QD_D + 64 * (i >> 2) + 16 * t + 4 * (i & 3);
#pragma unroll
      for (int e = 0; e < 4; ++e)
        f[e] = (p.q_dtype == MXB_F32   ? load_elem<MXB_F32>(p.q, off + e)
                : p.q_dtype == MXB_F16 ? load_elem<MXB_F16>(p.q, off + e)
                                       : load_elem<MXB_BF16>(p.q, off + e)) * p.scale_log2;
    }
    const __half2 lo = __floats2half2_rn(f[0], f[1]), hi = __floats2half2_rn(f[2], f[3]);
    qb_s[(i * 2 + 0) * 32 + lane] = *reinterpret_cast<const uint32_t*>(&lo);
    qb_s[(i * 2 + 1) * 32 + lane] = *reinterpret_cast<const uint32_t*>(&hi);
  }
  }
  __syncthreads();
  // sums of q (as the MMA reads it) over each group, in the accumulator layout: qsum[grp][e] = head 2 t + e
  float qsum[4][2];
#pragma unroll
  for (int grp = 0; grp < 4; ++grp) {
    float c[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int w = 0; w < 4; ++w)
      mma_f16_16816(c, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, 0x3C003C00u, qb_s[((4 * grp + w) * 2 + 0) * 32 + lane],
                    qb_s[((4 * grp + w) * 2 + 1) * 32 + lane]);
    qsum[grp][0] = c[0];
    qsum[grp][1] = c[1];
  }

  float m_run[2] = {-INFINITY, -INFINITY};   // heads 2 t, 2 t + 1 (the same in the eight lanes that share t)
  float l_run[2] = {0.f, 0.f};               // ... over this lane's keys only
  float o[16][4];   // o[i][c]: head 2 t + c % 2, dim 64 (i / 4) + 16 (g / 2) + 4 (i % 4) + 2 (c / 2) + g % 2
#pragma unroll
  for (int i = 0; i < 16; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  // what the byte operands leave out, per group and head 2 t + e, over this lane's keys only:
  // sum of P * (bias - 1024 scale)  (P as the value MMA reads it: rounded, times the rounded scale)
  float ofix[4][2];
#pragma unroll
  for (int grp = 0; grp < 4; ++grp) ofix[grp][0] = ofix[grp][1] = 0.f;

  const int per = (p.P + p.nsplit - 1) / p.nsplit;
  const int k_lo = min(split * per, p.P), k_hi = min(k_lo + per, p.P);
  const int ntiles = (k_hi - k_lo + QD_TILE - 1) / QD_TILE;
  const int64_t hb = (int64_t)kvh * p.head_stride_rows;
  const int esz = ST == MXB_F32 ? 4 : 2;
  auto issue_tile = [&](int tile, int stage) {   // this lane's pieces of a tile, on their way into its staging slots
    if (tile < ntiles) {
      const int key0 = k_lo + tile * QD_TILE;
      const int64_t r0 = hb + min(key0 + g, k_hi - 1), r1 = hb + min(key0 + g + 8, k_hi - 1);   // clamped rows are masked later
      uint8_t* st = my_stage + (size_t)stage * STAGE_BYTES;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        stage16(st + ((0 + c) * 32 + lane) * 16, reinterpret_cast<const uint4*>(p.kp + r0 * 64) + c * 4 + t);
        stage16(st + ((4 + c) * 32 + lane) * 16, reinterpret_cast<const uint4*>(p.kp + r1 * 64) + c * 4 + t);
        stage16(st + ((8 + c) * 32 + lane) * 16, reinterpret_cast<const uint4*>(p.vp + r0 * 64) + c * 4 + t);
        stage16(st + ((12 + c) * 32 + lane) * 16, reinterpret_cast<const uint4*>(p.vp + r1 * 64) + c * 4 + t);
      }
      uint8_t* ss = st + 16 * 512;
      // slots: 0 ks(r0) 1 kb(r0) 2 ks(r1) 3 kb(r1) 4 vs(r0) 5 vb(r0) 6 vs(r1) 7 vb(r1); lane t copies slots t, t + 4
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int j = t + 4 * half;
        const void* base = half == 0 ? ((j & 1) ? p.kb : p.ks) : ((j & 1) ? p.vb : p.vs);
        const int64_t r = (j & 2) ? r1 : r0;
        const uint8_t* src = reinterpret_cast<const uint8_t*>(base) + r * 4 * esz;
        if constexpr (ST == MXB_F32) stage16(ss + (j * 8 + g) * SB, src);
        else stage8(ss + (j * 8 + g) * SB, src);
      }
    }
    asm volatile("cp.async.commit_group;" ::: "memory");   // (an empty group past the last tile keeps the count uniform)
  };
#pragma unroll
  for (int s0 = 0; s0 < QD_STAGES - 1; ++s0) issue_tile(warp + s0 * QD_WARPS, s0);
  int stage = 0;
  for (int tile = warp; tile < ntiles; tile += QD_WARPS) {
    const int key0 = k_lo + tile * QD_TILE;
    const bool ok0 = key0 + g < k_hi, ok1 = key0 + g + 8 < k_hi;
    __syncwarp();   // every lane is done with the slots that the next copies overwrite
    {
      int ahead = stage + QD_STAGES - 1;
      if (ahead >= QD_STAGES) ahead -= QD_STAGES;
      issue_tile(tile + (QD_STAGES - 1) * QD_WARPS, ahead);
    }
    asm volatile("cp.async.wait_group %0;" ::"n"(QD_STAGES - 1) : "memory");   // this tile's pieces have landed
    __syncwarp();                                                                // ... those of the other lanes of the quad too
    const uint8_t* st = my_stage + (size_t)stage * STAGE_BYTES;
    const uint8_t* ss = st + 16 * 512;
    stage = stage + 1 == QD_STAGES ? 0 : stage + 1;
    uint32_t kr0[16], kr1[16];   // bytes [16 t, 16 t + 16) of every group of key rows g and g + 8
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      *reinterpret_cast<uint4*>(&kr0[4 * c]) = *reinterpret_cast<const uint4*>(st + ((0 + c) * 32 + lane) * 16);
      *reinterpret_cast<uint4*>(&kr1[4 * c]) = *reinterpret_cast<const uint4*>(st + ((4 + c) * 32 + lane) * 16);
    }
    float ks0[4], kb0[4], ks1[4], kb1[4];
    staged_group4<ST>(ss + (0 * 8 + g) * SB, ks0); staged_group4<ST>(ss + (1 * 8 + g) * SB, kb0);
    staged_group4<ST>(ss + (2 * 8 + g) * SB, ks1); staged_group4<ST>(ss + (3 * 8 + g) * SB, kb1);

    // ---- S = K q^T (log2 units): c0, c1 = key g, heads 2 t, 2 t + 1; c2, c3 = key g + 8.  The bytes go into the
    // MMA as 1024 + u; per group, w = u * scale + bias = (1024 + u) * scale + (bias - 1024 scale), so
    // S += scale * (bytes . q) + (bias - 1024 scale) * (sum of q over the group).
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      float a[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const int i = 4 * grp + w;
        mma_f16_16816(a, byte_pair_f16(kr0[i], 0), byte_pair_f16(kr1[i], 0), byte_pair_f16(kr0[i], 1),
                      byte_pair_f16(kr1[i], 1), qb_s[(i * 2 + 0) * 32 + lane], qb_s[(i * 2 + 1) * 32 + lane]);
      }
      const float o0 = fmaf(-1024.f, ks0[grp], kb0[grp]), o1 = fmaf(-1024.f, ks1[grp], kb1[grp]);
      sc[0] += fmaf(ks0[grp], a[0], o0 * qsum[grp][0]);
      sc[1] += fmaf(ks0[grp], a[1], o0 * qsum[grp][1]);
      sc[2] += fmaf(ks1[grp], a[2], o1 * qsum[grp][0]);
      sc[3] += fmaf(ks1[grp], a[3], o1 * qsum[grp][1]);
    }
    if (!ok0) sc[0] = sc[1] = -INFINITY;
    if (!ok1) sc[2] = sc[3] = -INFINITY;
    float mt0 = fmaxf(sc[0], sc[2]), mt1 = fmaxf(sc[1], sc[3]);
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {   // over the eight lanes (keys) that share t
      mt0 = fmaxf(mt0, __shfl_xor_sync(0xffffffffu, mt0, off));
      mt1 = fmaxf(mt1, __shfl_xor_sync(0xffffffffu, mt1, off));
    }
    const float mn0 = fmaxf(m_run[0], mt0), mn1 = fmaxf(m_run[1], mt1);
    if (__any_sync(0xffffffffu, mn0 > m_run[0] || mn1 > m_run[1])) {   // a maximum moved: bring O^T and l along
      const float c0 = m_run[0] == -INFINITY ? 0.f : exp2f(m_run[0] - mn0);
      const float c1 = m_run[1] == -INFINITY ? 0.f : exp2f(m_run[1] - mn1);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        o[i][0] *= c0; o[i][2] *= c0;
        o[i][1] *= c1; o[i][3] *= c1;
      }
#pragma unroll
      for (int grp = 0; grp < 4; ++grp) {
        ofix[grp][0] *= c0;
        ofix[grp][1] *= c1;
      }
      l_run[0] *= c0;
      l_run[1] *= c1;
      m_run[0] = mn0;
      m_run[1] = mn1;
    }
    // ---- P (fp16) and its sums; rows without a key weigh nothing
    const float p00 = ok0 ? exp2f(sc[0] - m_run[0]) : 0.f, p01 = ok0 ? exp2f(sc[1] - m_run[1]) : 0.f;
    const float p10 = ok1 ? exp2f(sc[2] - m_run[0]) : 0.f, p11 = ok1 ? exp2f(sc[3] - m_run[1]) : 0.f;
    const __half2 plo = __floats2half2_rn(p00, p01), phi = __floats2half2_rn(p10, p11);
    l_run[0] += __low2float(plo) + __low2float(phi);   // the weights as the MMA reads them
    l_run[1] += __high2float(plo) + __high2float(phi);

    uint32_t vr0[16], vr1[16];   // the value rows, read from the staging slots only now
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      *reinterpret_cast<uint4*>(&vr0[4 * c]) = *reinterpret_cast<const uint4*>(st + ((8 + c) * 32 + lane) * 16);
      *reinterpret_cast<uint4*>(&vr1[4 * c]) = *reinterpret_cast<const uint4*>(st + ((12 + c) * 32 + lane) * 16);
    }
    float vs0[4], vb0[4], vs1[4], vb1[4];
    staged_group4<ST>(ss + (4 * 8 + g) * SB, vs0); staged_group4<ST>(ss + (5 * 8 + g) * SB, vb0);
    staged_group4<ST>(ss + (6 * 8 + g) * SB, vs1); staged_group4<ST>(ss + (7 * 8 + g) * SB, vb1);
    // ---- O^T += V^T P, 16 dims of ONE group per MMA: the value bytes go in as 1024 + u, the key's scale for that
    // group goes into P (rounded to fp16: what the MMA reads), and the rest, sum of P * scale * (bias / scale - 1024),
    // is kept beside the accumulators with the same rounded weights
#pragma unroll
    for (int grp = 0; grp < 4; ++grp) {
      const __half2 w0 = __hmul2(plo, __float2half2_rn(vs0[grp])), w1 = __hmul2(phi, __float2half2_rn(vs1[grp]));
      const uint32_t pb0 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&w0));   // head g, keys 2 t, 2 t + 1
      const uint32_t pb1 = movmatrix_trans(*reinterpret_cast<const uint32_t*>(&w1));   // head g, keys 2 t + 8, 2 t + 9
      // bias * P - 1024 * (P * scale as rounded)
      ofix[grp][0] += fmaf(__low2float(plo), vb0[grp], fmaf(__low2float(phi), vb1[grp], -1024.f * (__low2float(w0) + __low2float(w1))));
      ofix[grp][1] += fmaf(__high2float(plo), vb0[grp], fmaf(__high2float(phi), vb1[grp], -1024.f * (__high2float(w0) + __high2float(w1))));
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const int i = 4 * grp + w;
        const uint32_t a0 = movmatrix_trans(byte_pair_f16(vr0[i], 0));
        const uint32_t a1 = movmatrix_trans(byte_pair_f16(vr0[i], 1));
        const uint32_t a2 = movmatrix_trans(byte_pair_f16(vr1[i], 0));
        const uint32_t a3 = movmatrix_trans(byte_pair_f16(vr1[i], 1));
        mma_f16_16816(o[i], a0, a1, a2, a3, pb0, pb1);
      }
    }
  }
  // the left-out terms, summed over the eight lanes (keys) that share t, join every dim of their group
#pragma unroll
  for (int grp = 0; grp < 4; ++grp) {
#pragma unroll
    for (int off = 4; off < 32; off <<= 1) {
      ofix[grp][0] += __shfl_xor_sync(0xffffffffu, ofix[grp][0], off);
      ofix[grp][1] += __shfl_xor_sync(0xffffffffu, ofix[grp][1], off);
    }
#pragma unroll
    for (int w = 0; w < 4; ++w) {
      o[4 * grp + w][0] += ofix[grp][0]; o[4 * grp + w][2] += ofix[grp][0];
      o[4 * grp + w][1] += ofix[grp][1]; o[4 * grp + w][3] += ofix[grp][1];
    }
  }

  // ---- merge the warps in warp order
#pragma unroll
  for (int off = 4; off < 32; off <<= 1) {
    l_run[0] += __shfl_xor_sync(0xffffffffu, l_run[0], off);
    l_run[1] += __shfl_xor_sync(0xffffffffu, l_run[1], off);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();   // the staging memory becomes the accumulator exchange
  if (g == 0) {
    m_s[warp][2 * t] = m_run[0];
    m_s[warp][2 * t + 1] = m_run[1];
    l_s[warp][2 * t] = l_run[0];
    l_s[warp][2 * t + 1] = l_run[1];
  }
#pragma unroll
  for (int i = 0; i < 16; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c)
      o_s[warp][2 * t + (c & 1)][64 * (i >> 2) + 16 * (g >> 1) + 4 * (i & 3) + 2 * (c >> 1) + (g & 1)] = o[i][c];
  __syncthreads();
  for (int i = tid; i < G * QD_D; i += QD_WARPS * 32) {
    const int h = i / QD_D, d = i % QD_D;
    float mm = -INFINITY;
    for (int w = 0; w < QD_WARPS; ++w) mm = fmaxf(mm, m_s[w][h]);
    float acc = 0.f, ll = 0.f;
    for (int w = 0; w < QD_WARPS; ++w) {
      const float f = m_s[w][h] == -INFINITY ? 0.f : exp2f(m_s[w][h] - mm);
      acc = fmaf(o_s[w][h][d], f, acc);
      ll = fmaf(l_s[w][h], f, ll);
    }
    const int hq = kvh * G + h;
    p.o_parts[((int64_t)split * p.Hq + hq) * QD_D + d] = acc;
    if (d == 0) {
      // (m, l) in natural-log units for the merge kernel
      p.ml_parts[((int64_t)split * p.Hq + hq) * 2] = mm == -INFINITY ? -INFINITY : mm * 0.6931471805599453f;
      p.ml_parts[((int64_t)split * p.Hq + hq) * 2 + 1] = ll;
    }
  }
}

}  // namespace mxb

using namespace mxb;

static int q8_check(const mxb_affine_q8_args* a, const char* what) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "%s: null args", what);
  MXB_REQUIRE(a->n_rows > 0 && a->width > 0 && a->width % Q8_GROUP == 0, MXB_ERR_INVALID,
              "%s: rows must be non-empty and their width a multiple of the group size 64", what);
  MXB_REQUIRE(a->x && a->packed && a->scales && a->biases, MXB_ERR_INVALID, "%s: null tensor", what);
  MXB_REQUIRE(a->x_dtype == MXB_F32 || a->x_dtype == MXB_F16 || a->x_dtype == MXB_BF16, MXB_ERR_INVALID,
              "%s: rows must be float32, float16 or bfloat16", what);
  MXB_REQUIRE(a->sb_dtype == MXB_F32 || a->sb_dtype == MXB_F16 || a->sb_dtype == MXB_BF16, MXB_ERR_INVALID,
              "%s: scales and biases must be float32, float16 or bfloat16", what);
  MXB_REQUIRE((reinterpret_cast<uintptr_t>(a->packed) & 7) == 0, MXB_ERR_INVALID, "%s: packed words must be 8-byte aligned", what);
  return MXB_OK;
}

extern "C" int mxb_affine_q8_quantize(const mxb_affine_q8_args* a, void* stream) {
  int rc = q8_check(a, "affine q8 quantise");
  if (rc != MXB_OK) return rc;
  MXB_REQUIRE(a->sb_dtype == a->x_dtype, MXB_ERR_INVALID, "affine q8 quantise: scales and biases take the rows' type");
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
  uint32_t* pk = reinterpret_cast<uint32_t*>(a->packed);
#define MXB_Q(XT) affine_q8_quantize_kernel<XT><<<grid, 128, 0, st>>>(a->x, a->x_row_stride, pk, a->scales, a->biases, a->n_rows, a->width)
  if (a->x_dtype == MXB_F32) MXB_Q(MXB_F32);
  else if (a->x_dtype == MXB_F16) MXB_Q(MXB_F16);
  else MXB_Q(MXB_BF16);
#undef MXB_Q
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_affine_q8_dequantize(const mxb_affine_q8_args* a, void* stream) {
  int rc = q8_check(a, "affine q8 dequantise");
  if (rc != MXB_OK) return rc;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const unsigned grid = (unsigned)ceil_div(a->n_rows, 4);
  const uint32_t* pk = reinterpret_cast<const uint32_t*>(a->packed);
  void* out = const_cast<void*>(a->x);
#define MXB_DQ(ST, OT) \
  if (a->sb_dtype == ST && a->x_dtype == OT)                                                                          \
    affine_q8_dequantize_kernel<ST, OT><<<grid, 128, 0, st>>>(pk, a->scales, a->biases, out, a->x_row_stride, a->n_rows, a->width); \
  else
  MXB_DQ(MXB_F32, MXB_F32) MXB_DQ(MXB_F32, MXB_F16) MXB_DQ(MXB_F32, MXB_BF16)
  MXB_DQ(MXB_F16, MXB_F32) MXB_DQ(MXB_F16, MXB_F16) MXB_DQ(MXB_F16, MXB_BF16)
  MXB_DQ(MXB_BF16, MXB_F32) MXB_DQ(MXB_BF16, MXB_F16) MXB_DQ(MXB_BF16, MXB_BF16)
  return fail(MXB_ERR_UNSUPPORTED, "affine q8 dequantise: unsupported type pair");
#undef MXB_DQ
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}

extern "C" int mxb_sdpa_decode_q8(const mxb_sdpa_decode_q8_args* a, void* stream) {
  MXB_REQUIRE(a != nullptr, MXB_ERR_INVALID, "q8 decode: null args");
  MXB_REQUIRE(a->D == QD_D, MXB_ERR_INVALID, "q8 decode requires head_dim=256");
  MXB_REQUIRE(a->Hq > 0 && a->Hkv > 0 && a->Hq % a->Hkv == 0 && a->Hq / a->Hkv <= QD_MAXG, MXB_ERR_INVALID,
              "q8 decode: query heads must be a multiple (at most 8x) of kv heads");
  MXB_REQUIRE(a->P >= 1, MXB_ERR_INVALID, "q8 decode needs at least one cached key");
  MXB_REQUIRE(a->n_splits >= 1 && a->n_splits <= 1024, MXB_ERR_INVALID, "q8 decode: splits must be between 1 and 1024");
  MXB_REQUIRE(a->q && a->k_packed && a->k_scales && a->k_biases && a->v_packed && a->v_scales && a->v_biases &&
                  a->o_parts && a->ml_parts,
              MXB_ERR_INVALID, "q8 decode: null tensor");
  MXB_REQUIRE(((reinterpret_cast<uintptr_t>(a->k_packed) | reinterpret_cast<uintptr_t>(a->v_packed)) & 15) == 0,
              MXB_ERR_INVALID, "q8 decode: packed words must be 16-byte aligned");
  {
    const uintptr_t sb = reinterpret_cast<uintptr_t>(a->k_scales) | reinterpret_cast<uintptr_t>(a->k_biases) |
                         reinterpret_cast<uintptr_t>(a->v_scales) | reinterpret_cast<uintptr_t>(a->v_biases);
    MXB_REQUIRE((sb & (a->sb_dtype == MXB_F32 ? 15u : 7u)) == 0, MXB_ERR_INVALID,
                "q8 decode: scales and biases must be aligned to the four values of a row");
  }
  Q8DecodeParams p{};
  p.q = a->q; p.q_dtype = a->q_dtype;
  p.kp = reinterpret_cast<const uint32_t*>(a->k_packed); p.ks = a->k_scales; p.kb = a->k_biases;
  p.vp = reinterpret_cast<const uint32_t*>(a->v_packed); p.vs = a->v_scales; p.vb = a->v_biases;
  p.head_stride_rows = a->head_stride_rows; p.sb_dtype = a->sb_dtype;
  p.P = a->P; p.Hq = a->Hq; p.Hkv = a->Hkv; p.nsplit = a->n_splits;
  p.scale_log2 = a->scale * 1.4426950408889634f;
  p.o_parts = a->o_parts; p.ml_parts = a->ml_parts;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  dim3 grid((unsigned)a->n_splits, (unsigned)a->Hkv);
#define MXB_QD(ST)                                                                                              \
  {                                                                                                             \
    const int stage_bytes = QD_WARPS * QD_STAGES * (16 * 512 + 8 * 8 * ((ST) == MXB_F32 ? 16 : 8)) + 16 * 2 * 32 * 4; \
    const int out_bytes = QD_WARPS * QD_MAXG * QD_D * 4;                                                         \
    const int smem = stage_bytes > out_bytes ? stage_bytes : out_bytes;                                          \
    MXB_CUDA_OK(cudaFuncSetAttribute(q8_decode_kernel<ST>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem)); \
    q8_decode_kernel<ST><<<grid, QD_WARPS * 32, smem, st>>>(p);                                                 \
  }
  if (a->sb_dtype == MXB_F32) MXB_QD(MXB_F32)
  else if (a->sb_dtype == MXB_F16) MXB_QD(MXB_F16)
  else if (a->sb_dtype == MXB_BF16) MXB_QD(MXB_BF16)
  else return fail(MXB_ERR_INVALID, "q8 decode: scales and biases must be float32, float16 or bfloat16");
#undef MXB_QD
  note_launch();
  MXB_CUDA_OK(cudaGetLastError());
  return MXB_OK;
}
