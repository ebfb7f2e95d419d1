// Tensor-core causal attention (forward and backward) for head sizes 32 / 64 / 128 and S <= 256.
//
// One CTA = one (sample, head, block of 64 query or key rows); 4 warps, each owning a 16-row tile and issuing
// mma.sync m16n8k16 (bf16 in, fp32 accumulate).  Q, K (rotary embedding applied while loading), V and -- in
// backward -- dO of the head sit in shared memory as bf16 rows of HD + 8 elements (the padding makes both the
// 32-bit fragment loads and the 16-byte ldmatrix rows bank-conflict free).  Operands that the MMA wants
// "transposed" (V in P.V, K in dS.K, dO in P^T.dO, Q in dS^T.Q) are fetched with ldmatrix.trans from the same
// row-major tiles, so no transposed copy exists.  Scores never leave registers; backward recomputes the
// probabilities from the saved log-sum-exp in two sweeps (query-major for dQ, key-major for dK and dV), which
// keeps it free of atomics and bitwise reproducible.
#pragma once

#include "rte_common.cuh"

namespace attn_mma {

constexpr int QB = 64;          // rows per CTA
constexpr int NTHR = 128;

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// B fragment (k = 16 rows of a row-major tile, n = 8 columns starting at the given address), transposed on load.
__device__ __forceinline__ void ldsm_x2_trans(uint32_t& b0, uint32_t& b1, const __nv_bfloat16* row_ptr) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(row_ptr));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
}
__device__ __forceinline__ uint32_t ld32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }

__device__ __forceinline__ float inv_freq(int pair, int hd) { return 1.0f / powf(10000.0f, (float)(2 * pair) / (float)hd); }
// cos/sin of position `pos`, rotary pair `pair`: from the caller's table [S, hd/2, 2] when given, else computed.
__device__ __forceinline__ void rope_cs(const float* __restrict__ table, int pos, int pair, int hd, float& cs, float& sn) {
  if (table != nullptr) {
    const float2 v = *reinterpret_cast<const float2*>(table + ((size_t)pos * (hd / 2) + pair) * 2);
    cs = v.x; sn = v.y;
  } else {
    sincosf((float)pos * inv_freq(pair, hd), &sn, &cs);
  }
}

// rows [row0, row0 + n_rows) of one head -> smem rows [0, pad_rows) (bf16, row stride HD + 8); rows past n_rows are
// zeroed.  Each thread moves 8 consecutive dims (4 rotary pairs) with one 16-byte load; rotary positions are absolute
// (row0 + r).  When `dsum` is given, also accumulates sum_c x[r,c] * other[r,c] per row into dsum[r] (used for
// D = rowsum(dO * O) in backward): the HD/8 threads of a row are neighbouring lanes.
template <int HD, bool ROPE>
__device__ __forceinline__ void load_rows(const __nv_bfloat16* __restrict__ src, int ld, int n_rows, int pad_rows,
                                          __nv_bfloat16* dst, const float* __restrict__ rope = nullptr, int row0 = 0,
                                          const __nv_bfloat16* __restrict__ other = nullptr, int ld_other = 0,
                                          float* dsum = nullptr) {
  constexpr int LDS = HD + 8, CPR = HD / 8;      // 16-byte chunks per row
  for (int idx = threadIdx.x; idx < pad_rows * CPR; idx += blockDim.x) {
    const int r = idx / CPR, ch = idx % CPR;
    uint4 raw = make_uint4(0u, 0u, 0u, 0u);
    float part = 0.f;
    if (r < n_rows) {
      raw = *reinterpret_cast<const uint4*>(src + (size_t)(row0 + r) * ld + 8 * ch);
      if (ROPE) {
        uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          float cs, sn;
          rope_cs(rope, row0 + r, 4 * ch + q, HD, cs, sn);
          const float2 v = rte::unpack_bf16x2(w[q]);
          w[q] = rte::pack_bf16x2(v.x * cs - v.y * sn, v.y * cs + v.x * sn);
        }
        raw = make_uint4(w[0], w[1], w[2], w[3]);
      }
      if (other != nullptr) {
        const uint4 o = *reinterpret_cast<const uint4*>(other + (size_t)(row0 + r) * ld_other + 8 * ch);
        const uint32_t a4[4] = {raw.x, raw.y, raw.z, raw.w}, b4[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const float2 x = rte::unpack_bf16x2(a4[q]), y = rte::unpack_bf16x2(b4[q]);
          part += x.x * y.x + x.y * y.y;
        }
      }
    }
    *reinterpret_cast<uint4*>(dst + r * LDS + 8 * ch) = raw;
    if (dsum != nullptr) {
#pragma unroll
      for (int o = 1; o < CPR; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
      if (ch == 0) dsum[r] = part;
    }
  }
}

// ---- asynchronous tile loads.  All tiles of a CTA are requested at once with cp.async (16-byte pieces straight into
// shared memory, nothing held in registers), so a CTA has its whole working set in flight instead of one dependent
// load per thread at a time; the rotary embedding is then applied in place by the thread that copied the piece.
__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gsrc) {
  const uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
  asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}

// rows [row0, row0 + n_rows) of one head -> smem rows [0, pad_rows) (row stride HD + 8), rows past n_rows zeroed.
template <int HD>
__device__ __forceinline__ void tile_async(const __nv_bfloat16* __restrict__ src, int ld, int n_rows, int pad_rows,
                                           __nv_bfloat16* dst, int row0 = 0) {
  constexpr int LDS = HD + 8, CPR = HD / 8;
  for (int idx = threadIdx.x; idx < pad_rows * CPR; idx += blockDim.x) {
    const int r = idx / CPR, ch = idx % CPR;
    __nv_bfloat16* d = dst + r * LDS + 8 * ch;
    if (r < n_rows) cp_async16(d, src + (size_t)(row0 + r) * ld + 8 * ch);
    else *reinterpret_cast<uint4*>(d) = make_uint4(0u, 0u, 0u, 0u);
  }
}

// Rotary embedding in place on a tile loaded by tile_async: every thread rotates exactly the pieces it copied (same
// index mapping), so it only needs its own copies to have landed (cp_async_wait_all), not a CTA barrier.
template <int HD>
__device__ __forceinline__ void rotate_tile(__nv_bfloat16* tile, int n_rows, int pad_rows, const float* __restrict__ rope, int row0 = 0) {
  constexpr int LDS = HD + 8, CPR = HD / 8;
  for (int idx = threadIdx.x; idx < pad_rows * CPR; idx += blockDim.x) {
    const int r = idx / CPR, ch = idx % CPR;
    if (r >= n_rows) continue;
    uint4* p = reinterpret_cast<uint4*>(tile + r * LDS + 8 * ch);
    const uint4 raw = *p;
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
    float cs[4], sn[4];
    if (rope != nullptr) {            // (cos, sin) of 4 consecutive pairs = 32 contiguous bytes of the table
      const float4* t4 = reinterpret_cast<const float4*>(rope + ((size_t)(row0 + r) * (HD / 2) + 4 * ch) * 2);
      const float4 a = t4[0], b = t4[1];
      cs[0] = a.x; sn[0] = a.y; cs[1] = a.z; sn[1] = a.w; cs[2] = b.x; sn[2] = b.y; cs[3] = b.z; sn[3] = b.w;
    } else {
#pragma unroll
      for (int q = 0; q < 4; ++q) rope_cs(nullptr, row0 + r, 4 * ch + q, HD, cs[q], sn[q]);
    }
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 v = rte::unpack_bf16x2(w[q]);
      w[q] = rte::pack_bf16x2(v.x * cs[q] - v.y * sn[q], v.y * cs[q] + v.x * sn[q]);
    }
    *p = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// dsum[r] = sum_c tile[r, c] * other[row r of global `other`, c] (D = rowsum(dO * O) of backward): the HD/8 threads
// of a row are neighbouring lanes.  `tile` pieces are the thread's own (loaded by tile_async with the same mapping).
template <int HD>
__device__ __forceinline__ void rowdot_tile(const __nv_bfloat16* tile, int n_rows, int pad_rows, const __nv_bfloat16* __restrict__ other,
                                            int ld_other, float* dsum) {
  constexpr int LDS = HD + 8, CPR = HD / 8;
  for (int idx = threadIdx.x; idx < pad_rows * CPR; idx += blockDim.x) {
    const int r = idx / CPR, ch = idx % CPR;
    float part = 0.f;
    if (r < n_rows) {
      const uint4 a = *reinterpret_cast<const uint4*>(tile + r * LDS + 8 * ch);
      const uint4 o = *reinterpret_cast<const uint4*>(other + (size_t)r * ld_other + 8 * ch);
      const uint32_t a4[4] = {a.x, a.y, a.z, a.w}, b4[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const float2 x = rte::unpack_bf16x2(a4[q]), y = rte::unpack_bf16x2(b4[q]);
        part += x.x * y.x + x.y * y.y;
      }
    }
#pragma unroll
    for (int o = 1; o < CPR; o <<= 1) part += __shfl_xor_sync(0xffffffffu, part, o);
    if (ch == 0) dsum[r] = part;
  }
}

// A fragments (16 rows starting at row0, all HD columns) of a row-major smem tile.
template <int HD>
__device__ __forceinline__ void load_a_frags(const __nv_bfloat16* tile, int row0, int g, int t, uint32_t (&f)[HD / 16][4]) {
  constexpr int LDS = HD + 8;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const __nv_bfloat16* p = tile + (row0 + g) * LDS + 16 * ks + 2 * t;
    f[ks][0] = ld32(p);
    f[ks][1] = ld32(p + 8 * LDS);
    f[ks][2] = ld32(p + 8);
    f[ks][3] = ld32(p + 8 * LDS + 8);
  }
}

// 16 x 8 tile of A . B^T where B rows (n) start at brow0 of a row-major tile: acc[.] = sum_k A[., k] * B[brow0 + n, k]
template <int HD>
__device__ __forceinline__ void rowrow_tile(float (&acc)[4], const uint32_t (&a)[HD / 16][4], const __nv_bfloat16* btile,
                                            int brow0, int g, int t) {
  constexpr int LDS = HD + 8;
  acc[0] = acc[1] = acc[2] = acc[3] = 0.f;
#pragma unroll
  for (int ks = 0; ks < HD / 16; ++ks) {
    const __nv_bfloat16* p = btile + (brow0 + g) * LDS + 16 * ks + 2 * t;
    mma16816(acc, a[ks], ld32(p), ld32(p + 8));
  }
}

// ------------------------------------------------------------------ forward
template <int HD, int SMAX>
__global__ void __launch_bounds__(NTHR, (SMAX <= 64 && HD <= 64) ? 6 : 1)
fwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int sec, __nv_bfloat16* __restrict__ y, int ldy,
           float* __restrict__ lse, const float* __restrict__ rope, int S, int H,
           __nv_bfloat16* __restrict__ ym, const int32_t* __restrict__ mask_row, const float* __restrict__ mask_tab) {
  constexpr int LDS = HD + 8, KT = SMAX / 8;
  extern __shared__ __align__(16) uint8_t smraw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smraw);       // [QB][LDS]
  __nv_bfloat16* sk = sq + QB * LDS;                                  // [SMAX][LDS]
  __nv_bfloat16* sv = sk + SMAX * LDS;                                // [SMAX][LDS]
  const int b = blockIdx.x / H, h = blockIdx.x % H, qb0 = blockIdx.y * QB;
  const int kv_rows = min(S, qb0 + QB);                               // causal: later keys are never read
  const int kv_pad = min(SMAX, (kv_rows + 15) & ~15);
  const __nv_bfloat16* base = qkv + (size_t)b * S * ld + h * HD;
  const int q_rows = max(0, min(QB, S - qb0));
  tile_async<HD>(base, ld, q_rows, QB, sq, qb0);
  tile_async<HD>(base + sec, ld, kv_rows, kv_pad, sk);
  tile_async<HD>(base + 2 * sec, ld, kv_rows, kv_pad, sv);
  cp_async_wait_all();
  rotate_tile<HD>(sq, q_rows, QB, rope, qb0);
  rotate_tile<HD>(sk, kv_rows, kv_pad, rope);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int r0 = warp * 16, q0 = qb0 + r0;
  if (q0 >= S) return;
  uint32_t qf[HD / 16][4];
  load_a_frags<HD>(sq, r0, g, t, qf);
  const int ntiles = min(kv_pad, q0 + 16) / 8;                        // even: kv_pad and q0 are multiples of 16
  const float scale = rsqrtf((float)HD);
  float sc[KT][4];
  float m0 = -INFINITY, m1 = -INFINITY;
  const int row_a = q0 + g, row_b = q0 + g + 8;
#pragma unroll
  for (int nb = 0; nb < KT; ++nb) {
    if (nb < ntiles) {
      rowrow_tile<HD>(sc[nb], qf, sk, nb * 8, g, t);
      const int c0 = nb * 8 + 2 * t, c1 = c0 + 1;
      sc[nb][0] = (c0 <= row_a && c0 < S) ? sc[nb][0] * scale : -INFINITY;
      sc[nb][1] = (c1 <= row_a && c1 < S) ? sc[nb][1] * scale : -INFINITY;
      sc[nb][2] = (c0 <= row_b && c0 < S) ? sc[nb][2] * scale : -INFINITY;
      sc[nb][3] = (c1 <= row_b && c1 < S) ? sc[nb][3] * scale : -INFINITY;
      m0 = fmaxf(m0, fmaxf(sc[nb][0], sc[nb][1]));
      m1 = fmaxf(m1, fmaxf(sc[nb][2], sc[nb][3]));
    }
  }
  m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 1)); m0 = fmaxf(m0, __shfl_xor_sync(0xffffffffu, m0, 2));
  m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 1)); m1 = fmaxf(m1, __shfl_xor_sync(0xffffffffu, m1, 2));
  float s0 = 0.f, s1 = 0.f;
#pragma unroll
  for (int nb = 0; nb < KT; ++nb) {
    if (nb < ntiles) {
      sc[nb][0] = __expf(sc[nb][0] - m0); sc[nb][1] = __expf(sc[nb][1] - m0);
      sc[nb][2] = __expf(sc[nb][2] - m1); sc[nb][3] = __expf(sc[nb][3] - m1);
      s0 += sc[nb][0] + sc[nb][1];
      s1 += sc[nb][2] + sc[nb][3];
    }
  }
  s0 += __shfl_xor_sync(0xffffffffu, s0, 1); s0 += __shfl_xor_sync(0xffffffffu, s0, 2);
  s1 += __shfl_xor_sync(0xffffffffu, s1, 1); s1 += __shfl_xor_sync(0xffffffffu, s1, 2);
  float o[HD / 8][4];
#pragma unroll
  for (int nd = 0; nd < HD / 8; ++nd) o[nd][0] = o[nd][1] = o[nd][2] = o[nd][3] = 0.f;
#pragma unroll
  for (int j = 0; j < KT / 2; ++j) {
    if (2 * j < ntiles) {
      uint32_t a[4];
      a[0] = rte::pack_bf16x2(sc[2 * j][0], sc[2 * j][1]);
      a[1] = rte::pack_bf16x2(sc[2 * j][2], sc[2 * j][3]);
      a[2] = rte::pack_bf16x2(sc[2 * j + 1][0], sc[2 * j + 1][1]);
      a[3] = rte::pack_bf16x2(sc[2 * j + 1][2], sc[2 * j + 1][3]);
#pragma unroll
      for (int nd = 0; nd < HD / 8; ++nd) {
        uint32_t b0, b1;
        ldsm_x2_trans(b0, b1, sv + (16 * j + (lane & 15)) * LDS + nd * 8);
        mma16816(o[nd], a, b0, b1);
      }
    }
  }
  const float i0 = 1.f / s0, i1 = 1.f / s1;
  // optional second output: the same rows times a per-sample column mask (ym = bf16(y) * mask_tab[mask_row[b]][col],
  // exactly what a separate pass over the stored y would give)
  const float* mt = ym ? mask_tab + (size_t)mask_row[b] * (H * HD) + h * HD : nullptr;
  if (row_a < S) {
    __nv_bfloat16* yo = y + (size_t)(b * S + row_a) * ldy + h * HD;
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(o[nd][0] * i0, o[nd][1] * i0);
      *reinterpret_cast<__nv_bfloat162*>(yo + nd * 8 + 2 * t) = v;
      if (ym) {
        const float2 w = *reinterpret_cast<const float2*>(mt + nd * 8 + 2 * t);
        *reinterpret_cast<__nv_bfloat162*>(ym + (size_t)(b * S + row_a) * ldy + h * HD + nd * 8 + 2 * t) =
            __floats2bfloat162_rn(__low2float(v) * w.x, __high2float(v) * w.y);
      }
    }
    if (t == 0) lse[((size_t)b * H + h) * S + row_a] = m0 + __logf(s0);
  }
  if (row_b < S) {
    __nv_bfloat16* yo = y + (size_t)(b * S + row_b) * ldy + h * HD;
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      const __nv_bfloat162 v = __floats2bfloat162_rn(o[nd][2] * i1, o[nd][3] * i1);
      *reinterpret_cast<__nv_bfloat162*>(yo + nd * 8 + 2 * t) = v;
      if (ym) {
        const float2 w = *reinterpret_cast<const float2*>(mt + nd * 8 + 2 * t);
        *reinterpret_cast<__nv_bfloat162*>(ym + (size_t)(b * S + row_b) * ldy + h * HD + nd * 8 + 2 * t) =
            __floats2bfloat162_rn(__low2float(v) * w.x, __high2float(v) * w.y);
      }
    }
    if (t == 0) lse[((size_t)b * H + h) * S + row_b] = m1 + __logf(s1);
  }
}

// ------------------------------------------------------------------ backward
__device__ __forceinline__ void unrope_pair(float& a, float& b, int pos, int pair, int hd, const float* __restrict__ rope) {
  float sn, cs;
  rope_cs(rope, pos, pair, hd, cs, sn);
  const float x = a, y = b;
  a = x * cs + y * sn;
  b = -x * sn + y * cs;
}

// tile[r][c] *= mask[c] on the pieces this thread copied itself (the mapping of tile_async), one bf16 rounding
template <int HD>
__device__ __forceinline__ void colscale_tile(__nv_bfloat16* tile, int n_rows, int pad_rows, const float* __restrict__ mask) {
  constexpr int LDS = HD + 8, CPR = HD / 8;
  for (int idx = threadIdx.x; idx < pad_rows * CPR; idx += blockDim.x) {
    const int r = idx / CPR, ch = idx % CPR;
    if (r >= n_rows) continue;
    uint4* p = reinterpret_cast<uint4*>(tile + r * LDS + 8 * ch);
    const uint4 raw = *p;
    uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const float2 v = rte::unpack_bf16x2(w[q]);
      w[q] = rte::pack_bf16x2(v.x * mask[8 * ch + 2 * q], v.y * mask[8 * ch + 2 * q + 1]);
    }
    *p = make_uint4(w[0], w[1], w[2], w[3]);
  }
}

// MASKED: the upstream gradient is dy[row, c] * mask_tab[mask_row[sample]][c] (the banked core's recipe mask on the
// attention output, layers.py:702-728); the mask is applied to the dy tile in shared memory.
template <int HD, int SMAX, bool MASKED>
__global__ void __launch_bounds__(NTHR, (SMAX <= 64 && HD <= 64) ? 4 : 1)
bwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int sec, const __nv_bfloat16* __restrict__ y,
           const __nv_bfloat16* __restrict__ dy, int ldy, const float* __restrict__ lse,
           __nv_bfloat16* __restrict__ dqkv, const float* __restrict__ rope, int S, int H,
           const int32_t* __restrict__ mask_row, const float* __restrict__ mask_tab) {
  constexpr int LDS = HD + 8;
  extern __shared__ __align__(16) uint8_t smraw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smraw);
  __nv_bfloat16* sk = sq + SMAX * LDS;
  __nv_bfloat16* sv = sk + SMAX * LDS;
  __nv_bfloat16* sdo = sv + SMAX * LDS;
  float* slse = reinterpret_cast<float*>(sdo + SMAX * LDS);
  float* sD = slse + SMAX;
  const int b = blockIdx.x / H, h = blockIdx.x % H, blk0 = blockIdx.y * QB;
  const int s_pad = min(SMAX, (S + 15) & ~15);
  const __nv_bfloat16* base = qkv + (size_t)b * S * ld + h * HD;
  tile_async<HD>(base, ld, S, s_pad, sq);
  tile_async<HD>(base + sec, ld, S, s_pad, sk);
  tile_async<HD>(base + 2 * sec, ld, S, s_pad, sv);
  tile_async<HD>(dy + (size_t)b * S * ldy + h * HD, ldy, S, s_pad, sdo);
  cp_async_wait_all();
  rotate_tile<HD>(sq, S, s_pad, rope);
  rotate_tile<HD>(sk, S, s_pad, rope);
  if (MASKED) colscale_tile<HD>(sdo, S, s_pad, mask_tab + (size_t)mask_row[b] * (H * HD) + h * HD);
  rowdot_tile<HD>(sdo, S, s_pad, y + (size_t)b * S * ldy + h * HD, ldy, sD);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  for (int i = threadIdx.x; i < s_pad; i += NTHR) slse[i] = (i < S) ? lse[((size_t)b * H + h) * S + i] : 0.f;
  __syncthreads();
  const float scale = rsqrtf((float)HD);
  const int r0 = blk0 + warp * 16;
  if (r0 >= S) return;
  __nv_bfloat16* dbase = dqkv + (size_t)b * S * ld + h * HD;
  const int row_a = r0 + g, row_b = r0 + g + 8;

  // With few (sample, head) pairs the launch is split in two along z: one CTA per sweep, half the latency.
  const int only = gridDim.z == 2 ? (int)blockIdx.z : -1;

  // ---- sweep 1: dQ of query rows r0 .. r0+15 over key blocks j <= r0/16
  if (only != 1) {
    uint32_t qf[HD / 16][4], dof[HD / 16][4];
    load_a_frags<HD>(sq, r0, g, t, qf);
    load_a_frags<HD>(sdo, r0, g, t, dof);
    const float la = slse[row_a], lb = slse[row_b], Da = sD[row_a], Db = sD[row_b];
    float dq[HD / 8][4];
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) dq[nd][0] = dq[nd][1] = dq[nd][2] = dq[nd][3] = 0.f;
    for (int j = 0; j <= r0 / 16; ++j) {
      float ds[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int nb = 2 * j + half;
        float st[4], dp[4];
        rowrow_tile<HD>(st, qf, sk, nb * 8, g, t);
        rowrow_tile<HD>(dp, dof, sv, nb * 8, g, t);
        const int c0 = nb * 8 + 2 * t, c1 = c0 + 1;
        ds[half][0] = (c0 <= row_a && c0 < S) ? __expf(st[0] * scale - la) * (dp[0] - Da) : 0.f;
        ds[half][1] = (c1 <= row_a && c1 < S) ? __expf(st[1] * scale - la) * (dp[1] - Da) : 0.f;
        ds[half][2] = (c0 <= row_b && c0 < S) ? __expf(st[2] * scale - lb) * (dp[2] - Db) : 0.f;
        ds[half][3] = (c1 <= row_b && c1 < S) ? __expf(st[3] * scale - lb) * (dp[3] - Db) : 0.f;
      }
      uint32_t a[4] = {rte::pack_bf16x2(ds[0][0], ds[0][1]), rte::pack_bf16x2(ds[0][2], ds[0][3]),
                       rte::pack_bf16x2(ds[1][0], ds[1][1]), rte::pack_bf16x2(ds[1][2], ds[1][3])};
#pragma unroll
      for (int nd = 0; nd < HD / 8; ++nd) {
        uint32_t b0, b1;
        ldsm_x2_trans(b0, b1, sk + (16 * j + (lane & 15)) * LDS + nd * 8);
        mma16816(dq[nd], a, b0, b1);
      }
    }
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      const int pair = nd * 4 + t;
      float a0 = dq[nd][0] * scale, a1 = dq[nd][1] * scale, b0 = dq[nd][2] * scale, b1 = dq[nd][3] * scale;
      unrope_pair(a0, a1, min(row_a, S - 1), pair, HD, rope);
      unrope_pair(b0, b1, min(row_b, S - 1), pair, HD, rope);
      if (row_a < S) *reinterpret_cast<__nv_bfloat162*>(dbase + (size_t)row_a * ld + nd * 8 + 2 * t) = __floats2bfloat162_rn(a0, a1);
      if (row_b < S) *reinterpret_cast<__nv_bfloat162*>(dbase + (size_t)row_b * ld + nd * 8 + 2 * t) = __floats2bfloat162_rn(b0, b1);
    }
  }

  // ---- sweep 2: dK, dV of key rows r0 .. r0+15 over query blocks j >= r0/16
  if (only != 0) {
    uint32_t kf[HD / 16][4], vf[HD / 16][4];
    load_a_frags<HD>(sk, r0, g, t, kf);
    load_a_frags<HD>(sv, r0, g, t, vf);
    float dk[HD / 8][4], dv[HD / 8][4];
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      dk[nd][0] = dk[nd][1] = dk[nd][2] = dk[nd][3] = 0.f;
      dv[nd][0] = dv[nd][1] = dv[nd][2] = dv[nd][3] = 0.f;
    }
    for (int j = r0 / 16; j < s_pad / 16; ++j) {
      float pr[2][4], ds[2][4];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        const int nb = 2 * j + half;
        float st[4], dp[4];
        rowrow_tile<HD>(st, kf, sq, nb * 8, g, t);      // st[key, query]
        rowrow_tile<HD>(dp, vf, sdo, nb * 8, g, t);     // (V . dO^T)[key, query]
        const int q0 = nb * 8 + 2 * t, q1 = q0 + 1;
        const float l0 = slse[q0], l1 = slse[q1], D0 = sD[q0], D1 = sD[q1];
        pr[half][0] = (row_a <= q0 && q0 < S) ? __expf(st[0] * scale - l0) : 0.f;
        pr[half][1] = (row_a <= q1 && q1 < S) ? __expf(st[1] * scale - l1) : 0.f;
        pr[half][2] = (row_b <= q0 && q0 < S) ? __expf(st[2] * scale - l0) : 0.f;
        pr[half][3] = (row_b <= q1 && q1 < S) ? __expf(st[3] * scale - l1) : 0.f;
        ds[half][0] = pr[half][0] * (dp[0] - D0);
        ds[half][1] = pr[half][1] * (dp[1] - D1);
        ds[half][2] = pr[half][2] * (dp[2] - D0);
        ds[half][3] = pr[half][3] * (dp[3] - D1);
      }
      uint32_t ap[4] = {rte::pack_bf16x2(pr[0][0], pr[0][1]), rte::pack_bf16x2(pr[0][2], pr[0][3]),
                        rte::pack_bf16x2(pr[1][0], pr[1][1]), rte::pack_bf16x2(pr[1][2], pr[1][3])};
      uint32_t ad[4] = {rte::pack_bf16x2(ds[0][0], ds[0][1]), rte::pack_bf16x2(ds[0][2], ds[0][3]),
                        rte::pack_bf16x2(ds[1][0], ds[1][1]), rte::pack_bf16x2(ds[1][2], ds[1][3])};
#pragma unroll
      for (int nd = 0; nd < HD / 8; ++nd) {
        uint32_t b0, b1;
        ldsm_x2_trans(b0, b1, sdo + (16 * j + (lane & 15)) * LDS + nd * 8);
        mma16816(dv[nd], ap, b0, b1);
        ldsm_x2_trans(b0, b1, sq + (16 * j + (lane & 15)) * LDS + nd * 8);
        mma16816(dk[nd], ad, b0, b1);
      }
    }
#pragma unroll
    for (int nd = 0; nd < HD / 8; ++nd) {
      const int pair = nd * 4 + t;
      float a0 = dk[nd][0] * scale, a1 = dk[nd][1] * scale, b0 = dk[nd][2] * scale, b1 = dk[nd][3] * scale;
      unrope_pair(a0, a1, min(row_a, S - 1), pair, HD, rope);
      unrope_pair(b0, b1, min(row_b, S - 1), pair, HD, rope);
      if (row_a < S) {
        *reinterpret_cast<__nv_bfloat162*>(dbase + (size_t)row_a * ld + sec + nd * 8 + 2 * t) = __floats2bfloat162_rn(a0, a1);
        *reinterpret_cast<__nv_bfloat162*>(dbase + (size_t)row_a * ld + 2 * sec + nd * 8 + 2 * t) = __floats2bfloat162_rn(dv[nd][0], dv[nd][1]);
      }
      if (row_b < S) {
        *reinterpret_cast<__nv_bfloat162*>(dbase + (size_t)row_b * ld + sec + nd * 8 + 2 * t) = __floats2bfloat162_rn(b0, b1);
        *reinterpret_cast<__nv_bfloat162*>(dbase + (size_t)row_b * ld + 2 * sec + nd * 8 + 2 * t) = __floats2bfloat162_rn(dv[nd][2], dv[nd][3]);
      }
    }
  }
}

template <int HD, int SMAX>
int launch_fwd(const void* qkv, int ld, int sec, void* y, int ldy, float* lse, const float* rope, int B, int S, int H, cudaStream_t st,
               void* ym = nullptr, const int32_t* mask_row = nullptr, const float* mask_tab = nullptr) {
  constexpr int smem = (QB + 2 * SMAX) * (HD + 8) * 2;
  static bool set = false;
  if (!set && smem > 48 * 1024) {
    if (cudaFuncSetAttribute(fwd_kernel<HD, SMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess) return RTE_ERR_LAUNCH;
    set = true;
  }
  fwd_kernel<HD, SMAX><<<dim3(B * H, rte::ceil_div(S, QB)), NTHR, smem, st>>>(
      reinterpret_cast<const __nv_bfloat16*>(qkv), ld, sec, reinterpret_cast<__nv_bfloat16*>(y), ldy, lse, rope, S, H,
      reinterpret_cast<__nv_bfloat16*>(ym), mask_row, mask_tab);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

template <int HD, int SMAX>
int launch_bwd(const void* qkv, int ld, int sec, const void* y, const void* dy, int ldy, const float* lse, void* dqkv,
               const float* rope, int B, int S, int H, cudaStream_t st, const int32_t* mask_row = nullptr,
               const float* mask_tab = nullptr) {
  constexpr int smem = 4 * SMAX * (HD + 8) * 2 + 2 * SMAX * 4;
  static bool set = false;
  if (!set && smem > 48 * 1024) {
    if (cudaFuncSetAttribute(bwd_kernel<HD, SMAX, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess ||
        cudaFuncSetAttribute(bwd_kernel<HD, SMAX, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem) != cudaSuccess)
      return RTE_ERR_LAUNCH;
    set = true;
  }
  const int ctas = B * H * rte::ceil_div(S, QB);
  const dim3 grid(B * H, rte::ceil_div(S, QB), ctas < 148 ? 2 : 1);
  const auto* q16 = reinterpret_cast<const __nv_bfloat16*>(qkv);
  const auto* y16 = reinterpret_cast<const __nv_bfloat16*>(y);
  const auto* dy16 = reinterpret_cast<const __nv_bfloat16*>(dy);
  auto* dq16 = reinterpret_cast<__nv_bfloat16*>(dqkv);
  if (mask_row != nullptr)
    bwd_kernel<HD, SMAX, true><<<grid, NTHR, smem, st>>>(q16, ld, sec, y16, dy16, ldy, lse, dq16, rope, S, H, mask_row, mask_tab);
  else
    bwd_kernel<HD, SMAX, false><<<grid, NTHR, smem, st>>>(q16, ld, sec, y16, dy16, ldy, lse, dq16, rope, S, H, nullptr, nullptr);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

}  // namespace attn_mma
