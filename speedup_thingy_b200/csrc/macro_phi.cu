// The macro operator Phi of the recursive model, forward and backward, on device:
//   out = h + s_cfg * scale * tanh(gain * h + silu(z @ v) @ u + bias),
//   z   = [rmsnorm(h), mean_S rmsnorm(h), h0],  h == h0 on the hot path (the consistency term applies Phi to a state
//   h != h0: the kernels that touch the h0 slice take it as a second pointer `hx`, equal to `h` on the hot path),
// with gain / v / u / bias / scale selected PER SAMPLE by (recipe id, stride id).
//
// The per-sample low-rank weights are small (3d x m and m x d, m <= 64), so these are SIMT kernels
// tiled through shared memory; the weight gather is pointer arithmetic, the concat `z` is never
// materialised (three K-slices; the pooled slice collapses to one m-vector per sample).
// Parameter gradients are produced per sample and then summed per (recipe, stride) key in sample
// order, so results are bitwise reproducible and keys no sample used receive exact zeros.

#include "rte_common.cuh"

namespace {

constexpr int TT = 32;        // tokens per CTA tile
constexpr int NTHR = 256;
constexpr int CH = 64;        // d-chunk staged in shared memory
constexpr int MMAX = 64;      // largest supported macro rank

struct PhiDims { int B, S, d, m, K; };

__device__ __forceinline__ size_t key_of(const int32_t* rid, const int32_t* sid, int b, int K) {
  return (size_t)rid[b] * K + sid[b];
}

// rstd per token, pooled = mean_S(rmsnorm(h0)) per sample, pa = pooled @ v[d:2d, :]
__global__ void __launch_bounds__(NTHR)
phi_prep_kernel(const float* __restrict__ h0, const float* __restrict__ v, const int32_t* __restrict__ rid,
                const int32_t* __restrict__ sid, float* __restrict__ rstd, float* __restrict__ pooled,
                float* __restrict__ pa, PhiDims D, float eps) {
  extern __shared__ float sm[];            // rstd_s[S] then pooled_s[d]
  float* rs = sm;
  float* ps = sm + D.S;
  const int b = blockIdx.x, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* hb = h0 + (size_t)b * D.S * D.d;
  for (int s = warp; s < D.S; s += NTHR / 32) {
    float ss = 0.f;
    for (int c = lane; c < D.d; c += 32) { const float x = hb[(size_t)s * D.d + c]; ss += x * x; }
    ss = rte::warp_sum(ss);
    if (lane == 0) { const float r = rsqrtf(ss / (float)D.d + eps); rs[s] = r; rstd[(size_t)b * D.S + s] = r; }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < D.d; c += NTHR) {
    float acc = 0.f;
    for (int s = 0; s < D.S; ++s) acc += hb[(size_t)s * D.d + c] * rs[s];
    acc /= (float)D.S;
    ps[c] = acc;
    pooled[(size_t)b * D.d + c] = acc;
  }
  __syncthreads();
  const float* v2 = v + (key_of(rid, sid, b, D.K) * 3 * D.d + D.d) * D.m;
  for (int j = warp; j < D.m; j += NTHR / 32) {
    float acc = 0.f;
    for (int c = lane; c < D.d; c += 32) acc += ps[c] * v2[(size_t)c * D.m + j];
    acc = rte::warp_sum(acc);
    if (lane == 0) pa[(size_t)b * D.m + j] = acc;
  }
}

// act[tok, j] = pa[b, j] + sum_c (h0[tok,c] * rstd[tok] * v1[c,j] + hx[tok,c] * v3[c,j])      (hx == h0 on the hot path)
__global__ void __launch_bounds__(NTHR)
phi_act_kernel(const float* __restrict__ h0, const float* __restrict__ hx, const float* __restrict__ rstd,
               const float* __restrict__ pa, const float* __restrict__ v, const int32_t* __restrict__ rid,
               const int32_t* __restrict__ sid, float* __restrict__ act, PhiDims D) {
  __shared__ float sx[TT][CH + 1];
  __shared__ float sv1[CH][MMAX];
  __shared__ float sv3[CH][MMAX];
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* vb = v + key_of(rid, sid, b, D.K) * 3 * D.d * D.m;
  const bool own3 = hx != h0;                        // kernel-uniform
  float acc[4][2], rs[4];
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int s = tok0 + warp * 4 + t;
    rs[t] = (s < D.S) ? rstd[(size_t)b * D.S + s] : 0.f;
#pragma unroll
    for (int q = 0; q < 2; ++q) { const int j = lane + 32 * q; acc[t][q] = (j < D.m) ? pa[(size_t)b * D.m + j] : 0.f; }
  }
  for (int c0 = 0; c0 < D.d; c0 += CH) {
    for (int i = threadIdx.x; i < TT * CH; i += NTHR) {
      const int t = i / CH, c = i % CH, s = tok0 + t;
      sx[t][c] = (s < D.S && c0 + c < D.d) ? h0[((size_t)b * D.S + s) * D.d + c0 + c] : 0.f;
    }
    for (int i = threadIdx.x; i < CH * D.m; i += NTHR) {
      const int c = i / D.m, j = i % D.m;
      const bool ok = c0 + c < D.d;
      sv1[c][j] = ok ? vb[(size_t)(c0 + c) * D.m + j] : 0.f;
      sv3[c][j] = ok ? vb[(size_t)(2 * D.d + c0 + c) * D.m + j] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int c = 0; c < CH; ++c) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int j = lane + 32 * q;
        if (j < D.m) {
          const float w1 = sv1[c][j], w3 = sv3[c][j];
#pragma unroll
          for (int t = 0; t < 4; ++t) { const float x = sx[warp * 4 + t][c]; acc[t][q] += own3 ? x * rs[t] * w1 : x * (rs[t] * w1 + w3); }
        }
      }
    }
    if (own3) {                                    // the v3 slice multiplies the injected state: second sweep over its tile
      __syncthreads();
      for (int i = threadIdx.x; i < TT * CH; i += NTHR) {
        const int t = i / CH, c = i % CH, s = tok0 + t;
        sx[t][c] = (s < D.S && c0 + c < D.d) ? hx[((size_t)b * D.S + s) * D.d + c0 + c] : 0.f;
      }
      __syncthreads();
#pragma unroll 4
      for (int c = 0; c < CH; ++c) {
#pragma unroll
        for (int q = 0; q < 2; ++q) {
          const int j = lane + 32 * q;
          if (j < D.m) {
            const float w3 = sv3[c][j];
#pragma unroll
            for (int t = 0; t < 4; ++t) acc[t][q] += sx[warp * 4 + t][c] * w3;
          }
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int s = tok0 + warp * 4 + t;
    if (s < D.S) {
#pragma unroll
      for (int q = 0; q < 2; ++q) { const int j = lane + 32 * q; if (j < D.m) act[((size_t)b * D.S + s) * D.m + j] = acc[t][q]; }
    }
  }
}

// MODE 0 (forward):  out = h + s_cfg*scale*tanh(gain*h + silu(act) @ u + bias)
// MODE 1 (backward): dupd = dout*s_cfg*scale*(1 - tanh^2);  dh0 = dout + gain*dupd   (dupd -> scratch)
template <int MODE, int MP>
__global__ void __launch_bounds__(NTHR)
phi_out_kernel(const float* __restrict__ h0, const float* __restrict__ act, const float* __restrict__ gain,
               const float* __restrict__ u, const float* __restrict__ bias, const float* __restrict__ scale,
               const int32_t* __restrict__ rid, const int32_t* __restrict__ sid, float s_cfg,
               const float* __restrict__ dout, float* __restrict__ out, float* __restrict__ dupd, PhiDims D) {
  __shared__ float ssa[TT][MMAX];
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const size_t key = key_of(rid, sid, b, D.K);
  for (int i = threadIdx.x; i < TT * MP; i += NTHR) {           // columns past the rank are zero (they meet ur[j] = 0)
    const int t = i / MP, j = i % MP, s = tok0 + t;
    ssa[t][j] = (s < D.S && j < D.m) ? rte::silu_f(act[((size_t)b * D.S + s) * D.m + j]) : 0.f;
  }
  __syncthreads();
  const float* ub = u + key * D.m * D.d;
  for (int c = threadIdx.x; c < D.d; c += NTHR) {
    float ur[MP];                 // MP = macro rank rounded up to 32 or 64
#pragma unroll
    for (int j = 0; j < MP; ++j) ur[j] = (j < D.m) ? ub[(size_t)j * D.d + c] : 0.f;
    const float g = gain[key * D.d + c], bs = bias[key * D.d + c], sc = s_cfg * scale[key * D.d + c];
    const int t_end = min(TT, D.S - tok0);
#pragma unroll 4
    for (int t = 0; t < t_end; ++t) {
      const int s = tok0 + t;
      float low = 0.f;
#pragma unroll
      for (int j = 0; j < MP; ++j) low += ssa[t][j] * ur[j];
      const size_t idx = ((size_t)b * D.S + s) * D.d + c;
      const float h = h0[idx];
      const float th = tanhf(g * h + low + bs);
      if (MODE == 0) {
        out[idx] = h + sc * th;
      } else {
        const float du = dout[idx] * sc * (1.f - th * th);
        dupd[idx] = du;
        out[idx] = dout[idx] + g * du;
      }
    }
  }
}

// da[tok, j] = silu'(act[tok,j]) * sum_c dupd[tok,c] * u[j,c]
__global__ void __launch_bounds__(NTHR)
phi_da_kernel(const float* __restrict__ dupd, const float* __restrict__ act, const float* __restrict__ u,
              const int32_t* __restrict__ rid, const int32_t* __restrict__ sid, float* __restrict__ da, PhiDims D) {
  __shared__ float sd[TT][CH + 1];
  __shared__ float su[MMAX][CH + 1];
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* ub = u + key_of(rid, sid, b, D.K) * D.m * D.d;
  float acc[4][2];
#pragma unroll
  for (int t = 0; t < 4; ++t) acc[t][0] = acc[t][1] = 0.f;
  for (int c0 = 0; c0 < D.d; c0 += CH) {
    for (int i = threadIdx.x; i < TT * CH; i += NTHR) {
      const int t = i / CH, c = i % CH, s = tok0 + t;
      sd[t][c] = (s < D.S && c0 + c < D.d) ? dupd[((size_t)b * D.S + s) * D.d + c0 + c] : 0.f;
    }
    for (int i = threadIdx.x; i < D.m * CH; i += NTHR) {
      const int j = i / CH, c = i % CH;
      su[j][c] = (c0 + c < D.d) ? ub[(size_t)j * D.d + c0 + c] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int c = 0; c < CH; ++c) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int j = lane + 32 * q;
        if (j < D.m) {
          const float w = su[j][c];
#pragma unroll
          for (int t = 0; t < 4; ++t) acc[t][q] += sd[warp * 4 + t][c] * w;
        }
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) {
    const int s = tok0 + warp * 4 + t;
    if (s < D.S) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const int j = lane + 32 * q;
        if (j < D.m) {
          const size_t idx = ((size_t)b * D.S + s) * D.m + j;
          const float a = act[idx], sg = rte::sigmoid_f(a);
          da[idx] = acc[t][q] * sg * (1.f + a * (1.f - sg));
        }
      }
    }
  }
}

// ---- Tensor-core versions of the two data-gradient products (taken when d % 8 == 0): TF32 mma with the 3xTF32
// error compensation, so results stay at fp32 accuracy.
// Operand fragments of mma.m16n8k8 come straight from global memory: a quad of lanes reads 16 contiguous bytes of a
// row and the two k-halves of a step complete the 32-byte sector, so no shared-memory staging (and no barrier) is
// needed; the per-key weights stay in L1/L2.  Warp tile: 16 tokens; a CTA covers TT = 32 tokens of one sample.
__device__ __forceinline__ uint32_t to_tf32(float x) {
  uint32_t r;
  asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
  return r;
}

__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// fp32-accurate product from TF32 pieces: x = hi + lo with both representable in TF32, and
// a*b ~= a_lo*b_hi + a_hi*b_lo + a_hi*b_hi (the dropped lo*lo term is below fp32 rounding).
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = to_tf32(x);
  lo = to_tf32(x - __uint_as_float(hi));
}

__device__ __forceinline__ void mma_3xtf32(float (&c)[4], const uint32_t (&ah)[4], const uint32_t (&al)[4],
                                           const uint32_t (&bh)[2], const uint32_t (&bl)[2]) {
  mma_tf32(c, al, bh);
  mma_tf32(c, ah, bl);
  mma_tf32(c, ah, bh);
}

// Both kernels read their operands with 16-byte loads.  Inside a chunk of 32 reduction indices the mma's logical
// k-slot (step s, slot t or t+4) is mapped to the physical index 8t+s or 8t+4+s: lane t then needs the eight
// consecutive values [8t, 8t+8) of its rows -- two float4 -- and A and B use the same permutation, so the sum is
// unchanged.
struct Frag8 { float4 lo, hi; };     // physical indices 8t..8t+3 and 8t+4..8t+7 of one row
__device__ __forceinline__ Frag8 load8(const float* p, bool ok) {
  Frag8 f;
  if (ok) { f.lo = *reinterpret_cast<const float4*>(p); f.hi = *reinterpret_cast<const float4*>(p + 4); }
  else { f.lo = make_float4(0.f, 0.f, 0.f, 0.f); f.hi = f.lo; }
  return f;
}
__device__ __forceinline__ float pick(const float4& v, int s) { return s == 0 ? v.x : s == 1 ? v.y : s == 2 ? v.z : v.w; }

// da[tok, j] = silu'(act[tok,j]) * sum_c dupd[tok,c] * u[j,c]:  M = tokens, N = rank, K = d  (d % 32 == 0).
// Eight warps = 2 token tiles x 4 column groups; group ng owns rank columns [8ng, 8ng+8) and [8ng+32, 8ng+40).
__global__ void __launch_bounds__(NTHR)
phi_da_mma_kernel(const float* __restrict__ dupd, const float* __restrict__ act, const float* __restrict__ u,
                  const int32_t* __restrict__ rid, const int32_t* __restrict__ sid, float* __restrict__ da, PhiDims D) {
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int mt = warp & 1, ng = warp >> 1;
  const int n_tiles = rte::ceil_div(D.m, 8);
  if (ng >= n_tiles) return;                         // warp-uniform; the kernel has no barrier
  const bool two = ng + 4 < n_tiles;
  const float* ub = u + key_of(rid, sid, b, D.K) * D.m * D.d;
  const int r0 = tok0 + mt * 16 + g, r1 = r0 + 8;
  const bool ok0 = r0 < D.S, ok1 = r1 < D.S;
  const float* a0p = dupd + ((size_t)b * D.S + (ok0 ? r0 : 0)) * D.d + 8 * t;
  const float* a1p = dupd + ((size_t)b * D.S + (ok1 ? r1 : 0)) * D.d + 8 * t;
  const int j0 = ng * 8 + g, j1 = j0 + 32;
  const bool okb0 = j0 < D.m, okb1 = two && j1 < D.m;
  const float* b0p = ub + (size_t)(okb0 ? j0 : 0) * D.d + 8 * t;
  const float* b1p = ub + (size_t)(okb1 ? j1 : 0) * D.d + 8 * t;
  float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
  for (int k0 = 0; k0 < D.d; k0 += 32) {
    const Frag8 x0 = load8(a0p + k0, ok0), x1 = load8(a1p + k0, ok1);
    const Frag8 w0 = load8(b0p + k0, okb0);
    Frag8 w1;
    if (two) w1 = load8(b1p + k0, okb1);
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      uint32_t a[4], al[4], f[2], fl[2];
      split_tf32(pick(x0.lo, s), a[0], al[0]);
      split_tf32(pick(x1.lo, s), a[1], al[1]);
      split_tf32(pick(x0.hi, s), a[2], al[2]);
      split_tf32(pick(x1.hi, s), a[3], al[3]);
      split_tf32(pick(w0.lo, s), f[0], fl[0]);
      split_tf32(pick(w0.hi, s), f[1], fl[1]);
      mma_3xtf32(c0, a, al, f, fl);
      if (two) {
        split_tf32(pick(w1.lo, s), f[0], fl[0]);
        split_tf32(pick(w1.hi, s), f[1], fl[1]);
        mma_3xtf32(c1, a, al, f, fl);
      }
    }
  }
  auto put = [&](int row, int col, float x) {
    if (row < D.S && col < D.m) {
      const size_t idx = ((size_t)b * D.S + row) * D.m + col;
      const float av = act[idx], sg = rte::sigmoid_f(av);
      da[idx] = x * sg * (1.f + av * (1.f - sg));
    }
  };
  const int col0 = ng * 8 + 2 * t;
  put(r0, col0, c0[0]); put(r0, col0 + 1, c0[1]); put(r1, col0, c0[2]); put(r1, col0 + 1, c0[3]);
  if (two) { put(r0, col0 + 32, c1[0]); put(r0, col0 + 33, c1[1]); put(r1, col0 + 32, c1[2]); put(r1, col0 + 33, c1[3]); }
}

// ---- Forward products on tensor cores.  They need the reduction index contiguous per output column, i.e. the
// TRANSPOSED parameters: wt = vt [m][keys*3d] (vt[j][key*3d + c] = v[key][c][j]) followed by
// ut [d][keys*m] (ut[c][key*m + j] = u[key][j][c]), refreshed once per step by rte_macro_phi_prepare.

// act[tok, j] = pa[b, j] + rstd[tok] * (h0 @ v1)[tok, j] + (hx @ v3)[tok, j]:  M = tokens, N = rank, K = d (d % 32 == 0).
// Same warp layout as phi_da_mma_kernel; two accumulators per rank tile (with hx == h0, the hot path, the v1 and v3
// slices share the A fragments; otherwise the v3 slice gets fragments of its own).
template <bool OWN3>
__global__ void __launch_bounds__(NTHR)
phi_act_mma_kernel(const float* __restrict__ h0, const float* __restrict__ hx, const float* __restrict__ rstd,
                   const float* __restrict__ pa, const float* __restrict__ vt, long long vt_ld,
                   const int32_t* __restrict__ rid, const int32_t* __restrict__ sid, float* __restrict__ act, PhiDims D) {
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int mt = warp & 1, ng = warp >> 1;
  const int n_tiles = rte::ceil_div(D.m, 8);
  if (ng >= n_tiles) return;                         // warp-uniform; the kernel has no barrier
  const bool two = ng + 4 < n_tiles;
  const size_t koff = key_of(rid, sid, b, D.K) * 3 * D.d;
  const int r0 = tok0 + mt * 16 + g, r1 = r0 + 8;
  const bool ok0 = r0 < D.S, ok1 = r1 < D.S;
  const float* a0p = h0 + ((size_t)b * D.S + (ok0 ? r0 : 0)) * D.d + 8 * t;
  const float* a1p = h0 + ((size_t)b * D.S + (ok1 ? r1 : 0)) * D.d + 8 * t;
  // OWN3: hx is a different tensor than h0 (a compile-time switch: the hot path keeps its register footprint)
  const float* x0p = hx + ((size_t)b * D.S + (ok0 ? r0 : 0)) * D.d + 8 * t;
  const float* x1p = hx + ((size_t)b * D.S + (ok1 ? r1 : 0)) * D.d + 8 * t;
  const int j0 = ng * 8 + g, j1 = j0 + 32;
  const bool okb0 = j0 < D.m, okb1 = two && j1 < D.m;
  const float* b0p = vt + (size_t)(okb0 ? j0 : 0) * vt_ld + koff + 8 * t;
  const float* b1p = vt + (size_t)(okb1 ? j1 : 0) * vt_ld + koff + 8 * t;
  float p1[2][4], p3[2][4];
#pragma unroll
  for (int q = 0; q < 2; ++q)
#pragma unroll
    for (int e = 0; e < 4; ++e) p1[q][e] = p3[q][e] = 0.f;
#pragma unroll 2
  for (int k0 = 0; k0 < D.d; k0 += 32) {
    const Frag8 x0 = load8(a0p + k0, ok0), x1 = load8(a1p + k0, ok1);
    Frag8 z0 = x0, z1 = x1;                          // A operand of the v3 slice
    if constexpr (OWN3) { z0 = load8(x0p + k0, ok0); z1 = load8(x1p + k0, ok1); }
    const Frag8 w1 = load8(b0p + k0, okb0), w3 = load8(b0p + 2 * D.d + k0, okb0);
    Frag8 y1, y3;
    if (two) { y1 = load8(b1p + k0, okb1); y3 = load8(b1p + 2 * D.d + k0, okb1); }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      uint32_t a[4], al[4], c[4], cl[4], f[2], fl[2];
      split_tf32(pick(x0.lo, s), a[0], al[0]);
      split_tf32(pick(x1.lo, s), a[1], al[1]);
      split_tf32(pick(x0.hi, s), a[2], al[2]);
      split_tf32(pick(x1.hi, s), a[3], al[3]);
      if constexpr (OWN3) {
        split_tf32(pick(z0.lo, s), c[0], cl[0]);
        split_tf32(pick(z1.lo, s), c[1], cl[1]);
        split_tf32(pick(z0.hi, s), c[2], cl[2]);
        split_tf32(pick(z1.hi, s), c[3], cl[3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) { c[e] = a[e]; cl[e] = al[e]; }
      }
      split_tf32(pick(w1.lo, s), f[0], fl[0]);
      split_tf32(pick(w1.hi, s), f[1], fl[1]);
      mma_3xtf32(p1[0], a, al, f, fl);
      split_tf32(pick(w3.lo, s), f[0], fl[0]);
      split_tf32(pick(w3.hi, s), f[1], fl[1]);
      mma_3xtf32(p3[0], c, cl, f, fl);
      if (two) {
        split_tf32(pick(y1.lo, s), f[0], fl[0]);
        split_tf32(pick(y1.hi, s), f[1], fl[1]);
        mma_3xtf32(p1[1], a, al, f, fl);
        split_tf32(pick(y3.lo, s), f[0], fl[0]);
        split_tf32(pick(y3.hi, s), f[1], fl[1]);
        mma_3xtf32(p3[1], c, cl, f, fl);
      }
    }
  }
  const float rs0 = ok0 ? rstd[(size_t)b * D.S + r0] : 0.f, rs1 = ok1 ? rstd[(size_t)b * D.S + r1] : 0.f;
  auto put = [&](int row, int col, float rs, float a1v, float a3v) {
    if (row < D.S && col < D.m) act[((size_t)b * D.S + row) * D.m + col] = pa[(size_t)b * D.m + col] + rs * a1v + a3v;
  };
#pragma unroll
  for (int q = 0; q < 2; ++q) {
    if (q == 1 && !two) break;
    const int col0 = ng * 8 + 2 * t + 32 * q;
    put(r0, col0, rs0, p1[q][0], p3[q][0]); put(r0, col0 + 1, rs0, p1[q][1], p3[q][1]);
    put(r1, col0, rs1, p1[q][2], p3[q][2]); put(r1, col0 + 1, rs1, p1[q][3], p3[q][3]);
  }
}

// MODE 0 (forward):  out = h + s_cfg*scale*tanh(gain*h + silu(act) @ u + bias)
// MODE 1 (backward): dupd = dout*s_cfg*scale*(1 - tanh^2);  out (= dh0) = dout + gain*dupd
// M = tokens, N = d, K = rank (d % 32 == 0, rank % 4 == 0); warp layout, operand permutations and float4 epilogue
// as in phi_dz_mma_kernel; the A operand is silu(act) of the warp's 16 tokens, held in registers.
template <int MODE, int KC>
__global__ void __launch_bounds__(NTHR, KC == 1 ? 2 : 1)
phi_out_mma_kernel(const float* __restrict__ h0, const float* __restrict__ act, const float* __restrict__ gain,
                   const float* __restrict__ ut, long long ut_ld, const float* __restrict__ bias,
                   const float* __restrict__ scale, const int32_t* __restrict__ rid, const int32_t* __restrict__ sid,
                   float s_cfg, const float* __restrict__ dout, float* __restrict__ out, float* __restrict__ dupd, PhiDims D) {
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int mt = warp & 1, cq = warp >> 1;
  const size_t key = key_of(rid, sid, b, D.K);
  const float* ub = ut + key * D.m;                 // row c of this key's u^T: ub + c * ut_ld
  const int r0 = tok0 + mt * 16 + g, r1 = r0 + 8;
  const bool ok0 = r0 < D.S, ok1 = r1 < D.S;
  const size_t row0 = (size_t)b * D.S + (ok0 ? r0 : 0), row1 = (size_t)b * D.S + (ok1 ? r1 : 0);
  uint32_t ah[KC][4][4], al[KC][4][4];
#pragma unroll
  for (int ch = 0; ch < KC; ++ch) {
    const int k = 32 * ch + 8 * t;
    Frag8 y0 = load8(act + row0 * D.m + k, ok0 && k + 8 <= D.m), y1 = load8(act + row1 * D.m + k, ok1 && k + 8 <= D.m);
    if (k < D.m && k + 8 > D.m) {
      if (ok0) y0.lo = *reinterpret_cast<const float4*>(act + row0 * D.m + k);
      if (ok1) y1.lo = *reinterpret_cast<const float4*>(act + row1 * D.m + k);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      const bool in_lo = k + s < D.m, in_hi = k + 4 + s < D.m;      // silu(0) = 0 anyway; keep padded slots exact zeros
      split_tf32(in_lo ? rte::silu_f(pick(y0.lo, s)) : 0.f, ah[ch][s][0], al[ch][s][0]);
      split_tf32(in_lo ? rte::silu_f(pick(y1.lo, s)) : 0.f, ah[ch][s][1], al[ch][s][1]);
      split_tf32(in_hi ? rte::silu_f(pick(y0.hi, s)) : 0.f, ah[ch][s][2], al[ch][s][2]);
      split_tf32(in_hi ? rte::silu_f(pick(y1.hi, s)) : 0.f, ah[ch][s][3], al[ch][s][3]);
    }
  }
  const int n_blocks = D.d / 32;
  const int pc0 = 8 * (g >> 1) + (g & 1);
  const float* gk = gain + key * D.d;
  const float* bk = bias + key * D.d;
  const float* sk = scale + key * D.d;
  for (int nb = cq; nb < n_blocks; nb += 4) {
    const int cb = nb * 32, col = cb + 8 * t;
    float c[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
      const float* wr = ub + (size_t)(cb + pc0 + 2 * j) * ut_ld;
#pragma unroll
      for (int ch = 0; ch < KC; ++ch) {
        const int k = 32 * ch + 8 * t;
        Frag8 f = load8(wr + k, k + 8 <= D.m);
        if (k < D.m && k + 8 > D.m) f.lo = *reinterpret_cast<const float4*>(wr + k);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          uint32_t fh[2], fl[2];
          split_tf32(pick(f.lo, s), fh[0], fl[0]);
          split_tf32(pick(f.hi, s), fh[1], fl[1]);
          mma_3xtf32(c[j], ah[ch][s], al[ch][s], fh, fl);
        }
      }
    }
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!(half ? ok1 : ok0)) continue;
      const size_t row = half ? row1 : row0;
      const float low[8] = {c[0][2 * half], c[0][2 * half + 1], c[1][2 * half], c[1][2 * half + 1],
                            c[2][2 * half], c[2][2 * half + 1], c[3][2 * half], c[3][2 * half + 1]};
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        const size_t idx = row * D.d + col + 4 * q;
        const float4 h = *reinterpret_cast<const float4*>(h0 + idx);
        const float4 gv = *reinterpret_cast<const float4*>(gk + col + 4 * q);
        const float4 bv = *reinterpret_cast<const float4*>(bk + col + 4 * q);
        float4 sc = *reinterpret_cast<const float4*>(sk + col + 4 * q);
        sc.x *= s_cfg; sc.y *= s_cfg; sc.z *= s_cfg; sc.w *= s_cfg;
        const float t0 = tanhf(gv.x * h.x + low[4 * q] + bv.x), t1 = tanhf(gv.y * h.y + low[4 * q + 1] + bv.y);
        const float t2 = tanhf(gv.z * h.z + low[4 * q + 2] + bv.z), t3 = tanhf(gv.w * h.w + low[4 * q + 3] + bv.w);
        if (MODE == 0) {
          *reinterpret_cast<float4*>(out + idx) = make_float4(h.x + sc.x * t0, h.y + sc.y * t1, h.z + sc.z * t2, h.w + sc.w * t3);
        } else {
          const float4 dv = *reinterpret_cast<const float4*>(dout + idx);
          const float4 du = make_float4(dv.x * sc.x * (1.f - t0 * t0), dv.y * sc.y * (1.f - t1 * t1),
                                        dv.z * sc.z * (1.f - t2 * t2), dv.w * sc.w * (1.f - t3 * t3));
          *reinterpret_cast<float4*>(dupd + idx) = du;
          *reinterpret_cast<float4*>(out + idx) = make_float4(dv.x + gv.x * du.x, dv.y + gv.y * du.y, dv.z + gv.z * du.z, dv.w + gv.w * du.w);
        }
      }
    }
  }
}

// Per-sample parameter gradients of u, gain, bias:  pu[b][j,c], pg[b][c], pb[b][c].
__global__ void __launch_bounds__(NTHR)
phi_pu_kernel(const float* __restrict__ h0, const float* __restrict__ act, const float* __restrict__ dupd,
              float* __restrict__ pu, float* __restrict__ pg, float* __restrict__ pb, PhiDims D) {
  extern __shared__ float ssa[];     // [S][m]
  const int cblocks = rte::ceil_div(D.d, NTHR);
  const int b = blockIdx.x / cblocks, c = (blockIdx.x % cblocks) * NTHR + threadIdx.x;
  for (int i = threadIdx.x; i < D.S * D.m; i += NTHR) ssa[i] = rte::silu_f(act[(size_t)b * D.S * D.m + i]);
  __syncthreads();
  if (c >= D.d) return;
  float au[MMAX];
#pragma unroll
  for (int j = 0; j < MMAX; ++j) au[j] = 0.f;
  float ag = 0.f, ab = 0.f;
  if (D.m % 4 == 0) {                 // four ranks per shared-memory read
    const int m4 = D.m >> 2;
#pragma unroll 2
    for (int s = 0; s < D.S; ++s) {
      const size_t idx = ((size_t)b * D.S + s) * D.d + c;
      const float du = dupd[idx];
      ag += du * h0[idx];
      ab += du;
      const float4* row = reinterpret_cast<const float4*>(ssa + s * D.m);
#pragma unroll
      for (int j4 = 0; j4 < MMAX / 4; ++j4) {
        if (j4 < m4) {
          const float4 sv = row[j4];
          au[4 * j4] += sv.x * du; au[4 * j4 + 1] += sv.y * du; au[4 * j4 + 2] += sv.z * du; au[4 * j4 + 3] += sv.w * du;
        }
      }
    }
  } else {
    for (int s = 0; s < D.S; ++s) {
      const size_t idx = ((size_t)b * D.S + s) * D.d + c;
      const float du = dupd[idx];
      ag += du * h0[idx];
      ab += du;
#pragma unroll
      for (int j = 0; j < MMAX; ++j) if (j < D.m) au[j] += ssa[s * D.m + j] * du;
    }
  }
  pg[(size_t)b * D.d + c] = ag;
  pb[(size_t)b * D.d + c] = ab;
#pragma unroll
  for (int j = 0; j < MMAX; ++j) if (j < D.m) pu[((size_t)b * D.m + j) * D.d + c] = au[j];
}

// Per-sample gradient of v:  pv[b][c', j] for c' in [0, 3d):
//   c' <  d  : sum_s h0[s,c]*rstd[s] * da[s,j]
//   c' < 2d  : pooled[b,c] * sum_s da[s,j]
//   else     : sum_s hx[s,c] * da[s,j]          (hx == h0 on the hot path)
constexpr int PV_ROWS = 32;       // rows of v per CTA (one 128-byte line of h0 per token)

__global__ void __launch_bounds__(NTHR)
phi_pv_kernel(const float* __restrict__ h0, const float* __restrict__ hx, const float* __restrict__ rstd,
              const float* __restrict__ pooled, const float* __restrict__ da, float* __restrict__ pv, PhiDims D) {
  extern __shared__ float sm[];      // sda[S][m], rs[S], sx[S][PV_ROWS], sx3[S][PV_ROWS]
  float* sda = sm;
  float* rs = sm + D.S * D.m;
  float* sx = rs + D.S;
  float* sx3 = sx + D.S * PV_ROWS;
  constexpr int ROWS = PV_ROWS;
  const int rblocks = rte::ceil_div(D.d, ROWS);
  const int b = blockIdx.x / rblocks, c0 = (blockIdx.x % rblocks) * ROWS;
  for (int i = threadIdx.x; i < D.S * D.m; i += NTHR) sda[i] = da[(size_t)b * D.S * D.m + i];
  for (int i = threadIdx.x; i < D.S; i += NTHR) rs[i] = rstd[(size_t)b * D.S + i];
  for (int i = threadIdx.x; i < D.S * ROWS; i += NTHR) {
    const int s = i / ROWS, r = i % ROWS;
    sx[i] = (c0 + r < D.d) ? h0[((size_t)b * D.S + s) * D.d + c0 + r] : 0.f;
    sx3[i] = (c0 + r < D.d) ? hx[((size_t)b * D.S + s) * D.d + c0 + r] : 0.f;
  }
  __syncthreads();
  float* pvb = pv + (size_t)b * 3 * D.d * D.m;
  for (int o = threadIdx.x; o < ROWS * D.m; o += NTHR) {
    const int r = o / D.m, j = o % D.m, c = c0 + r;
    if (c >= D.d) continue;
    float a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int s = 0; s < D.S; ++s) {
      const float dv = sda[s * D.m + j], x = sx[s * ROWS + r];
      a1 += x * rs[s] * dv;
      a2 += dv;
      a3 += sx3[s * ROWS + r] * dv;
    }
    pvb[(size_t)c * D.m + j] = a1;
    pvb[(size_t)(D.d + c) * D.m + j] = pooled[(size_t)b * D.d + c] * a2;
    pvb[(size_t)(2 * D.d + c) * D.m + j] = a3;
  }
}

// sda[b, j] = sum_s da[b,s,j]  ->  dpool[b, c] = (1/S) * sum_j sda[b,j] * v2[c,j]
__global__ void __launch_bounds__(NTHR)
phi_dpool_kernel(const float* __restrict__ da, const float* __restrict__ v, const int32_t* __restrict__ rid,
                 const int32_t* __restrict__ sid, float* __restrict__ dpool, PhiDims D) {
  __shared__ float ssum[MMAX];
  const int b = blockIdx.x;
  for (int j = threadIdx.x; j < D.m; j += NTHR) {
    float a = 0.f;
    for (int s = 0; s < D.S; ++s) a += da[((size_t)b * D.S + s) * D.m + j];
    ssum[j] = a;
  }
  __syncthreads();
  const float* v2 = v + (key_of(rid, sid, b, D.K) * 3 * D.d + D.d) * D.m;
  for (int c = threadIdx.x; c < D.d; c += NTHR) {
    float a = 0.f;
    for (int j = 0; j < D.m; ++j) a += ssum[j] * v2[(size_t)c * D.m + j];
    dpool[(size_t)b * D.d + c] = a / (float)D.S;
  }
}

// dhx[tok,:] += da @ v3^T;  dh0[tok,:] += rmsnorm_backward(da @ v1^T + dpool[b,:])     (one warp per token; dhx may be dh0)
__global__ void __launch_bounds__(NTHR)
phi_dz_kernel(const float* __restrict__ h0, const float* __restrict__ rstd, const float* __restrict__ da,
              const float* __restrict__ dpool, const float* __restrict__ v, const int32_t* __restrict__ rid,
              const int32_t* __restrict__ sid, float* dh0, float* dhx, PhiDims D) {
  __shared__ float sv1[CH][MMAX + 1];
  __shared__ float sv3[CH][MMAX + 1];
  __shared__ float sda[TT][MMAX];
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* vb = v + key_of(rid, sid, b, D.K) * 3 * D.d * D.m;
  for (int i = threadIdx.x; i < TT * D.m; i += NTHR) {
    const int t = i / D.m, j = i % D.m, s = tok0 + t;
    sda[t][j] = (s < D.S) ? da[((size_t)b * D.S + s) * D.m + j] : 0.f;
  }
  // pass 1: dh0 += da @ v3^T and the row dot products <dn, xhat>; pass 2 recomputes dn per chunk
  float dot[4] = {0.f, 0.f, 0.f, 0.f};
  const int nchunks = rte::ceil_div(D.d, CH);
  for (int ch = 0; ch < nchunks; ++ch) {
    const int c0 = ch * CH;
    __syncthreads();
    for (int i = threadIdx.x; i < CH * D.m; i += NTHR) {
      const int c = i / D.m, j = i % D.m;
      const bool ok = c0 + c < D.d;
      sv1[c][j] = ok ? vb[(size_t)(c0 + c) * D.m + j] : 0.f;
      sv3[c][j] = ok ? vb[(size_t)(2 * D.d + c0 + c) * D.m + j] : 0.f;
    }
    __syncthreads();
    float a1[4][2], a3[4][2];
#pragma unroll
    for (int t = 0; t < 4; ++t) a1[t][0] = a1[t][1] = a3[t][0] = a3[t][1] = 0.f;
#pragma unroll 4
    for (int j = 0; j < D.m; ++j) {
      const float w1a = sv1[lane][j], w1b = sv1[lane + 32][j], w3a = sv3[lane][j], w3b = sv3[lane + 32][j];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float dv = sda[warp * 4 + t][j];
        a1[t][0] += dv * w1a; a1[t][1] += dv * w1b;
        a3[t][0] += dv * w3a; a3[t][1] += dv * w3b;
      }
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int cl = lane + 32 * q, c = c0 + cl;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int s = tok0 + warp * 4 + t;
        if (s < D.S && c < D.d) {
          const size_t idx = ((size_t)b * D.S + s) * D.d + c;
          const float dnv = a1[t][q] + dpool[(size_t)b * D.d + c];
          dhx[idx] += a3[t][q];
          dot[t] += dnv * h0[idx] * rstd[(size_t)b * D.S + s];
        }
      }
    }
  }
#pragma unroll
  for (int t = 0; t < 4; ++t) dot[t] = rte::warp_sum(dot[t]) / (float)D.d;
  // second pass: recompute dn per chunk and finish dx = rstd * (dn - xhat * dot)
  for (int ch = 0; ch < nchunks; ++ch) {
    const int c0 = ch * CH;
    __syncthreads();
    for (int i = threadIdx.x; i < CH * D.m; i += NTHR) {
      const int c = i / D.m, j = i % D.m;
      sv1[c][j] = (c0 + c < D.d) ? vb[(size_t)(c0 + c) * D.m + j] : 0.f;
    }
    __syncthreads();
    float a1[4][2];
#pragma unroll
    for (int t = 0; t < 4; ++t) a1[t][0] = a1[t][1] = 0.f;
#pragma unroll 4
    for (int j = 0; j < D.m; ++j) {
      const float w1a = sv1[lane][j], w1b = sv1[lane + 32][j];
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const float dv = sda[warp * 4 + t][j];
        a1[t][0] += dv * w1a; a1[t][1] += dv * w1b;
      }
    }
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const int cl = lane + 32 * q, c = c0 + cl;
#pragma unroll
      for (int t = 0; t < 4; ++t) {
        const int s = tok0 + warp * 4 + t;
        if (s < D.S && c < D.d) {
          const size_t idx = ((size_t)b * D.S + s) * D.d + c;
          const float r = rstd[(size_t)b * D.S + s];
          const float dnv = a1[t][q] + dpool[(size_t)b * D.d + c];
          dh0[idx] += r * (dnv - h0[idx] * r * dot[t]);
        }
      }
    }
  }
}

// dhx[tok,:] += da @ v3^T;  dh0[tok,:] += rmsnorm_backward(da @ v1^T + dpool[b,:])  (dhx may be dh0):  M = tokens, N = d,
// K = rank (tensor-core form;
// d % 32 == 0, rank % 4 == 0).  Eight warps = 2 token tiles x 4 column groups; a group takes 32-column blocks
// cq, cq+4, ...  The A operand (16 tokens x rank) lives in registers (KC chunks of 32 rank indices, permuted as
// above).  Output columns are permuted too: mma tile j of a block holds, for lane t, the physical columns
// 8t+2j and 8t+2j+1, so a lane owns the eight consecutive columns [8t, 8t+8) of its two rows and the epilogue moves
// float4.  Pass 1 forms the row dot products <dn, xhat>; pass 2 recomputes the small products and finishes with one
// read-modify-write of dh0.
template <int KC>
__global__ void __launch_bounds__(NTHR, KC == 1 ? 2 : 1)
phi_dz_mma_kernel(const float* __restrict__ h0, const float* __restrict__ rstd, const float* __restrict__ da,
                  const float* __restrict__ dpool, const float* __restrict__ v, const int32_t* __restrict__ rid,
                  const int32_t* __restrict__ sid, float* dh0, float* dhx, PhiDims D) {
  __shared__ float sdot[TT][4];
  const int tiles = rte::ceil_div(D.S, TT);
  const int b = blockIdx.x / tiles, tok0 = (blockIdx.x % tiles) * TT;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;
  const int mt = warp & 1, cq = warp >> 1;
  const float* v1 = v + key_of(rid, sid, b, D.K) * 3 * D.d * D.m;
  const float* v3 = v1 + (size_t)2 * D.d * D.m;
  const int r0 = tok0 + mt * 16 + g, r1 = r0 + 8;
  const bool ok0 = r0 < D.S, ok1 = r1 < D.S;
  const size_t row0 = (size_t)b * D.S + (ok0 ? r0 : 0), row1 = (size_t)b * D.S + (ok1 ? r1 : 0);
  uint32_t ah[KC][4][4], al[KC][4][4];          // [chunk][k-step][fragment register]
#pragma unroll
  for (int ch = 0; ch < KC; ++ch) {
    const int k = 32 * ch + 8 * t;
    const bool in = k < D.m;                     // rank % 4 == 0 and 8-wide pieces: guard each half
    const Frag8 x0 = load8(da + row0 * D.m + k, ok0 && in && k + 8 <= D.m);
    const Frag8 x1 = load8(da + row1 * D.m + k, ok1 && in && k + 8 <= D.m);
    Frag8 y0 = x0, y1 = x1;
    if (in && k + 8 > D.m) {                     // only the first four of the eight exist
      if (ok0) y0.lo = *reinterpret_cast<const float4*>(da + row0 * D.m + k);
      if (ok1) y1.lo = *reinterpret_cast<const float4*>(da + row1 * D.m + k);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      split_tf32(pick(y0.lo, s), ah[ch][s][0], al[ch][s][0]);
      split_tf32(pick(y1.lo, s), ah[ch][s][1], al[ch][s][1]);
      split_tf32(pick(y0.hi, s), ah[ch][s][2], al[ch][s][2]);
      split_tf32(pick(y1.hi, s), ah[ch][s][3], al[ch][s][3]);
    }
  }
  const float rs0 = ok0 ? rstd[row0] : 0.f, rs1 = ok1 ? rstd[row1] : 0.f;
  const int n_blocks = D.d / 32;
  const float* dpb = dpool + (size_t)b * D.d;
  // rows of v this lane loads for mma tile j of a 32-column block: physical column 8*(g>>1) + 2j + (g&1)
  const int pc0 = 8 * (g >> 1) + (g & 1);

  auto product = [&](const float* w, int cb, float (&c)[4][4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      c[j][0] = c[j][1] = c[j][2] = c[j][3] = 0.f;
      const float* wr = w + (size_t)(cb + pc0 + 2 * j) * D.m;
#pragma unroll
      for (int ch = 0; ch < KC; ++ch) {
        const int k = 32 * ch + 8 * t;
        Frag8 f = load8(wr + k, k + 8 <= D.m);
        if (k < D.m && k + 8 > D.m) f.lo = *reinterpret_cast<const float4*>(wr + k);
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          uint32_t fh[2], fl[2];
          split_tf32(pick(f.lo, s), fh[0], fl[0]);
          split_tf32(pick(f.hi, s), fh[1], fl[1]);
          mma_3xtf32(c[j], ah[ch][s], al[ch][s], fh, fl);
        }
      }
    }
  };
  // the lane's eight consecutive columns of row 0 / row 1 as two float4 each
  auto row_vals = [](const float (&c)[4][4], int half, float4& lo, float4& hi) {
    lo = make_float4(c[0][2 * half], c[0][2 * half + 1], c[1][2 * half], c[1][2 * half + 1]);
    hi = make_float4(c[2][2 * half], c[2][2 * half + 1], c[3][2 * half], c[3][2 * half + 1]);
  };
  auto dot4 = [](const float4& a, const float4& p, const float4& x) {
    return (a.x + p.x) * x.x + (a.y + p.y) * x.y + (a.z + p.z) * x.z + (a.w + p.w) * x.w;
  };

  float dot0 = 0.f, dot1 = 0.f;
  for (int nb = cq; nb < n_blocks; nb += 4) {
    const int cb = nb * 32, col = cb + 8 * t;
    float c1[4][4];
    product(v1, cb, c1);
    const float4 dpa = *reinterpret_cast<const float4*>(dpb + col), dpc = *reinterpret_cast<const float4*>(dpb + col + 4);
    float4 lo, hi;
    if (ok0) {
      row_vals(c1, 0, lo, hi);
      const float4 ha = *reinterpret_cast<const float4*>(h0 + row0 * D.d + col), hb = *reinterpret_cast<const float4*>(h0 + row0 * D.d + col + 4);
      dot0 += (dot4(lo, dpa, ha) + dot4(hi, dpc, hb)) * rs0;
    }
    if (ok1) {
      row_vals(c1, 1, lo, hi);
      const float4 ha = *reinterpret_cast<const float4*>(h0 + row1 * D.d + col), hb = *reinterpret_cast<const float4*>(h0 + row1 * D.d + col + 4);
      dot1 += (dot4(lo, dpa, ha) + dot4(hi, dpc, hb)) * rs1;
    }
  }
  dot0 += __shfl_xor_sync(0xffffffffu, dot0, 1); dot0 += __shfl_xor_sync(0xffffffffu, dot0, 2);
  dot1 += __shfl_xor_sync(0xffffffffu, dot1, 1); dot1 += __shfl_xor_sync(0xffffffffu, dot1, 2);
  if (t == 0) { sdot[mt * 16 + g][cq] = dot0; sdot[mt * 16 + g + 8][cq] = dot1; }
  __syncthreads();
  {
    const float* q0 = sdot[mt * 16 + g];
    const float* q1 = sdot[mt * 16 + g + 8];
    dot0 = (q0[0] + q0[1] + q0[2] + q0[3]) / (float)D.d;
    dot1 = (q1[0] + q1[1] + q1[2] + q1[3]) / (float)D.d;
  }
  const bool own3 = dhx != dh0;                      // kernel-uniform: the v3 slice's gradient has a buffer of its own
  auto finish = [&](float4& o, const float4& a1v, const float4& a3v, const float4& dp, const float4& hv, float rs, float dot) {
    o.x += a3v.x + rs * ((a1v.x + dp.x) - hv.x * rs * dot);
    o.y += a3v.y + rs * ((a1v.y + dp.y) - hv.y * rs * dot);
    o.z += a3v.z + rs * ((a1v.z + dp.z) - hv.z * rs * dot);
    o.w += a3v.w + rs * ((a1v.w + dp.w) - hv.w * rs * dot);
  };
  const float4 zero4 = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int nb = cq; nb < n_blocks; nb += 4) {
    const int cb = nb * 32, col = cb + 8 * t;
    float c1[4][4], c3[4][4];
    product(v1, cb, c1);
    product(v3, cb, c3);
    const float4 dpa = *reinterpret_cast<const float4*>(dpb + col), dpc = *reinterpret_cast<const float4*>(dpb + col + 4);
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const bool ok = half ? ok1 : ok0;
      if (!ok) continue;
      const size_t row = half ? row1 : row0;
      const float rs = half ? rs1 : rs0, dot = half ? dot1 : dot0;
      float4 l1, h1, l3, h3;
      row_vals(c1, half, l1, h1);
      row_vals(c3, half, l3, h3);
      const float4 ha = *reinterpret_cast<const float4*>(h0 + row * D.d + col), hb = *reinterpret_cast<const float4*>(h0 + row * D.d + col + 4);
      float4* q = reinterpret_cast<float4*>(dh0 + row * D.d + col);
      float4 oa = q[0], ob = q[1];
      finish(oa, l1, own3 ? zero4 : l3, dpa, ha, rs, dot);
      finish(ob, h1, own3 ? zero4 : h3, dpc, hb, rs, dot);
      q[0] = oa; q[1] = ob;
      if (own3) {
        float4* qx = reinterpret_cast<float4*>(dhx + row * D.d + col);
        float4 xa = qx[0], xb = qx[1];
        xa.x += l3.x; xa.y += l3.y; xa.z += l3.z; xa.w += l3.w;
        xb.x += h3.x; xb.y += h3.y; xb.z += h3.z; xb.w += h3.w;
        qx[0] = xa; qx[1] = xb;
      }
    }
  }
}

// out[key][e] = sum over samples b with key(b) == key, in sample order, of partial[b][e]   (blockIdx.y = key)
__global__ void __launch_bounds__(NTHR)
phi_reduce_keys_kernel(const float* __restrict__ partial, const int32_t* __restrict__ rid, const int32_t* __restrict__ sid,
                       float* __restrict__ out, int B, int K, long long elems) {
  __shared__ int members[1024];
  __shared__ int n_members;
  const int key = blockIdx.y;
  if (threadIdx.x == 0) {
    int n = 0;
    for (int b = 0; b < B && n < 1024; ++b)
      if (rid[b] * K + sid[b] == key) members[n++] = b;
    n_members = n;
  }
  __syncthreads();
  const long long e = blockIdx.x * (long long)NTHR + threadIdx.x;
  if (e >= elems) return;
  float acc = 0.f;
  const int n = n_members;
#pragma unroll 4
  for (int i = 0; i < n; ++i) acc += partial[(size_t)members[i] * elems + e];
  out[(size_t)key * elems + e] = acc;
}

// Mean-squared-error pieces of the consistency term (macro.py:359): g[i] = coef * (a[i] - b[i]) and one partial sum of
// (a[i] - b[i])^2 per block (fixed grid, grid-stride: the summation order does not depend on anything but n).
constexpr int SQD_BLOCKS = 592;
__global__ void __launch_bounds__(256)
sqdiff_grad_kernel(const float* __restrict__ a, const float* __restrict__ b, long long n, float coef,
                   float* __restrict__ g, float* __restrict__ partial) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = blockIdx.x * 256LL + threadIdx.x; i < n; i += (long long)gridDim.x * 256) {
    const float dv = a[i] - b[i];
    g[i] = coef * dv;
    s += dv * dv;
  }
  s = rte::block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void sqdiff_final_kernel(const float* __restrict__ partial, int n, float* __restrict__ out, int accumulate) {
  __shared__ float red[32];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = rte::block_sum(s, red);
  if (threadIdx.x == 0) out[0] = accumulate ? out[0] + s : s;
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

namespace {
// The tensor-core forward / phi_out backward need the transposed parameters (p->wt, see rte_macro_phi_prepare),
// d % 32 == 0, rank % 4 == 0 and 16-byte aligned buffers; otherwise the scalar kernels run.
inline bool phi_tensor_path(const rte_phi_params* p, const void* a, const void* b, const void* c, int d, int m) {
  return p->wt != nullptr && p->n_keys > 0 && d % 32 == 0 && m % 4 == 0 &&
         ((reinterpret_cast<uintptr_t>(p->wt) | reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b) |
           reinterpret_cast<uintptr_t>(c) | reinterpret_cast<uintptr_t>(p->gain) | reinterpret_cast<uintptr_t>(p->bias) |
           reinterpret_cast<uintptr_t>(p->scale)) & 15) == 0;
}
}  // namespace

// wt (n_keys*(3d*m + m*d) floats) = [ v^T as [m][n_keys*3d] | u^T as [d][n_keys*m] ]: once per optimiser step.
extern "C" int rte_macro_phi_prepare(const float* v, const float* u, float* wt, int32_t n_keys, int32_t d, int32_t m,
                                     rte_stream_t stream) {
  RTE_CHECK_ARG(v && u && wt && n_keys > 0 && d > 0 && m > 0);
  int rc = rte_transpose_f32(v, wt, n_keys * 3 * d, m, 0, 0, stream);
  if (rc != RTE_OK) return rc;
  return rte_transpose_f32(u, wt + (size_t)m * n_keys * 3 * d, n_keys * m, d, 0, 0, stream);
}

namespace {
// `h0`: the state Phi is applied to (norm, pooled mean, gain and residual terms); `hx`: the injected state of the third
// slice of z (the same pointer on the hot path).
int phi_fwd_impl(const float* h0, const float* hx, const rte_phi_params* p, const int32_t* recipe_id,
                 const int32_t* stride_id, float s_cfg, float* out, float* rstd, float* pooled,
                 float* act, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                 float eps, rte_stream_t stream) {
  RTE_CHECK_ARG(h0 && hx && p && p->gain && p->v && p->u && p->bias && p->scale && recipe_id && stride_id && out && rstd &&
                pooled && act && B > 0 && S > 0 && d > 0 && m > 0 && K_strides > 0);
  if (m > MMAX) return RTE_ERR_UNSUPPORTED;
  PhiDims D{B, S, d, m, K_strides};
  const int tiles = rte::ceil_div(S, TT);
  // `act` doubles as the home of pa (B*m floats) is NOT safe; pa lives at the tail of `pooled`'s
  // companion: callers give pooled >= B*d + B*m floats.
  float* pa = pooled + (size_t)B * d;
  phi_prep_kernel<<<B, NTHR, (size_t)(S + d) * sizeof(float), ST(stream)>>>(h0, p->v, recipe_id, stride_id, rstd, pooled, pa, D, eps);
  RTE_LAUNCH_CHECK();
  if (phi_tensor_path(p, h0, out, act, d, m) && (reinterpret_cast<uintptr_t>(hx) & 15) == 0) {
    const long long vt_ld = (long long)p->n_keys * 3 * d, ut_ld = (long long)p->n_keys * m;
    const float* ut = p->wt + (size_t)m * vt_ld;
    if (hx != h0) phi_act_mma_kernel<true><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, hx, rstd, pa, p->wt, vt_ld, recipe_id, stride_id, act, D);
    else phi_act_mma_kernel<false><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, hx, rstd, pa, p->wt, vt_ld, recipe_id, stride_id, act, D);
    RTE_LAUNCH_CHECK();
    if (m <= 32)
      phi_out_mma_kernel<0, 1><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, ut, ut_ld, p->bias, p->scale, recipe_id,
                                                                   stride_id, s_cfg, nullptr, out, nullptr, D);
    else
      phi_out_mma_kernel<0, 2><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, ut, ut_ld, p->bias, p->scale, recipe_id,
                                                                   stride_id, s_cfg, nullptr, out, nullptr, D);
    RTE_LAUNCH_CHECK();
    return RTE_OK;
  }
  phi_act_kernel<<<B * tiles, NTHR, 0, ST(stream)>>>(h0, hx, rstd, pa, p->v, recipe_id, stride_id, act, D);
  RTE_LAUNCH_CHECK();
  if (m <= 32)
    phi_out_kernel<0, 32><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, p->u, p->bias, p->scale, recipe_id, stride_id,
                                                              s_cfg, nullptr, out, nullptr, D);
  else
    phi_out_kernel<0, 64><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, p->u, p->bias, p->scale, recipe_id, stride_id,
                                                              s_cfg, nullptr, out, nullptr, D);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
}  // namespace

extern "C" int rte_macro_phi_fwd(const float* h0, const rte_phi_params* p, const int32_t* recipe_id,
                                 const int32_t* stride_id, float s_cfg, float* out, float* rstd, float* pooled,
                                 float* act, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                                 float eps, rte_stream_t stream) {
  return phi_fwd_impl(h0, h0, p, recipe_id, stride_id, s_cfg, out, rstd, pooled, act, B, S, d, m, K_strides, eps, stream);
}

extern "C" int rte_macro_phi_fwd_hx(const float* h, const float* h0, const rte_phi_params* p, const int32_t* recipe_id,
                                    const int32_t* stride_id, float s_cfg, float* out, float* rstd, float* pooled,
                                    float* act, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                                    float eps, rte_stream_t stream) {
  return phi_fwd_impl(h, h0, p, recipe_id, stride_id, s_cfg, out, rstd, pooled, act, B, S, d, m, K_strides, eps, stream);
}

namespace {
struct PhiBwdScratch { float *dupd, *da, *dpool, *pu, *pg, *pb, *pv; };
// scratch layout (floats): dupd[M*d] | da[M*m] | dpool[B*d] | pu[B*m*d] | pg[B*d] | pb[B*d] | pv[B*3d*m]
inline PhiBwdScratch phi_scratch(float* scratch, int B, int S, int d, int m) {
  const size_t M = (size_t)B * S;
  PhiBwdScratch x;
  x.dupd = scratch;
  x.da = x.dupd + M * d;
  x.dpool = x.da + M * m;
  x.pu = x.dpool + (size_t)B * d;
  x.pg = x.pu + (size_t)B * m * d;
  x.pb = x.pg + (size_t)B * d;
  x.pv = x.pb + (size_t)B * d;
  return x;
}
}  // namespace

namespace {
// dh0 (overwritten): gradient wrt the state Phi was applied to; dhx (accumulated into; may be dh0): gradient wrt the
// injected state of z's third slice.
int phi_bwd_data_impl(const float* h0, const float* dout, const rte_phi_params* p, const int32_t* recipe_id,
                      const int32_t* stride_id, float s_cfg, const float* rstd, const float* act, float* dh0, float* dhx,
                      float* scratch, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                      rte_stream_t stream) {
  RTE_CHECK_ARG(h0 && dhx && dout && p && recipe_id && stride_id && rstd && act && dh0 && scratch && B > 0 && S > 0 && d > 0 && m > 0 &&
                K_strides > 0);
  if (m > MMAX || B > 1024) return RTE_ERR_UNSUPPORTED;
  PhiDims D{B, S, d, m, K_strides};
  const int tiles = rte::ceil_div(S, TT);
  const PhiBwdScratch x = phi_scratch(scratch, B, S, d, m);
  if (phi_tensor_path(p, h0, dout, dh0, d, m) && (reinterpret_cast<uintptr_t>(scratch) & 15) == 0) {
    const long long vt_ld = (long long)p->n_keys * 3 * d, ut_ld = (long long)p->n_keys * m;
    const float* ut = p->wt + (size_t)m * vt_ld;
    if (m <= 32)
      phi_out_mma_kernel<1, 1><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, ut, ut_ld, p->bias, p->scale, recipe_id,
                                                                   stride_id, s_cfg, dout, dh0, x.dupd, D);
    else
      phi_out_mma_kernel<1, 2><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, ut, ut_ld, p->bias, p->scale, recipe_id,
                                                                   stride_id, s_cfg, dout, dh0, x.dupd, D);
  } else if (m <= 32)
    phi_out_kernel<1, 32><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, p->u, p->bias, p->scale, recipe_id, stride_id,
                                                              s_cfg, dout, dh0, x.dupd, D);
  else
    phi_out_kernel<1, 64><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, act, p->gain, p->u, p->bias, p->scale, recipe_id, stride_id,
                                                              s_cfg, dout, dh0, x.dupd, D);
  RTE_LAUNCH_CHECK();
  // tensor-core (3xTF32) products with 16-byte operand loads; other shapes keep the scalar kernels
  const bool mma = d % 32 == 0 && m % 4 == 0 && ((reinterpret_cast<uintptr_t>(scratch) | reinterpret_cast<uintptr_t>(h0) |
                   reinterpret_cast<uintptr_t>(dh0) | reinterpret_cast<uintptr_t>(dhx) | reinterpret_cast<uintptr_t>(p->u) |
                   reinterpret_cast<uintptr_t>(p->v)) & 15) == 0;
  if (mma) phi_da_mma_kernel<<<B * tiles, NTHR, 0, ST(stream)>>>(x.dupd, act, p->u, recipe_id, stride_id, x.da, D);
  else phi_da_kernel<<<B * tiles, NTHR, 0, ST(stream)>>>(x.dupd, act, p->u, recipe_id, stride_id, x.da, D);
  RTE_LAUNCH_CHECK();
  phi_dpool_kernel<<<B, NTHR, 0, ST(stream)>>>(x.da, p->v, recipe_id, stride_id, x.dpool, D);
  RTE_LAUNCH_CHECK();
  if (mma && m <= 32) phi_dz_mma_kernel<1><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, rstd, x.da, x.dpool, p->v, recipe_id, stride_id, dh0, dhx, D);
  else if (mma) phi_dz_mma_kernel<2><<<B * tiles, NTHR, 0, ST(stream)>>>(h0, rstd, x.da, x.dpool, p->v, recipe_id, stride_id, dh0, dhx, D);
  else phi_dz_kernel<<<B * tiles, NTHR, 0, ST(stream)>>>(h0, rstd, x.da, x.dpool, p->v, recipe_id, stride_id, dh0, dhx, D);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
}  // namespace

// Data-gradient half: dh0 (the chain the rest of backward waits for); leaves dupd and da in `scratch`.
extern "C" int rte_macro_phi_bwd_data(const float* h0, const float* dout, const rte_phi_params* p, const int32_t* recipe_id,
                                      const int32_t* stride_id, float s_cfg, const float* rstd, const float* act, float* dh0,
                                      float* scratch, int32_t B, int32_t S, int32_t d, int32_t m, int32_t K_strides,
                                      rte_stream_t stream) {
  return phi_bwd_data_impl(h0, dout, p, recipe_id, stride_id, s_cfg, rstd, act, dh0, dh0, scratch, B, S, d, m, K_strides, stream);
}

// Parameter-gradient half: reads dupd and da left in `scratch` by rte_macro_phi_bwd_data (may run on another
// stream, ordered after it); nothing downstream in backward depends on it.
namespace {
int phi_bwd_params_impl(const float* h0, const float* hx, const int32_t* recipe_id, const int32_t* stride_id, const float* rstd,
                        const float* pooled, const float* act, const rte_phi_grads* g, float* scratch,
                        int32_t B, int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides,
                        rte_stream_t stream) {
  RTE_CHECK_ARG(h0 && hx && recipe_id && stride_id && rstd && pooled && act && g && scratch && B > 0 && S > 0 && d > 0 && m > 0 &&
                R > 0 && K_strides > 0);
  RTE_CHECK_ARG(g->gain && g->v && g->u && g->bias);
  if (m > MMAX || B > 1024) return RTE_ERR_UNSUPPORTED;
  PhiDims D{B, S, d, m, K_strides};
  const PhiBwdScratch x = phi_scratch(scratch, B, S, d, m);
  const size_t smem_pu = (size_t)S * m * sizeof(float);
  const size_t smem_pv = ((size_t)S * m + S + 2 * (size_t)S * PV_ROWS) * sizeof(float);
  if (smem_pu > 48 * 1024 || smem_pv > 48 * 1024) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(phi_pu_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess ||
          cudaFuncSetAttribute(phi_pv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024) != cudaSuccess)
        return RTE_ERR_LAUNCH;
      set = true;
    }
  }
  phi_pu_kernel<<<B * rte::ceil_div(d, NTHR), NTHR, smem_pu, ST(stream)>>>(h0, act, x.dupd, x.pu, x.pg, x.pb, D);
  RTE_LAUNCH_CHECK();
  phi_pv_kernel<<<B * rte::ceil_div(d, PV_ROWS), NTHR, smem_pv, ST(stream)>>>(h0, hx, rstd, pooled, x.da, x.pv, D);
  RTE_LAUNCH_CHECK();
  const int n_keys = R * K_strides;
  const long long eu = (long long)m * d, ev = (long long)3 * d * m, ed = d;
  phi_reduce_keys_kernel<<<dim3((unsigned)rte::ceil_div64(eu, NTHR), n_keys), NTHR, 0, ST(stream)>>>(x.pu, recipe_id, stride_id, g->u, B, K_strides, eu);
  RTE_LAUNCH_CHECK();
  phi_reduce_keys_kernel<<<dim3((unsigned)rte::ceil_div64(ev, NTHR), n_keys), NTHR, 0, ST(stream)>>>(x.pv, recipe_id, stride_id, g->v, B, K_strides, ev);
  RTE_LAUNCH_CHECK();
  phi_reduce_keys_kernel<<<dim3((unsigned)rte::ceil_div64(ed, NTHR), n_keys), NTHR, 0, ST(stream)>>>(x.pg, recipe_id, stride_id, g->gain, B, K_strides, ed);
  RTE_LAUNCH_CHECK();
  phi_reduce_keys_kernel<<<dim3((unsigned)rte::ceil_div64(ed, NTHR), n_keys), NTHR, 0, ST(stream)>>>(x.pb, recipe_id, stride_id, g->bias, B, K_strides, ed);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
}  // namespace

extern "C" int rte_macro_phi_bwd_params(const float* h0, const int32_t* recipe_id, const int32_t* stride_id, const float* rstd,
                                        const float* pooled, const float* act, const rte_phi_grads* g, float* scratch,
                                        int32_t B, int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides,
                                        rte_stream_t stream) {
  return phi_bwd_params_impl(h0, h0, recipe_id, stride_id, rstd, pooled, act, g, scratch, B, S, d, m, R, K_strides, stream);
}

// Phi applied to a state h that is not the injected h0 (macro.py:342-359, the consistency term's second application):
// dh (overwritten) and dh0 (ACCUMULATED into) are separate; parameter gradients as in rte_macro_phi_bwd.
extern "C" int rte_macro_phi_bwd_hx(const float* h, const float* h0, const float* dout, const rte_phi_params* p,
                                    const int32_t* recipe_id, const int32_t* stride_id, float s_cfg, const float* rstd,
                                    const float* pooled, const float* act, float* dh, float* dh0, const rte_phi_grads* g,
                                    float* scratch, int32_t B, int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides,
                                    rte_stream_t stream) {
  RTE_CHECK_ARG(g != nullptr && R > 0 && dh != dh0);
  const int rc = phi_bwd_data_impl(h, dout, p, recipe_id, stride_id, s_cfg, rstd, act, dh, dh0, scratch, B, S, d, m, K_strides, stream);
  if (rc != RTE_OK) return rc;
  return phi_bwd_params_impl(h, h0, recipe_id, stride_id, rstd, pooled, act, g, scratch, B, S, d, m, R, K_strides, stream);
}

// Both halves on one stream.
extern "C" int rte_macro_phi_bwd(const float* h0, const float* dout, const rte_phi_params* p, const int32_t* recipe_id,
                                 const int32_t* stride_id, float s_cfg, const float* rstd, const float* pooled,
                                 const float* act, float* dh0, const rte_phi_grads* g, float* scratch, int32_t B,
                                 int32_t S, int32_t d, int32_t m, int32_t R, int32_t K_strides, float eps,
                                 rte_stream_t stream) {
  (void)eps;
  RTE_CHECK_ARG(g != nullptr && R > 0);
  const int rc = rte_macro_phi_bwd_data(h0, dout, p, recipe_id, stride_id, s_cfg, rstd, act, dh0, scratch, B, S, d, m, K_strides, stream);
  if (rc != RTE_OK) return rc;
  return rte_macro_phi_bwd_params(h0, recipe_id, stride_id, rstd, pooled, act, g, scratch, B, S, d, m, R, K_strides, stream);
}

// g = coef * (a - b);  sum_out (+)= sum (a - b)^2.  `partial`: >= 1024 floats of scratch.
extern "C" int rte_sqdiff_grad(const float* a, const float* b, int64_t n, float coef, float* g, float* partial, float* sum_out,
                               int32_t accumulate, rte_stream_t stream) {
  RTE_CHECK_ARG(a && b && g && partial && sum_out && n > 0);
  sqdiff_grad_kernel<<<SQD_BLOCKS, 256, 0, ST(stream)>>>(a, b, n, coef, g, partial);
  RTE_LAUNCH_CHECK();
  sqdiff_final_kernel<<<1, 1024, 0, ST(stream)>>>(partial, SQD_BLOCKS, sum_out, accumulate);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
