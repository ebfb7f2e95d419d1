// Causal self-attention with rotary embedding, forward and backward, for the short sequences of
// the training step (S <= 256).  One CTA per (sample, head): the head's roped Q, K and V (and dO in
// backward) live in shared memory as bf16, all arithmetic is fp32.  Forward keeps log-sum-exp per
// query row; backward recomputes the probabilities from it (no S x S matrix ever reaches HBM) in two
// deterministic sweeps: query-major for dQ, key-major for dK and dV (no atomics).
//
// Layout contract: qkv is [B*S, ld] bf16 with the head's q at column h*HD, k at sec + h*HD and v at
// 2*sec + h*HD.  Rotary pairs are ADJACENT elements (2i, 2i+1), angle = pos * 10000^(-2i/HD).

#include "rte_common.cuh"
#include "attention_mma.cuh"

namespace {

constexpr int ATT_THREADS = 256;
constexpr int ATT_WARPS = ATT_THREADS / 32;

template <int HD>
struct AttCfg {
  static constexpr int DPL = (HD >= 32) ? HD / 32 : 1;   // head dims per lane in the "c-parallel" phases
  static constexpr int LDS = HD + 2;                     // padded smem row (bf16 elements)
};

__device__ __forceinline__ float rope_inv_freq(int pair, int hd) {
  return 1.0f / powf(10000.0f, (float)(2 * pair) / (float)hd);
}

// Loads rows [0,S) of one head's slice into smem (bf16), optionally applying the rotary embedding.
template <int HD, bool ROPE>
__device__ __forceinline__ void load_head(const __nv_bfloat16* __restrict__ src, int ld, int S, __nv_bfloat16* dst,
                                          const float* __restrict__ rope = nullptr) {
  constexpr int LDS = AttCfg<HD>::LDS;
  for (int idx = threadIdx.x; idx < S * (HD / 2); idx += blockDim.x) {
    const int s = idx / (HD / 2), pr = idx % (HD / 2);
    const __nv_bfloat162 in = *reinterpret_cast<const __nv_bfloat162*>(src + (size_t)s * ld + 2 * pr);
    float2 v = __bfloat1622float2(in);
    if (ROPE) {
      float sn, cs;
      attn_mma::rope_cs(rope, s, pr, HD, cs, sn);
      v = make_float2(v.x * cs - v.y * sn, v.y * cs + v.x * sn);
    }
    *reinterpret_cast<__nv_bfloat162*>(dst + s * LDS + 2 * pr) = __floats2bfloat162_rn(v.x, v.y);
  }
}

template <int HD>
__device__ __forceinline__ float dot_rows(const __nv_bfloat16* a, const __nv_bfloat16* b) {
  float acc = 0.f;
#pragma unroll
  for (int c = 0; c < HD / 2; ++c) {
    const float2 x = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(a + 2 * c));
    const float2 y = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(b + 2 * c));
    acc += x.x * y.x + x.y * y.y;
  }
  return acc;
}

// ------------------------------------------------------------------ forward
template <int HD, int SMAX>
__global__ void __launch_bounds__(ATT_THREADS)
attn_fwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int sec, __nv_bfloat16* __restrict__ y, int ldy,
                float* __restrict__ lse, const float* __restrict__ rope, int S, int H) {
  constexpr int LDS = AttCfg<HD>::LDS, DPL = AttCfg<HD>::DPL, NT = SMAX / 32;
  extern __shared__ __align__(16) uint8_t smraw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smraw);
  __nv_bfloat16* sk = sq + SMAX * LDS;
  __nv_bfloat16* sv = sk + SMAX * LDS;
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const __nv_bfloat16* base = qkv + (size_t)b * S * ld + h * HD;
  load_head<HD, true>(base, ld, S, sq, rope);
  load_head<HD, true>(base + sec, ld, S, sk, rope);
  load_head<HD, false>(base + 2 * sec, ld, S, sv);
  __syncthreads();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float scale = rsqrtf((float)HD);
  for (int i = warp; i < S; i += ATT_WARPS) {
    float p[NT];
    float mx = -INFINITY;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int j = lane + 32 * t;
      p[t] = (j <= i) ? dot_rows<HD>(sq + i * LDS, sk + j * LDS) * scale : -INFINITY;
      mx = fmaxf(mx, p[t]);
    }
    mx = rte::warp_max(mx);
    float sum = 0.f;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      p[t] = (lane + 32 * t <= i) ? __expf(p[t] - mx) : 0.f;
      sum += p[t];
    }
    sum = rte::warp_sum(sum);
    const float inv = 1.f / sum;
    float acc[DPL];
#pragma unroll
    for (int c = 0; c < DPL; ++c) acc[c] = 0.f;
    const int c0 = lane * DPL;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (32 * t > i) break;
      const int jmax = min(31, i - 32 * t);
      for (int jj = 0; jj <= jmax; ++jj) {
        const float pj = __shfl_sync(0xffffffffu, p[t], jj);
        if (c0 < HD) {
#pragma unroll
          for (int c = 0; c < DPL; ++c) acc[c] += pj * __bfloat162float(sv[(32 * t + jj) * LDS + c0 + c]);
        }
      }
    }
    if (c0 < HD) {
      __nv_bfloat16* yo = y + (size_t)(b * S + i) * ldy + h * HD + c0;
#pragma unroll
      for (int c = 0; c < DPL; ++c) yo[c] = __float2bfloat16_rn(acc[c] * inv);
    }
    if (lane == 0) lse[((size_t)b * H + h) * S + i] = mx + __logf(sum);
  }
}

// Inverse rotary embedding of a gradient vector held `DPL` consecutive dims per lane.
template <int HD>
__device__ __forceinline__ void unrope_inplace(float (&g)[AttCfg<HD>::DPL], int c0, int pos, int lane,
                                               const float* __restrict__ rope) {
  constexpr int DPL = AttCfg<HD>::DPL;
  if constexpr (DPL >= 2) {
    if (c0 < HD) {
#pragma unroll
      for (int c = 0; c < DPL; c += 2) {
        float sn, cs;
        attn_mma::rope_cs(rope, pos, (c0 + c) / 2, HD, cs, sn);
        const float a = g[c], bq = g[c + 1];
        g[c] = a * cs + bq * sn;
        g[c + 1] = -a * sn + bq * cs;
      }
    }
  } else {
    const float other = __shfl_xor_sync(0xffffffffu, g[0], 1);
    if (c0 < HD) {
      float sn, cs;
      attn_mma::rope_cs(rope, pos, c0 / 2, HD, cs, sn);
      g[0] = (c0 & 1) ? (-other * sn + g[0] * cs) : (g[0] * cs + other * sn);
    }
  }
}

// ------------------------------------------------------------------ backward
template <int HD, int SMAX>
__global__ void __launch_bounds__(ATT_THREADS)
attn_bwd_kernel(const __nv_bfloat16* __restrict__ qkv, int ld, int sec, const __nv_bfloat16* __restrict__ y,
                const __nv_bfloat16* __restrict__ dy, int ldy, const float* __restrict__ lse,
                __nv_bfloat16* __restrict__ dqkv, const float* __restrict__ rope, int S, int H) {
  constexpr int LDS = AttCfg<HD>::LDS, DPL = AttCfg<HD>::DPL, NT = SMAX / 32;
  extern __shared__ __align__(16) uint8_t smraw[];
  __nv_bfloat16* sq = reinterpret_cast<__nv_bfloat16*>(smraw);
  __nv_bfloat16* sk = sq + SMAX * LDS;
  __nv_bfloat16* sv = sk + SMAX * LDS;
  __nv_bfloat16* sdo = sv + SMAX * LDS;
  float* slse = reinterpret_cast<float*>(sdo + SMAX * LDS);
  float* sD = slse + SMAX;
  const int b = blockIdx.x / H, h = blockIdx.x % H;
  const __nv_bfloat16* base = qkv + (size_t)b * S * ld + h * HD;
  load_head<HD, true>(base, ld, S, sq, rope);
  load_head<HD, true>(base + sec, ld, S, sk, rope);
  load_head<HD, false>(base + 2 * sec, ld, S, sv);
  load_head<HD, false>(dy + (size_t)b * S * ldy + h * HD, ldy, S, sdo);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = warp; i < S; i += ATT_WARPS) {
    // D_i = sum_c dO[i,c] * O[i,c]
    float part = 0.f;
    for (int c = lane; c < HD; c += 32)
      part += __bfloat162float(dy[(size_t)(b * S + i) * ldy + h * HD + c]) * __bfloat162float(y[(size_t)(b * S + i) * ldy + h * HD + c]);
    part = rte::warp_sum(part);
    if (lane == 0) { sD[i] = part; slse[i] = lse[((size_t)b * H + h) * S + i]; }
  }
  __syncthreads();
  const float scale = rsqrtf((float)HD);
  const int c0 = lane * DPL;
  __nv_bfloat16* dbase = dqkv + (size_t)b * S * ld + h * HD;

  // sweep 1: query-major, dQ_i = scale * sum_{j<=i} dS_ij K_j
  for (int i = warp; i < S; i += ATT_WARPS) {
    float ds[NT];
    const float li = slse[i], Di = sD[i];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int j = lane + 32 * t;
      float v = 0.f;
      if (j <= i) {
        const float pij = __expf(dot_rows<HD>(sq + i * LDS, sk + j * LDS) * scale - li);
        const float dp = dot_rows<HD>(sdo + i * LDS, sv + j * LDS);
        v = pij * (dp - Di);
      }
      ds[t] = v;
    }
    float acc[DPL];
#pragma unroll
    for (int c = 0; c < DPL; ++c) acc[c] = 0.f;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (32 * t > i) break;
      const int jmax = min(31, i - 32 * t);
      for (int jj = 0; jj <= jmax; ++jj) {
        const float d = __shfl_sync(0xffffffffu, ds[t], jj);
        if (c0 < HD) {
#pragma unroll
          for (int c = 0; c < DPL; ++c) acc[c] += d * __bfloat162float(sk[(32 * t + jj) * LDS + c0 + c]);
        }
      }
    }
#pragma unroll
    for (int c = 0; c < DPL; ++c) acc[c] *= scale;
    unrope_inplace<HD>(acc, c0, i, lane, rope);
    if (c0 < HD) {
#pragma unroll
      for (int c = 0; c < DPL; ++c) dbase[(size_t)i * ld + c0 + c] = __float2bfloat16_rn(acc[c]);
    }
  }

  // sweep 2: key-major, dV_j = sum_{i>=j} P_ij dO_i ; dK_j = scale * sum_{i>=j} dS_ij Q_i
  for (int j = warp; j < S; j += ATT_WARPS) {
    float pr[NT], ds[NT];
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      const int i = lane + 32 * t;
      float pv = 0.f, dv = 0.f;
      if (i >= j && i < S) {
        pv = __expf(dot_rows<HD>(sq + i * LDS, sk + j * LDS) * scale - slse[i]);
        const float dp = dot_rows<HD>(sdo + i * LDS, sv + j * LDS);
        dv = pv * (dp - sD[i]);
      }
      pr[t] = pv; ds[t] = dv;
    }
    float av[DPL], ak[DPL];
#pragma unroll
    for (int c = 0; c < DPL; ++c) av[c] = ak[c] = 0.f;
#pragma unroll
    for (int t = 0; t < NT; ++t) {
      if (32 * t + 31 < j) continue;
      if (32 * t >= S) break;
      const int i_lo = max(0, j - 32 * t), i_hi = min(31, S - 1 - 32 * t);
      for (int ii = i_lo; ii <= i_hi; ++ii) {
        const float pv = __shfl_sync(0xffffffffu, pr[t], ii);
        const float dv = __shfl_sync(0xffffffffu, ds[t], ii);
        if (c0 < HD) {
#pragma unroll
          for (int c = 0; c < DPL; ++c) {
            av[c] += pv * __bfloat162float(sdo[(32 * t + ii) * LDS + c0 + c]);
            ak[c] += dv * __bfloat162float(sq[(32 * t + ii) * LDS + c0 + c]);
          }
        }
      }
    }
#pragma unroll
    for (int c = 0; c < DPL; ++c) ak[c] *= scale;
    unrope_inplace<HD>(ak, c0, j, lane, rope);
    if (c0 < HD) {
#pragma unroll
      for (int c = 0; c < DPL; ++c) {
        dbase[(size_t)j * ld + sec + c0 + c] = __float2bfloat16_rn(ak[c]);
        dbase[(size_t)j * ld + 2 * sec + c0 + c] = __float2bfloat16_rn(av[c]);
      }
    }
  }
}

template <int HD, int SMAX>
int launch_fwd(const void* qkv, int ld, int sec, void* y, int ldy, float* lse, const float* rope, int B, int S, int H, cudaStream_t st) {
  constexpr size_t smem = (size_t)3 * SMAX * AttCfg<HD>::LDS * 2;
  static bool set = false;
  if (!set && smem > 48 * 1024) {
    if (cudaFuncSetAttribute(attn_fwd_kernel<HD, SMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return RTE_ERR_LAUNCH;
    set = true;
  }
  attn_fwd_kernel<HD, SMAX><<<B * H, ATT_THREADS, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(qkv), ld, sec,
      reinterpret_cast<__nv_bfloat16*>(y), ldy, lse, rope, S, H);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
template <int HD, int SMAX>
int launch_bwd(const void* qkv, int ld, int sec, const void* y, const void* dy, int ldy, const float* lse, void* dqkv,
               const float* rope, int B, int S, int H, cudaStream_t st) {
  constexpr size_t smem = (size_t)4 * SMAX * AttCfg<HD>::LDS * 2 + (size_t)2 * SMAX * 4;
  static bool set = false;
  if (!set && smem > 48 * 1024) {
    if (cudaFuncSetAttribute(attn_bwd_kernel<HD, SMAX>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) != cudaSuccess)
      return RTE_ERR_LAUNCH;
    set = true;
  }
  attn_bwd_kernel<HD, SMAX><<<B * H, ATT_THREADS, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(qkv), ld, sec,
      reinterpret_cast<const __nv_bfloat16*>(y), reinterpret_cast<const __nv_bfloat16*>(dy), ldy, lse,
      reinterpret_cast<__nv_bfloat16*>(dqkv), rope, S, H);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

__global__ void rope_table_kernel(float* __restrict__ out, int S, int hd) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= S * (hd / 2)) return;
  float sn, cs;
  sincosf((float)(i / (hd / 2)) * rope_inv_freq(i % (hd / 2), hd), &sn, &cs);
  out[2 * i] = cs;
  out[2 * i + 1] = sn;
}

// Stand-alone rotary application over [rows, S, hd] tensors (rows = B*H) with caller-supplied cos/sin [S, hd]
// (the layout of the reference's cached buffers after repeat_interleave).  adjoint != 0 applies the transpose
// of the rotation (the backward pass of the same operator).
template <typename T>
__global__ void rope_apply_kernel(const T* __restrict__ x, const float* __restrict__ cs, const float* __restrict__ sn,
                                  T* __restrict__ out, long long pairs, int S, int hd, int adjoint) {
  const int hp = hd / 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < pairs; i += (long long)gridDim.x * blockDim.x) {
    const int pr = (int)(i % hp);
    const int pos = (int)((i / hp) % S);
    const float a = (float)x[2 * i], b = (float)x[2 * i + 1];
    const float c0 = cs[pos * hd + 2 * pr], c1 = cs[pos * hd + 2 * pr + 1];
    const float s0 = sn[pos * hd + 2 * pr], s1 = sn[pos * hd + 2 * pr + 1];
    float o0, o1;
    if (!adjoint) { o0 = a * c0 - b * s0; o1 = b * c1 + a * s1; }       // x*cos + rotate_half(x)*sin
    else          { o0 = a * c0 + b * s1; o1 = b * c1 - a * s0; }
    out[2 * i] = (T)o0;
    out[2 * i + 1] = (T)o1;
  }
}

}  // namespace

#define RTE_ATT_DISPATCH(FN, ...)                                              \
  do {                                                                         \
    const int smax = S <= 32 ? 32 : S <= 64 ? 64 : S <= 128 ? 128 : 256;       \
    switch (head_dim * 1000 + smax) {                                          \
      case 8032: return FN<8, 32>(__VA_ARGS__);                                \
      case 8064: return FN<8, 64>(__VA_ARGS__);                                \
      case 16032: return FN<16, 32>(__VA_ARGS__);                              \
      case 16064: return FN<16, 64>(__VA_ARGS__);                              \
      case 32032: return FN<32, 32>(__VA_ARGS__);                              \
      case 32064: return FN<32, 64>(__VA_ARGS__);                              \
      case 32128: return FN<32, 128>(__VA_ARGS__);                             \
      case 64032: return FN<64, 32>(__VA_ARGS__);                              \
      case 64064: return FN<64, 64>(__VA_ARGS__);                              \
      case 64128: return FN<64, 128>(__VA_ARGS__);                             \
      case 64256: return FN<64, 256>(__VA_ARGS__);                             \
      case 128064: return FN<128, 64>(__VA_ARGS__);                            \
      case 128128: return FN<128, 128>(__VA_ARGS__);                           \
      default: return RTE_ERR_UNSUPPORTED;                                     \
    }                                                                          \
  } while (0)

// Tensor-core path for the head sizes the mma.sync tiles cover; everything else falls through to the
// SIMT kernels above (tiny heads of the test configurations).  Needs 16-byte aligned rows for ldmatrix.
#define RTE_ATT_MMA_DISPATCH(FN, ...)                                          \
  do {                                                                         \
    if (ld_qkv % 8 == 0 && sec % 8 == 0 && ld_y % 8 == 0) {                    \
      const int smax = S <= 64 ? 64 : S <= 128 ? 128 : 256;                    \
      switch (head_dim * 1000 + smax) {                                        \
        case 32064: return FN<32, 64>(__VA_ARGS__);                            \
        case 32128: return FN<32, 128>(__VA_ARGS__);                           \
        case 32256: return FN<32, 256>(__VA_ARGS__);                           \
        case 64064: return FN<64, 64>(__VA_ARGS__);                            \
        case 64128: return FN<64, 128>(__VA_ARGS__);                           \
        case 64256: return FN<64, 256>(__VA_ARGS__);                           \
        case 128064: return FN<128, 64>(__VA_ARGS__);                          \
        case 128128: return FN<128, 128>(__VA_ARGS__);                         \
        default: break;                                                        \
      }                                                                        \
    }                                                                          \
  } while (0)

extern "C" int rte_rope_table(float* out, int32_t S, int32_t head_dim, rte_stream_t stream) {
  RTE_CHECK_ARG(out && S > 0 && head_dim > 0 && head_dim % 2 == 0);
  const int n = S * (head_dim / 2);
  rope_table_kernel<<<rte::ceil_div(n, 256), 256, 0, reinterpret_cast<cudaStream_t>(stream)>>>(out, S, head_dim);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_rope_apply(const void* x, const float* cos_tab, const float* sin_tab, void* out, int64_t rows, int32_t S,
                              int32_t head_dim, int32_t is_bf16, int32_t adjoint, rte_stream_t stream) {
  RTE_CHECK_ARG(x && cos_tab && sin_tab && out && rows > 0 && S > 0 && head_dim > 0 && head_dim % 2 == 0);
  const long long pairs = rows * (long long)S * (head_dim / 2);
  long long g = (pairs + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (is_bf16)
    rope_apply_kernel<__nv_bfloat16><<<(int)g, 256, 0, st>>>(reinterpret_cast<const __nv_bfloat16*>(x), cos_tab, sin_tab,
                                                            reinterpret_cast<__nv_bfloat16*>(out), pairs, S, head_dim, adjoint);
  else
    rope_apply_kernel<float><<<(int)g, 256, 0, st>>>(reinterpret_cast<const float*>(x), cos_tab, sin_tab,
                                                    reinterpret_cast<float*>(out), pairs, S, head_dim, adjoint);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_attn_fwd(const void* qkv, int32_t ld_qkv, int32_t sec, void* y, int32_t ld_y, float* lse,
                            const float* rope_table, int32_t B, int32_t S, int32_t n_heads, int32_t head_dim,
                            rte_stream_t stream) {
  RTE_CHECK_ARG(qkv && y && lse && B > 0 && S > 0 && S <= 256 && n_heads > 0 && ld_qkv % 2 == 0 && sec % 2 == 0);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  RTE_ATT_MMA_DISPATCH(attn_mma::launch_fwd, qkv, ld_qkv, sec, y, ld_y, lse, rope_table, B, S, n_heads, st);
  RTE_ATT_DISPATCH(launch_fwd, qkv, ld_qkv, sec, y, ld_y, lse, rope_table, B, S, n_heads, st);
}

// Attention forward with a second, column-masked copy of the output (the banked core's recipe mask,
// layers.py:702-728): ym[row, c] = y[row, c] * mask_table[mask_row[row / S]][c].  One launch on the tensor-core
// path; otherwise the plain forward followed by rte_colmask_mul_bf16.  y and ym share the leading dimension.
extern "C" int rte_attn_fwd_masked(const void* qkv, int32_t ld_qkv, int32_t sec, void* y, void* y_masked, int32_t ld_y,
                                   float* lse, const float* rope_table, const int32_t* mask_row, const float* mask_table,
                                   int32_t B, int32_t S, int32_t n_heads, int32_t head_dim, rte_stream_t stream) {
  RTE_CHECK_ARG(qkv && y && y_masked && lse && mask_row && mask_table && B > 0 && S > 0 && S <= 256 && n_heads > 0 &&
                ld_qkv % 2 == 0 && sec % 2 == 0);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ld_y == n_heads * head_dim && (reinterpret_cast<uintptr_t>(mask_table) & 7) == 0) {
    RTE_ATT_MMA_DISPATCH(attn_mma::launch_fwd, qkv, ld_qkv, sec, y, ld_y, lse, rope_table, B, S, n_heads, st, y_masked, mask_row,
                         mask_table);
  }
  const int rc = rte_attn_fwd(qkv, ld_qkv, sec, y, ld_y, lse, rope_table, B, S, n_heads, head_dim, stream);
  if (rc != RTE_OK) return rc;
  if (ld_y != n_heads * head_dim) return RTE_ERR_UNSUPPORTED;
  return rte_colmask_mul_bf16(y, mask_row, mask_table, S, y_masked, B * S, n_heads * head_dim, stream);
}

// Attention backward whose upstream gradient is dy times the per-sample column mask of rte_attn_fwd_masked (the banked
// core applies the recipe mask to the attention output before the output projection).  One launch on the tensor-core
// path (the mask is applied to the dy tile in shared memory, dy itself is left alone); otherwise dy is masked IN PLACE
// by rte_colmask_mul_bf16 and the plain backward follows.
extern "C" int rte_attn_bwd_masked(const void* qkv, int32_t ld_qkv, int32_t sec, const void* y, void* dy, int32_t ld_y,
                                   const float* lse, void* dqkv, const float* rope_table, const int32_t* mask_row,
                                   const float* mask_table, int32_t B, int32_t S, int32_t n_heads, int32_t head_dim,
                                   rte_stream_t stream) {
  RTE_CHECK_ARG(qkv && y && dy && lse && dqkv && mask_row && mask_table && B > 0 && S > 0 && S <= 256 && n_heads > 0 &&
                ld_qkv % 2 == 0 && sec % 2 == 0 && ld_y % 2 == 0);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ld_y == n_heads * head_dim) {
    RTE_ATT_MMA_DISPATCH(attn_mma::launch_bwd, qkv, ld_qkv, sec, y, dy, ld_y, lse, dqkv, rope_table, B, S, n_heads, st, mask_row,
                         mask_table);
  } else {
    return RTE_ERR_UNSUPPORTED;
  }
  const int rc = rte_colmask_mul_bf16(dy, mask_row, mask_table, S, dy, B * S, n_heads * head_dim, stream);
  if (rc != RTE_OK) return rc;
  return rte_attn_bwd(qkv, ld_qkv, sec, y, dy, ld_y, lse, dqkv, rope_table, B, S, n_heads, head_dim, stream);
}

extern "C" int rte_attn_bwd(const void* qkv, int32_t ld_qkv, int32_t sec, const void* y, const void* dy, int32_t ld_y,
                            const float* lse, void* dqkv, const float* rope_table, int32_t B, int32_t S, int32_t n_heads,
                            int32_t head_dim, rte_stream_t stream) {
  RTE_CHECK_ARG(qkv && y && dy && lse && dqkv && B > 0 && S > 0 && S <= 256 && n_heads > 0 && ld_qkv % 2 == 0 &&
                sec % 2 == 0 && ld_y % 2 == 0);
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  RTE_ATT_MMA_DISPATCH(attn_mma::launch_bwd, qkv, ld_qkv, sec, y, dy, ld_y, lse, dqkv, rope_table, B, S, n_heads, st);
  RTE_ATT_DISPATCH(launch_bwd, qkv, ld_qkv, sec, y, dy, ld_y, lse, dqkv, rope_table, B, S, n_heads, st);
}
