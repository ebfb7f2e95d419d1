// HBM-bound kernels of the training step: embedding gather/scatter, RMSNorm forward/backward
// (with the recurrent core's FiLM), per-token cross entropy with its gradient, split-K reduction,
// fp32->bf16 weight shadows, fused multi-tensor AdamW and the global gradient norm.
// All loads/stores are 16-byte vectors along the contiguous axis; grids are sized from the data
// (one warp or one CTA per row), which at the step's sizes is many waves of 148 SMs.

#include "rte_common.cuh"

namespace {

using rte::block_max;
using rte::block_sum;
using rte::warp_sum;

// ------------------------------------------------------------------ embedding
__global__ void embed_fwd_kernel(const int64_t* __restrict__ tokens, const float* __restrict__ table,
                                 float* __restrict__ out, int n_tokens, int d, int vocab, int* status) {
  const int d4 = d >> 2;
  const long long total = (long long)n_tokens * d4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / d4), c = int(i % d4);
    long long tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
      if (status) atomicExch(status, RTE_DEV_INDEX_OUT_OF_RANGE);
      tok = 0;
    }
    reinterpret_cast<float4*>(out)[i] = reinterpret_cast<const float4*>(table)[tok * d4 + c];
  }
}

// The scatter-add of token-row gradients into the table is ORDER-FREE: every addend is converted to 64-bit fixed
// point (scale 2^40: resolution 9e-13, range +-8.4e6), integer atomics are associative, and the sum is converted
// back once per table element, so repeated runs produce the same bits whatever order the adds land in.
constexpr float EMBED_FX_SCALE = 1099511627776.f;          // 2^40

__global__ void embed_bwd_accum_kernel(const int64_t* __restrict__ tokens, const float* __restrict__ dx,
                                       unsigned long long* __restrict__ accum, float* __restrict__ dtable,
                                       int n_tokens, int d, int vocab, int* status) {
  const long long total = (long long)n_tokens * d;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int t = int(i / d), c = int(i % d);
    const long long tok = tokens[t];
    if (tok < 0 || tok >= vocab) {
      if (status) atomicExch(status, RTE_DEV_INDEX_OUT_OF_RANGE);
      continue;
    }
    const float x = dx[i];
    if (!isfinite(x)) { dtable[tok * d + c] = x - x; continue; }      // NaN stays NaN through the final add
    atomicAdd(accum + tok * d + c, (unsigned long long)__float2ll_rn(x * EMBED_FX_SCALE));
  }
}

__global__ void embed_bwd_apply_kernel(const unsigned long long* __restrict__ accum, float* __restrict__ dtable, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const long long q = (long long)accum[i];
    if (q != 0) dtable[i] += __ll2float_rn(q) * (1.f / EMBED_FX_SCALE);
  }
}

// ------------------------------------------------------------------ RMSNorm
// One warp per row, row held in registers (d <= 32 * 4 * RN_MAX_V4).
constexpr int RN_MAX_V4 = 16;   // d up to 2048

template <int NV>
__global__ void __launch_bounds__(256)
rmsnorm_fwd_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ fg,
                   const float* __restrict__ fb, __nv_bfloat16* __restrict__ y16, float* __restrict__ y32,
                   float* __restrict__ rstd, int rows, int d, float eps) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int d4 = d >> 2;
  const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * d);
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < d4) {
      v[i] = xr[c];
      ss += v[i].x * v[i].x + v[i].y * v[i].y + v[i].z * v[i].z + v[i].w * v[i].w;
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)d + eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < d4) {
      float4 o = make_float4(v[i].x * r, v[i].y * r, v[i].z * r, v[i].w * r);
      if (w) {
        const float4 ww = reinterpret_cast<const float4*>(w)[c];
        o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w;
      }
      if (fg) {
        const float4 g = reinterpret_cast<const float4*>(fg)[c], b = reinterpret_cast<const float4*>(fb)[c];
        o.x = o.x * (1.f + g.x) + b.x; o.y = o.y * (1.f + g.y) + b.y;
        o.z = o.z * (1.f + g.z) + b.z; o.w = o.w * (1.f + g.w) + b.w;
      }
      if (y32) reinterpret_cast<float4*>(y32 + (size_t)row * d)[c] = o;
      if (y16) {
        uint2 pk = make_uint2(rte::pack_bf16x2(o.x, o.y), rte::pack_bf16x2(o.z, o.w));
        reinterpret_cast<uint2*>(y16 + (size_t)row * d)[c] = pk;
      }
    }
  }
}

// Residual update(s) fused in front of the norm (one warp per row):
//   x1 = (active == NULL || active[row / S]) ? base + *scale * branch : passthrough      -> x1_out (optional)
//   x  = add2 ? x1 + *scale2 * add2 : x1                                                  -> x_out
//   y  = rmsnorm(x) * w [* (1 + fg) + fb]
template <int NV>
__global__ void __launch_bounds__(256)
residual_rmsnorm_fwd_kernel(const float* __restrict__ base, const float* __restrict__ branch, const float* __restrict__ scale,
                            const int32_t* __restrict__ active, const float* __restrict__ passthrough, int S,
                            const float* __restrict__ add2, const float* __restrict__ scale2, float* __restrict__ x1_out,
                            float* __restrict__ x_out, const float* __restrict__ w, const float* __restrict__ fg,
                            const float* __restrict__ fb, __nv_bfloat16* __restrict__ y16, float* __restrict__ rstd, int rows, int d,
                            float eps, int branch_splits, long long branch_stride, float* __restrict__ branch_out) {
  // branch_splits > 1: `branch` holds that many split-K partials of the branch, branch_stride floats apart; they are
  // summed here in split order (what rte_reduce_splits would have produced) and the sum is kept in branch_out.
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const int d4 = d >> 2;
  const size_t off = (size_t)row * d;
  const bool on = active == nullptr || active[row / S] != 0;
  const float s1 = *scale, s2 = add2 ? *scale2 : 0.f;
  float4 v[NV];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < d4) {
      float4 x;
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (on || branch_out) {
        b = reinterpret_cast<const float4*>(branch + off)[c];
        for (int s = 1; s < branch_splits; ++s) {
          const float4 t = reinterpret_cast<const float4*>(branch + (size_t)s * branch_stride + off)[c];
          b.x += t.x; b.y += t.y; b.z += t.z; b.w += t.w;
        }
        if (branch_out) reinterpret_cast<float4*>(branch_out + off)[c] = b;
      }
      if (on) {
        const float4 a = reinterpret_cast<const float4*>(base + off)[c];
        x = make_float4(a.x + s1 * b.x, a.y + s1 * b.y, a.z + s1 * b.z, a.w + s1 * b.w);
      } else {
        x = reinterpret_cast<const float4*>(passthrough + off)[c];
      }
      if (x1_out) reinterpret_cast<float4*>(x1_out + off)[c] = x;
      if (add2) {
        const float4 e = reinterpret_cast<const float4*>(add2 + off)[c];
        x.x += s2 * e.x; x.y += s2 * e.y; x.z += s2 * e.z; x.w += s2 * e.w;
      }
      reinterpret_cast<float4*>(x_out + off)[c] = x;
      v[i] = x;
      ss += x.x * x.x + x.y * x.y + x.z * x.z + x.w * x.w;
    }
  }
  ss = warp_sum(ss);
  const float r = rsqrtf(ss / (float)d + eps);
  if (lane == 0 && rstd) rstd[row] = r;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < d4) {
      float4 o = make_float4(v[i].x * r, v[i].y * r, v[i].z * r, v[i].w * r);
      if (w) {
        const float4 ww = reinterpret_cast<const float4*>(w)[c];
        o.x *= ww.x; o.y *= ww.y; o.z *= ww.z; o.w *= ww.w;
      }
      if (fg) {
        const float4 g = reinterpret_cast<const float4*>(fg)[c], b = reinterpret_cast<const float4*>(fb)[c];
        o.x = o.x * (1.f + g.x) + b.x; o.y = o.y * (1.f + g.y) + b.y;
        o.z = o.z * (1.f + g.z) + b.z; o.w = o.w * (1.f + g.w) + b.w;
      }
      uint2 pk = make_uint2(rte::pack_bf16x2(o.x, o.y), rte::pack_bf16x2(o.z, o.w));
      reinterpret_cast<uint2*>(y16 + off)[c] = pk;
    }
  }
}

// Backward.  y = xhat * w * (1 + fg) + fb with xhat = x * rstd.
//   g  = dy * (1 + fg) * w          (gradient wrt xhat)
//   dx = rstd * (g - xhat * mean(g * xhat)) + dres
//   dw += dy * (1 + fg) * xhat,  dfg += dy * xhat * w,  dfb += dy
// Each CTA walks rows blockIdx.x, blockIdx.x + gridDim.x, ...; column-wise partial sums for the
// parameter gradients are kept in registers per warp, combined through shared memory at the end
// and written to row blockIdx.x of the partial buffers (deterministic, no atomics).
// FILM = false drops the FiLM accumulators (and a third of the registers) for the plain-norm launches.
template <int NV, bool FILM>
__global__ void __launch_bounds__(256, NV <= 4 ? 2 : 1)
rmsnorm_bwd_kernel(const float* __restrict__ x, const float* __restrict__ w, const float* __restrict__ fg,
                   const float* __restrict__ rstd, const __nv_bfloat16* __restrict__ dy16,
                   const float* __restrict__ dy32, const float* __restrict__ dres, float* __restrict__ dx32,
                   __nv_bfloat16* __restrict__ dx16, float* __restrict__ dw_part, float* __restrict__ dg_part,
                   float* __restrict__ db_part, int rows, int d, int dy_splits, long long dy_stride) {
  // dy_splits > 1: dy32 holds that many split-K partials of dy, dy_stride floats apart, summed here in split order
  extern __shared__ float sm[];   // [3][warps][d] when parameter gradients are requested
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const int d4 = d >> 2;
  constexpr int NF = FILM ? NV : 1;
  float4 aw[NV], ag[NF], ab[NF];
#pragma unroll
  for (int i = 0; i < NV; ++i) aw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
  for (int i = 0; i < NF; ++i) ag[i] = ab[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool want_w = dw_part != nullptr, want_f = FILM && dg_part != nullptr;

  int row = blockIdx.x * nwarp + warp;
  const int stride = gridDim.x * nwarp;
  if constexpr (!FILM && NV <= 4) {
    // Two rows per trip with all loads of both rows issued before the first use: a warp that walks its rows one at a
    // time keeps too few bytes in flight to cover the memory latency (the plain-norm launches of the hot pass).
    for (; dy_splits <= 1 && row + stride < rows; row += 2 * stride) {
      const int rw[2] = {row, row + stride};
      float rr[2];
      float4 xh[2][NV], g[2][NV], dyv[2][NV];
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        rr[u] = rstd[rw[u]];
        const float4* xr = reinterpret_cast<const float4*>(x + (size_t)rw[u] * d);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + 32 * i;
          if (c < d4) {
            xh[u][i] = xr[c];
            if (dy16) {
              const uint2 pk = reinterpret_cast<const uint2*>(dy16 + (size_t)rw[u] * d)[c];
              const float2 a = rte::unpack_bf16x2(pk.x), b = rte::unpack_bf16x2(pk.y);
              dyv[u][i] = make_float4(a.x, a.y, b.x, b.y);
            } else {
              dyv[u][i] = reinterpret_cast<const float4*>(dy32 + (size_t)rw[u] * d)[c];
            }
          }
        }
      }
      float dot[2] = {0.f, 0.f};
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < d4) {
          const float4 ww = w ? reinterpret_cast<const float4*>(w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const float r = rr[u];
            const float4 xv = xh[u][i], dv = dyv[u][i];
            const float4 h = make_float4(xv.x * r, xv.y * r, xv.z * r, xv.w * r);
            xh[u][i] = h;
            if (want_w) { aw[i].x += dv.x * h.x; aw[i].y += dv.y * h.y; aw[i].z += dv.z * h.z; aw[i].w += dv.w * h.w; }
            g[u][i] = make_float4(dv.x * ww.x, dv.y * ww.y, dv.z * ww.z, dv.w * ww.w);
            dot[u] += g[u][i].x * h.x + g[u][i].y * h.y + g[u][i].z * h.z + g[u][i].w * h.w;
          }
        }
      }
      dot[0] = warp_sum(dot[0]) / (float)d;
      dot[1] = warp_sum(dot[1]) / (float)d;
      if (dres) {                                    // the residual gradient of both rows, loads first
#pragma unroll
        for (int u = 0; u < 2; ++u)
#pragma unroll
          for (int i = 0; i < NV; ++i) {
            const int c = lane + 32 * i;
            if (c < d4) dyv[u][i] = reinterpret_cast<const float4*>(dres + (size_t)rw[u] * d)[c];
          }
      }
#pragma unroll
      for (int u = 0; u < 2; ++u)
#pragma unroll
        for (int i = 0; i < NV; ++i) {
          const int c = lane + 32 * i;
          if (c < d4) {
            const float r = rr[u], dt = dot[u];
            float4 o = make_float4(r * (g[u][i].x - xh[u][i].x * dt), r * (g[u][i].y - xh[u][i].y * dt),
                                   r * (g[u][i].z - xh[u][i].z * dt), r * (g[u][i].w - xh[u][i].w * dt));
            if (dres) { const float4 t = dyv[u][i]; o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w; }
            if (dx32) reinterpret_cast<float4*>(dx32 + (size_t)rw[u] * d)[c] = o;
            if (dx16) {
              uint2 pk = make_uint2(rte::pack_bf16x2(o.x, o.y), rte::pack_bf16x2(o.z, o.w));
              reinterpret_cast<uint2*>(dx16 + (size_t)rw[u] * d)[c] = pk;
            }
          }
        }
    }
  }
  for (; row < rows; row += stride) {
    const float r = rstd[row];
    const float4* xr = reinterpret_cast<const float4*>(x + (size_t)row * d);
    float4 xh[NV], g[NV];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < d4) {
        float4 xv = xr[c];
        xh[i] = make_float4(xv.x * r, xv.y * r, xv.z * r, xv.w * r);
        float4 dyv;
        if (dy16) {
          const uint2 pk = reinterpret_cast<const uint2*>(dy16 + (size_t)row * d)[c];
          const float2 a = rte::unpack_bf16x2(pk.x), b = rte::unpack_bf16x2(pk.y);
          dyv = make_float4(a.x, a.y, b.x, b.y);
        } else {
          dyv = reinterpret_cast<const float4*>(dy32 + (size_t)row * d)[c];
          for (int s = 1; s < dy_splits; ++s) {
            const float4 t = reinterpret_cast<const float4*>(dy32 + (size_t)s * dy_stride + (size_t)row * d)[c];
            dyv.x += t.x; dyv.y += t.y; dyv.z += t.z; dyv.w += t.w;
          }
        }
        float4 ww = w ? reinterpret_cast<const float4*>(w)[c] : make_float4(1.f, 1.f, 1.f, 1.f);
        float4 f1 = make_float4(1.f, 1.f, 1.f, 1.f);
        if (FILM && fg) {
          const float4 t = reinterpret_cast<const float4*>(fg)[c];
          f1 = make_float4(1.f + t.x, 1.f + t.y, 1.f + t.z, 1.f + t.w);
        }
        if (want_w) {
          aw[i].x += dyv.x * f1.x * xh[i].x; aw[i].y += dyv.y * f1.y * xh[i].y;
          aw[i].z += dyv.z * f1.z * xh[i].z; aw[i].w += dyv.w * f1.w * xh[i].w;
        }
        if constexpr (FILM) {
          if (want_f) {
            ag[i].x += dyv.x * xh[i].x * ww.x; ag[i].y += dyv.y * xh[i].y * ww.y;
            ag[i].z += dyv.z * xh[i].z * ww.z; ag[i].w += dyv.w * xh[i].w * ww.w;
            ab[i].x += dyv.x; ab[i].y += dyv.y; ab[i].z += dyv.z; ab[i].w += dyv.w;
          }
        }
        g[i] = make_float4(dyv.x * f1.x * ww.x, dyv.y * f1.y * ww.y, dyv.z * f1.z * ww.z, dyv.w * f1.w * ww.w);
        dot += g[i].x * xh[i].x + g[i].y * xh[i].y + g[i].z * xh[i].z + g[i].w * xh[i].w;
      }
    }
    dot = warp_sum(dot) / (float)d;
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < d4) {
        float4 o = make_float4(r * (g[i].x - xh[i].x * dot), r * (g[i].y - xh[i].y * dot),
                               r * (g[i].z - xh[i].z * dot), r * (g[i].w - xh[i].w * dot));
        if (dres) {
          const float4 t = reinterpret_cast<const float4*>(dres + (size_t)row * d)[c];
          o.x += t.x; o.y += t.y; o.z += t.z; o.w += t.w;
        }
        if (dx32) reinterpret_cast<float4*>(dx32 + (size_t)row * d)[c] = o;
        if (dx16) {
          uint2 pk = make_uint2(rte::pack_bf16x2(o.x, o.y), rte::pack_bf16x2(o.z, o.w));
          reinterpret_cast<uint2*>(dx16 + (size_t)row * d)[c] = pk;
        }
      }
    }
  }
  if (!want_w && !want_f) return;
  // combine the warps' column sums
  float* sw = sm;
  float* sg = sm + (size_t)nwarp * d;
  float* sb = sm + (size_t)2 * nwarp * d;
#pragma unroll
  for (int i = 0; i < NV; ++i) {
    const int c = lane + 32 * i;
    if (c < d4) {
      if (want_w) reinterpret_cast<float4*>(sw + (size_t)warp * d)[c] = aw[i];
      if constexpr (FILM) {
        if (want_f) {
          reinterpret_cast<float4*>(sg + (size_t)warp * d)[c] = ag[i];
          reinterpret_cast<float4*>(sb + (size_t)warp * d)[c] = ab[i];
        }
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < d; c += blockDim.x) {
    float tw = 0.f, tg = 0.f, tb = 0.f;
    for (int k = 0; k < nwarp; ++k) {
      if (want_w) tw += sw[(size_t)k * d + c];
      if (want_f) { tg += sg[(size_t)k * d + c]; tb += sb[(size_t)k * d + c]; }
    }
    if (want_w) dw_part[(size_t)blockIdx.x * d + c] = tw;
    if (want_f) { dg_part[(size_t)blockIdx.x * d + c] = tg; db_part[(size_t)blockIdx.x * d + c] = tb; }
  }
}

// 32 columns x 32 row-groups per CTA: thirty-two partial sums per column, combined through shared memory in a
// fixed order (deterministic).
__global__ void __launch_bounds__(1024)
colsum_kernel(const float* __restrict__ part, int n_rows, int d, float* __restrict__ out, int accumulate) {
  __shared__ float sm[32][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < d) {
#pragma unroll 4
    for (int r = ty; r < n_rows; r += 32) s += part[(size_t)r * d + c];
  }
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sm[k][tx];
    out[c] = accumulate ? out[c] + t : t;
  }
}

// Up to three column sums of equally shaped partial buffers in one launch (blockIdx.y selects the buffer).
struct ColsumJob { const float* part; float* out; int accumulate; };
struct ColsumJobs { ColsumJob j[3]; };

__global__ void __launch_bounds__(1024)
colsum3_kernel(ColsumJobs jobs, int n_rows, int d) {
  __shared__ float sm[32][33];
  const ColsumJob job = jobs.j[blockIdx.y];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + tx;
  float s = 0.f;
  if (c < d) {
#pragma unroll 4
    for (int r = ty; r < n_rows; r += 32) s += job.part[(size_t)r * d + c];
  }
  sm[ty][tx] = s;
  __syncthreads();
  if (ty == 0 && c < d) {
    float t = 0.f;
#pragma unroll
    for (int k = 0; k < 32; ++k) t += sm[k][tx];
    job.out[c] = job.accumulate ? job.out[c] + t : t;
  }
}

// ------------------------------------------------------------------ cross entropy
// One CTA per token row; logits read twice from L2/HBM (max+sum pass, gradient pass).
__global__ void __launch_bounds__(256)
ce_kernel(const __nv_bfloat16* __restrict__ logits, int ldl, const int64_t* __restrict__ targets,
          const float* __restrict__ row_weight, int S, float* __restrict__ loss_tok,
          __nv_bfloat16* __restrict__ dlogits, int rows, int V, int* status) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  if (row >= rows) return;
  const __nv_bfloat16* lr = logits + (size_t)row * ldl;
  long long tgt = targets[row];
  if (tgt < 0 || tgt >= V) {
    if (status && threadIdx.x == 0) atomicExch(status, RTE_DEV_INDEX_OUT_OF_RANGE);
    tgt = 0;
  }
  const int V8 = ((ldl % 8) == 0 && (reinterpret_cast<uintptr_t>(logits) & 15) == 0) ? (V >> 3) : 0;
  float mx = -INFINITY;
  for (int c = threadIdx.x; c < V8; c += blockDim.x) {
    const uint4 pk = reinterpret_cast<const uint4*>(lr)[c];
    const float2 a = rte::unpack_bf16x2(pk.x), b = rte::unpack_bf16x2(pk.y), cc = rte::unpack_bf16x2(pk.z), dd = rte::unpack_bf16x2(pk.w);
    mx = fmaxf(mx, fmaxf(fmaxf(fmaxf(a.x, a.y), fmaxf(b.x, b.y)), fmaxf(fmaxf(cc.x, cc.y), fmaxf(dd.x, dd.y))));
  }
  for (int c = V8 * 8 + threadIdx.x; c < V; c += blockDim.x) mx = fmaxf(mx, __bfloat162float(lr[c]));
  mx = block_max(mx, red);
  float se = 0.f;
  for (int c = threadIdx.x; c < V8; c += blockDim.x) {
    const uint4 pk = reinterpret_cast<const uint4*>(lr)[c];
    const float2 a = rte::unpack_bf16x2(pk.x), b = rte::unpack_bf16x2(pk.y), cc = rte::unpack_bf16x2(pk.z), dd = rte::unpack_bf16x2(pk.w);
    se += __expf(a.x - mx) + __expf(a.y - mx) + __expf(b.x - mx) + __expf(b.y - mx) + __expf(cc.x - mx) +
          __expf(cc.y - mx) + __expf(dd.x - mx) + __expf(dd.y - mx);
  }
  for (int c = V8 * 8 + threadIdx.x; c < V; c += blockDim.x) se += __expf(__bfloat162float(lr[c]) - mx);
  se = block_sum(se, red);
  const float lse = mx + __logf(se);
  const float tl = __bfloat162float(lr[tgt]);
  if (threadIdx.x == 0) loss_tok[row] = lse - tl;
  if (dlogits == nullptr) return;
  __syncthreads();   // every thread has read lr[tgt] before an aliasing dlogits row is overwritten
  const float wgt = row_weight[row / S];
  __nv_bfloat16* dr = dlogits + (size_t)row * ldl;
  for (int c = threadIdx.x; c < V8; c += blockDim.x) {
    const uint4 pk = reinterpret_cast<const uint4*>(lr)[c];
    const float2 a = rte::unpack_bf16x2(pk.x), b = rte::unpack_bf16x2(pk.y), cc = rte::unpack_bf16x2(pk.z), dd = rte::unpack_bf16x2(pk.w);
    float v[8] = {a.x, a.y, b.x, b.y, cc.x, cc.y, dd.x, dd.y};
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float pr = __expf(v[j] - lse);
      v[j] = wgt * (pr - ((c * 8 + j) == tgt ? 1.f : 0.f));
    }
    uint4 o;
    o.x = rte::pack_bf16x2(v[0], v[1]); o.y = rte::pack_bf16x2(v[2], v[3]);
    o.z = rte::pack_bf16x2(v[4], v[5]); o.w = rte::pack_bf16x2(v[6], v[7]);
    reinterpret_cast<uint4*>(dr)[c] = o;
  }
  for (int c = V8 * 8 + threadIdx.x; c < V; c += blockDim.x) {
    const float pr = __expf(__bfloat162float(lr[c]) - lse);
    dr[c] = __float2bfloat16_rn(wgt * (pr - (c == tgt ? 1.f : 0.f)));
  }
}

__global__ void segment_sum_kernel(const float* __restrict__ in, float* __restrict__ out, int n_seg, int seg_len) {
  __shared__ float red[32];
  const int seg = blockIdx.x;
  if (seg >= n_seg) return;
  float s = 0.f;
  for (int i = threadIdx.x; i < seg_len; i += blockDim.x) s += in[(size_t)seg * seg_len + i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) out[seg] = s;
}

// ------------------------------------------------------------------ small vector kernels
__global__ void reduce_splits_kernel(const float* __restrict__ ws, int splits, long long stride, long long n4,
                                     float* __restrict__ out, int accumulate) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    float4 acc = accumulate ? reinterpret_cast<float4*>(out)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < splits; ++s) {
      const float4 t = reinterpret_cast<const float4*>(ws + (size_t)s * stride)[i];
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    reinterpret_cast<float4*>(out)[i] = acc;
  }
}
__global__ void reduce_splits_tail_kernel(const float* __restrict__ ws, int splits, long long stride, long long start,
                                          long long n, float* __restrict__ out, int accumulate) {
  const long long i = start + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if (i >= n) return;
  float acc = accumulate ? out[i] : 0.f;
  for (int s = 0; s < splits; ++s) acc += ws[(size_t)s * stride + i];
  out[i] = acc;
}

__global__ void cast_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
  const long long n4 = n >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 t = reinterpret_cast<const float4*>(src)[i];
    reinterpret_cast<uint2*>(dst)[i] = make_uint2(rte::pack_bf16x2(t.x, t.y), rte::pack_bf16x2(t.z, t.w));
  }
  for (long long i = n4 * 4 + blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    dst[i] = __float2bfloat16_rn(src[i]);
}
__global__ void fill_kernel(float* __restrict__ dst, float value, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] = value;
}
__global__ void add_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] += src[i];
}
__global__ void add_guarded_kernel(float* __restrict__ dst, const float* __restrict__ src, long long n, const int32_t* __restrict__ skip) {
  if (*skip != 0) return;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) dst[i] += src[i];
}
__global__ void axpy_rows_kernel(float* __restrict__ dst, const float* __restrict__ vec, float alpha, int rows, int seg, int d) {
  const long long total = (long long)rows * d;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / d), c = int(i % d);
    dst[i] += alpha * vec[(size_t)(r / seg) * d + c];
  }
}

// ------------------------------------------------------------------ AdamW
// `skip` (optional device flag): non-zero turns the whole launch into a no-op -- parameters, moments, shadows and step
// counters stay as they are (the reference drops a step whose loss is not finite, training.py:448-452).
// `metric_partial` (optional, [chunks][2]): per-chunk sums of (grad_scale * g)^2 and of p^2 BEFORE the update, the
// raw material of the per-group gradient / parameter norms (training.py:386-443); reduced by adamw_metric_kernel.
__global__ void __launch_bounds__(256)
adamw_kernel(const rte_adamw_tensor* __restrict__ table, const int32_t* __restrict__ chunk_tensor,
             const int32_t* __restrict__ chunk_index, const float* __restrict__ lr_table,
             const int32_t* __restrict__ step_count, float beta1, float beta2, float eps, float wd,
             const float* __restrict__ grad_scale, const int32_t* __restrict__ skip, float* __restrict__ metric_partial,
             const int32_t* __restrict__ absent_flag, const uint8_t* __restrict__ absent_mask) {
  __shared__ float red[32];
  const int ti = chunk_tensor[blockIdx.x];
  // dropped step, or a tensor that received no gradient in this step (torch.optim.AdamW skips `grad is None`: no decay,
  // no moment update, no step count)
  if ((skip != nullptr && *skip != 0) || (absent_flag != nullptr && *absent_flag != 0 && absent_mask[ti] != 0)) {
    if (metric_partial != nullptr && threadIdx.x == 0) { metric_partial[2 * blockIdx.x] = 0.f; metric_partial[2 * blockIdx.x + 1] = 0.f; }
    return;
  }
  const rte_adamw_tensor t = table[ti];
  const long long base = (long long)chunk_index[blockIdx.x] * RTE_ADAMW_CHUNK;
  const float lr = lr_table[t.lr_group];
  const float step = (float)(step_count[t.step_slot] + 1);   // incremented by adamw_step_kernel afterwards
  const float bc1 = 1.f - powf(beta1, step), bc2 = 1.f - powf(beta2, step);
  const float gs = grad_scale ? *grad_scale : 1.f;
  const float step_size = lr / bc1, inv_sqrt_bc2 = rsqrtf(bc2), decay = 1.f - lr * wd;
  __nv_bfloat16* shadow = reinterpret_cast<__nv_bfloat16*>(t.bf16_shadow);
  float gsq = 0.f, psq = 0.f;
#pragma unroll 4
  for (int j = threadIdx.x; j < RTE_ADAMW_CHUNK; j += blockDim.x) {
    const long long i = base + j;
    if (i >= t.n) break;
    const float g = t.g[i] * gs;
    const float p0 = t.p[i];
    gsq += g * g; psq += p0 * p0;
    float p = p0 * decay;
    const float m = beta1 * t.m[i] + (1.f - beta1) * g;
    const float v = beta2 * t.v[i] + (1.f - beta2) * g * g;
    p -= step_size * m / (sqrtf(v) * inv_sqrt_bc2 + eps);
    t.p[i] = p; t.m[i] = m; t.v[i] = v;
    if (shadow) shadow[i] = __float2bfloat16_rn(p);
  }
  if (metric_partial != nullptr) {       // uniform branch: every thread of the block takes part in the reductions
    gsq = block_sum(gsq, red);
    psq = block_sum(psq, red);
    if (threadIdx.x == 0) { metric_partial[2 * blockIdx.x] = gsq; metric_partial[2 * blockIdx.x + 1] = psq; }
  }
}
__global__ void adamw_step_kernel(const rte_adamw_tensor* __restrict__ table, int n_tensors, int32_t* step_count,
                                  const int32_t* __restrict__ skip, const int32_t* __restrict__ absent_flag,
                                  const uint8_t* __restrict__ absent_mask) {
  if (skip != nullptr && *skip != 0) return;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_tensors && !(absent_flag != nullptr && *absent_flag != 0 && absent_mask[i] != 0)) step_count[table[i].step_slot] += 1;
}
// out[2*g] = sum of grad^2, out[2*g+1] = sum of param^2 over the chunks of the tensors of metric group g = blockIdx.x
// (fixed summation order: reproducible).
__global__ void __launch_bounds__(256)
adamw_metric_kernel(const int32_t* __restrict__ chunk_tensor, const int32_t* __restrict__ metric_group, long long total_chunks,
                    const float* __restrict__ partial, float* __restrict__ out) {
  __shared__ float red[32];
  float a = 0.f, b = 0.f;
  for (long long c = threadIdx.x; c < total_chunks; c += blockDim.x)
    if (metric_group[chunk_tensor[c]] == (int)blockIdx.x) { a += partial[2 * c]; b += partial[2 * c + 1]; }
  a = block_sum(a, red);
  b = block_sum(b, red);
  if (threadIdx.x == 0) { out[2 * blockIdx.x] = a; out[2 * blockIdx.x + 1] = b; }
}
// skip = 1 (and flag_out = 1.0) when any of the listed values is not finite, else 0.
__global__ void __launch_bounds__(256)
nonfinite_guard_kernel(const float* __restrict__ a, int na, const float* __restrict__ b, int nb, const float* __restrict__ c, int nc,
                       int32_t* skip, float* flag_out) {
  __shared__ int bad;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  int mine = 0;
  for (int i = threadIdx.x; i < na; i += blockDim.x) mine |= !isfinite(a[i]);
  for (int i = threadIdx.x; i < nb; i += blockDim.x) mine |= !isfinite(b[i]);
  for (int i = threadIdx.x; i < nc; i += blockDim.x) mine |= !isfinite(c[i]);
  if (mine) atomicOr(&bad, 1);
  __syncthreads();
  if (threadIdx.x == 0) { *skip = bad; if (flag_out) *flag_out = bad ? 1.f : 0.f; }
}

__global__ void __launch_bounds__(256)
gradnorm_partial_kernel(const rte_adamw_tensor* __restrict__ table, const int32_t* __restrict__ chunk_tensor,
                        const int32_t* __restrict__ chunk_index, float* __restrict__ partial) {
  __shared__ float red[32];
  const rte_adamw_tensor t = table[chunk_tensor[blockIdx.x]];
  const long long base = (long long)chunk_index[blockIdx.x] * RTE_ADAMW_CHUNK;
  float s = 0.f;
  for (int j = threadIdx.x; j < RTE_ADAMW_CHUNK; j += blockDim.x) {
    const long long i = base + j;
    if (i < t.n) { const float g = t.g[i]; s += g * g; }
  }
  s = block_sum(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}
__global__ void gradnorm_final_kernel(const float* __restrict__ partial, long long n, float* sumsq, float max_norm, float* clip_coef) {
  __shared__ float red[32];
  float s = 0.f;
  for (long long i = threadIdx.x; i < n; i += blockDim.x) s += partial[i];
  s = block_sum(s, red);
  if (threadIdx.x == 0) {
    sumsq[0] = s;
    if (clip_coef) clip_coef[0] = max_norm > 0.f ? fminf(1.f, max_norm / (sqrtf(s) + 1e-6f)) : 1.f;
  }
}

// ------------------------------------------------------------------ built-in scratch for the no-allocation gradient norm
// Lives in the library image: every GPU that loads the library carries these 256 KB until the process ends.
// In HOST code the name `g_gradnorm_scratch` is only a stand-in for the symbol, not a device address, so the
// launcher below asks the runtime for the real address (once per device) and hands that to the kernels.
constexpr long long GRADNORM_STATIC_MAX_CHUNKS = 65536;   // 65536 chunks x 4096 elements = 268M gradient elements
static __device__ __align__(256) float g_gradnorm_scratch[GRADNORM_STATIC_MAX_CHUNKS];

constexpr int MAX_DEVICES = 64;
float* g_gradnorm_scratch_addr[MAX_DEVICES] = {nullptr};

// Returns the device address of the scratch array on the CURRENT device (looked up on first use).  The cache is
// written without a lock: two host threads that make the first call on a device at the same time both look the
// address up and store the same value, which is harmless.
int gradnorm_scratch_for_current_device(float** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return RTE_ERR_NO_DEVICE;
  if (g_gradnorm_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    if (cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_gradnorm_scratch) != cudaSuccess || ptr == nullptr)
      return RTE_ERR_LAUNCH;
    g_gradnorm_scratch_addr[dev] = ptr;
  }
  *out = g_gradnorm_scratch_addr[dev];
  return RTE_OK;
}

// ------------------------------------------------------------------ top-k, ties to the lowest index
// One warp per row.  k rounds of a warp arg-max over (value desc, index asc); a selected entry is
// masked by remembering the previous winner's (value, index) and only admitting strictly "later"
// candidates in that order, so no scratch copy of the row is needed.
__global__ void __launch_bounds__(256)
topk_kernel(const float* __restrict__ scores, int ld, int rows, int n, int k, int32_t* __restrict__ idx, float* __restrict__ vals) {
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= rows) return;
  const float* sr = scores + (size_t)row * ld;
  float pv = INFINITY; int pi = -1;      // previous winner; first round admits everything
  for (int r = 0; r < k; ++r) {
    float bv = -INFINITY; int bi = 0x7fffffff;
    for (int c = lane; c < n; c += 32) {
      const float v = sr[c];
      const bool after_prev = (v < pv) || (v == pv && c > pi);
      const bool better = (v > bv) || (v == bv && c < bi);
      if (after_prev && better) { bv = v; bi = c; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if (lane == 0) {
      if (idx) idx[(size_t)row * k + r] = bi;
      if (vals) vals[(size_t)row * k + r] = bv;
    }
    pv = bv; pi = bi;
  }
}

inline int grid_for(long long n, int block, int cap = 148 * 16) {
  long long g = (n + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

// SwiGLU as a pass of its own over a saved (up | gate) buffer: 8 hidden units per thread, 16-byte accesses.
__device__ __forceinline__ void unpack8(const uint4& t, float (&v)[8]) {
  const float2 a = rte::unpack_bf16x2(t.x), b = rte::unpack_bf16x2(t.y), c = rte::unpack_bf16x2(t.z), d = rte::unpack_bf16x2(t.w);
  v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y; v[4] = c.x; v[5] = c.y; v[6] = d.x; v[7] = d.y;
}
__device__ __forceinline__ uint4 pack8(const float (&v)[8]) {
  return make_uint4(rte::pack_bf16x2(v[0], v[1]), rte::pack_bf16x2(v[2], v[3]), rte::pack_bf16x2(v[4], v[5]), rte::pack_bf16x2(v[6], v[7]));
}
__global__ void __launch_bounds__(256)
swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ ug, __nv_bfloat16* __restrict__ z, long long rows, int F) {
  const int f8 = F >> 3;
  const long long total = rows * f8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / f8;
    const int j = int(i % f8) << 3;
    float up[8], g[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(ug + r * 2 * F + j), up);
    unpack8(*reinterpret_cast<const uint4*>(ug + r * 2 * F + F + j), g);
#pragma unroll
    for (int k = 0; k < 8; ++k) o[k] = up[k] * rte::silu_f(g[k]);
    *reinterpret_cast<uint4*>(z + r * F + j) = pack8(o);
  }
}
__global__ void __launch_bounds__(256)
swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ ug, const __nv_bfloat16* __restrict__ dz, __nv_bfloat16* __restrict__ dug,
                  long long rows, int F) {
  const int f8 = F >> 3;
  const long long total = rows * f8;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / f8;
    const int j = int(i % f8) << 3;
    float up[8], g[8], d[8], du[8], dg[8];
    unpack8(*reinterpret_cast<const uint4*>(ug + r * 2 * F + j), up);
    unpack8(*reinterpret_cast<const uint4*>(ug + r * 2 * F + F + j), g);
    unpack8(*reinterpret_cast<const uint4*>(dz + r * F + j), d);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = rte::sigmoid_f(g[k]);
      du[k] = d[k] * g[k] * sg;
      dg[k] = d[k] * up[k] * sg * (1.f + g[k] * (1.f - sg));
    }
    *reinterpret_cast<uint4*>(dug + r * 2 * F + j) = pack8(du);
    *reinterpret_cast<uint4*>(dug + r * 2 * F + F + j) = pack8(dg);
  }
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" const char* rte_backend_name(void) { return "cuda_sm100a_ext"; }

extern "C" const char* rte_status_string(int code) {
  switch (code) {
    case RTE_OK: return "ok";
    case RTE_ERR_BAD_ARG: return "bad argument";
    case RTE_ERR_ALIGNMENT: return "pointer or stride not 16-byte aligned";
    case RTE_ERR_TENSOR_MAP: return "tensor map creation failed";
    case RTE_ERR_LAUNCH: return "kernel launch failed";
    case RTE_ERR_UNSUPPORTED: return "unsupported size";
    case RTE_ERR_NO_DEVICE: return "no CUDA device";
    case RTE_ERR_SCRATCH_CAPACITY: return "size exceeds the capacity of the library's built-in scratch array";
    case RTE_DEV_WAIT_TIMEOUT_PRODUCER: return "device: TMA producer wait ran out";
    case RTE_DEV_WAIT_TIMEOUT_MMA: return "device: MMA issuer wait ran out";
    case RTE_DEV_WAIT_TIMEOUT_EPILOGUE: return "device: epilogue wait ran out";
    case RTE_DEV_WAIT_TIMEOUT_PEER: return "device: wait for a data-parallel peer ran out";
    case RTE_DEV_INDEX_OUT_OF_RANGE: return "device: index out of range";
    case RTE_DEV_CAPACITY_OVERFLOW: return "device: packed rows exceed the caller's capacity";
    default: return "unknown";
  }
}

extern "C" int rte_embed_fwd(const int64_t* tokens, const float* table, float* out, int32_t n_tokens, int32_t d,
                             int32_t vocab, int32_t* status, rte_stream_t stream) {
  RTE_CHECK_ARG(tokens && table && out && n_tokens > 0 && d > 0 && d % 4 == 0);
  embed_fwd_kernel<<<grid_for((long long)n_tokens * (d / 4), 256), 256, 0, ST(stream)>>>(tokens, table, out, n_tokens, d, vocab, status);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
extern "C" int rte_embed_bwd(const int64_t* tokens, const float* dx, float* dtable, int64_t* accum, int32_t n_tokens,
                             int32_t d, int32_t vocab, int32_t* status, rte_stream_t stream) {
  RTE_CHECK_ARG(tokens && dx && dtable && accum && n_tokens > 0 && d > 0 && vocab > 0);
  const long long n = (long long)vocab * d;
  if (cudaMemsetAsync(accum, 0, (size_t)n * sizeof(int64_t), ST(stream)) != cudaSuccess) return RTE_ERR_LAUNCH;
  embed_bwd_accum_kernel<<<grid_for((long long)n_tokens * d, 256), 256, 0, ST(stream)>>>(
      tokens, dx, reinterpret_cast<unsigned long long*>(accum), dtable, n_tokens, d, vocab, status);
  embed_bwd_apply_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(reinterpret_cast<const unsigned long long*>(accum), dtable, n);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_rmsnorm_fwd(const float* x, const float* w, const float* film_gamma, const float* film_beta,
                               void* y_bf16, float* y_f32, float* rstd, int32_t rows, int32_t d, float eps,
                               rte_stream_t stream) {
  RTE_CHECK_ARG(x && rows > 0 && d > 0 && d % 4 == 0 && (y_bf16 || y_f32));
  RTE_CHECK_ARG((film_gamma == nullptr) == (film_beta == nullptr));
  if (d > 128 * RN_MAX_V4) return RTE_ERR_UNSUPPORTED;
#define RTE_RN_FWD(NV)                                                                            \
  rmsnorm_fwd_kernel<NV><<<rte::ceil_div(rows, 8), 256, 0, ST(stream)>>>(x, w, film_gamma, film_beta, \
      reinterpret_cast<__nv_bfloat16*>(y_bf16), y_f32, rstd, rows, d, eps)
  if (d <= 128) RTE_RN_FWD(1);
  else if (d <= 256) RTE_RN_FWD(2);
  else if (d <= 512) RTE_RN_FWD(4);
  else if (d <= 1024) RTE_RN_FWD(8);
  else RTE_RN_FWD(16);
#undef RTE_RN_FWD
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_residual_rmsnorm_fwd(const float* base, const float* branch, const float* scale, const int32_t* active,
                                        const float* passthrough, int32_t S, const float* add2, const float* scale2,
                                        float* x1_out, float* x_out, const float* w, const float* film_gamma,
                                        const float* film_beta, void* y_bf16, float* rstd, int32_t rows, int32_t d, float eps,
                                        rte_stream_t stream) {
  return rte_residual_rmsnorm_fwd_splits(base, branch, 1, 0, nullptr, scale, active, passthrough, S, add2, scale2, x1_out, x_out,
                                         w, film_gamma, film_beta, y_bf16, rstd, rows, d, eps, stream);
}

extern "C" int rte_residual_rmsnorm_fwd_splits(const float* base, const float* branch, int32_t branch_splits,
                                               int64_t branch_split_stride, float* branch_out, const float* scale,
                                               const int32_t* active, const float* passthrough, int32_t S, const float* add2,
                                               const float* scale2, float* x1_out, float* x_out, const float* w,
                                               const float* film_gamma, const float* film_beta, void* y_bf16, float* rstd,
                                               int32_t rows, int32_t d, float eps, rte_stream_t stream) {
  RTE_CHECK_ARG(base && branch && scale && x_out && y_bf16 && rows > 0 && d > 0 && d % 4 == 0 && S > 0);
  RTE_CHECK_ARG(branch_splits >= 1 && (branch_splits == 1 || (branch_split_stride % 4 == 0 && branch_split_stride >= (int64_t)rows * d)));
  RTE_CHECK_ARG((active == nullptr || passthrough != nullptr) && (add2 == nullptr || scale2 != nullptr));
  RTE_CHECK_ARG((film_gamma == nullptr) == (film_beta == nullptr));
  if (d > 128 * RN_MAX_V4) return RTE_ERR_UNSUPPORTED;
#define RTE_RRN_FWD(NV)                                                                                              \
  residual_rmsnorm_fwd_kernel<NV><<<rte::ceil_div(rows, 8), 256, 0, ST(stream)>>>(base, branch, scale, active, passthrough, \
      S, add2, scale2, x1_out, x_out, w, film_gamma, film_beta, reinterpret_cast<__nv_bfloat16*>(y_bf16), rstd, rows, d, eps, \
      branch_splits, (long long)branch_split_stride, branch_out)
  if (d <= 128) RTE_RRN_FWD(1);
  else if (d <= 256) RTE_RRN_FWD(2);
  else if (d <= 512) RTE_RRN_FWD(4);
  else if (d <= 1024) RTE_RRN_FWD(8);
  else RTE_RRN_FWD(16);
#undef RTE_RRN_FWD
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_rmsnorm_bwd(const float* x, const float* w, const float* film_gamma, const float* rstd,
                               const void* dy_bf16, const float* dy_f32, const float* dres, float* dx_f32,
                               void* dx_bf16, float* dw_partial, float* dgamma_partial, float* dbeta_partial,
                               int32_t rows, int32_t d, int32_t max_partials, int32_t* n_partials,
                               rte_stream_t stream) {
  return rte_rmsnorm_bwd_splits(x, w, film_gamma, rstd, dy_bf16, dy_f32, 1, 0, dres, dx_f32, dx_bf16, dw_partial, dgamma_partial,
                                dbeta_partial, rows, d, max_partials, n_partials, stream);
}

extern "C" int rte_rmsnorm_bwd_splits(const float* x, const float* w, const float* film_gamma, const float* rstd,
                                      const void* dy_bf16, const float* dy_f32, int32_t dy_splits, int64_t dy_split_stride,
                                      const float* dres, float* dx_f32, void* dx_bf16, float* dw_partial,
                                      float* dgamma_partial, float* dbeta_partial, int32_t rows, int32_t d,
                                      int32_t max_partials, int32_t* n_partials, rte_stream_t stream) {
  RTE_CHECK_ARG(x && rstd && rows > 0 && d > 0 && d % 4 == 0 && (dy_bf16 || dy_f32) && (dx_f32 || dx_bf16));
  RTE_CHECK_ARG(dy_splits >= 1 && (dy_splits == 1 || (dy_f32 && !dy_bf16 && dy_split_stride % 4 == 0 &&
                                                      dy_split_stride >= (int64_t)rows * d)));
  RTE_CHECK_ARG((dgamma_partial == nullptr) == (dbeta_partial == nullptr));
  if (d > 128 * RN_MAX_V4) return RTE_ERR_UNSUPPORTED;
  const bool grads = dw_partial || dgamma_partial;
  int grid = rte::ceil_div(rows, 8);
  // one wave of CTAs (each writes one partial row): three fit an SM without FiLM accumulators at d <= 512
  const int cap = 148 * ((film_gamma || dgamma_partial || d > 512) ? 2 : 3);
  if (grid > cap) grid = cap;
  if (grads) {
    RTE_CHECK_ARG(max_partials >= 1);
    if (grid > max_partials) grid = max_partials;
  }
  if (n_partials) *n_partials = grid;
  const size_t smem = grads ? (size_t)(dgamma_partial ? 3 : 1) * 8 * d * sizeof(float) : 0;
#define RTE_RN_BWD(NV)                                                                                           \
  do {                                                                                                           \
    if (film_gamma || dgamma_partial) RTE_RN_BWD_F(NV, true); else RTE_RN_BWD_F(NV, false);                      \
  } while (0)
#define RTE_RN_BWD_F(NV, FILM)                                                                                   \
  do {                                                                                                           \
    if (smem > 48 * 1024) {                                                                                      \
      static bool set = false;                                                                                   \
      if (!set) {                                                                                                \
        if (cudaFuncSetAttribute(rmsnorm_bwd_kernel<NV, FILM>, cudaFuncAttributeMaxDynamicSharedMemorySize,            \
                                 200 * 1024) != cudaSuccess)                                                     \
          return RTE_ERR_LAUNCH;                                                                                 \
        set = true;                                                                                              \
      }                                                                                                          \
    }                                                                                                            \
    rmsnorm_bwd_kernel<NV, FILM><<<grid, 256, smem, ST(stream)>>>(x, w, film_gamma, rstd,                              \
        reinterpret_cast<const __nv_bfloat16*>(dy_bf16), dy_f32, dres, dx_f32,                                   \
        reinterpret_cast<__nv_bfloat16*>(dx_bf16), dw_partial, dgamma_partial, dbeta_partial, rows, d,           \
        dy_splits, (long long)dy_split_stride);                                                                  \
  } while (0)
  if (d <= 128) RTE_RN_BWD(1);
  else if (d <= 256) RTE_RN_BWD(2);
  else if (d <= 512) RTE_RN_BWD(4);
  else if (d <= 1024) RTE_RN_BWD(8);
  else RTE_RN_BWD(16);
#undef RTE_RN_BWD
#undef RTE_RN_BWD_F
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_colsum_partials(const float* partial, int32_t n_rows, int32_t d, float* out, int32_t accumulate,
                                   rte_stream_t stream) {
  RTE_CHECK_ARG(partial && out && n_rows > 0 && d > 0);
  colsum_kernel<<<rte::ceil_div(d, 32), 1024, 0, ST(stream)>>>(partial, n_rows, d, out, accumulate);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_colsum_partials3(const float* const* partials, float* const* outs, const int32_t* accumulate, int32_t count,
                                    int32_t n_rows, int32_t d, rte_stream_t stream) {
  RTE_CHECK_ARG(partials && outs && accumulate && count >= 1 && count <= 3 && n_rows > 0 && d > 0);
  ColsumJobs jobs;
  for (int i = 0; i < 3; ++i) {
    const int k = i < count ? i : 0;
    RTE_CHECK_ARG(partials[k] && outs[k]);
    jobs.j[i] = ColsumJob{partials[k], outs[k], accumulate[k]};
  }
  colsum3_kernel<<<dim3(rte::ceil_div(d, 32), count), 1024, 0, ST(stream)>>>(jobs, n_rows, d);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_ce_fwd_bwd(const void* logits, int32_t ldl, const int64_t* targets, const float* row_weight,
                              int32_t S, float* loss_tok, void* dlogits, int32_t rows, int32_t V, int32_t* status,
                              rte_stream_t stream) {
  RTE_CHECK_ARG(logits && targets && loss_tok && rows > 0 && V > 0 && ldl >= V && S > 0);
  RTE_CHECK_ARG(dlogits == nullptr || row_weight != nullptr);
  ce_kernel<<<rows, 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(logits), ldl, targets, row_weight, S,
                                          loss_tok, reinterpret_cast<__nv_bfloat16*>(dlogits), rows, V, status);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_segment_sum(const float* in, float* out, int32_t n_seg, int32_t seg_len, rte_stream_t stream) {
  RTE_CHECK_ARG(in && out && n_seg > 0 && seg_len > 0);
  segment_sum_kernel<<<n_seg, 128, 0, ST(stream)>>>(in, out, n_seg, seg_len);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_reduce_splits(const float* ws, int32_t splits, int64_t split_stride, int64_t n, float* out,
                                 int32_t accumulate, rte_stream_t stream) {
  RTE_CHECK_ARG(ws && out && splits >= 1 && n > 0);
  const bool vec = (split_stride % 4 == 0) && ((reinterpret_cast<uintptr_t>(ws) & 15) == 0) &&
                   ((reinterpret_cast<uintptr_t>(out) & 15) == 0);
  const long long n4 = vec ? (n >> 2) : 0;
  if (n4 > 0) {
    reduce_splits_kernel<<<grid_for(n4, 256), 256, 0, ST(stream)>>>(ws, splits, split_stride, n4, out, accumulate);
    RTE_LAUNCH_CHECK();
  }
  const long long rest = n - n4 * 4;
  if (rest > 0) {
    reduce_splits_tail_kernel<<<(int)rte::ceil_div64(rest, 256), 256, 0, ST(stream)>>>(ws, splits, split_stride, n4 * 4, n, out, accumulate);
    RTE_LAUNCH_CHECK();
  }
  return RTE_OK;
}

extern "C" int rte_swiglu_fwd(const void* ug, void* z, int64_t rows, int32_t F, rte_stream_t stream) {
  RTE_CHECK_ARG(ug && z && rows > 0 && F > 0 && F % 8 == 0);
  if ((reinterpret_cast<uintptr_t>(ug) & 15) || (reinterpret_cast<uintptr_t>(z) & 15)) return RTE_ERR_ALIGNMENT;
  swiglu_fwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(ug),
                                                                          reinterpret_cast<__nv_bfloat16*>(z), rows, F);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
extern "C" int rte_swiglu_bwd(const void* ug, const void* dz, void* dug, int64_t rows, int32_t F, rte_stream_t stream) {
  RTE_CHECK_ARG(ug && dz && dug && rows > 0 && F > 0 && F % 8 == 0);
  if ((reinterpret_cast<uintptr_t>(ug) & 15) || (reinterpret_cast<uintptr_t>(dz) & 15) || (reinterpret_cast<uintptr_t>(dug) & 15))
    return RTE_ERR_ALIGNMENT;
  swiglu_bwd_kernel<<<grid_for(rows * (F / 8), 256), 256, 0, ST(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(ug), reinterpret_cast<const __nv_bfloat16*>(dz), reinterpret_cast<__nv_bfloat16*>(dug), rows, F);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_cast_f32_bf16(const float* src, void* dst, int64_t n, rte_stream_t stream) {
  RTE_CHECK_ARG(src && dst && n > 0);
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 7)) return RTE_ERR_ALIGNMENT;
  cast_kernel<<<grid_for(n / 4 + 1, 256), 256, 0, ST(stream)>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), n);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
extern "C" int rte_fill_f32(float* dst, float value, int64_t n, rte_stream_t stream) {
  RTE_CHECK_ARG(dst && n > 0);
  fill_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(dst, value, n);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
extern "C" int rte_add_f32(float* dst, const float* src, int64_t n, rte_stream_t stream) {
  RTE_CHECK_ARG(src && dst && n > 0);
  add_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(dst, src, n);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
extern "C" int rte_axpy_rows_f32(float* dst, const float* vec, float alpha, int32_t rows, int32_t seg, int32_t d,
                                 rte_stream_t stream) {
  RTE_CHECK_ARG(dst && vec && rows > 0 && seg > 0 && d > 0);
  axpy_rows_kernel<<<grid_for((long long)rows * d, 256), 256, 0, ST(stream)>>>(dst, vec, alpha, rows, seg, d);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_adamw_multi_tensor_ex(const rte_adamw_tensor* table, int32_t n_tensors, int64_t total_chunks,
                                         const int32_t* chunk_tensor, const int32_t* chunk_index, const float* lr_table,
                                         int32_t* step_count, float beta1, float beta2, float eps, float weight_decay,
                                         const float* grad_scale, const rte_adamw_extras* ex, rte_stream_t stream) {
  RTE_CHECK_ARG(table && chunk_tensor && chunk_index && lr_table && step_count && n_tensors > 0 && total_chunks > 0);
  const int32_t* skip = ex ? ex->skip : nullptr;
  const int32_t* absent_flag = ex ? ex->absent_flag : nullptr;
  const uint8_t* absent_mask = ex ? ex->absent_mask : nullptr;
  RTE_CHECK_ARG((absent_flag == nullptr) == (absent_mask == nullptr));
  float* mpart = nullptr;
  if (ex && ex->metric_out) {
    RTE_CHECK_ARG(ex->metric_partial && ex->metric_group && ex->n_metric_groups > 0);
    mpart = ex->metric_partial;
  }
  adamw_kernel<<<(unsigned)total_chunks, 256, 0, ST(stream)>>>(table, chunk_tensor, chunk_index, lr_table, step_count,
                                                               beta1, beta2, eps, weight_decay, grad_scale, skip, mpart,
                                                               absent_flag, absent_mask);
  RTE_LAUNCH_CHECK();
  adamw_step_kernel<<<rte::ceil_div(n_tensors, 128), 128, 0, ST(stream)>>>(table, n_tensors, step_count, skip, absent_flag,
                                                                           absent_mask);
  RTE_LAUNCH_CHECK();
  if (mpart) {
    adamw_metric_kernel<<<ex->n_metric_groups, 256, 0, ST(stream)>>>(chunk_tensor, ex->metric_group, total_chunks, mpart,
                                                                     ex->metric_out);
    RTE_LAUNCH_CHECK();
  }
  return RTE_OK;
}

extern "C" int rte_adamw_multi_tensor(const rte_adamw_tensor* table, int32_t n_tensors, int64_t total_chunks,
                                      const int32_t* chunk_tensor, const int32_t* chunk_index, const float* lr_table,
                                      int32_t* step_count, float beta1, float beta2, float eps, float weight_decay,
                                      const float* grad_scale, rte_stream_t stream) {
  return rte_adamw_multi_tensor_ex(table, n_tensors, total_chunks, chunk_tensor, chunk_index, lr_table, step_count, beta1,
                                   beta2, eps, weight_decay, grad_scale, nullptr, stream);
}

extern "C" int rte_add_f32_guarded(float* dst, const float* src, int64_t n, const int32_t* skip, rte_stream_t stream) {
  RTE_CHECK_ARG(dst && src && skip && n > 0);
  add_guarded_kernel<<<grid_for(n, 256), 256, 0, ST(stream)>>>(dst, src, n, skip);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_nonfinite_guard(const float* a, int32_t na, const float* b, int32_t nb, const float* c, int32_t nc,
                                   int32_t* skip, float* flag_out, rte_stream_t stream) {
  RTE_CHECK_ARG(skip && na >= 0 && nb >= 0 && nc >= 0 && (a || na == 0) && (b || nb == 0) && (c || nc == 0));
  nonfinite_guard_kernel<<<1, 256, 0, ST(stream)>>>(a, na, b, nb, c, nc, skip, flag_out);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_grad_norm_multi_tensor(const rte_adamw_tensor* table, int64_t total_chunks, const int32_t* chunk_tensor,
                                          const int32_t* chunk_index, float* partial, float* sumsq, float max_norm,
                                          float* clip_coef, rte_stream_t stream) {
  RTE_CHECK_ARG(table && chunk_tensor && chunk_index && partial && sumsq && total_chunks > 0);
  gradnorm_partial_kernel<<<(unsigned)total_chunks, 256, 0, ST(stream)>>>(table, chunk_tensor, chunk_index, partial);
  RTE_LAUNCH_CHECK();
  gradnorm_final_kernel<<<1, 1024, 0, ST(stream)>>>(partial, total_chunks, sumsq, max_norm, clip_coef);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

// Same result as rte_grad_norm_multi_tensor, but the per-chunk partial sums go to the library's own
// built-in array instead of a caller-supplied buffer: nothing is allocated here or by the caller.
// The first call on a device looks up the array's device address (a host-side runtime query, not a launch).
// Each call first overwrites every slot it later reads, so nothing has to be cleared between calls; but all
// calls on one device share the one array, so two calls whose kernels overlap in time would corrupt each other.
extern "C" int rte_grad_norm_multi_tensor_static(const rte_adamw_tensor* table, int64_t total_chunks,
                                                 const int32_t* chunk_tensor, const int32_t* chunk_index, float* sumsq,
                                                 float max_norm, float* clip_coef, rte_stream_t stream) {
  RTE_CHECK_ARG(table && chunk_tensor && chunk_index && sumsq && total_chunks > 0);
  if (total_chunks > GRADNORM_STATIC_MAX_CHUNKS) return RTE_ERR_SCRATCH_CAPACITY;
  float* partial = nullptr;
  const int rc = gradnorm_scratch_for_current_device(&partial);
  if (rc != RTE_OK) return rc;
  gradnorm_partial_kernel<<<(unsigned)total_chunks, 256, 0, ST(stream)>>>(table, chunk_tensor, chunk_index, partial);
  RTE_LAUNCH_CHECK();
  gradnorm_final_kernel<<<1, 1024, 0, ST(stream)>>>(partial, total_chunks, sumsq, max_norm, clip_coef);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_topk_lowest_index(const float* scores, int32_t ld, int32_t rows, int32_t n, int32_t k,
                                     int32_t* idx, float* vals, rte_stream_t stream) {
  RTE_CHECK_ARG(scores && rows > 0 && n > 0 && k > 0 && k <= n && ld >= n && (idx || vals));
  topk_kernel<<<rte::ceil_div(rows, 8), 256, 0, ST(stream)>>>(scores, ld, rows, n, k, idx, vals);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
