// Helpers of the exact-audit replay: the audited samples (a fixed, small count per batch) are run through the
// banked recurrent core with the router's per-pass recipe choices applied as COLUMN MASKS read from tables, so
// that no tensor shape depends on a routing decision and the replay can sit in the same CUDA graph as the hot
// pass.  Everything here is small (n*S tokens, n = audited samples) and bandwidth-trivial; the point of these
// kernels is to keep the whole step on the device without host branches.

#include <cooperative_groups.h>

#include "rte_common.cuh"

namespace cg = cooperative_groups;

namespace {

constexpr int NTHR = 256;

inline int grid_for(long long n, int block, int cap = 148 * 8) {
  long long g = (n + block - 1) / block;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return (int)g;
}

__global__ void gather_rows_kernel(const uint4* __restrict__ src, const int32_t* __restrict__ idx, uint4* __restrict__ dst,
                                   int n, long long row16) {
  const long long total = (long long)n * row16;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / row16);
    dst[i] = src[(long long)idx[r] * row16 + (i % row16)];
  }
}

__global__ void scatter_add_rows_kernel(float* __restrict__ dst, const int32_t* __restrict__ idx, const float* __restrict__ src,
                                        int n, long long row) {
  const long long total = (long long)n * row;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / row);
    if (idx[r] < 0) continue;                       // unused slot of a capacity-padded subset
    dst[(long long)idx[r] * row + (i % row)] += src[i];
  }
}

__global__ void audit_route_kernel(const int32_t* __restrict__ by_pass, const int32_t* __restrict__ depth,
                                   const int32_t* __restrict__ idx, int32_t* __restrict__ rid, int32_t* __restrict__ active,
                                   int n, int T) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n * T) return;
  const int t = i / n, s = i % n, b = idx[s];
  rid[i] = by_pass[b * T + t];
  active[i] = depth[b] > t ? 1 : 0;
}

__global__ void colmask_mul_kernel(const __nv_bfloat16* __restrict__ x, const int32_t* __restrict__ rid,
                                   const float* __restrict__ table, int S, __nv_bfloat16* __restrict__ out, int rows, int cols) {
  const long long total = (long long)rows * cols;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / cols), c = int(i % cols);
    out[i] = __float2bfloat16_rn(__bfloat162float(x[i]) * table[(size_t)rid[r / S] * cols + c]);
  }
}

__global__ void swiglu_masked_fwd_kernel(const __nv_bfloat16* __restrict__ ug, const int32_t* __restrict__ rid,
                                         const float* __restrict__ table, int S, __nv_bfloat16* __restrict__ z, int rows, int F) {
  const long long total = (long long)rows * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / F), j = int(i % F);
    const float up = __bfloat162float(ug[(size_t)r * 2 * F + j]), g = __bfloat162float(ug[(size_t)r * 2 * F + F + j]);
    z[i] = __float2bfloat16_rn(up * rte::silu_f(g) * table[(size_t)rid[r / S] * F + j]);
  }
}

__global__ void swiglu_masked_bwd_kernel(const __nv_bfloat16* __restrict__ ug, const __nv_bfloat16* __restrict__ dz,
                                         const int32_t* __restrict__ rid, const float* __restrict__ table, int S,
                                         __nv_bfloat16* __restrict__ dug, int rows, int F) {
  const long long total = (long long)rows * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / F), j = int(i % F);
    const float up = __bfloat162float(ug[(size_t)r * 2 * F + j]), g = __bfloat162float(ug[(size_t)r * 2 * F + F + j]);
    const float d = __bfloat162float(dz[i]) * table[(size_t)rid[r / S] * F + j];
    const float sg = rte::sigmoid_f(g);
    dug[(size_t)r * 2 * F + j] = __float2bfloat16_rn(d * g * sg);
    dug[(size_t)r * 2 * F + F + j] = __float2bfloat16_rn(d * up * sg * (1.f + g * (1.f - sg)));
  }
}

__global__ void scaled_residual_fwd_kernel(const float* __restrict__ base, const float* __restrict__ branch,
                                           const float* __restrict__ scale, const int32_t* __restrict__ active,
                                           const float* __restrict__ pass, float* __restrict__ out, int n, long long se) {
  const float s = *scale;
  const long long total = (long long)n * se;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const bool on = active == nullptr || active[i / se] != 0;
    out[i] = on ? base[i] + s * branch[i] : pass[i];
  }
}

__global__ void __launch_bounds__(NTHR)
scaled_residual_bwd_kernel(const float* __restrict__ dout, const float* __restrict__ branch, const float* __restrict__ scale,
                           const int32_t* __restrict__ active, float* __restrict__ dbase, __nv_bfloat16* __restrict__ db16,
                           float* __restrict__ db32, float* __restrict__ dpass, float* __restrict__ dscale_part,
                           const int32_t* __restrict__ frozen_active, const float* __restrict__ frozen_src, int n,
                           long long se) {
  __shared__ float red[32];
  const float s = *scale;
  const long long total = (long long)n * se;
  float acc = 0.f;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const bool on = active == nullptr || active[i / se] != 0;
    const float g = dout[i];
    if (on) acc += g * branch[i];
    if (dpass && !on) dpass[i] += g;
    if (db16) db16[i] = __float2bfloat16_rn(on ? s * g : 0.f);
    if (db32 && on) db32[i] += s * g;
    if (dbase) {
      float o = on ? g : 0.f;
      if (frozen_src && frozen_active[i / se] == 0) o += frozen_src[i];     // samples frozen in this pass: hand-through
      dbase[i] = o;
    }
  }
  acc = rte::block_sum(acc, red);
  if (threadIdx.x == 0 && dscale_part) dscale_part[blockIdx.x] = acc;
}

__device__ __forceinline__ float smooth_l1(float x) { const float a = fabsf(x); return a < 1.f ? 0.5f * x * x : a - 0.5f; }
__device__ __forceinline__ float clamp1(float x) { return fminf(1.f, fmaxf(-1.f, x)); }

// One thread-block cluster of DISTILL_CTAS CTAs per audited sample, one warp per token row.  Phase A: every warp
// reduces its rows for the direction / rms terms; the CTAs' partial sums meet through distributed shared memory
// (summed in rank order by every CTA, so all of them hold the same bits).  Phase B: the two smooth-L1 terms per row
// (the normed one goes back through the row's rmsnorm) and the gradient with respect to the hot endpoint.
constexpr int DISTILL_CTAS = 8;

__global__ void __cluster_dims__(DISTILL_CTAS, 1, 1) __launch_bounds__(NTHR)
macro_distill_kernel(const float* __restrict__ hot, const float* __restrict__ exact, const float* __restrict__ h0,
                     float l_dir, float l_rms, float l_normed, float l_raw, float* __restrict__ terms,
                     float* __restrict__ dhot, int n, int S, int d) {
  constexpr int NW = NTHR / 32;
  __shared__ float wpart[NW][3];
  __shared__ float cta_part[3];        // read by the other CTAs of the cluster
  __shared__ float cta_sl1[2];         // read by rank 0
  __shared__ float wsl1[NW][2];
  cg::cluster_group cluster = cg::this_cluster();
  const int rank = (int)cluster.block_rank();
  const int i = blockIdx.x / DISTILL_CTAS, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int gw = rank * NW + warp, GW = DISTILL_CTAS * NW;
  const long long N = (long long)S * d;
  const float* hp = hot + (size_t)i * N;
  const float* ep = exact + (size_t)i * N;
  const float* zp = h0 + (size_t)i * N;
  float* gp = dhot + (size_t)i * N;
  float dot = 0.f, pp = 0.f, ee = 0.f;
  for (int s = gw; s < S; s += GW) {
    const size_t o = (size_t)s * d;
    for (int c = lane; c < d; c += 32) {
      const float z = zp[o + c], a = hp[o + c] - z, b = ep[o + c] - z;
      dot += a * b; pp += a * a; ee += b * b;
    }
  }
  dot = rte::warp_sum(dot); pp = rte::warp_sum(pp); ee = rte::warp_sum(ee);
  if (lane == 0) { wpart[warp][0] = dot; wpart[warp][1] = pp; wpart[warp][2] = ee; }
  __syncthreads();
  if (threadIdx.x < 3) {
    float t = 0.f;
    for (int w = 0; w < NW; ++w) t += wpart[w][threadIdx.x];
    cta_part[threadIdx.x] = t;
  }
  cluster.sync();
  dot = pp = ee = 0.f;
  for (int r = 0; r < DISTILL_CTAS; ++r) {
    const float* rp_ = cluster.map_shared_rank(cta_part, r);
    dot += rp_[0]; pp += rp_[1]; ee += rp_[2];
  }
  const float np = fmaxf(sqrtf(pp), 1e-8f), ne = fmaxf(sqrtf(ee), 1e-8f);
  const float cosv = dot / (np * ne);
  const float rp = fmaxf(sqrtf(pp / (float)N), 1e-8f), re = fmaxf(sqrtf(ee / (float)N), 1e-8f);
  const float delta = logf(rp) - logf(re);
  const float c_dir = -l_dir / (float)n, c_rms = l_rms / (float)n * 2.f * delta / ((float)N * rp * rp);
  const float c_el = 1.f / ((float)n * (float)N);
  float sl1n = 0.f, sl1r = 0.f;
  for (int s = gw; s < S; s += GW) {
    const float* hr = hp + (size_t)s * d;
    const float* er = ep + (size_t)s * d;
    float sh = 0.f, se = 0.f;
    for (int c = lane; c < d; c += 32) { sh += hr[c] * hr[c]; se += er[c] * er[c]; }
    sh = rte::warp_sum(sh); se = rte::warp_sum(se);
    const float rh = rsqrtf(sh / (float)d + 1e-5f), rx = rsqrtf(se / (float)d + 1e-5f);
    float rowdot = 0.f;
    for (int c = lane; c < d; c += 32) {
      const float hn = hr[c] * rh, df = hn - er[c] * rx;
      sl1n += smooth_l1(df);
      rowdot += clamp1(df) * hn;
    }
    rowdot = rte::warp_sum(rowdot) / (float)d;
    for (int c = lane; c < d; c += 32) {
      const float hn = hr[c] * rh, df = hn - er[c] * rx, raw = hr[c] - er[c];
      sl1r += smooth_l1(raw);
      const float a = hr[c] - zp[(size_t)s * d + c], b = er[c] - zp[(size_t)s * d + c];
      float g = l_normed * c_el * rh * (clamp1(df) - hn * rowdot);
      g += l_raw * c_el * clamp1(raw);
      g += c_dir * (b / (np * ne) - cosv * a / (np * np));
      g += c_rms * a;
      gp[(size_t)s * d + c] = g;
    }
  }
  sl1n = rte::warp_sum(sl1n); sl1r = rte::warp_sum(sl1r);
  if (lane == 0) { wsl1[warp][0] = sl1n; wsl1[warp][1] = sl1r; }
  __syncthreads();
  if (threadIdx.x < 2) {
    float t = 0.f;
    for (int w = 0; w < NW; ++w) t += wsl1[w][threadIdx.x];
    cta_sl1[threadIdx.x] = t;
  }
  cluster.sync();
  if (rank == 0 && threadIdx.x == 0) {
    float a = 0.f, b = 0.f;
    for (int r = 0; r < DISTILL_CTAS; ++r) {
      const float* q = cluster.map_shared_rank(cta_sl1, r);
      a += q[0]; b += q[1];
    }
    terms[i * 4 + 0] = 1.f - cosv;
    terms[i * 4 + 1] = delta * delta;
    terms[i * 4 + 2] = a;
    terms[i * 4 + 3] = b;
  }
  cluster.sync();          // no CTA leaves while rank 0 may still read its shared memory
}

// One CTA per token row of the audited subset.  SEPARATE: the gradient coef*(p_hot - p_exact) goes to the dense f32
// buffer dsep [rows, V] (added to the hot dlogits later by add_rows_f32_to_bf16_kernel) instead of into dlog.
template <bool SEPARATE>
__global__ void __launch_bounds__(NTHR)
kl_distill_kernel(const __nv_bfloat16* __restrict__ hot, const __nv_bfloat16* __restrict__ exact, float inv_temp, float coef,
                  const int32_t* __restrict__ idx, int S, __nv_bfloat16* __restrict__ dlog, int ld, float* __restrict__ dsep,
                  float* __restrict__ kl_rows, float* __restrict__ kl1_rows, int V) {
  __shared__ float red[32];
  const int row = blockIdx.x;
  const __nv_bfloat16* hr = hot + (size_t)row * V;
  const __nv_bfloat16* er = exact + (size_t)row * V;
  float mh = -INFINITY, me = -INFINITY;
  for (int c = threadIdx.x; c < V; c += NTHR) {
    mh = fmaxf(mh, __bfloat162float(hr[c]) * inv_temp);
    me = fmaxf(me, __bfloat162float(er[c]) * inv_temp);
  }
  mh = rte::block_max(mh, red);
  me = rte::block_max(me, red);
  // (kl1_rows: the same divergence at temperature 1 as a by-product; max(x) = max(x / T) * T for T > 0)
  const float mh1 = mh / inv_temp, me1 = me / inv_temp;
  float sh = 0.f, se = 0.f, sh1 = 0.f, se1 = 0.f;
  for (int c = threadIdx.x; c < V; c += NTHR) {
    const float xh = __bfloat162float(hr[c]), xe = __bfloat162float(er[c]);
    sh += __expf(xh * inv_temp - mh);
    se += __expf(xe * inv_temp - me);
    if (kl1_rows) { sh1 += __expf(xh - mh1); se1 += __expf(xe - me1); }
  }
  sh = rte::block_sum(sh, red);
  se = rte::block_sum(se, red);
  const float lh = mh + __logf(sh), le = me + __logf(se);
  float lh1 = 0.f, le1 = 0.f;
  if (kl1_rows) {
    sh1 = rte::block_sum(sh1, red);
    se1 = rte::block_sum(se1, red);
    lh1 = mh1 + __logf(sh1);
    le1 = me1 + __logf(se1);
  }
  __nv_bfloat16* dr = SEPARATE ? nullptr : dlog + ((size_t)idx[row / S] * S + (row % S)) * ld;
  float kl = 0.f, kl1 = 0.f;
  for (int c = threadIdx.x; c < V; c += NTHR) {
    const float lph = __bfloat162float(hr[c]) * inv_temp - lh, lpe = __bfloat162float(er[c]) * inv_temp - le;
    const float ph = __expf(lph), pe = __expf(lpe);
    kl += pe * (lpe - lph);
    if (kl1_rows) {
      const float a = __bfloat162float(hr[c]) - lh1, b = __bfloat162float(er[c]) - le1;
      kl1 += __expf(b) * (b - a);
    }
    if (SEPARATE) { if (dsep) dsep[(size_t)row * V + c] = coef * (ph - pe); }
    else dr[c] = __float2bfloat16_rn(__bfloat162float(dr[c]) + coef * (ph - pe));
  }
  kl = rte::block_sum(kl, red);
  if (threadIdx.x == 0) kl_rows[row] = kl;
  if (kl1_rows) {
    kl1 = rte::block_sum(kl1, red);
    if (threadIdx.x == 0) kl1_rows[row] = kl1;
  }
}

// dst[(idx[row / S] * S + row % S) * ld + c] += src[row * V + c]   (bf16 destination, f32 addend, one rounding)
__global__ void add_rows_f32_to_bf16_kernel(__nv_bfloat16* __restrict__ dst, int ld, const int32_t* __restrict__ idx, int S,
                                            const float* __restrict__ src, int rows, int V) {
  const long long total = (long long)rows * V;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = int(i / V), c = int(i % V);
    if (idx[row / S] < 0) continue;                 // unused slot of a capacity-padded subset
    __nv_bfloat16* q = dst + ((size_t)idx[row / S] * S + (row % S)) * ld + c;
    *q = __float2bfloat16_rn(__bfloat162float(*q) + src[i]);
  }
}

// Residual clip of the control variate (audit.py:306-321): corrected = hot + clamp(exact - hot, -c, c) / p.  Inside the
// clip the derivative is (1 - 1/p) on the hot loss and 1/p on the exact loss; outside it is 1 and 0.  The two cross-entropy
// launches have already written their gradients with the weights 1 (hot) and 1/p (exact), so the factors are
//   f_hot = inside ? 1 - 1/p : 1,   f_exact = inside ? 1 : 0.
__global__ void audit_clip_kernel(const float* __restrict__ hot_loss, const float* __restrict__ exact_loss,
                                  const int32_t* __restrict__ idx, int n, float inv_p, const float* __restrict__ inv_p_slot,
                                  float clip, float* __restrict__ f_hot, float* __restrict__ f_exact) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= n) return;
  if (inv_p_slot) inv_p = inv_p_slot[j];            // per-sample inclusion probabilities (Bernoulli sampler)
  const float r = exact_loss[j] - hot_loss[idx[j]];
  const bool inside = fabsf(r) <= clip;             // (a NaN residual counts as clipped: no gradient through it)
  f_hot[j] = inside ? 1.f - inv_p : 1.f;
  f_exact[j] = inside ? 1.f : 0.f;
}

// x[(row_of(r)) * ld + c] *= scale[r / S]  with row_of(r) = idx ? idx[r / S] * S + r % S : r   (bf16, one rounding)
__global__ void scale_rows_bf16_kernel(__nv_bfloat16* __restrict__ x, int ld, const int32_t* __restrict__ idx, int S,
                                       const float* __restrict__ scale, int rows, int V) {
  const long long total = (long long)rows * V;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int row = int(i / V), c = int(i % V);
    const float f = scale[row / S];
    if (f == 1.f || (idx && idx[row / S] < 0)) continue;
    const size_t phys = idx ? (size_t)idx[row / S] * S + (row % S) : (size_t)row;
    __nv_bfloat16* q = x + phys * ld + c;
    *q = __float2bfloat16_rn(__bfloat162float(*q) * f);
  }
}

// ---- Bernoulli audit sampler with adaptive probability and cap (audit.py:79-132), one CTA of 1024 threads (B <= 1024)
//   p_b   = clamp(p_min + alpha * entropy_b / (R + K) + beta * recent_residual + gamma * deficit(recipe_b), p_min, p_max)
//           deficit(r) = max(coverage_min - ema[r], 0) / max(coverage_min, 1e-12)            (ema BEFORE this step's update)
//   mask  = u_b < p_b                       (u: the uniforms torch.bernoulli would draw, staged by the host)
//   cap   : more than `cap` candidates -> the candidates at positions perm[0..cap) of the ascending candidate list
//           (perm: the row of `perm_table` for this candidate count), inclusion probability p_b * cap / candidates
// Outputs for the replay's fixed-capacity slots (ascending sample order, unused slots point at sample 0 with weight 0):
//   idx, valid (1/0), inv_p (1 / max(p_inc, 1e-12) or 0), dist_scale (n_cap / audited for valid slots: turns the replay's
//   means over n_cap slots into means over the audited samples), the hot rows' loss weights and the replay's.
// Then the coverage average of the audited recipes (audit.py:70-77): ema = beta_c * ema + (1 - beta_c) * counts / max(sum, 1).
struct AuditSampleParams {
  float p_min, p_max, alpha, beta, gamma, cov_min, cov_beta, inv_rk, w0;
  int B, R, cap, n_cap, weight_mode;      // weight_mode 0: plain hot weights (no gradient correction, or residual clip:
};                                        // the factor is applied later); 1: hot weight w0 * (1 - 1/p_inc) on audited rows

__global__ void __launch_bounds__(1024)
audit_sample_kernel(const float* __restrict__ entropy, const int32_t* __restrict__ recipe_id, const float* __restrict__ u,
                    const int32_t* __restrict__ perm_table, float* __restrict__ ema, const float* __restrict__ recent,
                    AuditSampleParams P, int32_t* __restrict__ idx, int32_t* __restrict__ idx_scatter,
                    float* __restrict__ valid, float* __restrict__ inv_p,
                    float* __restrict__ dist_scale, float* __restrict__ row_weight, float* __restrict__ row_weight_a,
                    float* __restrict__ stats, int32_t* __restrict__ none_audited, int* __restrict__ status) {
  __shared__ int scan[1024];
  __shared__ int sel[1024];
  __shared__ int chosen[1024];
  __shared__ int rcount[64];
  __shared__ float red[32];
  const int b = threadIdx.x;
  const bool in = b < P.B;
  float p = 0.f;
  int m = 0;
  if (in) {
    const int r = recipe_id[b];
    const float deficit = fmaxf(P.cov_min - ema[r], 0.f) / fmaxf(P.cov_min, 1e-12f);
    p = P.p_min + P.alpha * (entropy[b] * P.inv_rk) + P.beta * recent[0] + P.gamma * deficit;
    p = fminf(fmaxf(p, P.p_min), P.p_max);
    m = u[b] < p ? 1 : 0;
  }
  // inclusive scan of m over the block (ascending sample index)
  auto block_scan = [&](int v) -> int {
    scan[b] = v;
    __syncthreads();
    for (int off = 1; off < 1024; off <<= 1) {
      const int add = b >= off ? scan[b - off] : 0;
      __syncthreads();
      scan[b] += add;
      __syncthreads();
    }
    return scan[b];
  };
  int incl = block_scan(m);
  const int candidates = scan[1023];
  __syncthreads();
  float p_inc = p;
  int fin = m;
  if (P.cap >= 0 && candidates > P.cap) {
    if (m) sel[incl - 1] = b;
    chosen[b] = 0;
    __syncthreads();
    const int32_t* perm = perm_table + (size_t)(candidates - P.cap - 1) * P.cap;
    if (b < P.cap) chosen[sel[perm[b]]] = 1;
    __syncthreads();
    fin = chosen[b];
    p_inc = p * ((float)P.cap / (float)candidates);
    incl = block_scan(fin);
  }
  const int audited = scan[1023];
  __syncthreads();
  if (audited > P.n_cap && b == 0 && status) atomicExch(status, RTE_DEV_CAPACITY_OVERFLOW);
  const float scale = audited > 0 ? (float)P.n_cap / (float)audited : 0.f;
  if (in) {
    const float ip = 1.f / fmaxf(p_inc, 1e-12f);
    if (fin && incl - 1 < P.n_cap) {
      const int j = incl - 1;
      idx[j] = b; idx_scatter[j] = b; valid[j] = 1.f; inv_p[j] = ip; dist_scale[j] = scale; row_weight_a[j] = P.w0 * ip;
    }
    row_weight[b] = (fin && P.weight_mode == 1) ? P.w0 * (1.f - ip) : P.w0;
  }
  for (int j = min(audited, P.n_cap) + b; j < P.n_cap; j += 1024) {
    idx[j] = 0; idx_scatter[j] = -1; valid[j] = 0.f; inv_p[j] = 0.f; dist_scale[j] = 0.f; row_weight_a[j] = 0.f;
  }
  // coverage average of the audited recipes
  if (b < 64) rcount[b] = 0;
  __syncthreads();
  if (in && fin) atomicAdd(&rcount[recipe_id[b]], 1);
  __syncthreads();
  if (b < P.R) {
    const float probs = (float)rcount[b] / fmaxf((float)audited, 1.f);
    ema[b] = ema[b] * P.cov_beta + probs * (1.f - P.cov_beta);
  }
  // statistics: candidates, audited, mean requested p, mean inclusion p
  float s_req = rte::block_sum(in ? p : 0.f, red);
  float s_inc = rte::block_sum(in ? p_inc : 0.f, red);
  if (b == 0) {
    stats[0] = (float)candidates; stats[1] = (float)audited; stats[2] = s_req / (float)P.B; stats[3] = s_inc / (float)P.B;
    if (none_audited) none_audited[0] = audited == 0 ? 1 : 0;
  }
}

// x[j, :] *= factor[j]  (fp32 rows of row_len elements)
__global__ void scale_rows_f32_kernel(float* __restrict__ x, const float* __restrict__ factor, int n, long long row_len) {
  const long long total = (long long)n * row_len;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x)
    x[i] *= factor[i / row_len];
}

// cos[j] = <a_j, b_j> / (max(|a_j|, eps) * max(|b_j|, eps)) over rows of row_len elements (F.cosine_similarity, eps 1e-8);
// then recent = max(1 - sum_j valid_j cos_j / sum_j valid_j, 0) when any slot is valid (audit.py:213-218), else unchanged.
__global__ void __launch_bounds__(NTHR)
rows_cosine_kernel(const float* __restrict__ a, const float* __restrict__ b, long long row_len, float* __restrict__ cos_out) {
  __shared__ float red[32];
  const float* x = a + (size_t)blockIdx.x * row_len;
  const float* y = b + (size_t)blockIdx.x * row_len;
  float sxy = 0.f, sxx = 0.f, syy = 0.f;
  for (long long i = threadIdx.x; i < row_len; i += NTHR) { const float p = x[i], q = y[i]; sxy += p * q; sxx += p * p; syy += q * q; }
  sxy = rte::block_sum(sxy, red); sxx = rte::block_sum(sxx, red); syy = rte::block_sum(syy, red);
  if (threadIdx.x == 0) cos_out[blockIdx.x] = sxy / (fmaxf(sqrtf(sxx), 1e-8f) * fmaxf(sqrtf(syy), 1e-8f));
}
__global__ void audit_recent_kernel(const float* __restrict__ cos_in, const float* __restrict__ valid, int n, float* __restrict__ recent) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  float s = 0.f, c = 0.f;
  for (int j = 0; j < n; ++j) { s += valid[j] * cos_in[j]; c += valid[j]; }
  if (c > 0.f) recent[0] = fmaxf(1.f - s / c, 0.f);
}

// Sums behind macro_alignment_metrics (macro.py:499-546) for one audited sample per CTA: with a = macro endpoint,
// b = exact endpoint, z = h0 (rows of row_len floats): out[j] = (a.b, a.a, b.b, |a-b|^2, |a-z|^2, |b-z|^2, (a-z).(b-z), untouched).
__global__ void __launch_bounds__(1024)
alignment_sums_kernel(const float* __restrict__ a, const float* __restrict__ b, const float* __restrict__ z, long long row_len,
                      float* __restrict__ out) {
  __shared__ float red[32];
  const float* x = a + (size_t)blockIdx.x * row_len;
  const float* y = b + (size_t)blockIdx.x * row_len;
  const float* w = z + (size_t)blockIdx.x * row_len;
  float s[7] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  auto take = [&](float p, float q, float r) {
    const float dp = p - r, dq = q - r, df = p - q;
    s[0] += p * q; s[1] += p * p; s[2] += q * q; s[3] += df * df; s[4] += dp * dp; s[5] += dq * dq; s[6] += dp * dq;
  };
  // one CTA per sample (a handful of samples, tens of thousands of elements each): 1024 threads, 16-byte loads
  const bool vec = (row_len % 4 == 0) && (((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y) |
                                            reinterpret_cast<uintptr_t>(w)) & 15) == 0);
  if (vec) {
    const float4* x4 = reinterpret_cast<const float4*>(x);
    const float4* y4 = reinterpret_cast<const float4*>(y);
    const float4* w4 = reinterpret_cast<const float4*>(w);
    for (long long i = threadIdx.x; i < row_len / 4; i += blockDim.x) {
      const float4 p = x4[i], q = y4[i], r = w4[i];
      take(p.x, q.x, r.x); take(p.y, q.y, r.y); take(p.z, q.z, r.z); take(p.w, q.w, r.w);
    }
  } else {
    for (long long i = threadIdx.x; i < row_len; i += blockDim.x) take(x[i], y[i], w[i]);
  }
#pragma unroll
  for (int k = 0; k < 7; ++k) {
    const float t = rte::block_sum(s[k], red);
    if (threadIdx.x == 0) out[(size_t)blockIdx.x * 8 + k] = t;
  }
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int rte_audit_clip(const float* hot_loss, const float* exact_loss, const int32_t* idx, int32_t n, float inv_p,
                              const float* inv_p_slot, float clip, float* f_hot, float* f_exact, rte_stream_t stream) {
  RTE_CHECK_ARG(hot_loss && exact_loss && idx && f_hot && f_exact && n > 0 && clip >= 0.f);
  audit_clip_kernel<<<rte::ceil_div(n, 128), 128, 0, ST(stream)>>>(hot_loss, exact_loss, idx, n, inv_p, inv_p_slot, clip, f_hot,
                                                                   f_exact);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_scale_rows_bf16(void* x_bf16, int32_t ld, const int32_t* idx, int32_t S, const float* scale, int32_t rows,
                                   int32_t V, rte_stream_t stream) {
  RTE_CHECK_ARG(x_bf16 && scale && S > 0 && rows > 0 && V > 0 && ld >= V);
  scale_rows_bf16_kernel<<<grid_for((long long)rows * V, NTHR), NTHR, 0, ST(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(x_bf16), ld, idx, S, scale, rows, V);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_gather_rows(const void* src, const int32_t* idx, void* dst, int32_t n, int64_t row_bytes, rte_stream_t stream) {
  RTE_CHECK_ARG(src && idx && dst && n > 0 && row_bytes > 0);
  if ((row_bytes % 16) || (reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dst) & 15)) return RTE_ERR_ALIGNMENT;
  const long long row16 = row_bytes / 16;
  gather_rows_kernel<<<grid_for((long long)n * row16, NTHR), NTHR, 0, ST(stream)>>>(
      reinterpret_cast<const uint4*>(src), idx, reinterpret_cast<uint4*>(dst), n, row16);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_scatter_add_rows_f32(float* dst, const int32_t* idx, const float* src, int32_t n, int64_t row_elems,
                                        rte_stream_t stream) {
  RTE_CHECK_ARG(dst && idx && src && n > 0 && row_elems > 0);
  scatter_add_rows_kernel<<<grid_for((long long)n * row_elems, NTHR), NTHR, 0, ST(stream)>>>(dst, idx, src, n, row_elems);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_audit_route(const int32_t* recipe_id_by_pass, const int32_t* depth, const int32_t* idx, int32_t* rid_out,
                               int32_t* active_out, int32_t n, int32_t T, rte_stream_t stream) {
  RTE_CHECK_ARG(recipe_id_by_pass && depth && idx && rid_out && active_out && n > 0 && T > 0);
  audit_route_kernel<<<rte::ceil_div(n * T, 128), 128, 0, ST(stream)>>>(recipe_id_by_pass, depth, idx, rid_out, active_out, n, T);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_colmask_mul_bf16(const void* x, const int32_t* rid, const float* table, int32_t S, void* out, int32_t rows,
                                    int32_t cols, rte_stream_t stream) {
  RTE_CHECK_ARG(x && rid && table && out && S > 0 && rows > 0 && cols > 0);
  colmask_mul_kernel<<<grid_for((long long)rows * cols, NTHR), NTHR, 0, ST(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(x), rid, table, S, reinterpret_cast<__nv_bfloat16*>(out), rows, cols);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_swiglu_masked_fwd(const void* ug, const int32_t* rid, const float* table, int32_t S, void* z, int32_t rows,
                                     int32_t F, rte_stream_t stream) {
  RTE_CHECK_ARG(ug && rid && table && z && S > 0 && rows > 0 && F > 0);
  swiglu_masked_fwd_kernel<<<grid_for((long long)rows * F, NTHR), NTHR, 0, ST(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(ug), rid, table, S, reinterpret_cast<__nv_bfloat16*>(z), rows, F);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_swiglu_masked_bwd(const void* ug, const void* dz, const int32_t* rid, const float* table, int32_t S,
                                     void* dug, int32_t rows, int32_t F, rte_stream_t stream) {
  RTE_CHECK_ARG(ug && dz && rid && table && dug && S > 0 && rows > 0 && F > 0);
  swiglu_masked_bwd_kernel<<<grid_for((long long)rows * F, NTHR), NTHR, 0, ST(stream)>>>(
      reinterpret_cast<const __nv_bfloat16*>(ug), reinterpret_cast<const __nv_bfloat16*>(dz), rid, table, S,
      reinterpret_cast<__nv_bfloat16*>(dug), rows, F);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_scaled_residual_fwd(const float* base, const float* branch, const float* scale, const int32_t* active,
                                       const float* passthrough, float* out, int32_t n, int64_t sample_elems,
                                       rte_stream_t stream) {
  RTE_CHECK_ARG(base && branch && scale && out && n > 0 && sample_elems > 0 && (active == nullptr || passthrough != nullptr));
  scaled_residual_fwd_kernel<<<grid_for((long long)n * sample_elems, NTHR), NTHR, 0, ST(stream)>>>(base, branch, scale, active,
                                                                                                 passthrough, out, n, sample_elems);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_scaled_residual_bwd(const float* dout, const float* branch, const float* scale, const int32_t* active,
                                       float* dbase, void* dbranch_bf16, float* dbranch_f32_accum, float* dpassthrough,
                                       float* dscale_partial, int32_t max_partials, int32_t* n_partials,
                                       const int32_t* frozen_active, const float* frozen_src, int32_t n,
                                       int64_t sample_elems, rte_stream_t stream) {
  RTE_CHECK_ARG(dout && branch && scale && n > 0 && sample_elems > 0);
  RTE_CHECK_ARG((frozen_active == nullptr) == (frozen_src == nullptr) && (frozen_src == nullptr || dbase != nullptr));
  int grid = grid_for((long long)n * sample_elems, NTHR, 64);
  if (dscale_partial) {
    RTE_CHECK_ARG(max_partials >= 1);
    if (grid > max_partials) grid = max_partials;
  }
  if (n_partials) *n_partials = grid;
  scaled_residual_bwd_kernel<<<grid, NTHR, 0, ST(stream)>>>(dout, branch, scale, active, dbase,
      reinterpret_cast<__nv_bfloat16*>(dbranch_bf16), dbranch_f32_accum, dpassthrough, dscale_partial, frozen_active,
      frozen_src, n, sample_elems);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_macro_distill(const float* hot, const float* exact, const float* h0, float l_dir, float l_rms,
                                 float l_normed, float l_raw, float* terms, float* dhot, int32_t n, int32_t S, int32_t d,
                                 rte_stream_t stream) {
  RTE_CHECK_ARG(hot && exact && h0 && terms && dhot && n > 0 && S > 0 && d > 0);
  macro_distill_kernel<<<n * DISTILL_CTAS, NTHR, 0, ST(stream)>>>(hot, exact, h0, l_dir, l_rms, l_normed, l_raw, terms, dhot, n, S, d);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_kl_distill(const void* hot_logits, const void* exact_logits, float temp, float coef, const int32_t* idx,
                              int32_t S, void* dlogits_hot, int32_t ld_dlogits, float* kl_rows, int32_t rows, int32_t V,
                              rte_stream_t stream) {
  RTE_CHECK_ARG(hot_logits && exact_logits && idx && dlogits_hot && kl_rows && temp > 0.f && S > 0 && rows > 0 && V > 0 &&
                ld_dlogits >= V);
  kl_distill_kernel<false><<<rows, NTHR, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(hot_logits),
      reinterpret_cast<const __nv_bfloat16*>(exact_logits), 1.f / temp, coef, idx, S,
      reinterpret_cast<__nv_bfloat16*>(dlogits_hot), ld_dlogits, nullptr, kl_rows, nullptr, V);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_kl_distill_grad(const void* hot_logits, const void* exact_logits, float temp, float coef, float* dgrad,
                                   float* kl_rows, float* kl1_rows, int32_t rows, int32_t V, rte_stream_t stream) {
  RTE_CHECK_ARG(hot_logits && exact_logits && kl_rows && temp > 0.f && rows > 0 && V > 0);
  kl_distill_kernel<true><<<rows, NTHR, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(hot_logits),
      reinterpret_cast<const __nv_bfloat16*>(exact_logits), 1.f / temp, coef, nullptr, 1, nullptr, 0, dgrad, kl_rows, kl1_rows, V);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_add_rows_f32_to_bf16(void* dst_bf16, int32_t ld, const int32_t* idx, int32_t S, const float* src,
                                        int32_t rows, int32_t V, rte_stream_t stream) {
  RTE_CHECK_ARG(dst_bf16 && idx && src && S > 0 && rows > 0 && V > 0 && ld >= V);
  add_rows_f32_to_bf16_kernel<<<grid_for((long long)rows * V, NTHR), NTHR, 0, ST(stream)>>>(
      reinterpret_cast<__nv_bfloat16*>(dst_bf16), ld, idx, S, src, rows, V);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_audit_sample_bernoulli(const float* entropy, const int32_t* recipe_id, const float* u, const int32_t* perm_table,
                                          float* ema, const float* recent, const rte_audit_sample_params* prm, int32_t* idx,
                                          int32_t* idx_scatter, float* valid, float* inv_p, float* dist_scale, float* row_weight, float* row_weight_a,
                                          float* stats, int32_t* none_audited, int32_t* status, rte_stream_t stream) {
  RTE_CHECK_ARG(entropy && recipe_id && u && ema && recent && prm && idx && idx_scatter && valid && inv_p && dist_scale && row_weight &&
                row_weight_a && stats);
  RTE_CHECK_ARG(prm->B > 0 && prm->B <= 1024 && prm->R > 0 && prm->R <= 64 && prm->n_cap > 0 && (prm->cap < 0 || perm_table));
  AuditSampleParams P;
  P.p_min = prm->p_min; P.p_max = prm->p_max; P.alpha = prm->alpha; P.beta = prm->beta; P.gamma = prm->gamma;
  P.cov_min = prm->coverage_min; P.cov_beta = prm->coverage_beta; P.inv_rk = prm->inv_r_plus_k; P.w0 = prm->w0;
  P.B = prm->B; P.R = prm->R; P.cap = prm->cap; P.n_cap = prm->n_cap; P.weight_mode = prm->weight_mode;
  audit_sample_kernel<<<1, 1024, 0, ST(stream)>>>(entropy, recipe_id, u, perm_table, ema, recent, P, idx, idx_scatter, valid, inv_p,
                                                  dist_scale, row_weight, row_weight_a, stats, none_audited, status);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_scale_rows_f32(float* x, const float* factor, int32_t n, int64_t row_len, rte_stream_t stream) {
  RTE_CHECK_ARG(x && factor && n > 0 && row_len > 0);
  scale_rows_f32_kernel<<<grid_for((long long)n * row_len, NTHR), NTHR, 0, ST(stream)>>>(x, factor, n, row_len);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_audit_recent_residual(const float* hot_end, const float* exact_end, const float* valid, int32_t n,
                                         int64_t row_len, float* cos_scratch, float* recent, rte_stream_t stream) {
  RTE_CHECK_ARG(hot_end && exact_end && valid && cos_scratch && recent && n > 0 && row_len > 0);
  rows_cosine_kernel<<<n, NTHR, 0, ST(stream)>>>(hot_end, exact_end, row_len, cos_scratch);
  RTE_LAUNCH_CHECK();
  audit_recent_kernel<<<1, 32, 0, ST(stream)>>>(cos_scratch, valid, n, recent);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_audit_alignment_sums(const float* hot_end, const float* exact_end, const float* h0, int32_t n, int64_t row_len,
                                        float* out, rte_stream_t stream) {
  RTE_CHECK_ARG(hot_end && exact_end && h0 && out && n > 0 && row_len > 0);
  alignment_sums_kernel<<<n, 1024, 0, ST(stream)>>>(hot_end, exact_end, h0, row_len, out);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
