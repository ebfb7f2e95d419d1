// Per-sample router of the recursive model and the backward pass of its auxiliary losses.
// One decision per SAMPLE from pooled = mean over the sequence of h0: two small MLPs
// (d -> hid -> R recipes, d -> hid -> K depths), softmaxes, arg-max ids with ties to the LOWEST
// index, per-pass recipe ids (logits + per-pass bias), entropies, expected depth.
// The matrices are tiny (hid x d floats, read once per sample from L2), so one CTA per sample.

#include "rte_common.cuh"

namespace {

constexpr int NTHR = 256;

__global__ void __launch_bounds__(NTHR)
pool_kernel(const float* __restrict__ h0, float* __restrict__ pooled, int S, int d) {
  const int b = blockIdx.y, c = blockIdx.x * NTHR + threadIdx.x;
  if (c >= d) return;
  float acc = 0.f;
  for (int s = 0; s < S; ++s) acc += h0[((size_t)b * S + s) * d + c];
  pooled[(size_t)b * d + c] = acc / (float)S;
}

__device__ __forceinline__ int argmax_lowest(const float* v, int n) {
  int best = 0;
  for (int i = 1; i < n; ++i) if (v[i] > v[best]) best = i;   // strict '>' keeps the lowest index on ties
  return best;
}
__device__ __forceinline__ void softmax_small(const float* logits, float* probs, int n) {
  float mx = logits[0];
  for (int i = 1; i < n; ++i) mx = fmaxf(mx, logits[i]);
  float s = 0.f;
  for (int i = 0; i < n; ++i) { probs[i] = expf(logits[i] - mx); s += probs[i]; }
  const float inv = 1.f / s;
  for (int i = 0; i < n; ++i) probs[i] *= inv;
}

// Hidden layer of one router MLP for 16 samples x 32 hidden rows per CTA: every weight row is read once per
// 16 samples (kept in registers as float4 chunks) and dotted with the samples' pooled vectors held in smem.
constexpr int RH_SAMPLES = 16, RH_ROWS = 32;
__global__ void __launch_bounds__(NTHR)
router_hidden_kernel(const float* __restrict__ pooled, const float* __restrict__ w0a, const float* __restrict__ b0a,
                     float* __restrict__ prea, const float* __restrict__ w0b, const float* __restrict__ b0b,
                     float* __restrict__ preb, int B, int d, int hid) {
  extern __shared__ float xs[];                 // [RH_SAMPLES][d]
  const float* w0 = blockIdx.z == 0 ? w0a : w0b;
  const float* b0 = blockIdx.z == 0 ? b0a : b0b;
  float* pre = blockIdx.z == 0 ? prea : preb;
  const int s0 = blockIdx.y * RH_SAMPLES, lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < RH_SAMPLES * d; i += NTHR) {
    const int s = s0 + i / d;
    xs[i] = s < B ? pooled[(size_t)s * d + i % d] : 0.f;
  }
  __syncthreads();
  const int d4 = d >> 2;
  for (int r = 0; r < RH_ROWS / (NTHR / 32); ++r) {
    const int j = blockIdx.x * RH_ROWS + warp * (RH_ROWS / (NTHR / 32)) + r;
    if (j >= hid) break;
    float acc[RH_SAMPLES];
#pragma unroll
    for (int q = 0; q < RH_SAMPLES; ++q) acc[q] = 0.f;
    for (int c = lane; c < d4; c += 32) {
      const float4 w = reinterpret_cast<const float4*>(w0 + (size_t)j * d)[c];
#pragma unroll
      for (int q = 0; q < RH_SAMPLES; ++q) {
        const float4 x = reinterpret_cast<const float4*>(xs + (size_t)q * d)[c];
        acc[q] += w.x * x.x + w.y * x.y + w.z * x.z + w.w * x.w;
      }
    }
#pragma unroll
    for (int q = 0; q < RH_SAMPLES; ++q) {
      const float v = rte::warp_sum(acc[q]);
      if (lane == 0 && s0 + q < B) pre[(size_t)(s0 + q) * hid + j] = v + b0[j];
    }
  }
}

__device__ void head_logits(const float* __restrict__ pre, const float* __restrict__ w2, const float* __restrict__ b2,
                            float* hs, float* logits, int hid, int nout) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int j = threadIdx.x; j < hid; j += NTHR) hs[j] = rte::silu_f(pre[j]);
  __syncthreads();
  for (int r = warp; r < nout; r += NTHR / 32) {
    float acc = 0.f;
#pragma unroll 4
    for (int j = lane; j < hid; j += 32) acc += w2[(size_t)r * hid + j] * hs[j];
    acc = rte::warp_sum(acc);
    if (lane == 0) logits[r] = acc + b2[r];
  }
  __syncthreads();
}

__global__ void __launch_bounds__(NTHR)
router_fwd_kernel(rte_router_weights w, const int32_t* __restrict__ depth_values, rte_router_out o, int d, int hid,
                  int R, int K, int T, int fixed_recipe, int fixed_depth_id) {
  extern __shared__ float sm[];   // hs[hid]
  __shared__ float rl[RTE_ROUTER_MAX_R], dl[RTE_ROUTER_MAX_K];
  float* hs = sm;
  const int b = blockIdx.x;
  head_logits(o.r_hidden_pre + (size_t)b * hid, w.r_w2, w.r_b2, hs, rl, hid, R);
  head_logits(o.d_hidden_pre + (size_t)b * hid, w.d_w2, w.d_b2, hs, dl, hid, K);
  if (threadIdx.x == 0) {
    float rp[RTE_ROUTER_MAX_R], dp[RTE_ROUTER_MAX_K], tmp[RTE_ROUTER_MAX_R], tp[RTE_ROUTER_MAX_R];
    softmax_small(rl, rp, R);
    softmax_small(dl, dp, K);
    float rent = 0.f, dent = 0.f, ed = 0.f;
    for (int r = 0; r < R; ++r) {
      o.recipe_logits[(size_t)b * R + r] = rl[r];
      o.recipe_probs[(size_t)b * R + r] = rp[r];
      rent -= logf(fmaxf(rp[r], 1e-9f)) * rp[r];
    }
    for (int k = 0; k < K; ++k) {
      o.depth_probs[(size_t)b * K + k] = dp[k];
      dent -= logf(fmaxf(dp[k], 1e-9f)) * dp[k];
      ed += dp[k] * (float)depth_values[k];
    }
    o.expected_depth[b] = ed;
    o.router_entropy[b] = rent + dent;
    o.recipe_id[b] = fixed_recipe >= 0 ? fixed_recipe : argmax_lowest(rp, R);
    for (int t = 0; t < T; ++t) {
      int id = fixed_recipe;
      if (fixed_recipe < 0) {
        for (int r = 0; r < R; ++r) tmp[r] = rl[r] + w.pass_recipe_bias[t * R + r];
        softmax_small(tmp, tp, R);
        id = argmax_lowest(tp, R);
      }
      o.recipe_id_by_pass[(size_t)b * T + t] = id;
    }
    const int did = fixed_depth_id >= 0 ? fixed_depth_id : argmax_lowest(dp, K);
    o.depth_id[b] = did;
    o.depth[b] = depth_values[did];
  }
}

// aux losses and the batch-mean of the recipe probabilities
__global__ void __launch_bounds__(NTHR)
aux_kernel(const float* __restrict__ recipe_probs, const float* __restrict__ expected_depth, float lambda_load,
           float lambda_depth, float* __restrict__ aux, float* __restrict__ mean_prob, const float* __restrict__ mean_given,
           int B, int R) {
  __shared__ float red[32];
  __shared__ float mp[RTE_ROUTER_MAX_R];
  for (int r = threadIdx.x; r < R; r += NTHR) {
    float acc = 0.f;
    if (mean_given != nullptr) {          // the batch mean over ALL data-parallel shards, reduced by the caller
      acc = mean_given[r];
    } else {
      for (int b = 0; b < B; ++b) acc += recipe_probs[(size_t)b * R + r];
      acc /= (float)B;
    }
    mp[r] = acc;
    mean_prob[r] = acc;
  }
  float ed = 0.f;
  for (int b = threadIdx.x; b < B; b += NTHR) ed += expected_depth[b];
  ed = rte::block_sum(ed, red);
  __syncthreads();
  if (threadIdx.x == 0) {
    float sq = 0.f;
    for (int r = 0; r < R; ++r) sq += mp[r] * mp[r];
    aux[0] = lambda_load * ((float)R * sq - 1.f);
    aux[1] = lambda_depth * ed / (float)B;
  }
}

// per-sample backward through softmax and both MLP heads; dh0 += dpooled / S
__device__ void mlp_backward_sample(const float* __restrict__ w0, const float* __restrict__ w2, const float* dlog,
                                    const float* __restrict__ pre, float* dpre_out, float* dhs, int d, int hid, int nout) {
  for (int j = threadIdx.x; j < hid; j += NTHR) {
    float acc = 0.f;
    for (int r = 0; r < nout; ++r) acc += w2[(size_t)r * hid + j] * dlog[r];
    const float a = pre[j], sg = rte::sigmoid_f(a);
    const float v = acc * sg * (1.f + a * (1.f - sg));
    dhs[j] = v;
    dpre_out[j] = v;
  }
  __syncthreads();
  (void)w0; (void)d;
}

__global__ void __launch_bounds__(NTHR)
router_bwd_sample_kernel(rte_router_weights w, rte_router_out o, const int32_t* __restrict__ depth_values,
                         const float* __restrict__ mean_prob, float lambda_load, float lambda_depth,
                         float* __restrict__ dpre_r, float* __restrict__ dpre_d, float* __restrict__ dlog_r,
                         float* __restrict__ dlog_d, float* __restrict__ dh0, int B, int S, int d, int hid, int R, int K) {
  extern __shared__ float sm[];   // dhr[hid], dhd[hid]
  __shared__ float dlr[RTE_ROUTER_MAX_R], dld[RTE_ROUTER_MAX_K];
  float* dhr = sm;
  float* dhd = sm + hid;
  const int b = blockIdx.x;
  if (threadIdx.x == 0) {
    float dot = 0.f;
    for (int r = 0; r < R; ++r) dot += o.recipe_probs[(size_t)b * R + r] * (lambda_load * (float)R * 2.f * mean_prob[r] / (float)B);
    for (int r = 0; r < R; ++r) {
      const float p = o.recipe_probs[(size_t)b * R + r];
      const float v = p * (lambda_load * (float)R * 2.f * mean_prob[r] / (float)B - dot);
      dlr[r] = v;
      dlog_r[(size_t)b * R + r] = v;
    }
    float dotd = 0.f;
    for (int k = 0; k < K; ++k) dotd += o.depth_probs[(size_t)b * K + k] * (lambda_depth * (float)depth_values[k] / (float)B);
    for (int k = 0; k < K; ++k) {
      const float p = o.depth_probs[(size_t)b * K + k];
      const float v = p * (lambda_depth * (float)depth_values[k] / (float)B - dotd);
      dld[k] = v;
      dlog_d[(size_t)b * K + k] = v;
    }
  }
  __syncthreads();
  mlp_backward_sample(w.r_w0, w.r_w2, dlr, o.r_hidden_pre + (size_t)b * hid, dpre_r + (size_t)b * hid, dhr, d, hid, R);
  mlp_backward_sample(w.d_w0, w.d_w2, dld, o.d_hidden_pre + (size_t)b * hid, dpre_d + (size_t)b * hid, dhd, d, hid, K);
}

// dst[r,:] += sum_p vec[p][r / seg,:]   (nparts partial vectors, part_stride floats apart, added in fixed order)
__global__ void bcast_add_kernel(float* __restrict__ dst, const float* __restrict__ vec, int rows, int seg, int d, int nparts,
                                 long long part_stride) {
  const long long total = (long long)rows * (d >> 2);
  const int d4 = d >> 2;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int r = int(i / d4), c = int(i % d4);
    float4 a = reinterpret_cast<float4*>(dst)[i];
    for (int p = 0; p < nparts; ++p) {
      const float4 v = reinterpret_cast<const float4*>(vec + p * part_stride)[(size_t)(r / seg) * d4 + c];
      a.x += v.x; a.y += v.y; a.z += v.z; a.w += v.w;
    }
    reinterpret_cast<float4*>(dst)[i] = a;
  }
}

// dpooled[part][b,:] = (dpre_r[b, J] @ W0r[J,:] + dpre_d[b, J] @ W0d[J,:]) / S over the part's slice J of the hidden
// dimension (blockIdx.y = part).  CTA = 4 samples x 128 columns; the two halves of the block split J again and are
// combined through shared memory.  The broadcast kernel adds the parts in fixed order.
__global__ void __launch_bounds__(NTHR)
router_dpooled_kernel(const float* __restrict__ w0r, const float* __restrict__ w0d, const float* __restrict__ dpre_r,
                      const float* __restrict__ dpre_d, float* __restrict__ dpooled, int B, int S, int d, int hid) {
  extern __shared__ float sm[];            // sr[4][hid], sd[4][hid], comb[4][128]
  float* sr = sm;
  float* sd = sm + 4 * hid;
  float* comb = sm + 8 * hid;
  const int cblocks = rte::ceil_div(d, 128);
  const int b0 = (blockIdx.x / cblocks) * 4, c = (blockIdx.x % cblocks) * 128 + (threadIdx.x & 127);
  const int half = threadIdx.x >> 7;
  const int part_len = (hid + (int)gridDim.y - 1) / (int)gridDim.y;
  const int p_lo = blockIdx.y * part_len, p_hi = min(hid, p_lo + part_len);
  dpooled += (size_t)blockIdx.y * B * d;
  for (int i = threadIdx.x; i < 4 * hid; i += NTHR) {
    const int bb = b0 + i / hid;
    sr[i] = bb < B ? dpre_r[(size_t)bb * hid + i % hid] : 0.f;
    sd[i] = bb < B ? dpre_d[(size_t)bb * hid + i % hid] : 0.f;
  }
  __syncthreads();
  float acc[4] = {0.f, 0.f, 0.f, 0.f};
  if (c < d) {
    const int jh = (p_hi - p_lo + 1) / 2, j_lo = p_lo + half * jh, j_hi = min(p_hi, j_lo + jh);
#pragma unroll 8
    for (int j = j_lo; j < j_hi; ++j) {
      const float wr = w0r[(size_t)j * d + c], wd = w0d[(size_t)j * d + c];
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q] += wr * sr[q * hid + j] + wd * sd[q * hid + j];
    }
  }
  if (half == 1) {
#pragma unroll
    for (int q = 0; q < 4; ++q) comb[q * 128 + (threadIdx.x & 127)] = acc[q];
  }
  __syncthreads();
  if (half == 0 && c < d) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int bb = b0 + q;
      if (bb >= B) break;
      dpooled[(size_t)bb * d + c] = (acc[q] + comb[q * 128 + threadIdx.x]) / (float)S;
    }
  }
}

// dW0[j,c] = sum_b dpre[b,j] * pooled[b,c];  db0[j] = sum_b dpre[b,j]
__global__ void __launch_bounds__(NTHR)
router_dw0_kernel(const float* __restrict__ dpre, const float* __restrict__ pooled, float* __restrict__ dw0,
                  float* __restrict__ db0, int B, int d, int hid) {
  const long long i = blockIdx.x * (long long)NTHR + threadIdx.x;
  if (i >= (long long)hid * d) return;
  const int j = int(i / d), c = int(i % d);
  float acc = 0.f, accb = 0.f;
#pragma unroll 8
  for (int b = 0; b < B; ++b) {
    const float v = dpre[(size_t)b * hid + j];
    acc += v * pooled[(size_t)b * d + c];
    accb += v;
  }
  dw0[i] = acc;
  if (c == 0) db0[j] = accb;
}
// dW2[r,j] = sum_b dlog[b,r] * silu(pre[b,j]);  db2[r] = sum_b dlog[b,r].  32 outputs x 8 sample groups per CTA.
__global__ void __launch_bounds__(NTHR)
router_dw2_kernel(const float* __restrict__ dlog, const float* __restrict__ pre, float* __restrict__ dw2,
                  float* __restrict__ db2, int B, int hid, int nout) {
  __shared__ float sa[8][33], sb[8][33];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int i = blockIdx.x * 32 + tx;
  float acc = 0.f, accb = 0.f;
  if (i < nout * hid) {
    const int r = i / hid, j = i % hid;
#pragma unroll 4
    for (int b = ty; b < B; b += 8) {
      const float v = dlog[(size_t)b * nout + r];
      acc += v * rte::silu_f(pre[(size_t)b * hid + j]);
      accb += v;
    }
  }
  sa[ty][tx] = acc; sb[ty][tx] = accb;
  __syncthreads();
  if (ty == 0 && i < nout * hid) {
    float t = 0.f, u = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) { t += sa[k][tx]; u += sb[k][tx]; }
    dw2[i] = t;
    if (i % hid == 0) db2[i / hid] = u;
  }
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int rte_router_fwd(const float* h0, const rte_router_weights* w, const int32_t* depth_values,
                              const rte_router_out* out, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                              int32_t K, int32_t T, int32_t fixed_recipe, int32_t fixed_depth_id, rte_stream_t stream) {
  RTE_CHECK_ARG(h0 && w && depth_values && out && B > 0 && S > 0 && d > 0 && hid > 0);
  RTE_CHECK_ARG(R > 0 && R <= RTE_ROUTER_MAX_R && K > 0 && K <= RTE_ROUTER_MAX_K && T > 0 && T <= RTE_ROUTER_MAX_T);
  RTE_CHECK_ARG(fixed_recipe < R && fixed_depth_id < K);
  RTE_CHECK_ARG(out->pooled && out->r_hidden_pre && out->d_hidden_pre && out->recipe_logits && out->recipe_probs &&
                out->depth_probs && out->expected_depth && out->router_entropy && out->recipe_id &&
                out->recipe_id_by_pass && out->depth_id && out->depth);
  const size_t smem = (size_t)hid * sizeof(float);
  const size_t smem_h = (size_t)RH_SAMPLES * d * sizeof(float);
  if (smem > 48 * 1024 || d % 4 != 0) return RTE_ERR_UNSUPPORTED;
  if (smem_h > 48 * 1024) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(router_hidden_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 128 * 1024) != cudaSuccess)
        return RTE_ERR_LAUNCH;
      set = true;
    }
  }
  pool_kernel<<<dim3(rte::ceil_div(d, NTHR), B), NTHR, 0, ST(stream)>>>(h0, out->pooled, S, d);
  RTE_LAUNCH_CHECK();
  router_hidden_kernel<<<dim3(rte::ceil_div(hid, RH_ROWS), rte::ceil_div(B, RH_SAMPLES), 2), NTHR, smem_h, ST(stream)>>>(
      out->pooled, w->r_w0, w->r_b0, out->r_hidden_pre, w->d_w0, w->d_b0, out->d_hidden_pre, B, d, hid);
  RTE_LAUNCH_CHECK();
  router_fwd_kernel<<<B, NTHR, smem, ST(stream)>>>(*w, depth_values, *out, d, hid, R, K, T, fixed_recipe, fixed_depth_id);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

// out[r] = scale * sum_b recipe_probs[b, r]: with scale = 1 / (B * world) the SUM of `out` over the data-parallel ranks is
// the batch mean over the global batch, which rte_router_aux_bwd_data then takes as `mean_prob_in`.
__global__ void __launch_bounds__(NTHR)
mean_prob_kernel(const float* __restrict__ recipe_probs, float* __restrict__ out, float scale, int B, int R) {
  for (int r = threadIdx.x; r < R; r += NTHR) {
    float acc = 0.f;
    for (int b = 0; b < B; ++b) acc += recipe_probs[(size_t)b * R + r];
    out[r] = acc * scale;
  }
}

extern "C" int rte_router_mean_prob(const float* recipe_probs, float* out, float scale, int32_t B, int32_t R, rte_stream_t stream) {
  RTE_CHECK_ARG(recipe_probs && out && B > 0 && R > 0 && R <= RTE_ROUTER_MAX_R);
  mean_prob_kernel<<<1, NTHR, 0, ST(stream)>>>(recipe_probs, out, scale, B, R);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

// Data-gradient half: the auxiliary losses, d(loss)/d(pre-activations) per sample (left in `scratch`), and
// dh0[b,s,:] += dpooled[b,:] / S -- what the rest of backward waits for.  None of it depends on an upstream
// gradient, so with dh0 == NULL everything but that last add can run as soon as the router's forward is done
// (rte_router_aux_add_dh0 performs the add later, from `scratch`).
extern "C" int rte_router_aux_bwd_data(const rte_router_weights* w, const rte_router_out* fwd, const int32_t* depth_values,
                                       float lambda_load, float lambda_depth, float* aux, float* dh0, float* scratch,
                                       const float* mean_prob_in, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                                       int32_t K, rte_stream_t stream) {
  RTE_CHECK_ARG(w && fwd && depth_values && aux && scratch && B > 0 && S > 0 && d > 0 && hid > 0);
  RTE_CHECK_ARG(R > 0 && R <= RTE_ROUTER_MAX_R && K > 0 && K <= RTE_ROUTER_MAX_K);
  float* mean_prob = scratch;                       // [RTE_ROUTER_MAX_R]
  float* dpre_r = scratch + RTE_ROUTER_MAX_R;       // [B, hid]
  float* dpre_d = dpre_r + (size_t)B * hid;         // [B, hid]
  float* dlog_r = dpre_d + (size_t)B * hid;         // [B, R]
  float* dlog_d = dlog_r + (size_t)B * R;           // [B, K]
  float* dpooled = scratch + (((size_t)RTE_ROUTER_MAX_R + (size_t)B * (2 * hid + R + K) + 3) & ~(size_t)3);   // [B, d], 16-byte aligned
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return RTE_ERR_ALIGNMENT;
  aux_kernel<<<1, NTHR, 0, ST(stream)>>>(fwd->recipe_probs, fwd->expected_depth, lambda_load, lambda_depth, aux, mean_prob,
                                         mean_prob_in, B, R);
  RTE_LAUNCH_CHECK();
  const size_t smem = (size_t)2 * hid * sizeof(float);
  if (smem > 48 * 1024) return RTE_ERR_UNSUPPORTED;
  router_bwd_sample_kernel<<<B, NTHR, smem, ST(stream)>>>(*w, *fwd, depth_values, mean_prob, lambda_load, lambda_depth,
                                                          dpre_r, dpre_d, dlog_r, dlog_d, dh0, B, S, d, hid, R, K);
  RTE_LAUNCH_CHECK();
  const size_t smem_dp = (size_t)(8 * hid + 4 * 128) * sizeof(float);
  if (smem_dp > 48 * 1024) return RTE_ERR_UNSUPPORTED;
  router_dpooled_kernel<<<dim3(rte::ceil_div(B, 4) * rte::ceil_div(d, 128), RTE_ROUTER_DPOOLED_PARTS), NTHR, smem_dp, ST(stream)>>>(
      w->r_w0, w->d_w0, dpre_r, dpre_d, dpooled, B, S, d, hid);
  RTE_LAUNCH_CHECK();
  if (d % 4 != 0) return RTE_ERR_UNSUPPORTED;
  if (dh0) {
    long long n4 = (long long)B * S * (d / 4);
    int grid = (int)((n4 + NTHR - 1) / NTHR);
    if (grid > 148 * 8) grid = 148 * 8;
    bcast_add_kernel<<<grid, NTHR, 0, ST(stream)>>>(dh0, dpooled, B * S, S, d, RTE_ROUTER_DPOOLED_PARTS, (long long)B * d);
    RTE_LAUNCH_CHECK();
  }
  return RTE_OK;
}

// dh0[b,s,:] += dpooled[b,:] / S from the `scratch` a call of rte_router_aux_bwd_data(dh0 = NULL) left behind.
extern "C" int rte_router_aux_add_dh0(float* dh0, const float* scratch, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                                      int32_t K, rte_stream_t stream) {
  RTE_CHECK_ARG(dh0 && scratch && B > 0 && S > 0 && d > 0 && hid > 0 && R > 0 && K > 0);
  if (d % 4 != 0) return RTE_ERR_UNSUPPORTED;
  if (reinterpret_cast<uintptr_t>(scratch) & 15) return RTE_ERR_ALIGNMENT;
  const float* dpooled = scratch + (((size_t)RTE_ROUTER_MAX_R + (size_t)B * (2 * hid + R + K) + 3) & ~(size_t)3);
  long long n4 = (long long)B * S * (d / 4);
  int grid = (int)((n4 + NTHR - 1) / NTHR);
  if (grid > 148 * 8) grid = 148 * 8;
  bcast_add_kernel<<<grid, NTHR, 0, ST(stream)>>>(dh0, dpooled, B * S, S, d, RTE_ROUTER_DPOOLED_PARTS, (long long)B * d);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

// Parameter-gradient half of the auxiliary-loss backward: reads dpre / dlog left in `scratch` by the data half.
extern "C" int rte_router_aux_bwd_params(const rte_router_out* fwd, const rte_router_grads* grads, float* scratch, int32_t B,
                                         int32_t d, int32_t hid, int32_t R, int32_t K, rte_stream_t stream) {
  RTE_CHECK_ARG(fwd && grads && scratch && B > 0 && d > 0 && hid > 0 && R > 0 && K > 0);
  RTE_CHECK_ARG(grads->r_w0 && grads->r_b0 && grads->r_w2 && grads->r_b2 && grads->d_w0 && grads->d_b0 && grads->d_w2 && grads->d_b2);
  float* dpre_r = scratch + RTE_ROUTER_MAX_R;
  float* dpre_d = dpre_r + (size_t)B * hid;
  float* dlog_r = dpre_d + (size_t)B * hid;
  float* dlog_d = dlog_r + (size_t)B * R;
  const int g0 = (int)rte::ceil_div64((long long)hid * d, NTHR);
  router_dw0_kernel<<<g0, NTHR, 0, ST(stream)>>>(dpre_r, fwd->pooled, grads->r_w0, grads->r_b0, B, d, hid);
  RTE_LAUNCH_CHECK();
  router_dw0_kernel<<<g0, NTHR, 0, ST(stream)>>>(dpre_d, fwd->pooled, grads->d_w0, grads->d_b0, B, d, hid);
  RTE_LAUNCH_CHECK();
  router_dw2_kernel<<<rte::ceil_div(R * hid, 32), NTHR, 0, ST(stream)>>>(dlog_r, fwd->r_hidden_pre, grads->r_w2, grads->r_b2, B, hid, R);
  RTE_LAUNCH_CHECK();
  router_dw2_kernel<<<rte::ceil_div(K * hid, 32), NTHR, 0, ST(stream)>>>(dlog_d, fwd->d_hidden_pre, grads->d_w2, grads->d_b2, B, hid, K);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

// Both halves on one stream.
extern "C" int rte_router_aux_bwd(const rte_router_weights* w, const rte_router_out* fwd, const int32_t* depth_values,
                                  float lambda_load, float lambda_depth, float* aux, const rte_router_grads* grads,
                                  float* dh0, float* scratch, int32_t B, int32_t S, int32_t d, int32_t hid, int32_t R,
                                  int32_t K, rte_stream_t stream) {
  RTE_CHECK_ARG(grads != nullptr);
  const int rc = rte_router_aux_bwd_data(w, fwd, depth_values, lambda_load, lambda_depth, aux, dh0, scratch, nullptr, B, S, d, hid, R, K,
                                         stream);
  if (rc != RTE_OK) return rc;
  return rte_router_aux_bwd_params(fwd, grads, scratch, B, d, hid, R, K, stream);
}
