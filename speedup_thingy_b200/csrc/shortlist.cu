// Vocabulary shortlist of the `recursive_macro_shortlist` mode (reference output.py:72-136).
//
// rte_shortlist_build: per token, the first K distinct ids of the candidate sequence
//   [target | members of the top clusters | hard negatives | random negatives | filler | target + 0..2K-1 (mod V)]
// in order of first appearance -- the reference's scatter_reduce(amin) + topk(largest=False) over a [tokens, V]
// table, done here by one warp per token walking the sequence 32 candidates at a time with a per-warp "seen"
// bitmap in shared memory (no [tokens, V] table).  Candidates are generated from their position, never stored.
// Bit-exact given the same top clusters and random negatives; the target always lands in slot 0.
//
// rte_shortlist_ce: logits over the shortlist (gathered embedding rows . hidden), cross entropy against slot 0,
// and the gradient written as a dense, otherwise-zero [tokens, V] bf16 row so that the backward pass reuses the
// tensor-core GEMMs of the full-vocabulary path.

#include "rte_common.cuh"

namespace {

constexpr int SB_WARPS = 8;

struct ShortlistDims { int V, C, TC, HN, RN, K, mpc; };

__device__ __forceinline__ int candidate_at(int p, long long target, const int32_t* __restrict__ top, const int32_t* __restrict__ rnd,
                                            const ShortlistDims& D) {
  if (p == 0) return (int)target;
  p -= 1;
  if (p < D.TC * D.mpc) {
    const int c = top[p / D.mpc], tok = c + (p % D.mpc) * D.C;      // cluster c owns ids c, c + C, c + 2C, ...
    return tok < D.V ? tok : 0;                                       // (member table padded with id 0)
  }
  p -= D.TC * D.mpc;
  if (p < D.HN) return p % D.V;
  p -= D.HN;
  if (p < D.RN) return rnd[p];
  p -= D.RN;
  if (p < D.K) return p % D.V;
  p -= D.K;
  return (int)((target + p) % D.V);
}

__global__ void __launch_bounds__(SB_WARPS * 32)
shortlist_build_kernel(const int64_t* __restrict__ targets, const int32_t* __restrict__ top_clusters,
                       const int32_t* __restrict__ random_negs, int32_t* __restrict__ shortlist,
                       int32_t* __restrict__ dup_count, int rows, ShortlistDims D, int* status) {
  extern __shared__ uint32_t seen_all[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int row = blockIdx.x * SB_WARPS + warp;
  const int words = (D.V + 31) / 32;
  uint32_t* seen = seen_all + (size_t)warp * words;
  if (row >= rows) return;
  for (int i = lane; i < words; i += 32) seen[i] = 0u;
  __syncwarp();
  long long target = targets[row];
  if (target < 0 || target >= D.V) {
    if (status && lane == 0) atomicExch(status, RTE_DEV_INDEX_OUT_OF_RANGE);
    target = 0;
  }
  const int32_t* top = top_clusters + (size_t)row * D.TC;
  const int32_t* rnd = random_negs + (size_t)row * D.RN;
  const int width = 1 + D.TC * D.mpc + D.HN + D.RN + D.K + 2 * D.K;
  int n_out = 0, n_unique = 0;
  for (int p0 = 0; p0 < width; p0 += 32) {
    const int p = p0 + lane;
    const bool valid = p < width;
    int id = valid ? candidate_at(p, target, top, rnd, D) : -1 - lane;     // invalid lanes get distinct dummies
    if (valid && (id < 0 || id >= D.V)) {
      if (status) atomicExch(status, RTE_DEV_INDEX_OUT_OF_RANGE);
      id = 0;
    }
    const unsigned same = __match_any_sync(0xffffffffu, id);
    const bool first_here = valid && ((same & ((1u << lane) - 1u)) == 0u);   // lowest lane holding this id
    const bool fresh = first_here && ((seen[id >> 5] >> (id & 31)) & 1u) == 0u;
    const unsigned fresh_mask = __ballot_sync(0xffffffffu, fresh);
    if (fresh) {
      const int slot = n_out + __popc(fresh_mask & ((1u << lane) - 1u));
      if (slot < D.K) shortlist[(size_t)row * D.K + slot] = id;
      atomicOr(&seen[id >> 5], 1u << (id & 31));
    }
    __syncwarp();
    n_out += __popc(fresh_mask);
    n_unique += __popc(fresh_mask);
    if (n_out >= D.K && dup_count == nullptr) break;
  }
  if (dup_count != nullptr && lane == 0) dup_count[row] = width - n_unique;
}

// one CTA per token: logits over the shortlist, CE vs slot 0, dense gradient row
__global__ void __launch_bounds__(128)
shortlist_ce_kernel(const __nv_bfloat16* __restrict__ hidden, const __nv_bfloat16* __restrict__ W,
                    const int32_t* __restrict__ shortlist, const float* __restrict__ row_weight, int S,
                    float* __restrict__ loss_tok, __nv_bfloat16* __restrict__ logits_out,
                    __nv_bfloat16* __restrict__ dense, int d, int V, int K) {
  extern __shared__ float sm[];          // hs[d], lg[K]
  __shared__ float red[32];
  float* hs = sm;
  float* lg = sm + d;
  const int row = blockIdx.x;
  for (int c = threadIdx.x; c < d; c += blockDim.x) hs[c] = __bfloat162float(hidden[(size_t)row * d + c]);
  if (dense != nullptr) {
    uint4* dr = reinterpret_cast<uint4*>(dense + (size_t)row * V);
    for (int i = threadIdx.x; i < V / 8; i += blockDim.x) dr[i] = make_uint4(0u, 0u, 0u, 0u);
  }
  __syncthreads();
  const int d8 = d >> 3;
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const uint4* wr = reinterpret_cast<const uint4*>(W + (size_t)shortlist[(size_t)row * K + k] * d);
    float acc = 0.f;
#pragma unroll 4
    for (int c = 0; c < d8; ++c) {
      const uint4 pk = wr[c];
      const float2 a = rte::unpack_bf16x2(pk.x), b = rte::unpack_bf16x2(pk.y), e = rte::unpack_bf16x2(pk.z), f = rte::unpack_bf16x2(pk.w);
      const float* h = hs + 8 * c;
      acc += a.x * h[0] + a.y * h[1] + b.x * h[2] + b.y * h[3] + e.x * h[4] + e.y * h[5] + f.x * h[6] + f.y * h[7];
    }
    acc = __bfloat162float(__float2bfloat16_rn(acc));      // the reference's logits are bf16 under autocast
    lg[k] = acc;
    if (logits_out) logits_out[(size_t)row * K + k] = __float2bfloat16_rn(acc);
  }
  __syncthreads();
  float mx = -INFINITY;
  for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, lg[k]);
  mx = rte::block_max(mx, red);
  float se = 0.f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) se += __expf(lg[k] - mx);
  se = rte::block_sum(se, red);
  const float lse = mx + __logf(se);
  if (threadIdx.x == 0) loss_tok[row] = lse - lg[0];
  if (dense == nullptr) return;
  const float wgt = row_weight[row / S];
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float g = wgt * (__expf(lg[k] - lse) - (k == 0 ? 1.f : 0.f));
    dense[(size_t)row * V + shortlist[(size_t)row * K + k]] = __float2bfloat16_rn(g);
  }
}

// The same cross entropy when the FULL logits row already exists (one tcgen05 GEMM over the vocabulary costs less than
// gathering K weight rows per token while the vocabulary is small): reads the K shortlisted logits of the row, then
// overwrites the row in place with the dense gradient (zero outside the shortlist).  One CTA per token.
__global__ void __launch_bounds__(128)
shortlist_ce_logits_kernel(__nv_bfloat16* __restrict__ logits, const int32_t* __restrict__ shortlist,
                           const float* __restrict__ row_weight, int S, float* __restrict__ loss_tok, int V, int K) {
  extern __shared__ float lg[];          // [K]
  __shared__ float red[32];
  const int row = blockIdx.x;
  __nv_bfloat16* lr = logits + (size_t)row * V;
  for (int k = threadIdx.x; k < K; k += blockDim.x) lg[k] = __bfloat162float(lr[shortlist[(size_t)row * K + k]]);
  __syncthreads();                        // every shortlisted logit has been read: the row may be overwritten
  uint4* dr = reinterpret_cast<uint4*>(lr);
  for (int i = threadIdx.x; i < V / 8; i += blockDim.x) dr[i] = make_uint4(0u, 0u, 0u, 0u);
  float mx = -INFINITY;
  for (int k = threadIdx.x; k < K; k += blockDim.x) mx = fmaxf(mx, lg[k]);
  mx = rte::block_max(mx, red);
  float se = 0.f;
  for (int k = threadIdx.x; k < K; k += blockDim.x) se += __expf(lg[k] - mx);
  se = rte::block_sum(se, red);           // (the reductions' barriers also order the zero fill before the scatter)
  const float lse = mx + __logf(se);
  if (threadIdx.x == 0) loss_tok[row] = lse - lg[0];
  const float wgt = row_weight[row / S];
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const float g = wgt * (__expf(lg[k] - lse) - (k == 0 ? 1.f : 0.f));
    lr[shortlist[(size_t)row * K + k]] = __float2bfloat16_rn(g);
  }
}

// dense[row, ids[row, k]] = vals[row, k], zero elsewhere (ids distinct within a row)
__global__ void __launch_bounds__(128)
scatter_cols_kernel(const __nv_bfloat16* __restrict__ vals, const int32_t* __restrict__ ids, __nv_bfloat16* __restrict__ dense,
                    int V, int K) {
  const int row = blockIdx.x;
  uint4* dr = reinterpret_cast<uint4*>(dense + (size_t)row * V);
  for (int i = threadIdx.x; i < V / 8; i += blockDim.x) dr[i] = make_uint4(0u, 0u, 0u, 0u);
  __syncthreads();
  for (int k = threadIdx.x; k < K; k += blockDim.x) {
    const int id = ids[(size_t)row * K + k];
    if (id >= 0 && id < V) dense[(size_t)row * V + id] = vals[(size_t)row * K + k];
  }
}

// out[i] = hash(seed, i) mod vocab  (counter-based, reproducible; used when no host-drawn negatives are supplied)
__global__ void random_tokens_kernel(int32_t* __restrict__ out, long long n, int vocab, const int64_t* __restrict__ seed) {
  const unsigned long long s = (unsigned long long)(*seed);
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    unsigned long long z = s * 0x9E3779B97F4A7C15ull + (unsigned long long)i + 0x632BE59BD9B4E019ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    out[i] = (int32_t)(z % (unsigned long long)vocab);
  }
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int rte_shortlist_build(const int64_t* targets, const int32_t* top_clusters, const int32_t* random_negs,
                                   int32_t* shortlist, int32_t* dup_count, int32_t rows, int32_t V, int32_t C, int32_t TC,
                                   int32_t HN, int32_t RN, int32_t K, int32_t* status, rte_stream_t stream) {
  RTE_CHECK_ARG(targets && top_clusters && shortlist && rows > 0 && V > 0 && C > 0 && TC > 0 && TC <= C && HN >= 0 && RN >= 0 &&
                K > 0 && K <= V && (RN == 0 || random_negs != nullptr));
  ShortlistDims D{V, C, TC, HN, RN, K, (V + C - 1) / C};
  const size_t smem = (size_t)SB_WARPS * ((V + 31) / 32) * sizeof(uint32_t);
  if (smem > 200 * 1024) return RTE_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(shortlist_build_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return RTE_ERR_LAUNCH;
      set = true;
    }
  }
  shortlist_build_kernel<<<rte::ceil_div(rows, SB_WARPS), SB_WARPS * 32, smem, ST(stream)>>>(
      targets, top_clusters, random_negs ? random_negs : top_clusters, shortlist, dup_count, rows, D, status);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_shortlist_ce(const void* hidden, const void* W, const int32_t* shortlist, const float* row_weight, int32_t S,
                                float* loss_tok, void* logits_out, void* dlogits_dense, int32_t rows, int32_t d, int32_t V,
                                int32_t K, rte_stream_t stream) {
  RTE_CHECK_ARG(hidden && W && shortlist && loss_tok && rows > 0 && d > 0 && d % 8 == 0 && V % 8 == 0 && K > 0 && S > 0);
  RTE_CHECK_ARG(dlogits_dense == nullptr || row_weight != nullptr);
  if ((reinterpret_cast<uintptr_t>(W) & 15) || (dlogits_dense && (reinterpret_cast<uintptr_t>(dlogits_dense) & 15))) return RTE_ERR_ALIGNMENT;
  const size_t smem = (size_t)(d + K) * sizeof(float);
  if (smem > 48 * 1024) return RTE_ERR_UNSUPPORTED;
  shortlist_ce_kernel<<<rows, 128, smem, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(hidden),
      reinterpret_cast<const __nv_bfloat16*>(W), shortlist, row_weight, S, loss_tok,
      reinterpret_cast<__nv_bfloat16*>(logits_out), reinterpret_cast<__nv_bfloat16*>(dlogits_dense), d, V, K);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_shortlist_ce_from_logits(void* logits_inout, const int32_t* shortlist, const float* row_weight, int32_t S,
                                           float* loss_tok, int32_t rows, int32_t V, int32_t K, rte_stream_t stream) {
  RTE_CHECK_ARG(logits_inout && shortlist && row_weight && loss_tok && rows > 0 && S > 0 && V > 0 && V % 8 == 0 && K > 0);
  if (reinterpret_cast<uintptr_t>(logits_inout) & 15) return RTE_ERR_ALIGNMENT;
  const size_t smem = (size_t)K * sizeof(float);
  if (smem > 48 * 1024) return RTE_ERR_UNSUPPORTED;
  shortlist_ce_logits_kernel<<<rows, 128, smem, ST(stream)>>>(reinterpret_cast<__nv_bfloat16*>(logits_inout), shortlist, row_weight,
                                                             S, loss_tok, V, K);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_scatter_cols_bf16(const void* vals, const int32_t* ids, void* dense, int32_t rows, int32_t V, int32_t K,
                                     rte_stream_t stream) {
  RTE_CHECK_ARG(vals && ids && dense && rows > 0 && V > 0 && V % 8 == 0 && K > 0);
  if (reinterpret_cast<uintptr_t>(dense) & 15) return RTE_ERR_ALIGNMENT;
  scatter_cols_kernel<<<rows, 128, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(vals), ids,
                                                    reinterpret_cast<__nv_bfloat16*>(dense), V, K);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_random_tokens(int32_t* out, int64_t n, int32_t vocab, const int64_t* seed, rte_stream_t stream) {
  RTE_CHECK_ARG(out && seed && n > 0 && vocab > 0);
  long long g = (n + 255) / 256;
  if (g > 148 * 8) g = 148 * 8;
  random_tokens_kernel<<<(int)g, 256, 0, ST(stream)>>>(out, n, vocab, seed);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
