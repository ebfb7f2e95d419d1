// Static cluster-pool sparse SwiGLU FFN: the pieces around the grouped tensor-core GEMMs
// (reference layers.py:188-220, kernels/cluster_pool_ffn.py:90-241).
//
//   route  : token -> centre with the largest score (lowest index on ties), scores = q . centre
//            (the reference L2-normalises q first; a positive per-token scale cannot change the arg-max)
//   pack   : stable counting sort of the tokens by cluster into ONE packed row order in which every cluster
//            starts on a 128-row boundary, so each 128-row GEMM tile belongs to exactly one cluster and
//            no shape ever depends on the routing (the reference pads every cluster to the largest one and
//            reads that size back to the host).  Emits the tile -> cluster table and the per-cluster
//            k-block ranges the grouped GEMMs consume.
//   gather : row gather with conversion and zero fill (pack x / dY, un-pack Y / dX)
//   reduce : pool-gradient rows summed into dense FFN rows through a CSR built once per codebook: a
//            gather-reduce in fixed order instead of the reference's index_add_ scatter (no atomics,
//            bitwise reproducible).
//   transpose: [R, C] fp32 -> [C, R] bf16 / fp32 (W_down is stored [d, F]; its pool rows are rows of W_down^T)

#include "rte_common.cuh"

namespace {

constexpr int PACK_THREADS = 1024;
constexpr int MAX_CLUSTERS = 64;

// one warp per token
__global__ void __launch_bounds__(256)
cluster_route_kernel(const float* __restrict__ q, int ldq, const float* __restrict__ centers, int32_t* __restrict__ assign,
                     float* __restrict__ scores_out, int n, int W, int C) {
  extern __shared__ float sc[];              // centres [C][W] when they fit
  const bool in_smem = (size_t)C * W * sizeof(float) <= 96 * 1024;
  if (in_smem) {
    for (int i = threadIdx.x; i < C * W; i += blockDim.x) sc[i] = centers[i];
    __syncthreads();
  }
  const float* cen = in_smem ? sc : centers;
  const int lane = threadIdx.x & 31;
  const int tok = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (tok >= n) return;
  const float* row = q + (size_t)tok * ldq;
  float best = -INFINITY;
  int best_c = 0;
  for (int c = 0; c < C; ++c) {
    float acc = 0.f;
    for (int k = lane; k < W; k += 32) acc += row[k] * cen[(size_t)c * W + k];
    acc = rte::warp_sum(acc);
    if (scores_out && lane == 0) scores_out[(size_t)tok * C + c] = acc;
    if (acc > best) { best = acc; best_c = c; }          // strict: the lowest index wins ties
  }
  if (lane == 0) assign[tok] = best_c;
}

// Single CTA.  perm[p] = token packed at row p (-1: padding row); pos[token] = its packed row.
__global__ void __launch_bounds__(PACK_THREADS)
cluster_pack_kernel(const int32_t* __restrict__ assign, int n, int C, int cap, int32_t* __restrict__ perm,
                    int32_t* __restrict__ pos, int32_t* __restrict__ counts, int32_t* __restrict__ offsets,
                    int32_t* __restrict__ tile_group, int32_t* __restrict__ kblocks, int* status) {
  __shared__ int cnt[MAX_CLUSTERS];
  __shared__ int base[MAX_CLUSTERS + 1];
  __shared__ int wc[PACK_THREADS / 32][MAX_CLUSTERS];
  __shared__ int bad;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  if (tid < MAX_CLUSTERS) cnt[tid] = 0;
  if (tid == 0) bad = 0;
  __syncthreads();
  for (int i = tid; i < n; i += PACK_THREADS) {
    const int a = assign[i];
    if (a < 0 || a >= C) bad = 1; else atomicAdd(&cnt[a], 1);
  }
  for (int i = tid; i < cap; i += PACK_THREADS) perm[i] = -1;
  __syncthreads();
  if (tid == 0) {
    int off = 0;
    for (int c = 0; c < C; ++c) {
      base[c] = off;
      offsets[c] = off;
      kblocks[c] = off / 64;
      counts[c] = cnt[c];
      off += (cnt[c] + 127) / 128 * 128;
    }
    base[C] = off;
    offsets[C] = off;
    kblocks[C] = off / 64;
    if (off > cap || bad) { if (status) atomicExch(status, off > cap ? RTE_DEV_CAPACITY_OVERFLOW : RTE_DEV_INDEX_OUT_OF_RANGE); bad = 1; }
  }
  __syncthreads();
  for (int b = tid; b < cap / 128; b += PACK_THREADS) {
    int g = -1;
    if (!bad)
      for (int c = 0; c < C; ++c)
        if (b * 128 >= base[c] && b * 128 < base[c + 1]) g = c;
    tile_group[b] = g;
  }
  if (bad) { for (int i = tid; i < n; i += PACK_THREADS) pos[i] = -1; return; }
  __syncthreads();
  // stable placement: token order is kept inside every cluster
  for (int i0 = 0; i0 < n; i0 += PACK_THREADS) {
    for (int i = tid; i < (PACK_THREADS / 32) * MAX_CLUSTERS; i += PACK_THREADS) (&wc[0][0])[i] = 0;
    __syncthreads();
    const int i = i0 + tid;
    const int a = (i < n) ? assign[i] : -1 - lane;           // idle lanes get distinct dummies
    const unsigned peers = __match_any_sync(0xffffffffu, a);
    const int rank_in_warp = __popc(peers & ((1u << lane) - 1u));
    if (a >= 0 && rank_in_warp == 0) wc[warp][a] = __popc(peers);
    __syncthreads();
    if (a >= 0) {
      int before = 0;
      for (int w = 0; w < warp; ++w) before += wc[w][a];
      const int p = base[a] + before + rank_in_warp;
      perm[p] = i;
      pos[i] = p;
    }
    __syncthreads();
    if (tid < C) {
      int tot = 0;
      for (int w = 0; w < PACK_THREADS / 32; ++w) tot += wc[w][tid];
      base[tid] += tot;
    }
    __syncthreads();
  }
}

// dst[i, :] = convert(src[idx[i], :]) or zeros when idx[i] < 0; 4 elements per thread
template <typename TS, typename TD>
__global__ void __launch_bounds__(256)
gather_convert_kernel(const TS* __restrict__ src, const int32_t* __restrict__ idx, TD* __restrict__ dst, long long n_out, int d) {
  const int d4 = d >> 2;
  const long long total = n_out * d4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / d4;
    const int c = int(i % d4) << 2;
    const int s = idx[r];
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    if (s >= 0) {
      const TS* p = src + (size_t)s * d + c;
#pragma unroll
      for (int k = 0; k < 4; ++k) v[k] = (float)p[k];
    }
    TD* o = dst + (size_t)r * d + c;
#pragma unroll
    for (int k = 0; k < 4; ++k) o[k] = (TD)v[k];
  }
}

// dense[f, :] (+)= sum over k in [row_ptr[f], row_ptr[f+1]) of src[rows[k], :]     (fixed order)
__global__ void __launch_bounds__(256)
csr_row_reduce_kernel(const float* __restrict__ src, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ rows,
                      float* __restrict__ dense, long long n_dense, int d, int accumulate) {
  const int d4 = d >> 2;
  const long long total = n_dense * d4;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long f = i / d4;
    const int c = int(i % d4) << 2;
    float4 acc = accumulate ? *reinterpret_cast<const float4*>(dense + (size_t)f * d + c) : make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = row_ptr[f]; k < row_ptr[f + 1]; ++k) {
      const float4 t = *reinterpret_cast<const float4*>(src + (size_t)rows[k] * d + c);
      acc.x += t.x; acc.y += t.y; acc.z += t.z; acc.w += t.w;
    }
    *reinterpret_cast<float4*>(dense + (size_t)f * d + c) = acc;
  }
}

template <typename TD>
__global__ void __launch_bounds__(256)
transpose_kernel(const float* __restrict__ src, TD* __restrict__ dst, int R, int C, int accumulate) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;          // 32 x 8
  for (int j = ty; j < 32; j += 8) {
    const int r = r0 + j, c = c0 + tx;
    tile[j][tx] = (r < R && c < C) ? src[(size_t)r * C + c] : 0.f;
  }
  __syncthreads();
  for (int j = ty; j < 32; j += 8) {
    const int c = c0 + j, r = r0 + tx;
    if (r < R && c < C) {
      const size_t o = (size_t)c * R + r;
      const float v = tile[tx][j] + (accumulate ? (float)dst[o] : 0.f);
      dst[o] = (TD)v;
    }
  }
}

inline int grid_for(long long n, int block, int cap = 148 * 16) {
  long long g = (n + block - 1) / block;
  return (int)(g < 1 ? 1 : (g > cap ? cap : g));
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int rte_cluster_route(const float* q, int32_t ldq, const float* centers, int32_t* assignments, float* scores_out,
                                 int32_t n_tokens, int32_t width, int32_t n_clusters, rte_stream_t stream) {
  RTE_CHECK_ARG(q && centers && assignments && n_tokens > 0 && width > 0 && n_clusters > 0 && ldq >= width);
  const size_t smem = (size_t)n_clusters * width * sizeof(float);
  const size_t use = smem <= 96 * 1024 ? smem : 0;
  if (use > 48 * 1024) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(cluster_route_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024) != cudaSuccess)
        return RTE_ERR_LAUNCH;
      set = true;
    }
  }
  cluster_route_kernel<<<rte::ceil_div(n_tokens, 8), 256, use, ST(stream)>>>(q, ldq, centers, assignments, scores_out, n_tokens,
                                                                            width, n_clusters);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_cluster_pack(const int32_t* assignments, int32_t n_tokens, int32_t n_clusters, int32_t capacity_rows,
                                int32_t* perm, int32_t* pos, int32_t* counts, int32_t* offsets, int32_t* tile_group,
                                int32_t* kblocks, int32_t* status, rte_stream_t stream) {
  RTE_CHECK_ARG(assignments && perm && pos && counts && offsets && tile_group && kblocks && n_tokens > 0 && n_clusters > 0);
  RTE_CHECK_ARG(capacity_rows > 0 && capacity_rows % 128 == 0);
  if (n_clusters > MAX_CLUSTERS) return RTE_ERR_UNSUPPORTED;
  cluster_pack_kernel<<<1, PACK_THREADS, 0, ST(stream)>>>(assignments, n_tokens, n_clusters, capacity_rows, perm, pos, counts,
                                                          offsets, tile_group, kblocks, status);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_gather_rows_convert(const void* src, int32_t src_bf16, const int32_t* idx, void* dst, int32_t dst_bf16,
                                       int64_t n_out, int32_t d, rte_stream_t stream) {
  RTE_CHECK_ARG(src && idx && dst && n_out > 0 && d > 0 && d % 4 == 0);
  const int g = grid_for(n_out * (d / 4), 256);
  using bf = __nv_bfloat16;
  if (src_bf16 && dst_bf16) gather_convert_kernel<bf, bf><<<g, 256, 0, ST(stream)>>>((const bf*)src, idx, (bf*)dst, n_out, d);
  else if (src_bf16) gather_convert_kernel<bf, float><<<g, 256, 0, ST(stream)>>>((const bf*)src, idx, (float*)dst, n_out, d);
  else if (dst_bf16) gather_convert_kernel<float, bf><<<g, 256, 0, ST(stream)>>>((const float*)src, idx, (bf*)dst, n_out, d);
  else gather_convert_kernel<float, float><<<g, 256, 0, ST(stream)>>>((const float*)src, idx, (float*)dst, n_out, d);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_csr_row_reduce_f32(const float* src, const int32_t* row_ptr, const int32_t* rows, float* dense,
                                      int64_t n_dense_rows, int32_t d, int32_t accumulate, rte_stream_t stream) {
  RTE_CHECK_ARG(src && row_ptr && rows && dense && n_dense_rows > 0 && d > 0 && d % 4 == 0);
  if ((reinterpret_cast<uintptr_t>(src) & 15) || (reinterpret_cast<uintptr_t>(dense) & 15)) return RTE_ERR_ALIGNMENT;
  csr_row_reduce_kernel<<<grid_for(n_dense_rows * (d / 4), 256), 256, 0, ST(stream)>>>(src, row_ptr, rows, dense, n_dense_rows, d,
                                                                                     accumulate);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_transpose_f32(const float* src, void* dst, int32_t rows, int32_t cols, int32_t dst_bf16, int32_t accumulate,
                                 rte_stream_t stream) {
  RTE_CHECK_ARG(src && dst && rows > 0 && cols > 0);
  dim3 grid(rte::ceil_div(cols, 32), rte::ceil_div(rows, 32));
  if (dst_bf16) transpose_kernel<__nv_bfloat16><<<grid, 256, 0, ST(stream)>>>(src, (__nv_bfloat16*)dst, rows, cols, accumulate);
  else transpose_kernel<float><<<grid, 256, 0, ST(stream)>>>(src, (float*)dst, rows, cols, accumulate);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
