// Few-row GEMM for the audit replay's launch chain: C[M,N] = A[M,K] * B^T with M of the order of one sample
// (64..256 rows).  The persistent tcgen05 kernel spends most of such a launch on set-up (barriers, TMEM
// allocation, tensor maps, TMA round trips) and covers N with a handful of CTAs; here every 64x64 output tile
// is its own 128-thread CTA that streams its operands with cp.async (an 8-deep ring of k-tiles) and issues
// mma.sync.m16n8k16, so a [64 x 1536 x 512] product is 24 CTAs of ~2 us instead of 6 CTAs of ~10 us.
// bf16 in, fp32 accumulate; B either K-major ([N,K], nn.Linear layout) or MN-major ([K,N], the banked layout);
// outputs bf16 or fp32 (+ fp32 residual), optional split along K into partial results (fp32, reduced by
// rte_reduce_splits in fixed order).
//
// The same kernel covers the replay's weight gradients dW[M,N] (+)= A^T B with A stored [K,M], B stored [K,N] and a
// reduction of only K = rows-of-one-sample (64..256): an update of rank K whose cost is reading and writing dW.
//
// These launches run beside a hot pass whose persistent GEMM owns all the shared memory of every SM it sits on, so
// what is left for them is a handful of SMs.  The ring of k-tiles is as deep as the reduction needs and no deeper
// (2, 4 or 8 stages), so that short reductions leave room for several CTAs per SM.

#include "rte_common.cuh"

namespace {

constexpr int BM = 64, BK = 64, LDS = BK + 8, THR = 128;       // BN (64 or 32) is a template parameter
constexpr int smem_bytes(int nst, int bn, bool b_mn) {       // nst stages of an A tile and a B tile
  return nst * (BM * LDS + (b_mn ? BK * (bn + 8) : bn * LDS)) * 2;
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool valid) {
  const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
  const int bytes = valid ? 16 : 0;                       // 0: the 16 bytes are zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void ldsm_x2_trans(uint32_t& b0, uint32_t& b1, const __nv_bfloat16* row_ptr) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(row_ptr));
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0,%1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&a)[4], const __nv_bfloat16* row_ptr) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(row_ptr));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(a[0]), "=r"(a[1]), "=r"(a[2]), "=r"(a[3]) : "r"(addr));
}
__device__ __forceinline__ uint32_t ld32(const __nv_bfloat16* p) { return *reinterpret_cast<const uint32_t*>(p); }

struct SmallParams {
  const __nv_bfloat16* A; int lda;
  const __nv_bfloat16* B; int ldb;
  void* C; int ldc;
  const float* R; int ldr;
  int M, N, K;
  int k_per_split; long long split_stride;
  int* counters; float* red_out; int red_accumulate;      // in-launch reduction of the split partials (or counters == NULL)
};

// The legacy mma.sync path peaks near 2 TFLOP/s per SM on this part, so a CTA's speed is set by how many MMAs it
// issues per k-tile: narrow (BN = 32) tiles double the CTA count when the wide grid would leave most SMs idle.
// A_MN: A is stored [K, M] (its tile sits in shared memory as [k][m] and the fragments come out of ldmatrix.trans).
// NST: k-tiles in flight (a ring of NST stages, NST - 1 of them prefetched).
template <bool A_MN, bool B_MN, bool OUT_F32, int BN, int NST>
__global__ void __launch_bounds__(THR)
gemm_small_kernel(const SmallParams p) {
  constexpr int LDB = B_MN ? BN + 8 : LDS;       // row stride of the B tile ([k][n] rows are BN long, [n][k] rows BK long)
  constexpr int B_ROWS = B_MN ? BK : BN;
  extern __shared__ __align__(16) uint8_t smraw[];
  __nv_bfloat16 (*sa)[BM * LDS] = reinterpret_cast<__nv_bfloat16 (*)[BM * LDS]>(smraw);
  __nv_bfloat16 (*sb)[B_ROWS * LDB] = reinterpret_cast<__nv_bfloat16 (*)[B_ROWS * LDB]>(smraw + NST * BM * LDS * 2);   // K-major B: [n][k]; MN-major: [k][n]
  static_assert(BM == BK, "the A tile has the same footprint in either orientation");
  const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
  const int k_lo = blockIdx.z * p.k_per_split, k_hi = min(p.K, k_lo + p.k_per_split);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, g = lane >> 2, t = lane & 3;

  auto load_tile = [&](int buf, int k0) {
    // out-of-range chunks are zero-filled; their source address is clamped to the matrix base (never dereferenced)
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int chunk = threadIdx.x + i * THR, r = chunk >> 3, c = (chunk & 7) * 8;
      if (!A_MN) {                                         // row r of the tile = output row, c = offset along k
        const bool va = (m0 + r) < p.M && (k0 + c) < k_hi;
        cp_async16(&sa[buf][r * LDS + c], va ? p.A + (size_t)(m0 + r) * p.lda + k0 + c : p.A, va);
      } else {                                             // row r of the tile = k, c = offset along the output rows
        const bool va = (k0 + r) < k_hi && (m0 + c) < p.M;
        cp_async16(&sa[buf][r * LDS + c], va ? p.A + (size_t)(k0 + r) * p.lda + m0 + c : p.A, va);
      }
    }
    if (!B_MN) {
#pragma unroll
      for (int i = 0; i < BN * 8 / THR; ++i) {            // BN rows of BK elements
        const int chunk = threadIdx.x + i * THR, r = chunk >> 3, c = (chunk & 7) * 8;
        const bool vb = (n0 + r) < p.N && (k0 + c) < k_hi;
        cp_async16(&sb[buf][r * LDB + c], vb ? p.B + (size_t)(n0 + r) * p.ldb + k0 + c : p.B, vb);
      }
    } else {
      constexpr int CPR = BN / 8;                         // 16-byte chunks per k-row
#pragma unroll
      for (int i = 0; i < BK * CPR / THR; ++i) {          // BK rows of BN elements
        const int chunk = threadIdx.x + i * THR, r = chunk / CPR, c = (chunk % CPR) * 8;
        const bool vb = (k0 + r) < k_hi && (n0 + c) < p.N;
        cp_async16(&sb[buf][r * LDB + c], vb ? p.B + (size_t)(k0 + r) * p.ldb + n0 + c : p.B, vb);
      }
    }
  };

  float acc[BN / 8][4];
#pragma unroll
  for (int nt = 0; nt < BN / 8; ++nt) acc[nt][0] = acc[nt][1] = acc[nt][2] = acc[nt][3] = 0.f;

  const int ktiles = (k_hi - k_lo + BK - 1) / BK;
  // NST-deep ring: one commit group per k-tile slot (empty groups keep the counting uniform)
#pragma unroll
  for (int s_ = 0; s_ < NST - 1; ++s_) {
    if (s_ < ktiles) load_tile(s_, k_lo + s_ * BK);
    cp_async_commit();
  }
  for (int kt = 0; kt < ktiles; ++kt) {
    const int buf = kt % NST;
    cp_async_wait<NST - 2>();                   // tile kt has landed
    __syncthreads();                            // ... for every thread, and everyone is done with tile kt-1
    {
      const int nx = kt + NST - 1;              // refill the slot tile kt-1 used
      if (nx < ktiles) load_tile(nx % NST, k_lo + nx * BK);
      cp_async_commit();
    }
    const __nv_bfloat16* a = sa[buf] + (warp * 16) * LDS;
    const __nv_bfloat16* b = sb[buf];
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t af[4];
      if (!A_MN) {
        af[0] = ld32(a + g * LDS + ks * 16 + 2 * t);
        af[1] = ld32(a + (g + 8) * LDS + ks * 16 + 2 * t);
        af[2] = ld32(a + g * LDS + ks * 16 + 8 + 2 * t);
        af[3] = ld32(a + (g + 8) * LDS + ks * 16 + 8 + 2 * t);
      } else {
        // four transposed 8x8 blocks of the [k][m] tile: (k lo, m lo), (k lo, m hi), (k hi, m lo), (k hi, m hi)
        const int j = lane >> 3, i = lane & 7;
        ldsm_x4_trans(af, sa[buf] + (ks * 16 + (j >> 1) * 8 + i) * LDS + warp * 16 + (j & 1) * 8);
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt) {
        uint32_t b0, b1;
        if (!B_MN) {
          b0 = ld32(b + (nt * 8 + g) * LDB + ks * 16 + 2 * t);
          b1 = ld32(b + (nt * 8 + g) * LDB + ks * 16 + 8 + 2 * t);
        } else {
          ldsm_x2_trans(b0, b1, b + (ks * 16 + (lane & 15)) * LDB + nt * 8);
        }
        mma16816(acc[nt], af, b0, b1);
      }
    }
  }
  cp_async_wait<0>();

  const int row_a = m0 + warp * 16 + g, row_b = row_a + 8;
#pragma unroll
  for (int nt = 0; nt < BN / 8; ++nt) {
    const int col = n0 + nt * 8 + 2 * t;
    if (col >= p.N) continue;
    const bool two = col + 1 < p.N;
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const int row = h ? row_b : row_a;
      if (row >= p.M) continue;
      float v0 = acc[nt][2 * h], v1 = acc[nt][2 * h + 1];
      if (OUT_F32) {
        float* out = reinterpret_cast<float*>(p.C) + (size_t)blockIdx.z * p.split_stride + (size_t)row * p.ldc + col;
        if (p.R) { const float* r = p.R + (size_t)row * p.ldr + col; v0 += r[0]; if (two) v1 += r[1]; }
        out[0] = v0;
        if (two) out[1] = v1;
      } else {
        __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + (size_t)row * p.ldc + col;
        out[0] = __float2bfloat16_rn(v0);
        if (two) out[1] = __float2bfloat16_rn(v1);
      }
    }
  }
  if (OUT_F32 && p.counters != nullptr && gridDim.z > 1) {
    // The last CTA to finish this output tile sums the tile's partials in split order (a fixed order: the result does
    // not depend on which CTA comes last) and writes the final values; the counter is left at zero for the next launch.
    __shared__ int last_s;
    __threadfence();
    __syncthreads();
    const int tile = blockIdx.y * gridDim.x + blockIdx.x;
    if (threadIdx.x == 0) last_s = (atomicAdd(p.counters + tile, 1) == (int)gridDim.z - 1) ? 1 : 0;
    __syncthreads();
    if (last_s) {
      __threadfence();
      const float* ws = reinterpret_cast<const float*>(p.C);
      for (int e = threadIdx.x; e < BM * BN; e += THR) {
        const int r = m0 + e / BN, c = n0 + e % BN;
        if (r >= p.M || c >= p.N) continue;
        const size_t o = (size_t)r * p.ldc + c;
        float acc = p.red_accumulate ? p.red_out[(size_t)r * p.N + c] : 0.f;
        for (int s_ = 0; s_ < (int)gridDim.z; ++s_) acc += ws[(size_t)s_ * p.split_stride + o];
        p.red_out[(size_t)r * p.N + c] = acc;
      }
      if (threadIdx.x == 0) p.counters[tile] = 0;
    }
  }
}

}  // namespace

extern "C" int rte_gemm_bf16_small(const rte_gemm_args* a, rte_stream_t stream) {
  RTE_CHECK_ARG(a != nullptr && a->A && a->B && a->C && a->M > 0 && a->N > 0 && a->K > 0);
  RTE_CHECK_ARG(a->tile_group == nullptr && a->split_kblocks == nullptr);
  RTE_CHECK_ARG(!a->a_mn_major || (a->b_mn_major && a->epilogue == RTE_EPI_F32));      // A^T only for weight gradients
  RTE_CHECK_ARG(a->epilogue == RTE_EPI_BF16 || a->epilogue == RTE_EPI_F32);
  const int splits = a->splits < 1 ? 1 : a->splits;
  RTE_CHECK_ARG(splits == 1 || (a->epilogue == RTE_EPI_F32 && a->R == nullptr));
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) || (a->lda % 8) || (a->ldb % 8) ||
      (a->K % 8) || (a->b_mn_major && (a->N % 8)) || (a->a_mn_major && (a->M % 8)))
    return RTE_ERR_ALIGNMENT;
  SmallParams p;
  p.A = reinterpret_cast<const __nv_bfloat16*>(a->A); p.lda = a->lda;
  p.B = reinterpret_cast<const __nv_bfloat16*>(a->B); p.ldb = a->ldb;
  p.C = a->C; p.ldc = a->ldc; p.R = reinterpret_cast<const float*>(a->R); p.ldr = a->ldr;
  p.M = a->M; p.N = a->N; p.K = a->K;
  const int ktiles = rte::ceil_div(a->K, BK);
  p.k_per_split = rte::ceil_div(ktiles, splits) * BK;
  RTE_CHECK_ARG(rte::ceil_div(a->K, p.k_per_split) == splits);      // every partial must be written
  p.split_stride = a->split_stride;
  p.counters = splits > 1 ? a->split_counters : nullptr;
  p.red_out = a->split_out;
  p.red_accumulate = a->split_accumulate;
  RTE_CHECK_ARG(p.counters == nullptr || (p.red_out != nullptr && rte::ceil_div(a->N, 32) * rte::ceil_div(a->M, BM) <= 1024));
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  const bool f32 = a->epilogue == RTE_EPI_F32;
  const int wide_ctas = rte::ceil_div(a->N, 64) * rte::ceil_div(a->M, BM) * splits;
  const bool narrow = wide_ctas < 74;                    // fewer CTAs than half the SMs: halve the tile width
  // k-tiles in flight: the whole reduction of a CTA up to eight tiles (one round trip to memory instead of several --
  // the launch is latency-bound), but no more stages than the reduction has tiles
  const int kt_cta = rte::ceil_div(p.k_per_split < a->K ? p.k_per_split : a->K, BK);
  const int depth = kt_cta > 4 ? 8 : kt_cta > 2 ? 4 : 2;
#define RTE_SMALL_LAUNCH(AMN, BMN, F32, BNV, NSTV)                                                                    \
  do {                                                                                                                \
    constexpr int SM_ = smem_bytes(NSTV, BNV, BMN);                                                                   \
    static bool set_ = false;                                                                                         \
    if (!set_) {                                                                                                      \
      if (cudaFuncSetAttribute(gemm_small_kernel<AMN, BMN, F32, BNV, NSTV>,                                           \
                               cudaFuncAttributeMaxDynamicSharedMemorySize, SM_) != cudaSuccess)                      \
        return RTE_ERR_LAUNCH;                                                                                        \
      set_ = true;                                                                                                    \
    }                                                                                                                 \
    gemm_small_kernel<AMN, BMN, F32, BNV, NSTV><<<dim3(rte::ceil_div(a->N, BNV), rte::ceil_div(a->M, BM), splits),   \
                                                  THR, SM_, st>>>(p);                                                 \
  } while (0)
#define RTE_SMALL_PICK(AMN, BMN, F32)                                                                                 \
  do {                                                                                                                \
    if (narrow) {                                                                                                     \
      if (depth == 8) RTE_SMALL_LAUNCH(AMN, BMN, F32, 32, 8);                                                         \
      else if (depth == 4) RTE_SMALL_LAUNCH(AMN, BMN, F32, 32, 4);                                                    \
      else RTE_SMALL_LAUNCH(AMN, BMN, F32, 32, 2);                                                                    \
    } else {                                                                                                          \
      if (depth == 8) RTE_SMALL_LAUNCH(AMN, BMN, F32, 64, 8);                                                         \
      else if (depth == 4) RTE_SMALL_LAUNCH(AMN, BMN, F32, 64, 4);                                                    \
      else RTE_SMALL_LAUNCH(AMN, BMN, F32, 64, 2);                                                                    \
    }                                                                                                                 \
  } while (0)
  if (a->a_mn_major) {
    RTE_SMALL_PICK(true, true, true);                    // weight gradient: both operands [K, *], fp32 out
  } else if (a->b_mn_major) {
    if (f32) RTE_SMALL_PICK(false, true, true); else RTE_SMALL_PICK(false, true, false);
  } else {
    if (f32) RTE_SMALL_PICK(false, false, true); else RTE_SMALL_PICK(false, false, false);
  }
#undef RTE_SMALL_PICK
#undef RTE_SMALL_LAUNCH
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
