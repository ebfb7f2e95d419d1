// Persistent warp-specialised bf16 GEMM for sm_100a:
//   C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory (TMEM),
//   operands staged by TMA into 128B-swizzled shared memory, MMAs issued by one
//   thread with tcgen05.mma.
//
// Two shapes of work unit (template parameter CTAS):
//   CTAS = 1: one CTA computes a 128 x BN tile (tcgen05.mma.cta_group::1, M = 128).
//   CTAS = 2: a cluster of two CTAs on neighbouring SMs computes a 256 x BN tile with
//             tcgen05.mma.cta_group::2 (M = 256): each CTA stages its own 128 rows of A and
//             its own HALF of the B tile (plain per-CTA TMA loads, no multicast), the MMA
//             of the leader CTA reads both halves, and each CTA's TMEM receives the
//             accumulators of its 128 rows.  Per FLOP this moves a third less operand
//             data from L2 into shared memory than two independent 128 x BN tiles,
//             which is what bounds the short-K products of the training step.
//
// Roles per CTA (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer (the leader CTA's only, with CTAS = 2), warps 2..9 = epilogue: warp w may
// read the TMEM lane quadrant w % 4 (32 rows); the two warps of a quadrant split the
// tile's columns.  Every epilogue warp owns private staging slots in shared memory
// and hands its 32 x 64 (bf16) or 32 x 32 (fp32) pieces to the TMA by itself, so no
// barrier couples the epilogue warps.  Two accumulator buffers in TMEM let the
// epilogue of tile i overlap the main loop of tile i+1.  Every wait is bounded: on
// expiry the role records a code in the caller's status word and all roles drain to
// the common teardown, which frees TMEM.
//
// Either operand may be "MN-major" (stored with the reduction dimension as the
// slow axis), which is what the weight- and data-gradient GEMMs of the training
// step need; no transposed copies are ever made.

#include <cuda.h>
#include <stdlib.h>

#include "rte_common.cuh"

namespace {

constexpr int BM = 128;         // rows of C per CTA (TMEM lanes)
constexpr int BK = 64;          // bf16 elements per k-block (= one 128-byte swizzle row)
constexpr int UMMA_K = 16;      // K per tcgen05.mma for 16-bit inputs
constexpr int NUM_THREADS = 320;   // warp 0 producer, warp 1 MMA issuer, warps 2..9 epilogue
constexpr int EPI_WARPS = 8;
constexpr int SLOT_BYTES = 4096;       // one epilogue staging slot: 32 rows x 128 bytes
constexpr int MAX_DYN_SMEM = 232448;   // 227 KB of dynamic shared memory per CTA
constexpr uint32_t WAIT_LIMIT = 24u * 1000u * 1000u;   // polls (with back-off) before a wait gives up

#ifdef RTE_GEMM_DIAG
constexpr bool DIAG = true;    // timing diagnostics: RTE_GEMM_DIAG_FLAGS bit 0 = no stores, 1 = no MMAs, 2 = no loads
#else
constexpr bool DIAG = false;
#endif

struct KParams {
  int diag;
  int M, N, K;
  int a_mn, b_mn;
  int epilogue;
  void* C; int ldc;
  const void* R; int ldr;
  void* C2; int ldc2;
  int pair_off;
  int splits; long long split_stride;
  int num_m_blocks, num_n_blocks, kblocks_total, kblocks_per_split;
  int tma_store;            // 1: outputs leave through shared-memory staging + TMA bulk stores
  int b_box_rows;           // K-major B: rows per TMA box
  const int* tile_group;    // grouped mode: group id of every 128-row block of A/C (< 0: block unused), else null
  int b_group_stride;       // grouped mode: rows of the stacked B between consecutive groups
  const int* split_kb;      // ragged split-K: k-block range [split_kb[s], split_kb[s+1]) of split s, else null
  int* status;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ uint32_t cluster_ctarank() {
  uint32_t r;
  asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
  return r;
}
// Address of this CTA's shared-memory location `addr` as seen in CTA `rank` of the cluster.
__device__ __forceinline__ uint32_t mapa_cluster(uint32_t addr, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(rank));
  return r;
}
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// Arrive on a barrier of another CTA of the cluster (`bar` is a shared::cluster address from mapa_cluster).
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar) {
  asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar) : "memory");
}
template <int CTAS>
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  if (CTAS == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  } else {      // arrivals may come from the peer CTA: cluster-scope acquire
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  }
  return ok != 0;
}
// Bounded wait: returns false when the limit ran out.
template <int CTAS>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_test<CTAS>(bar, parity)) return true;
    if (i > 128) __nanosleep(i > 4096 ? 128 : 32);
  }
  return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// `bar`: CTAS = 1 the CTA's own barrier; CTAS = 2 the LEADER CTA's barrier (shared::cluster address), which counts the
// bytes of both CTAs' loads.
template <int CTAS>
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  if (CTAS == 1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  } else {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
        : "memory");
  }
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap* map, uint32_t src, int x, int y, int z) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
               ::"l"(reinterpret_cast<uint64_t>(map)), "r"(src), "r"(x), "r"(y), "r"(z)
               : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void bulk_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

template <int CTAS>
__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  if (CTAS == 1) asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
  else asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_relinquish() {
  if (CTAS == 1) asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  else asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
template <int CTAS>
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  if (CTAS == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
  else asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// Arrives on `bar` once the MMAs issued so far have completed; CTAS = 2: on the barrier at the same offset in BOTH CTAs.
template <int CTAS>
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  if (CTAS == 1) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
  } else {
    const uint16_t both = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"(both) : "memory");
  }
}
template <int CTAS>
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  if (CTAS == 1) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  } else {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
  }
}
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor (128-byte swizzle, descriptor version 1 for sm_100).
//  K-major tile : rows of 128 B, 8-row groups 1024 B apart (stride byte offset), leading offset unused.
//  MN-major tile: 64-element (128 B) runs along MN, 8 k-rows per 1024 B atom (stride byte offset),
//                 next 64 MN elements 8192 B further (leading byte offset).
__device__ __forceinline__ uint64_t make_smem_desc(uint32_t saddr, bool mn_major) {
  uint64_t desc = static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  desc |= static_cast<uint64_t>(mn_major ? (8192u >> 4) : 1u) << 16;
  desc |= static_cast<uint64_t>(1024u >> 4) << 32;
  desc |= 1ull << 46;
  desc |= 2ull << 61;
  return desc;
}

// ------------------------------------------------------------------ epilogue helpers
// SiLU / sigmoid for the fused epilogues: ex2.approx + the fast divide (2 ulp), with no slow path for huge or
// denormal denominators (an IEEE divide takes hundreds of cycles there and would stall the whole epilogue warp).
// The results are rounded to bf16 right away, so the difference from the exact functions is far below one bf16 ulp.
__device__ __forceinline__ float fast_sigmoid(float g) { return __fdividef(1.f, 1.f + __expf(-g)); }
__device__ __forceinline__ float fast_silu(float g) { return __fdividef(g, 1.f + __expf(-g)); }

__device__ __forceinline__ void store_bf16x32(__nv_bfloat16* dst, const float (&v)[32], int ncols_valid) {
  if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    uint4* d4 = reinterpret_cast<uint4*>(dst);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 w;
      w.x = rte::pack_bf16x2(v[8 * q + 0], v[8 * q + 1]);
      w.y = rte::pack_bf16x2(v[8 * q + 2], v[8 * q + 3]);
      w.z = rte::pack_bf16x2(v[8 * q + 4], v[8 * q + 5]);
      w.w = rte::pack_bf16x2(v[8 * q + 6], v[8 * q + 7]);
      d4[q] = w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols_valid) dst[j] = __float2bfloat16_rn(v[j]);
  }
}
__device__ __forceinline__ void store_f32x32(float* dst, const float (&v)[32], int ncols_valid) {
  if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
    float4* d4 = reinterpret_cast<float4*>(dst);
#pragma unroll
    for (int q = 0; q < 8; ++q) d4[q] = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j)
      if (j < ncols_valid) dst[j] = v[j];
  }
}
__device__ __forceinline__ void load_f32x32(const float* src, float (&v)[32], int ncols_valid) {
  if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const float4* s4 = reinterpret_cast<const float4*>(src);
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      float4 t = s4[q];
      v[4 * q] = t.x; v[4 * q + 1] = t.y; v[4 * q + 2] = t.z; v[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < ncols_valid) ? src[j] : 0.f;
  }
}
__device__ __forceinline__ void load_bf16x32(const __nv_bfloat16* src, float (&v)[32], int ncols_valid) {
  if (ncols_valid >= 32 && (reinterpret_cast<uintptr_t>(src) & 15) == 0) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 t = s4[q];
      float2 a = rte::unpack_bf16x2(t.x), b = rte::unpack_bf16x2(t.y), c = rte::unpack_bf16x2(t.z), d = rte::unpack_bf16x2(t.w);
      v[8 * q] = a.x; v[8 * q + 1] = a.y; v[8 * q + 2] = b.x; v[8 * q + 3] = b.y;
      v[8 * q + 4] = c.x; v[8 * q + 5] = c.y; v[8 * q + 6] = d.x; v[8 * q + 7] = d.y;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 32; ++j) v[j] = (j < ncols_valid) ? __bfloat162float(src[j]) : 0.f;
  }
}
// 32 bf16 of one row as 16 packed pairs (zeros beyond ncols_valid); src must be 16-byte aligned.
__device__ __forceinline__ void load_bf16x32_packed(const __nv_bfloat16* src, uint32_t (&w)[16], int ncols_valid) {
  if (ncols_valid >= 32) {
    const uint4* s4 = reinterpret_cast<const uint4*>(src);
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      uint4 t = s4[q];
      w[4 * q] = t.x; w[4 * q + 1] = t.y; w[4 * q + 2] = t.z; w[4 * q + 3] = t.w;
    }
  } else {
#pragma unroll
    for (int j = 0; j < 16; ++j) {
      const float lo = (2 * j < ncols_valid) ? __bfloat162float(src[2 * j]) : 0.f;
      const float hi = (2 * j + 1 < ncols_valid) ? __bfloat162float(src[2 * j + 1]) : 0.f;
      w[j] = rte::pack_bf16x2(lo, hi);
    }
  }
}

template <int BN, int CTAS>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;            // this CTA's 128 rows of A: 16 KB
  static constexpr int B_ROWS = BN / CTAS;               // rows of the B tile this CTA stages
  static constexpr int B_BYTES = B_ROWS * BK * 2;
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int SLOTS = (BN == 256 && CTAS == 1) ? 1 : 2;     // staging slots per epilogue warp
  static constexpr int STAGING_BYTES = EPI_WARPS * SLOTS * SLOT_BYTES;
  static constexpr int BAR_BYTES = 512;
  static constexpr int STAGES_FIT = (MAX_DYN_SMEM - 1024 - BAR_BYTES - STAGING_BYTES) / STAGE_BYTES;
  static constexpr int STAGES = STAGES_FIT > 8 ? 8 : STAGES_FIT;
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;
  static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + BAR_BYTES + 1024;   // + slack for 1024-byte alignment
};

// ------------------------------------------------------------------ kernel
template <int BN, int CTAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_c2,
                    const KParams p) {
  using L = SmemLayout<BN, CTAS>;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t TMEM_COLS = 2 * BN;
  constexpr int HALF = BN / 2;               // columns of a tile per epilogue warp of a quadrant

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem ptr, error flag
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
  volatile uint32_t* err_flag = tmem_slot_ptr + 2;     // set by a role whose wait ran out

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
  const bool leader = cta_rank == 0;
  const int unit = blockIdx.x / CTAS, n_units = gridDim.x / CTAS;    // work units = CTAs or CTA pairs

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), EPI_WARPS * CTAS); }
    *err_flag = 0;
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc<CTAS>(tmem_slot, TMEM_COLS);     // CTAS = 2: one warp of EACH CTA of the pair takes part
    tmem_relinquish<CTAS>();
  }
  tc_fence_before();
  if (CTAS == 2) cluster_sync_all(); else __syncthreads();     // barriers of both CTAs are initialised beyond here
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int total_work = tiles * p.splits;

  if (warp == 0) {
    // ---------------- TMA producer (in both CTAs of a pair: each fills its own shared memory) ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int w = unit; w < total_work && ok; w += n_units) {
        const int split = w / tiles, t = w % tiles;
        const int mblk = t % p.num_m_blocks, nblk = t / p.num_m_blocks;
        const int m0 = (mblk * CTAS + int(cta_rank)) * BM, n0 = nblk * BN;
        int boff = 0;
        if (p.tile_group) {
          const int g = p.tile_group[mblk];
          if (g < 0) continue;
          boff = g * p.b_group_stride;
        }
        const int kb0 = p.split_kb ? p.split_kb[split] : split * p.kblocks_per_split;
        const int kb1 = p.split_kb ? p.split_kb[split + 1] : min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait<CTAS>(empty_bar(stage), phase ^ 1u)) {
            if (p.status) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_PRODUCER);
            *err_flag = 1;
            ok = false; break;
          }
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          if (DIAG && (p.diag & 4)) {
            if (leader) mbar_arrive(full_bar(stage));
            if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            continue;
          }
          // the leader's barrier counts the bytes of both CTAs' loads of this stage
          if (leader) mbar_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES * CTAS);
          const uint32_t fb = (CTAS == 2) ? mapa_cluster(full_bar(stage), 0) : full_bar(stage);
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d<CTAS>(sa, &tmap_a, fb, k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d<CTAS>(sa + j * 8192, &tmap_a, fb, m0 + 64 * j, k0);
          }
          // this CTA stages the tile's columns [c_lo, c_lo + B_ROWS)
          const int c_lo = int(cta_rank) * L::B_ROWS;
          if (!p.b_mn) {
            const int box = p.b_box_rows;
            for (int c = 0; c < L::B_ROWS; c += box) {
              const int tc = c_lo + c;               // column of the tile = row of B
              int brow;
              if (p.pair_off > 0 && p.epilogue == RTE_EPI_SWIGLU_FWD)     // tile = (up rows | matching gate rows)
                brow = (tc < HALF) ? nblk * HALF + tc : p.pair_off + nblk * HALF + (tc - HALF);
              else
                brow = n0 + tc;
              tma_load_2d<CTAS>(sb + uint32_t(c) * 128u, &tmap_b, fb, k0, boff + brow);
            }
          } else {
#pragma unroll
            for (int j = 0; j < L::B_ROWS / 64; ++j)
              tma_load_2d<CTAS>(sb + j * 8192, &tmap_b, fb, n0 + c_lo + 64 * j, boff + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer (one thread; with CTAS = 2 the leader CTA's, for both CTAs) ----------------
    if (lane == 0 && leader) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(p.a_mn) << 15) | (uint32_t(p.b_mn) << 16) |
                             (uint32_t(BN >> 3) << 17) | (uint32_t((BM * CTAS) >> 4) << 24);
      const uint32_t a_step = p.a_mn ? (UMMA_K * 128u) >> 4 : (UMMA_K * 2u) >> 4;
      const uint32_t b_step = p.b_mn ? (UMMA_K * 128u) >> 4 : (UMMA_K * 2u) >> 4;
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (int w = unit; w < total_work && ok; w += n_units) {
        const int split = w / tiles;
        if (p.tile_group && p.tile_group[(w % tiles) % p.num_m_blocks] < 0) continue;
        const int kb0 = p.split_kb ? p.split_kb[split] : split * p.kblocks_per_split;
        const int kb1 = p.split_kb ? p.split_kb[split + 1] : min(kb0 + p.kblocks_per_split, p.kblocks_total);
        if (!mbar_wait<CTAS>(tempty_bar(acc), acc_phase ^ 1u)) {
          if (p.status) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_MMA);
          *err_flag = 1;
          ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait<CTAS>(full_bar(stage), phase)) {
            if (p.status) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_MMA);
            *err_flag = 1;
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, p.a_mn != 0), bdesc = make_smem_desc(sb, p.b_mn != 0);
          if (!(DIAG && (p.diag & 2)))
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_bf16<CTAS>(d_tmem, adesc + uint64_t(k * a_step), bdesc + uint64_t(k * b_step), idesc,
                              (kb > kb0 || k > 0) ? 1u : 0u);
          tc_commit<CTAS>(empty_bar(stage));       // frees the stage (in both CTAs) once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit<CTAS>(tfull_bar(acc));           // accumulator complete -> epilogue (of both CTAs)
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9) ----------------
    // A warp may read the TMEM lane quadrant (warp % 4); warps 2..5 and 6..9 each cover all 128 rows and take one
    // half of the tile's columns.
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int grp = (warp - 2) >> 2;         // 0 or 1: which half of the columns
    const uint32_t tempty_remote0 = (CTAS == 2) ? mapa_cluster(tempty_bar(0), 0) : 0u;
    const uint32_t tempty_remote1 = (CTAS == 2) ? mapa_cluster(tempty_bar(1), 0) : 0u;
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    // TMA-store path: this warp's private staging slots; lane = row inside the warp's 32 rows.  A piece is written
    // into a slot with the 128-byte swizzle the store's tensor map expects, then lane 0 hands it to the TMA, which
    // clips rows / columns beyond M / N.  A slot is reused once the store that last read it has finished reading.
    const uint32_t wslots = smem_base + L::STAGING_OFFSET + uint32_t(warp - 2) * uint32_t(L::SLOTS * SLOT_BYTES);
    uint32_t job = 0;
    auto acquire = [&]() -> uint32_t {
      if (lane == 0) bulk_wait_read<L::SLOTS - 1>();
      __syncwarp();
      return wslots + (job % uint32_t(L::SLOTS)) * uint32_t(SLOT_BYTES);
    };
    auto submit = [&](const CUtensorMap* map, uint32_t slot, int x, int y, int z) {
      fence_proxy_async();
      __syncwarp();
      if (lane == 0 && !(DIAG && (p.diag & 32))) { tma_store_3d(map, slot, x, y, z); bulk_commit(); }
      ++job;
    };
    auto put16 = [&](uint32_t slot, uint32_t chunk, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
      st_shared_v4(slot + uint32_t(lane) * 128u + ((chunk ^ (uint32_t(lane) & 7u)) << 4), a, b, c, d);
    };

    auto epi_wait = [&](uint32_t bar, uint32_t parity) -> bool {
      return mbar_wait<CTAS>(bar, parity);
    };
    for (int w = unit; w < total_work && ok; w += n_units) {
      const int split = w / tiles, t = w % tiles;
      const int mblk = t % p.num_m_blocks, nblk = t / p.num_m_blocks;
      const int m0 = (mblk * CTAS + int(cta_rank)) * BM, n0 = nblk * BN;
      if (p.tile_group && p.tile_group[mblk] < 0) continue;
      // a split with an empty k-range never touched its accumulator: its partial is all zeros
      const bool empty_acc = p.split_kb && p.split_kb[split + 1] <= p.split_kb[split];
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const int y0 = m0 + quad * 32;           // first row of this warp's pieces
      const bool warp_rows = y0 < p.M && !(DIAG && (p.diag & 1));   // any of this warp's rows inside the matrix
      const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
      uint32_t raw[32];

      if (p.tma_store && p.epilogue == RTE_EPI_F32) {
        // ---- fp32 (+ residual): 32-column pieces; the residual of the next piece is fetched while this one is staged
        const float* Rf = reinterpret_cast<const float*>(p.R);
        float rres[32];
        const int c_first = grp * HALF;
        auto fetch_res = [&](int col) {
          if (Rf != nullptr) {
            if (row_ok && col < p.N) load_f32x32(Rf + size_t(row) * p.ldr + col, rres, p.N - col);
            else {
#pragma unroll
              for (int j = 0; j < 32; ++j) rres[j] = 0.f;
            }
          }
        };
        fetch_res(n0 + c_first);               // before the accumulator is complete
        if (!epi_wait(tfull_bar(acc), acc_phase)) {
          if (p.status && lane == 0) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_EPILOGUE);
          *err_flag = 1;
          ok = false; break;
        }
        tc_fence_after();
        for (int c0 = c_first; c0 < c_first + HALF; c0 += 32) {
          const int col = n0 + c0;
          if (col >= p.N) break;
          tmem_ld32(t_row + c0, raw);
          tmem_ld_wait();
          float v[32];
          if (Rf != nullptr) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = rres[j] + __uint_as_float(raw[j]);
            if (c0 + 32 < c_first + HALF) fetch_res(col + 32);
          } else {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = empty_acc ? 0.f : __uint_as_float(raw[j]);
          }
          if (warp_rows) {
            const uint32_t slot = acquire();
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c)
              put16(slot, c, __float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]), __float_as_uint(v[4 * c + 2]),
                    __float_as_uint(v[4 * c + 3]));
            submit(&tmap_c, slot, col, y0, split);
          }
        }
      } else {
        if (!epi_wait(tfull_bar(acc), acc_phase)) {
          if (p.status && lane == 0) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_EPILOGUE);
          *err_flag = 1;
          ok = false; break;
        }
        tc_fence_after();
        if (p.tma_store && p.epilogue == RTE_EPI_BF16) {
          // ---- bf16: 64-column pieces (128-byte rows)
          for (int c0 = grp * HALF; c0 < (grp + 1) * HALF; c0 += 64) {
            const int col = n0 + c0;
            if (col >= p.N) break;
            uint32_t raw2[32];
            tmem_ld32(t_row + c0, raw);
            tmem_ld32(t_row + c0 + 32, raw2);
            tmem_ld_wait();
            if (warp_rows) {
              const uint32_t slot = acquire();
#pragma unroll
              for (uint32_t c = 0; c < 4; ++c)
                put16(slot, c, rte::pack_bf16x2(__uint_as_float(raw[8 * c]), __uint_as_float(raw[8 * c + 1])),
                      rte::pack_bf16x2(__uint_as_float(raw[8 * c + 2]), __uint_as_float(raw[8 * c + 3])),
                      rte::pack_bf16x2(__uint_as_float(raw[8 * c + 4]), __uint_as_float(raw[8 * c + 5])),
                      rte::pack_bf16x2(__uint_as_float(raw[8 * c + 6]), __uint_as_float(raw[8 * c + 7])));
#pragma unroll
              for (uint32_t c = 0; c < 4; ++c)
                put16(slot, 4 + c, rte::pack_bf16x2(__uint_as_float(raw2[8 * c]), __uint_as_float(raw2[8 * c + 1])),
                      rte::pack_bf16x2(__uint_as_float(raw2[8 * c + 2]), __uint_as_float(raw2[8 * c + 3])),
                      rte::pack_bf16x2(__uint_as_float(raw2[8 * c + 4]), __uint_as_float(raw2[8 * c + 5])),
                      rte::pack_bf16x2(__uint_as_float(raw2[8 * c + 6]), __uint_as_float(raw2[8 * c + 7])));
              submit(&tmap_c, slot, col, y0, 0);
            }
          }
        } else if (p.tma_store && p.epilogue == RTE_EPI_SWIGLU_BWD) {
          // ---- acc = dz; (d up | d gate) from the saved (up | gate): two 64-column pieces per 64 columns of dz.
          // tmap_c views columns [0, F) of the output, tmap_c2 columns [F, 2F): each clips at its own edge.
          const int F = p.pair_off;
          for (int c0 = grp * HALF; c0 < (grp + 1) * HALF; c0 += 64) {
            const int col = n0 + c0;
            if (col >= p.N) break;
            uint32_t dgp[32];                  // d gate of the 64 columns, packed, until d up has left
            const uint32_t slot = acquire();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              const int cc = col + 32 * h;
              uint32_t upk[16], gpk[16];
              tmem_ld32(t_row + c0 + 32 * h, raw);
              if (row_ok && cc < p.N) {
                const __nv_bfloat16* ug = reinterpret_cast<const __nv_bfloat16*>(p.R) + size_t(row) * p.ldr;
                load_bf16x32_packed(ug + cc, upk, p.N - cc);
                load_bf16x32_packed(ug + F + cc, gpk, p.N - cc);
              } else {
#pragma unroll
                for (int j = 0; j < 16; ++j) { upk[j] = 0u; gpk[j] = 0u; }
              }
              tmem_ld_wait();
              uint32_t dup[16];
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float2 u_ = rte::unpack_bf16x2(upk[j]), g_ = rte::unpack_bf16x2(gpk[j]);
                const float dz0 = __uint_as_float(raw[2 * j]), dz1 = __uint_as_float(raw[2 * j + 1]);
                const float s0 = fast_sigmoid(g_.x), s1 = fast_sigmoid(g_.y);
                dup[j] = rte::pack_bf16x2(dz0 * g_.x * s0, dz1 * g_.y * s1);
                dgp[16 * h + j] = rte::pack_bf16x2(dz0 * u_.x * s0 * (1.f + g_.x * (1.f - s0)),
                                                   dz1 * u_.y * s1 * (1.f + g_.y * (1.f - s1)));
              }
#pragma unroll
              for (uint32_t c = 0; c < 4; ++c) put16(slot, 4 * h + c, dup[4 * c], dup[4 * c + 1], dup[4 * c + 2], dup[4 * c + 3]);
            }
            if (warp_rows) submit(&tmap_c, slot, col, y0, 0);
            const uint32_t slot2 = acquire();
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) put16(slot2, c, dgp[4 * c], dgp[4 * c + 1], dgp[4 * c + 2], dgp[4 * c + 3]);
            if (warp_rows) submit(&tmap_c2, slot2, col, y0, 0);
          }
        } else if (p.tma_store && p.epilogue == RTE_EPI_SWIGLU_FWD) {
          // ---- the tile holds BN/2 (up, gate) column pairs: columns [0, BN/2) = up_j, [BN/2, BN) = gate_j for hidden
          // units j0 .. j0 + BN/2; this warp takes BN/4 = 64 of them: the rounded up and gate values and
          // z = up * silu(gate) leave as three 64-column pieces.
          const int pq = grp * (BN / 4);
          const int col = nblk * HALF + pq;
          if (col < p.pair_off) {
            uint32_t upk[32], gpk[32];
            uint32_t slot = acquire();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              tmem_ld32(t_row + pq + 32 * h, raw);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) upk[16 * h + j] = rte::pack_bf16x2(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1]));
            }
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) put16(slot, c, upk[4 * c], upk[4 * c + 1], upk[4 * c + 2], upk[4 * c + 3]);
            if (warp_rows) submit(&tmap_c2, slot, col, y0, 0);
            slot = acquire();
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              tmem_ld32(t_row + HALF + pq + 32 * h, raw);
              tmem_ld_wait();
#pragma unroll
              for (int j = 0; j < 16; ++j) gpk[16 * h + j] = rte::pack_bf16x2(__uint_as_float(raw[2 * j]), __uint_as_float(raw[2 * j + 1]));
            }
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) put16(slot, c, gpk[4 * c], gpk[4 * c + 1], gpk[4 * c + 2], gpk[4 * c + 3]);
            if (warp_rows) submit(&tmap_c2, slot, p.pair_off + col, y0, 0);
            slot = acquire();
            // z from the ROUNDED up and gate: what backward re-reads must agree with what was multiplied here
#pragma unroll
            for (uint32_t c = 0; c < 8; ++c) {
              uint32_t zz[4];
#pragma unroll
              for (int i = 0; i < 4; ++i) {
                const float2 u_ = rte::unpack_bf16x2(upk[4 * c + i]), g_ = rte::unpack_bf16x2(gpk[4 * c + i]);
                zz[i] = rte::pack_bf16x2(u_.x * fast_silu(g_.x), u_.y * fast_silu(g_.y));
              }
              put16(slot, c, zz[0], zz[1], zz[2], zz[3]);
            }
            if (warp_rows) submit(&tmap_c, slot, col, y0, 0);
          }
        } else {
          // ---- direct stores (outputs whose addresses / strides the TMA cannot take): 32-column slices, the two
          // warps of a quadrant take alternate slices
          float v[32];
          if (p.epilogue == RTE_EPI_BF16) {
            for (int c = grp; c < BN / 32; c += 2) {
              tmem_ld32(t_row + c * 32, raw); tmem_ld_wait();
              const int col = n0 + c * 32;
              if (row_ok && col < p.N) {
#pragma unroll
                for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[j]);
                store_bf16x32(reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col, v, p.N - col);
              }
            }
          } else if (p.epilogue == RTE_EPI_F32) {
            float* Cf = reinterpret_cast<float*>(p.C) + size_t(split) * p.split_stride;
            for (int c = grp; c < BN / 32; c += 2) {
              tmem_ld32(t_row + c * 32, raw); tmem_ld_wait();
              const int col = n0 + c * 32;
              if (row_ok && col < p.N) {
                if (p.R != nullptr) {
                  load_f32x32(reinterpret_cast<const float*>(p.R) + size_t(row) * p.ldr + col, v, p.N - col);
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] += __uint_as_float(raw[j]);
                } else {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] = empty_acc ? 0.f : __uint_as_float(raw[j]);
                }
                store_f32x32(Cf + size_t(row) * p.ldc + col, v, p.N - col);
              }
            }
          } else if (p.epilogue == RTE_EPI_SWIGLU_FWD) {
            const int j0 = nblk * HALF;
            uint32_t rawg[32];
            for (int c = grp; c < BN / 64; c += 2) {
              tmem_ld32(t_row + c * 32, raw);
              tmem_ld32(t_row + HALF + c * 32, rawg);
              tmem_ld_wait();
              const int col = j0 + c * 32;
              if (row_ok && col < p.pair_off) {
                __nv_bfloat16* ug = reinterpret_cast<__nv_bfloat16*>(p.C2) + size_t(row) * p.ldc2;
                float up[32], gt[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  // round to bf16 first: the saved (up | gate) and z must agree with what backward re-reads
                  up[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(raw[j])));
                  gt[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(rawg[j])));
                  v[j] = up[j] * fast_silu(gt[j]);
                }
                const int nv = p.pair_off - col;
                store_bf16x32(ug + col, up, nv);
                store_bf16x32(ug + p.pair_off + col, gt, nv);
                store_bf16x32(reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col, v, nv);
              }
            }
          } else {  // RTE_EPI_SWIGLU_BWD
            const int F = p.pair_off;
            for (int c = grp; c < BN / 32; c += 2) {
              tmem_ld32(t_row + c * 32, raw); tmem_ld_wait();
              const int col = n0 + c * 32;
              if (row_ok && col < p.N) {
                const __nv_bfloat16* ug = reinterpret_cast<const __nv_bfloat16*>(p.R) + size_t(row) * p.ldr;
                float up[32], gt[32], dg[32];
                const int nv = p.N - col;
                load_bf16x32(ug + col, up, nv);
                load_bf16x32(ug + F + col, gt, nv);
#pragma unroll
                for (int j = 0; j < 32; ++j) {
                  const float dz = __uint_as_float(raw[j]);
                  const float sg = fast_sigmoid(gt[j]);
                  v[j] = dz * gt[j] * sg;                                    // d up
                  dg[j] = dz * up[j] * sg * (1.f + gt[j] * (1.f - sg));      // d gate
                }
                __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc;
                store_bf16x32(out + col, v, nv);
                store_bf16x32(out + F + col, dg, nv);
              }
            }
          }
        }
      }
      // the accumulator buffer is free once every epilogue warp (of both CTAs) has read its part
      tc_fence_before();
      __syncwarp();
      if (lane == 0) {
        if (CTAS == 2) mbar_arrive_cluster(acc ? tempty_remote1 : tempty_remote0);
        else mbar_arrive(tempty_bar(acc));
      }
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
    if (lane == 0) bulk_wait_all();            // this warp's stores have left shared memory and reached global memory
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  if (CTAS == 2) cluster_sync_all(); else __syncthreads();
  if (*err_flag != 0) {
    // a wait ran out: copies of this CTA (or, in a pair, of its peer) may still be in flight towards shared memory;
    // give them a bounded time to land before the CTA retires
    for (int i = 0; i < 64; ++i) __nanosleep(1000);
    if (CTAS == 2) cluster_sync_all(); else __syncthreads();
  }
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc<CTAS>(tmem_base, TMEM_COLS);
  }
}

// ------------------------------------------------------------------ host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* sym = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &sym, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess)
      return nullptr;
    fn = reinterpret_cast<EncodeTiledFn>(sym);
  }
  return fn;
}

// 2-D bf16 tensor map over a row-major [rows, cols] matrix with row stride ld: box = box_cols x box_rows,
// 128-byte swizzle, out-of-range elements read as zero.
int make_tmap(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, int box_cols, int box_rows) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return RTE_ERR_TENSOR_MAP;
  cuuint64_t dims[2] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows)};
  cuuint64_t strides[1] = {static_cast<cuuint64_t>(ld) * 2ull};
  cuuint32_t box[2] = {static_cast<cuuint32_t>(box_cols), static_cast<cuuint32_t>(box_rows)};
  cuuint32_t estr[2] = {1, 1};
  CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                  CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RTE_OK : RTE_ERR_TENSOR_MAP;
}

// 3-D tensor map for the epilogue's bulk stores: [planes, rows, cols] with a box of 32 rows x 128 bytes
// (64 bf16 or 32 fp32 columns) and the 128-byte swizzle of the staging slots.
int make_store_tmap(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, long long planes,
                    long long plane_stride, bool f32) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return RTE_ERR_TENSOR_MAP;
  const unsigned long long es = f32 ? 4ull : 2ull;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es, static_cast<cuuint64_t>(plane_stride) * es};
  cuuint32_t box[3] = {f32 ? 32u : 64u, 32, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                  CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RTE_OK : RTE_ERR_TENSOR_MAP;
}

// Tile shape of a product: BN columns per tile, one CTA (128 rows) or a CTA pair (256 rows) per tile.
struct TileConfig { int bn, ctas; };

TileConfig pick_tile(const rte_gemm_args* a) {
  const bool grouped = a->tile_group != nullptr || a->split_kblocks != nullptr;   // per-128-row-block bookkeeping
  TileConfig c;
  c.ctas = (!grouped && a->M > BM) ? 2 : 1;
  if (a->cta_pair == 1) c.ctas = 1;
  c.bn = (a->N >= 192) ? 256 : 128;
  if (a->tile_n == 128 || a->tile_n == 256) c.bn = a->tile_n;
  if (a->epilogue == RTE_EPI_SWIGLU_FWD) c.bn = 256;       // the paired epilogue takes 64 (up, gate) pairs per warp
  return c;
}

// Work units (CTAs or CTA pairs) that can run at the same time under `max_ctas`.
template <int BN, int CTAS>
int concurrent_units(int max_ctas, int sm_count) {
  using L = SmemLayout<BN, CTAS>;
  int ctas = max_ctas > 0 ? max_ctas : sm_count;
  if (CTAS == 1) return ctas;
  static int max_clusters = -1;
  if (max_clusters < 0) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return ctas / 2;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(sm_count / 2 * 2));
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = L::TOTAL;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr; cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, gemm_tcgen05_kernel<BN, CTAS>, &cfg) == cudaSuccess && n > 0) max_clusters = n;
    else { (void)cudaGetLastError(); max_clusters = sm_count / 2; }
  }
  int units = ctas / 2;
  return units < max_clusters ? units : max_clusters;
}

template <int BN, int CTAS>
int launch(const rte_gemm_args* a, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
           const CUtensorMap& tc2, KParams& kp, int sm_count, cudaStream_t st) {
  using L = SmemLayout<BN, CTAS>;
  static_assert(L::STAGES >= 3, "too few pipeline stages fit");
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN, CTAS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return RTE_ERR_LAUNCH;
    attr_set = true;
  }
  const int total = kp.num_m_blocks * kp.num_n_blocks * kp.splits;
  int units = concurrent_units<BN, CTAS>(a->max_ctas, sm_count);
  if (units > total) units = total;
  if (units < 1) units = 1;
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(unsigned(units * CTAS));
  cfg.blockDim = dim3(NUM_THREADS);
  cfg.dynamicSmemBytes = L::TOTAL;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = CTAS; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
  cfg.attrs = attr; cfg.numAttrs = (CTAS == 2) ? 1 : 0;
  if (cudaLaunchKernelEx(&cfg, gemm_tcgen05_kernel<BN, CTAS>, ta, tb, tc, tc2, kp) != cudaSuccess) {
    (void)cudaGetLastError();
    return RTE_ERR_LAUNCH;
  }
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

}  // namespace

extern "C" int rte_device_sm_count(void) {
  static int cached = 0;
  if (cached > 0) return cached;
  int dev = 0, n = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return RTE_ERR_NO_DEVICE;
  if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return RTE_ERR_NO_DEVICE;
  cached = n;
  return n;
}

extern "C" int rte_gemm_tile_plan(const rte_gemm_args* a, int32_t* tile_m, int32_t* tile_n, int32_t* concurrent) {
  RTE_CHECK_ARG(a != nullptr && a->M > 0 && a->N > 0);
  const TileConfig c = pick_tile(a);
  if (tile_m) *tile_m = BM * c.ctas;
  if (tile_n) *tile_n = c.bn;
  if (concurrent) {
    const int sms = rte_device_sm_count();
    if (sms <= 0) return RTE_ERR_NO_DEVICE;
    int u;
    if (c.ctas == 2) u = c.bn == 256 ? concurrent_units<256, 2>(a->max_ctas, sms) : concurrent_units<128, 2>(a->max_ctas, sms);
    else u = a->max_ctas > 0 ? a->max_ctas : sms;
    *concurrent = u;
  }
  return RTE_OK;
}

extern "C" int rte_gemm_bf16(const rte_gemm_args* a, rte_stream_t stream) {
  RTE_CHECK_ARG(a != nullptr && a->A && a->B && a->C);
  RTE_CHECK_ARG(a->M > 0 && a->N > 0 && a->K > 0);
  RTE_CHECK_ARG(a->epilogue >= RTE_EPI_BF16 && a->epilogue <= RTE_EPI_SWIGLU_BWD);
  const int splits = a->splits < 1 ? 1 : a->splits;
  RTE_CHECK_ARG(splits == 1 || (a->epilogue == RTE_EPI_F32 && a->R == nullptr));
  if ((reinterpret_cast<uintptr_t>(a->A) & 15) || (reinterpret_cast<uintptr_t>(a->B) & 15) || (a->lda % 8) || (a->ldb % 8))
    return RTE_ERR_ALIGNMENT;
  const bool swiglu_f = a->epilogue == RTE_EPI_SWIGLU_FWD, swiglu_b = a->epilogue == RTE_EPI_SWIGLU_BWD;
  if (swiglu_f) {
    RTE_CHECK_ARG(a->C2 != nullptr && a->b_pair_offset > 0 && a->N == 2 * a->b_pair_offset && !a->b_mn_major);
    RTE_CHECK_ARG(a->b_pair_offset % 64 == 0);
  }
  if (swiglu_b) RTE_CHECK_ARG(a->R != nullptr && a->b_pair_offset == a->N);

  const TileConfig tile = pick_tile(a);
  const int bn = tile.bn, ctas = tile.ctas;

  KParams kp;
  kp.diag = 0;
#ifdef RTE_GEMM_DIAG
  if (const char* e = getenv("RTE_GEMM_DIAG_FLAGS")) kp.diag = atoi(e);
#endif
  kp.M = a->M; kp.N = a->N; kp.K = a->K;
  kp.a_mn = a->a_mn_major ? 1 : 0; kp.b_mn = a->b_mn_major ? 1 : 0;
  kp.epilogue = a->epilogue;
  kp.C = a->C; kp.ldc = a->ldc; kp.R = a->R; kp.ldr = a->ldr; kp.C2 = a->C2; kp.ldc2 = a->ldc2;
  kp.pair_off = a->b_pair_offset;
  kp.splits = splits; kp.split_stride = a->split_stride;
  kp.num_m_blocks = rte::ceil_div(a->M, BM * ctas);
  kp.num_n_blocks = swiglu_f ? rte::ceil_div(a->b_pair_offset, bn / 2) : rte::ceil_div(a->N, bn);
  kp.kblocks_total = rte::ceil_div(a->K, BK);
  kp.kblocks_per_split = rte::ceil_div(kp.kblocks_total, splits);
  kp.status = a->status;
  kp.tile_group = a->tile_group;
  kp.b_group_stride = a->b_group_stride;
  kp.split_kb = a->split_kblocks;
  if (a->tile_group) {
    RTE_CHECK_ARG(a->n_groups >= 1 && a->b_group_stride > 0 && a->M % BM == 0);
    RTE_CHECK_ARG(!a->b_mn_major || a->K % BK == 0);          // a ragged k-block would read the next group's rows
  }
  if (a->split_kblocks) {
    RTE_CHECK_ARG(a->epilogue == RTE_EPI_F32 && a->R == nullptr && a->tile_group == nullptr);
  } else {
    kp.splits = rte::ceil_div(kp.kblocks_total, kp.kblocks_per_split);   // drop empty trailing splits
    // a dropped split would leave its partial unwritten: the caller reduces `splits` partials, so insist
    RTE_CHECK_ARG(kp.splits == splits);
  }

  CUtensorMap ta, tb;
  int rc;
  if (!kp.a_mn) rc = make_tmap(&ta, a->A, a->M, a->K, a->lda, BK, BM);
  else rc = make_tmap(&ta, a->A, a->K, a->M, a->lda, 64, BK);
  if (rc != RTE_OK) return rc;
  const long long b_groups = a->tile_group ? a->n_groups : 0;     // grouped mode: B is the stack of every group's matrix
  // K-major B: one TMA box holds up to 128 rows of this CTA's share of the tile; the paired (up | gate) tile never
  // lets a box straddle the two halves
  int box_rows = bn / ctas < 128 ? bn / ctas : 128;
  if (swiglu_f && box_rows > bn / 2) box_rows = bn / 2;
  kp.b_box_rows = box_rows;
  if (!kp.b_mn) {
    rc = make_tmap(&tb, a->B, b_groups ? b_groups * a->b_group_stride : a->N, a->K, a->ldb, BK, box_rows);
  } else {
    rc = make_tmap(&tb, a->B, b_groups ? b_groups * a->b_group_stride : a->K, a->N, a->ldb, 64, BK);
  }
  if (rc != RTE_OK) return rc;

  // Outputs through TMA bulk stores whenever their addresses and strides allow it (16-byte rules of the TMA);
  // otherwise the epilogue writes with plain vector stores.
  CUtensorMap tc = ta, tc2 = ta;
  const bool out_f32 = a->epilogue == RTE_EPI_F32;
  const long long es = out_f32 ? 4 : 2;
  auto aligned = [&](const void* ptr, long long ld) { return ptr && (reinterpret_cast<uintptr_t>(ptr) & 15) == 0 && (ld * es) % 16 == 0; };
  bool tma_ok = aligned(a->C, a->ldc) && a->M >= 1;
  if (splits > 1) tma_ok = tma_ok && (a->split_stride * es) % 16 == 0;
  if (out_f32 && a->R != nullptr) tma_ok = tma_ok && (reinterpret_cast<uintptr_t>(a->R) & 15) == 0 && (a->ldr % 4) == 0;
  if (swiglu_f) tma_ok = tma_ok && aligned(a->C2, a->ldc2);
  if (swiglu_b) tma_ok = tma_ok && (a->N % 8 == 0) && (reinterpret_cast<uintptr_t>(a->R) & 15) == 0 && (a->ldr % 8) == 0;
  if (tma_ok) {
    const long long plane = splits > 1 ? a->split_stride : (long long)a->M * a->ldc;
    if (swiglu_f) {
      rc = make_store_tmap(&tc, a->C, a->M, a->b_pair_offset, a->ldc, 1, (long long)a->M * a->ldc, false);
      if (rc == RTE_OK) rc = make_store_tmap(&tc2, a->C2, a->M, 2LL * a->b_pair_offset, a->ldc2, 1, (long long)a->M * a->ldc2, false);
    } else if (swiglu_b) {
      rc = make_store_tmap(&tc, a->C, a->M, a->N, a->ldc, 1, (long long)a->M * a->ldc, false);
      if (rc == RTE_OK)
        rc = make_store_tmap(&tc2, reinterpret_cast<const __nv_bfloat16*>(a->C) + a->N, a->M, a->N, a->ldc, 1, (long long)a->M * a->ldc, false);
    } else {
      rc = make_store_tmap(&tc, a->C, a->M, a->N, a->ldc, splits, plane, out_f32);
    }
    if (rc != RTE_OK) tma_ok = false;     // e.g. a stride the encoder rejects: use the direct path
  }
  kp.tma_store = tma_ok ? 1 : 0;
  if (DIAG && (kp.diag & 16)) kp.tma_store = 0;

  const int sms = rte_device_sm_count();
  if (sms <= 0) return RTE_ERR_NO_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  if (ctas == 2)
    return bn == 256 ? launch<256, 2>(a, ta, tb, tc, tc2, kp, sms, st) : launch<128, 2>(a, ta, tb, tc, tc2, kp, sms, st);
  return bn == 256 ? launch<256, 1>(a, ta, tb, tc, tc2, kp, sms, st) : launch<128, 1>(a, ta, tb, tc, tc2, kp, sms, st);
}
