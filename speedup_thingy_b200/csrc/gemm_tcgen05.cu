// Persistent warp-specialised bf16 GEMM for sm_100a:
//   C[M,N] = A[M,K] * B[N,K]^T, fp32 accumulation in tensor memory (TMEM),
//   operands staged by TMA into 128B-swizzled shared memory, MMAs issued by one
//   thread with tcgen05.mma (M=128, N=BN, K=16 per instruction).
//
// Roles per CTA (320 threads): warp 0 = TMA producer, warp 1 = TMEM owner + MMA
// issuer, warps 2..9 = two epilogue groups of four warps (each warp reads its 32-lane
// TMEM quadrant; the groups split a tile's columns).  Two
// accumulator buffers in TMEM let the epilogue of tile i overlap the main loop of
// tile i+1.  Every wait is bounded: on expiry the role records a code in the
// caller's status word and all roles drain to the common teardown, which frees TMEM.
//
// Either operand may be "MN-major" (stored with the reduction dimension as the
// slow axis), which is what the weight- and data-gradient GEMMs of the training
// step need; no transposed copies are ever made.

#include <cuda.h>

#include "rte_common.cuh"

namespace {

constexpr int BM = 128;         // rows of C per tile (TMEM lanes)
constexpr int BK = 64;          // bf16 elements per k-block (= one 128-byte swizzle row)
constexpr int UMMA_K = 16;      // K per tcgen05.mma for 16-bit inputs
constexpr int NUM_THREADS = 320;   // warp 0 producer, warp 1 MMA issuer, warps 2..9 two epilogue groups of four
constexpr uint32_t WAIT_LIMIT = 24u * 1000u * 1000u;   // polls (with back-off) before a wait gives up

struct KParams {
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
  const int* tile_group;    // grouped mode: group id of every 128-row block of A/C (< 0: block unused), else null
  int b_group_stride;       // grouped mode: rows of the stacked B between consecutive groups
  const int* split_kb;      // ragged split-K: k-block range [split_kb[s], split_kb[s+1]) of split s, else null
  int* status;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
  uint32_t ok;
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.u32 %0, 1, 0, p;\n\t}"
      : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
  return ok != 0;
}
// Bounded wait: returns false when the limit ran out.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
  for (uint32_t i = 0; i < WAIT_LIMIT; ++i) {
    if (mbar_test(bar, parity)) return true;
    if (i > 128) __nanosleep(i > 4096 ? 128 : 32);
  }
  return false;
}
__device__ __forceinline__ void fence_barrier_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
      ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
      : "memory");
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
__device__ __forceinline__ void epi_barrier(int group) { asm volatile("bar.sync %0, 128;" ::"r"(group + 1) : "memory"); }
__device__ __forceinline__ void st_shared_v4(uint32_t addr, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
  asm volatile("st.shared.v4.b32 [%0], {%1, %2, %3, %4};" ::"r"(addr), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ void prefetch_tmap(const CUtensorMap* map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(map)) : "memory");
}

__device__ __forceinline__ void tmem_alloc(uint32_t dst_smem, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(dst_smem), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
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

template <int BN>
struct SmemLayout {
  static constexpr int A_BYTES = BM * BK * 2;    // 16 KB
  static constexpr int B_BYTES = BN * BK * 2;    // 16/32 KB
  static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int STAGING_OFFSET = STAGES * STAGE_BYTES;     // output staging ring for TMA stores
  static constexpr int STAGING_BYTES = 32 * 1024;                 // 4 x [128 rows x 64 B] or 2 x [128 rows x 128 B]
  static constexpr int BAR_OFFSET = STAGING_OFFSET + STAGING_BYTES;
  static constexpr int TOTAL = BAR_OFFSET + 256 + 1024;   // barriers + slack for 1024-byte alignment
};

// ------------------------------------------------------------------ kernel
template <int BN>
__global__ void __launch_bounds__(NUM_THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_c, const __grid_constant__ CUtensorMap tmap_c2,
                    const KParams p) {
  using L = SmemLayout<BN>;
  constexpr int STAGES = L::STAGES;
  constexpr uint32_t TMEM_COLS = 2 * BN;

  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  const uint32_t bar_base = smem_base + L::BAR_OFFSET;
  // barrier slots (8 bytes each): full[STAGES], empty[STAGES], tmem_full[2], tmem_empty[2]; then tmem ptr
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (STAGES + s); };
  auto tfull_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + b); };
  auto tempty_bar = [&](int b) { return bar_base + 8u * (2 * STAGES + 2 + b); };
  const uint32_t tmem_slot = bar_base + 8u * (2 * STAGES + 4);
  volatile uint32_t* tmem_slot_ptr =
      reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(tfull_bar(b), 1); mbar_init(tempty_bar(b), 8); }
    fence_barrier_init();
    prefetch_tmap(&tmap_a);
    prefetch_tmap(&tmap_b);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot_ptr;

  const int tiles = p.num_m_blocks * p.num_n_blocks;
  const int total_work = tiles * p.splits;

  if (warp == 0) {
    // ---------------- TMA producer ----------------
    if (lane == 0) {
      int stage = 0; uint32_t phase = 0; bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w / tiles, t = w % tiles;
        const int m0 = (t % p.num_m_blocks) * BM, n0 = (t / p.num_m_blocks) * BN;
        int boff = 0;
        if (p.tile_group) {
          const int g = p.tile_group[t % p.num_m_blocks];
          if (g < 0) continue;
          boff = g * p.b_group_stride;
        }
        const int kb0 = p.split_kb ? p.split_kb[split] : split * p.kblocks_per_split;
        const int kb1 = p.split_kb ? p.split_kb[split + 1] : min(kb0 + p.kblocks_per_split, p.kblocks_total);
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
            if (p.status) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_PRODUCER);
            ok = false; break;
          }
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          mbar_arrive_expect_tx(full_bar(stage), L::STAGE_BYTES);
          const int k0 = kb * BK;
          if (!p.a_mn) {
            tma_load_2d(sa, &tmap_a, full_bar(stage), k0, m0);
          } else {
#pragma unroll
            for (int j = 0; j < BM / 64; ++j) tma_load_2d(sa + j * 8192, &tmap_a, full_bar(stage), m0 + 64 * j, k0);
          }
          if (!p.b_mn) {
            if (p.pair_off > 0 && p.epilogue == RTE_EPI_SWIGLU_FWD) {
              // first half of the tile = "up" rows, second half = the matching "gate" rows
              const int nh = boff + (t / p.num_m_blocks) * (BN / 2);
              if (BN == 256) {
                tma_load_2d(sb, &tmap_b, full_bar(stage), k0, nh);
                tma_load_2d(sb + 16384, &tmap_b, full_bar(stage), k0, p.pair_off + nh);
              } else {
                // box rows = 64 for BN = 128 pairing (see host: box_rows)
                tma_load_2d(sb, &tmap_b, full_bar(stage), k0, nh);
                tma_load_2d(sb + 8192, &tmap_b, full_bar(stage), k0, p.pair_off + nh);
              }
            } else {
#pragma unroll
              for (int j = 0; j < BN / 128; ++j) tma_load_2d(sb + j * 16384, &tmap_b, full_bar(stage), k0, boff + n0 + 128 * j);
            }
          } else {
#pragma unroll
            for (int j = 0; j < BN / 64; ++j) tma_load_2d(sb + j * 8192, &tmap_b, full_bar(stage), n0 + 64 * j, boff + k0);
          }
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      const uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | (uint32_t(p.a_mn) << 15) | (uint32_t(p.b_mn) << 16) |
                             (uint32_t(BN >> 3) << 17) | (uint32_t(BM >> 4) << 24);
      const uint32_t a_step = p.a_mn ? (UMMA_K * 128u) >> 4 : (UMMA_K * 2u) >> 4;
      const uint32_t b_step = p.b_mn ? (UMMA_K * 128u) >> 4 : (UMMA_K * 2u) >> 4;
      int stage = 0; uint32_t phase = 0; int acc = 0; uint32_t acc_phase = 0; bool ok = true;
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w / tiles;
        if (p.tile_group && p.tile_group[(w % tiles) % p.num_m_blocks] < 0) continue;
        const int kb0 = p.split_kb ? p.split_kb[split] : split * p.kblocks_per_split;
        const int kb1 = p.split_kb ? p.split_kb[split + 1] : min(kb0 + p.kblocks_per_split, p.kblocks_total);
        if (!mbar_wait(tempty_bar(acc), acc_phase ^ 1u)) {
          if (p.status) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_MMA);
          ok = false; break;
        }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb0; kb < kb1; ++kb) {
          if (!mbar_wait(full_bar(stage), phase)) {
            if (p.status) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_MMA);
            ok = false; break;
          }
          tc_fence_after();
          const uint32_t sa = smem_base + stage * L::STAGE_BYTES, sb = sa + L::A_BYTES;
          const uint64_t adesc = make_smem_desc(sa, p.a_mn != 0), bdesc = make_smem_desc(sb, p.b_mn != 0);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            tc_mma_bf16(d_tmem, adesc + uint64_t(k * a_step), bdesc + uint64_t(k * b_step), idesc,
                        (kb > kb0 || k > 0) ? 1u : 0u);
          tc_commit(empty_bar(stage));       // frees the smem stage once these MMAs have read it
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (!ok) break;
        tc_commit(tfull_bar(acc));           // accumulator complete -> epilogue
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
    }
  } else {
    // ---------------- epilogue (warps 2..9: two groups of four warps) ----------------
    // A warp may read the TMEM lane quadrant (warp % 4); each group of four consecutive warps covers all 128 rows.
    // The groups split a tile's columns between them (BN=256: group 0 takes [0,128), group 1 [128,256)), so two
    // 32-column slices are converted and staged at the same time.
    const int quad = warp & 3;               // TMEM lane quadrant this warp may read
    const int grp = (warp - 2) >> 2;         // 0 or 1
    int acc = 0; uint32_t acc_phase = 0; bool ok = true;
    if (p.tma_store) {
      // Each 32-column slice of the accumulator becomes one "store job": the group's 128 threads write their rows
      // into a swizzled staging slot, one thread hands the slot to the TMA (which clips rows/columns beyond M/N).
      // Per group: two 8 KB slots for 16-bit outputs, one 16 KB slot for 32-bit outputs.  Before a slot is
      // rewritten the store that last used it must have finished reading it (barrier A), and all rows must be in
      // place before the store is issued (barrier B).
      const uint32_t staging = smem_base + L::STAGING_OFFSET + uint32_t(grp) * 16384u;
      const bool issuer = (((warp - 2) & 3) == 0 && lane == 0);
      const int r = quad * 32 + lane;        // row of the tile this thread owns
      uint32_t job = 0;
      auto emit16 = [&](const CUtensorMap* map, int x, int y, const float (&v)[32]) {
        const uint32_t slot = staging + (job & 1u) * 8192u;
        if (issuer) bulk_wait_read<1>();
        epi_barrier(grp);
        const uint32_t base = slot + uint32_t(r) * 64u;
        const uint32_t sw = (uint32_t(r) >> 1) & 3u;
#pragma unroll
        for (uint32_t c = 0; c < 4; ++c)
          st_shared_v4(base + ((c ^ sw) << 4), rte::pack_bf16x2(v[8 * c], v[8 * c + 1]), rte::pack_bf16x2(v[8 * c + 2], v[8 * c + 3]),
                       rte::pack_bf16x2(v[8 * c + 4], v[8 * c + 5]), rte::pack_bf16x2(v[8 * c + 6], v[8 * c + 7]));
        fence_proxy_async();
        epi_barrier(grp);
        if (issuer) { tma_store_3d(map, slot, x, y, 0); bulk_commit(); }
        ++job;
      };
      auto emit32 = [&](const CUtensorMap* map, int x, int y, int z, const float (&v)[32]) {
        if (issuer) bulk_wait_read<0>();
        epi_barrier(grp);
        const uint32_t base = staging + uint32_t(r) * 128u;
        const uint32_t sw = uint32_t(r) & 7u;
#pragma unroll
        for (uint32_t c = 0; c < 8; ++c)
          st_shared_v4(base + ((c ^ sw) << 4), __float_as_uint(v[4 * c]), __float_as_uint(v[4 * c + 1]),
                       __float_as_uint(v[4 * c + 2]), __float_as_uint(v[4 * c + 3]));
        fence_proxy_async();
        epi_barrier(grp);
        if (issuer) { tma_store_3d(map, staging, x, y, z); bulk_commit(); }
        ++job;
      };
      for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
        const int split = w / tiles, t = w % tiles;
        const int m0 = (t % p.num_m_blocks) * BM, nblk = t / p.num_m_blocks, n0 = nblk * BN;
        if (p.tile_group && p.tile_group[t % p.num_m_blocks] < 0) continue;
        // a split with an empty k-range never touched its accumulator: its partial is all zeros
        const bool empty_acc = p.split_kb && p.split_kb[split + 1] <= p.split_kb[split];
        if (!mbar_wait(tfull_bar(acc), acc_phase)) {
          if (p.status && lane == 0) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_EPILOGUE);
          ok = false; break;
        }
        tc_fence_after();
        const int row = m0 + r;
        const bool row_ok = row < p.M;
        const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
        // two 32-column slices per TMEM wait
        uint32_t raw[2][32];
        float v[32];
        if (p.epilogue == RTE_EPI_BF16 || p.epilogue == RTE_EPI_F32 || p.epilogue == RTE_EPI_SWIGLU_BWD) {
          constexpr int HALF = BN / 2;                       // columns per group
          for (int s2 = 0; s2 < HALF / 64; ++s2) {
            const int cbase = grp * HALF + s2 * 64;          // column offset inside the tile
            if (n0 + cbase >= p.N) break;
#pragma unroll
            for (int q = 0; q < 2; ++q) tmem_ld32(t_row + cbase + q * 32, raw[q]);
            tmem_ld_wait();
#pragma unroll
            for (int q = 0; q < 2; ++q) {
              const int col = n0 + cbase + q * 32;
              if (col < p.N) {
                if (p.epilogue == RTE_EPI_BF16) {
#pragma unroll
                  for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(raw[q][j]);
                  emit16(&tmap_c, col, m0, v);
                } else if (p.epilogue == RTE_EPI_F32) {
                  if (p.R != nullptr) {
                    if (row_ok) load_f32x32(reinterpret_cast<const float*>(p.R) + size_t(row) * p.ldr + col, v, p.N - col);
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = (row_ok ? v[j] : 0.f) + __uint_as_float(raw[q][j]);
                  } else {
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = empty_acc ? 0.f : __uint_as_float(raw[q][j]);
                  }
                  emit32(&tmap_c, col, m0, split, v);
                } else {
                  const int F = p.pair_off;
                  float up[32], gt[32], dg[32];
                  if (row_ok) {
                    const __nv_bfloat16* ug = reinterpret_cast<const __nv_bfloat16*>(p.R) + size_t(row) * p.ldr;
                    load_bf16x32(ug + col, up, p.N - col);
                    load_bf16x32(ug + F + col, gt, p.N - col);
                  }
#pragma unroll
                  for (int j = 0; j < 32; ++j) {
                    const float dz = __uint_as_float(raw[q][j]);
                    const float g_ = row_ok ? gt[j] : 0.f, u_ = row_ok ? up[j] : 0.f;
                    const float sg = rte::sigmoid_f(g_);
                    v[j] = dz * g_ * sg;
                    dg[j] = dz * u_ * sg * (1.f + g_ * (1.f - sg));
                  }
                  // tmap_c views columns [0, F) of the output, tmap_c2 columns [F, 2F): each clips at its own edge
                  emit16(&tmap_c, col, m0, v);
                  emit16(&tmap_c2, col, m0, dg);
                }
              }
            }
          }
        } else {  // RTE_EPI_SWIGLU_FWD: the tile holds BN/2 (up, gate) column pairs; each group takes half of them
          const int j0 = nblk * (BN / 2);
          constexpr int PAIRS = BN / 64;                     // 32-column pairs per tile
          for (int pq = grp * (PAIRS / 2); pq < (grp + 1) * (PAIRS / 2); ++pq) {
            const int col = j0 + pq * 32;
            if (col >= p.pair_off) break;
            tmem_ld32(t_row + pq * 32, raw[0]);
            tmem_ld32(t_row + BN / 2 + pq * 32, raw[1]);
            tmem_ld_wait();
            float up[32], gt[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              up[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(raw[0][j])));
              gt[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(raw[1][j])));
              v[j] = up[j] * rte::silu_f(gt[j]);
            }
            emit16(&tmap_c2, col, m0, up);
            emit16(&tmap_c2, p.pair_off + col, m0, gt);
            emit16(&tmap_c, col, m0, v);
          }
        }
        tc_fence_before();
        __syncwarp();
        if (lane == 0) mbar_arrive(tempty_bar(acc));
        if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
      }
      if (issuer) bulk_wait_all();
    } else
    for (int w = blockIdx.x; w < total_work && ok; w += gridDim.x) {
      const int split = w / tiles, t = w % tiles;
      const int m0 = (t % p.num_m_blocks) * BM, nblk = t / p.num_m_blocks, n0 = nblk * BN;
      if (p.tile_group && p.tile_group[t % p.num_m_blocks] < 0) continue;
      const bool empty_acc = p.split_kb && p.split_kb[split + 1] <= p.split_kb[split];
      if (!mbar_wait(tfull_bar(acc), acc_phase)) {
        if (p.status && lane == 0) atomicExch(p.status, RTE_DEV_WAIT_TIMEOUT_EPILOGUE);
        ok = false; break;
      }
      tc_fence_after();
      const int row = m0 + quad * 32 + lane;
      const bool row_ok = row < p.M;
      const uint32_t t_row = tmem_base + (uint32_t(quad * 32) << 16) + acc * BN;
      uint32_t raw[32];
      float v[32];
      if (p.epilogue == RTE_EPI_BF16) {
        for (int c = grp; c < BN / 32; c += 2) {           // the two groups take alternate 32-column slices
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
        for (int c = grp; c < BN / 32; c += 2) {           // the two groups take alternate 32-column slices
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
        // tile columns [0, BN/2) = up_j, [BN/2, BN) = gate_j for hidden units j0 .. j0 + BN/2
        const int j0 = nblk * (BN / 2);
        uint32_t rawg[32];
        for (int c = grp; c < BN / 64; c += 2) {
          tmem_ld32(t_row + c * 32, raw);
          tmem_ld32(t_row + BN / 2 + c * 32, rawg);
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
              v[j] = up[j] * rte::silu_f(gt[j]);
            }
            const int nv = p.pair_off - col;
            store_bf16x32(ug + col, up, nv);
            store_bf16x32(ug + p.pair_off + col, gt, nv);
            store_bf16x32(reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc + col, v, nv);
          }
        }
      } else {  // RTE_EPI_SWIGLU_BWD
        const int F = p.pair_off;
        for (int c = grp; c < BN / 32; c += 2) {           // the two groups take alternate 32-column slices
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
              const float sg = rte::sigmoid_f(gt[j]);
              v[j] = dz * gt[j] * sg;                                    // d up
              dg[j] = dz * up[j] * sg * (1.f + gt[j] * (1.f - sg));      // d gate
            }
            __nv_bfloat16* out = reinterpret_cast<__nv_bfloat16*>(p.C) + size_t(row) * p.ldc;
            store_bf16x32(out + col, v, nv);
            store_bf16x32(out + F + col, dg, nv);
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(tempty_bar(acc));
      if (++acc == 2) { acc = 0; acc_phase ^= 1u; }
    }
  }

  // ---------------- teardown ----------------
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
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

// 3-D tensor map for the epilogue's bulk stores: [planes, rows, cols] with a 32-column x 128-row box and the swizzle
// that matches the staging layout (64-byte rows for 16-bit outputs, 128-byte rows for 32-bit outputs).
int make_store_tmap(CUtensorMap* map, const void* base, long long rows, long long cols, long long ld, long long planes,
                    long long plane_stride, bool f32) {
  EncodeTiledFn fn = get_encode_fn();
  if (!fn) return RTE_ERR_TENSOR_MAP;
  const unsigned long long es = f32 ? 4ull : 2ull;
  cuuint64_t dims[3] = {static_cast<cuuint64_t>(cols), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(planes)};
  cuuint64_t strides[2] = {static_cast<cuuint64_t>(ld) * es, static_cast<cuuint64_t>(plane_stride) * es};
  cuuint32_t box[3] = {32, 128, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = fn(map, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(base),
                  dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                  f32 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? RTE_OK : RTE_ERR_TENSOR_MAP;
}

template <int BN>
int launch(const rte_gemm_args* a, const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tc,
           const CUtensorMap& tc2, KParams& kp, int sm_count, cudaStream_t st) {
  using L = SmemLayout<BN>;
  static bool attr_set = false;
  if (!attr_set) {
    if (cudaFuncSetAttribute(gemm_tcgen05_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL) != cudaSuccess)
      return RTE_ERR_LAUNCH;
    attr_set = true;
  }
  const int total = kp.num_m_blocks * kp.num_n_blocks * kp.splits;
  int grid = a->max_ctas > 0 ? a->max_ctas : sm_count;
  if (grid > total) grid = total;
  gemm_tcgen05_kernel<BN><<<grid, NUM_THREADS, L::TOTAL, st>>>(ta, tb, tc, tc2, kp);
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

  int bn = (a->N >= 192) ? 256 : 128;
  if (swiglu_f && (a->b_pair_offset % 128 != 0)) bn = 128;

  KParams kp;
  kp.M = a->M; kp.N = a->N; kp.K = a->K;
  kp.a_mn = a->a_mn_major ? 1 : 0; kp.b_mn = a->b_mn_major ? 1 : 0;
  kp.epilogue = a->epilogue;
  kp.C = a->C; kp.ldc = a->ldc; kp.R = a->R; kp.ldr = a->ldr; kp.C2 = a->C2; kp.ldc2 = a->ldc2;
  kp.pair_off = a->b_pair_offset;
  kp.splits = splits; kp.split_stride = a->split_stride;
  kp.num_m_blocks = rte::ceil_div(a->M, BM);
  kp.num_n_blocks = rte::ceil_div(a->N, bn);
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
  if (!kp.b_mn) {
    const int box_rows = (swiglu_f && bn == 128) ? 64 : 128;
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
  if (swiglu_f) tma_ok = tma_ok && aligned(a->C2, a->ldc2) && (a->b_pair_offset % 32 == 0);
  if (swiglu_b) tma_ok = tma_ok && (a->N % 8 == 0);
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

  const int sms = rte_device_sm_count();
  if (sms <= 0) return RTE_ERR_NO_DEVICE;
  cudaStream_t st = reinterpret_cast<cudaStream_t>(stream);
  return bn == 256 ? launch<256>(a, ta, tb, tc, tc2, kp, sms, st) : launch<128>(a, ta, tb, tc, tc2, kp, sms, st);
}
