// In-place sum of a gradient range across the data-parallel ranks of one node, over NVLink peer memory: ONE kernel
// per rank does the whole exchange (no multimem, no library collective), and everything that crosses the link is a
// plain peer STORE -- remote loads pay the link's round trip per request and reached less than half of the stores'
// bandwidth when this exchange was built on them.
//
// Every rank holds device pointers to every rank's gradient buffer, staging buffer (same size and layout) and flag
// array (CUDA IPC mappings made by the caller).  A range of n floats is cut into `world` equal parts; part q belongs
// to rank q.
//   push   : rank r copies its own values of every foreign part q into rank q's staging buffer (row r of the part);
//            the last of its blocks to finish tells every peer "pushed";
//   reduce : once all peers have pushed, rank r sums its part in rank order 0..world-1 (its own values from its
//            buffer, the others' from its staging buffer: local loads), so that every rank ends with bit-identical
//            values, and stores the sum into every rank's buffer; the last block tells every peer "done" and waits
//            for theirs (their parts have then landed here).
// A rank leaves the kernel only after every peer's "done", i.e. after every peer has finished reading its staging
// buffer and its gradient range, so the next exchange may overwrite both at once.
// Flags carry an epoch that only grows, so nothing is ever reset; the epoch lives in device memory and is bumped by
// the kernel itself, which keeps the launch replayable from a CUDA graph.  Every wait is bounded: when it runs out
// the kernel records a code in the caller's status word and returns (the data is then not reduced).

#include <cstring>

#include "rte_common.cuh"

namespace {

constexpr uint32_t SPIN_LIMIT = 1u << 27;      // polls of a flag before a wait gives up (about a second)

struct Comm {
  float* buf[RTE_COMM_MAX_RANKS];
  float* stage[RTE_COMM_MAX_RANKS];            // stage[q]: rank q's staging buffer (as large as buf, plus slack)
  uint32_t* flags[RTE_COMM_MAX_RANKS];         // flags[q]: rank q's array [slots][2][RTE_COMM_MAX_RANKS]
  uint32_t* epoch;                             // this rank's counters [slots]
  uint32_t* done_count;                        // this rank's block counters [slots][2]
  int world, rank;
};

__device__ __forceinline__ void st_flag(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_flag(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Waits until every peer's flag of this (slot, phase) has reached `epoch`; false when the limit ran out.
__device__ __forceinline__ bool wait_peers(const Comm& c, int slot, int phase, uint32_t epoch) {
  const uint32_t* mine = c.flags[c.rank] + ((size_t)slot * 2 + phase) * RTE_COMM_MAX_RANKS;
  for (int q = threadIdx.x; q < c.world; q += blockDim.x) {
    if (q == c.rank) continue;
    uint32_t i = 0;
    while ((int32_t)(ld_flag(mine + q) - epoch) < 0) {
      if (++i > SPIN_LIMIT) return false;
      if (i > 64) __nanosleep(64);
    }
  }
  return true;
}
__device__ __forceinline__ void tell_peers(const Comm& c, int slot, int phase, uint32_t epoch) {
  if (threadIdx.x < c.world && threadIdx.x != c.rank)
    st_flag(c.flags[threadIdx.x] + ((size_t)slot * 2 + phase) * RTE_COMM_MAX_RANKS + c.rank, epoch);
}
// True in exactly one block of the grid: the last one to arrive (all threads of the block get the answer).
__device__ __forceinline__ bool last_block(uint32_t* counter) {
  __shared__ int last_s;
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x == 0) last_s = (atomicAdd(counter, 1u) == gridDim.x - 1) ? 1 : 0;
  __syncthreads();
  return last_s != 0;
}

// dst[i] = src[i] for i in [0, cnt) float4, U independent 16-byte loads in flight per thread
template <int U>
__device__ __forceinline__ void copy_part(float4* __restrict__ dst, const float4* __restrict__ src, long long cnt) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  for (; i + (U - 1) * stride < cnt; i += U * stride) {
    float4 v[U];
#pragma unroll
    for (int u = 0; u < U; ++u) v[u] = src[i + u * stride];
#pragma unroll
    for (int u = 0; u < U; ++u) dst[i + u * stride] = v[u];
  }
  for (; i < cnt; i += stride) dst[i] = src[i];
}

// W > 0: the world size as a compile-time constant (all loads of U consecutive strides are issued before the first
// add); W == 0: any world size, one element at a time.
template <int W, int U>
__device__ __forceinline__ void reduce_part(const Comm& c, long long offset, long long lo, long long hi, long long per) {
  const long long stride = (long long)gridDim.x * blockDim.x;
  const float4* own = reinterpret_cast<const float4*>(c.buf[c.rank] + offset);
  const float4* st = reinterpret_cast<const float4*>(c.stage[c.rank] + offset);       // row q at st + q * per
  long long i = lo + blockIdx.x * (long long)blockDim.x + threadIdx.x;
  if constexpr (W > 0) {
    for (; i + (U - 1) * stride < hi; i += U * stride) {
      float4 v[U][W];
#pragma unroll
      for (int u = 0; u < U; ++u)
#pragma unroll
        for (int q = 0; q < W; ++q)
          v[u][q] = (q == c.rank) ? own[i + u * stride] : st[q * per + (i + u * stride - lo)];
#pragma unroll
      for (int u = 0; u < U; ++u) {
        float4 acc = v[u][0];                               // rank order 0..W-1 on every rank: bit-identical sums
#pragma unroll
        for (int q = 1; q < W; ++q) { acc.x += v[u][q].x; acc.y += v[u][q].y; acc.z += v[u][q].z; acc.w += v[u][q].w; }
#pragma unroll
        for (int q = 0; q < W; ++q) reinterpret_cast<float4*>(c.buf[q] + offset)[i + u * stride] = acc;
      }
    }
  }
  for (; i < hi; i += stride) {
    float4 acc = (0 == c.rank) ? own[i] : st[i - lo];
    for (int q = 1; q < c.world; ++q) {
      const float4 v = (q == c.rank) ? own[i] : st[q * per + (i - lo)];
      acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
    }
    for (int q = 0; q < c.world; ++q) reinterpret_cast<float4*>(c.buf[q] + offset)[i] = acc;
  }
}

template <int W, int U>
__global__ void __launch_bounds__(512)
allreduce_sum_kernel(Comm c, long long offset, long long n, int slot, int* status) {
  __shared__ int ok_s;
  __shared__ uint32_t epoch_s;
  if (threadIdx.x == 0) { ok_s = 1; epoch_s = c.epoch[slot] + 1; }
  __syncthreads();
  const uint32_t epoch = epoch_s;
  const long long n4 = n / 4;                                   // the caller keeps ranges multiples of 4 floats
  const long long per = (n4 + c.world - 1) / c.world;           // float4 per part
  // ---- push: this rank's values of every foreign part go into the owner's staging buffer (row = this rank)
  for (int k = 1; k < c.world; ++k) {
    const int q = (c.rank + k) % c.world;                       // every rank starts with another peer
    const long long lo = (long long)q * per, hi = min(lo + per, n4);
    if (hi > lo)
      copy_part<U * 2>(reinterpret_cast<float4*>(c.stage[q] + offset) + (long long)c.rank * per,
                       reinterpret_cast<const float4*>(c.buf[c.rank] + offset) + lo, hi - lo);
  }
  if (last_block(c.done_count + slot * 2 + 0)) tell_peers(c, slot, 0, epoch);
  // ---- reduce: wait (on this rank's own memory) until every peer has pushed, then sum this rank's part
  if (threadIdx.x < 32 && !wait_peers(c, slot, 0, epoch)) ok_s = 0;
  __syncthreads();
  if (ok_s) {
    const long long lo = (long long)c.rank * per, hi = min(lo + per, n4);
    reduce_part<W, U>(c, offset, lo, hi, per);
  }
  // ---- done: the last block of this rank to finish tells the peers, waits for theirs, and advances the epoch
  if (!last_block(c.done_count + slot * 2 + 1)) {
    if (!ok_s && threadIdx.x == 0 && status) atomicExch(status, RTE_DEV_WAIT_TIMEOUT_PEER);
    return;
  }
  tell_peers(c, slot, 1, epoch);
  if (threadIdx.x < 32 && !wait_peers(c, slot, 1, epoch)) ok_s = 0;
  __syncthreads();
  if (threadIdx.x == 0) {
    c.done_count[slot * 2 + 0] = 0;
    c.done_count[slot * 2 + 1] = 0;
    c.epoch[slot] = epoch;
    if (!ok_s && status) atomicExch(status, RTE_DEV_WAIT_TIMEOUT_PEER);
  }
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

// ---- memory that other processes of the node can map (legacy CUDA IPC over a cudaMalloc allocation) ----------------
// The importing side opens the handle with ITS device current and cudaIpcMemLazyEnablePeerAccess: that is what makes
// the mapping reachable from kernels of the importing device.  (A mapping opened under the exporter's device ordinal
// is only reachable after an explicit cudaDeviceEnablePeerAccess; kernels that touch it without fault the context.)
static_assert(sizeof(cudaIpcMemHandle_t) == RTE_IPC_HANDLE_BYTES, "handle size");

extern "C" int rte_peer_alloc(int64_t bytes, void** ptr, uint8_t* handle) {
  RTE_CHECK_ARG(bytes > 0 && ptr != nullptr && handle != nullptr);
  void* p = nullptr;
  if (cudaMalloc(&p, (size_t)bytes) != cudaSuccess) { cudaGetLastError(); return RTE_ERR_LAUNCH; }
  cudaIpcMemHandle_t h;
  if (cudaMemset(p, 0, (size_t)bytes) != cudaSuccess || cudaIpcGetMemHandle(&h, p) != cudaSuccess) {
    cudaGetLastError();
    cudaFree(p);
    return RTE_ERR_LAUNCH;
  }
  memcpy(handle, &h, sizeof h);
  *ptr = p;
  return RTE_OK;
}

extern "C" int rte_peer_open(const uint8_t* handle, int32_t owner_device, void** ptr) {
  RTE_CHECK_ARG(handle != nullptr && ptr != nullptr);
  int cur = 0;
  if (cudaGetDevice(&cur) != cudaSuccess) return RTE_ERR_NO_DEVICE;
  if (owner_device >= 0 && owner_device != cur) {
    int can = 0;
    if (cudaDeviceCanAccessPeer(&can, cur, owner_device) != cudaSuccess || !can) { cudaGetLastError(); return RTE_ERR_UNSUPPORTED; }
  }
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof h);
  void* p = nullptr;
  if (cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess) != cudaSuccess) { cudaGetLastError(); return RTE_ERR_LAUNCH; }
  *ptr = p;
  return RTE_OK;
}

extern "C" int rte_peer_close(void* ptr) {
  RTE_CHECK_ARG(ptr != nullptr);
  if (cudaIpcCloseMemHandle(ptr) != cudaSuccess) { cudaGetLastError(); return RTE_ERR_LAUNCH; }
  return RTE_OK;
}

extern "C" int rte_peer_free(void* ptr) {
  RTE_CHECK_ARG(ptr != nullptr);
  if (cudaFree(ptr) != cudaSuccess) { cudaGetLastError(); return RTE_ERR_LAUNCH; }
  return RTE_OK;
}

extern "C" int rte_peer_allreduce_sum_f32(const rte_peer_comm* comm, int64_t offset, int64_t n, int32_t slot, int32_t max_ctas,
                                          int32_t* status, rte_stream_t stream) {
  RTE_CHECK_ARG(comm != nullptr && comm->world >= 2 && comm->world <= RTE_COMM_MAX_RANKS && comm->rank >= 0 && comm->rank < comm->world);
  RTE_CHECK_ARG(n > 0 && n % 4 == 0 && offset >= 0 && offset % 4 == 0 && slot >= 0 && slot < RTE_COMM_MAX_SLOTS);
  RTE_CHECK_ARG(comm->epoch != nullptr && comm->done_count != nullptr);
  Comm c;
  for (int q = 0; q < comm->world; ++q) {
    RTE_CHECK_ARG(comm->buf[q] != nullptr && comm->stage[q] != nullptr && comm->flags[q] != nullptr);
    if ((reinterpret_cast<uintptr_t>(comm->buf[q]) | reinterpret_cast<uintptr_t>(comm->stage[q])) & 15) return RTE_ERR_ALIGNMENT;
    c.buf[q] = comm->buf[q];
    c.stage[q] = comm->stage[q];
    c.flags[q] = comm->flags[q];
  }
  c.epoch = comm->epoch; c.done_count = comm->done_count; c.world = comm->world; c.rank = comm->rank;
  const long long per = (n / 4 + c.world - 1) / c.world;
  long long grid = (per + 511) / 512;
  const int cap = max_ctas > 0 ? max_ctas : 64;          // a share of the SMs: the rest keep computing
  if (grid > cap) grid = cap;
  if (grid < 1) grid = 1;
  switch (c.world) {
    case 2: allreduce_sum_kernel<2, 4><<<(int)grid, 512, 0, ST(stream)>>>(c, offset, n, slot, status); break;
    case 4: allreduce_sum_kernel<4, 4><<<(int)grid, 512, 0, ST(stream)>>>(c, offset, n, slot, status); break;
    case 8: allreduce_sum_kernel<8, 2><<<(int)grid, 512, 0, ST(stream)>>>(c, offset, n, slot, status); break;
    default: allreduce_sum_kernel<0, 1><<<(int)grid, 512, 0, ST(stream)>>>(c, offset, n, slot, status); break;
  }
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
