// SVD-factor sparse SwiGLU FFN (reference layers.py:342-643, mask mode; svd_sparse_ffn_triton.py:480-714):
// the per-token neuron selection.  Everything GEMM-shaped runs in the tcgen05 GEMM (selector factors, exact
// up/gate pre-activations of ALL neurons, the down projection over the masked activations); what remains is, per
// token, four "k largest of F" selections:
//   candidates = top up_m of |up_hat|*wn  U  top gate_m of |silu(gate_hat)|*wn  U  top product_m of |up_hat*silu(gate_hat)|*wn
//   selected   = top top_k of |z|*wn over the candidates,      z = up * silu(gate) (exact)
// and z_masked = selected ? z : 0, so the down projection is a dense GEMM whose zero rows cost nothing extra.
//
// One warp per token.  Each selection is an exact radix select on order-preserving 32-bit keys held in shared
// memory (4 passes of 8 bits, a 256-bin histogram per warp), followed by an index-ordered pass that takes the
// elements equal to the threshold in ascending index order: results are bit-exact with a stable sort by
// (value descending, index ascending), the tie rule of this build.

#include "rte_common.cuh"

namespace {

constexpr int SEL_WARPS = 4;

__device__ __forceinline__ uint32_t order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// Marks (ORs `bit` into flags[i]) the k largest keys; ties at the threshold go to the lowest indices.
// keys/flags/hist are this warp's shared-memory arrays.  All 32 lanes call it.
__device__ void warp_select_topk(const uint32_t* keys, int F, int k, uint8_t* flags, uint8_t bit, uint32_t* hist, int lane) {
  if (k <= 0) return;
  if (k >= F) { for (int i = lane; i < F; i += 32) flags[i] |= bit; __syncwarp(); return; }
  uint32_t prefix = 0, pmask = 0;
  int remaining = k;
  for (int shift = 24; shift >= 0; shift -= 8) {
    for (int b = lane; b < 256; b += 32) hist[b] = 0;
    __syncwarp();
    for (int i = lane; i < F; i += 32) {
      const uint32_t key = keys[i];
      if ((key & pmask) == prefix) atomicAdd(&hist[(key >> shift) & 255u], 1u);
    }
    __syncwarp();
    // lane l owns bins [8l, 8l+8); suffix sums from the top bin downwards
    uint32_t mine[8], lane_total = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) { mine[j] = hist[8 * lane + j]; lane_total += mine[j]; }
    uint32_t suffix = lane_total;                         // inclusive sum over this lane and all higher lanes
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const uint32_t t = __shfl_down_sync(0xffffffffu, suffix, o);
      if (lane + o < 32) suffix += t;
    }
    const uint32_t above = suffix - lane_total;           // elements in bins owned by higher lanes
    // the crossing lane: above < remaining <= above + lane_total
    const bool here = (int)above < remaining && remaining <= (int)(above + lane_total);
    int digit = -1, taken_above = 0;
    if (here) {
      uint32_t cum = above;
      for (int j = 7; j >= 0; --j) {
        if ((int)cum < remaining && remaining <= (int)(cum + mine[j])) { digit = 8 * lane + j; taken_above = (int)cum; break; }
        cum += mine[j];
      }
    }
    const unsigned who = __ballot_sync(0xffffffffu, here);
    const int src = __ffs(who) - 1;
    digit = __shfl_sync(0xffffffffu, digit, src);
    taken_above = __shfl_sync(0xffffffffu, taken_above, src);
    remaining -= taken_above;
    prefix |= (uint32_t)digit << shift;
    pmask |= 255u << shift;
    __syncwarp();
  }
  // prefix = the k-th largest key; `remaining` of the elements equal to it are taken, lowest indices first
  int eq_taken = 0;
  for (int i0 = 0; i0 < F; i0 += 32) {
    const int i = i0 + lane;
    const uint32_t key = (i < F) ? keys[i] : 0u;
    const bool gt = (i < F) && key > prefix, eq = (i < F) && key == prefix;
    const unsigned eqm = __ballot_sync(0xffffffffu, eq);
    const int rank = eq_taken + __popc(eqm & ((1u << lane) - 1u));
    if (gt || (eq && rank < remaining)) flags[i] |= bit;
    eq_taken += __popc(eqm);
  }
  __syncwarp();
}

// hats f32 [rows, 2F] = (up_hat | gate_hat); ug bf16 [rows, 2F] = exact (up | gate); wn f32 [F]
// z_masked bf16 [rows, F]; selected uint8 [rows, F] (1 = selected); cand_count int32 [rows] (optional)
__global__ void __launch_bounds__(SEL_WARPS * 32)
svd_select_kernel(const float* __restrict__ hats, const __nv_bfloat16* __restrict__ ug, const float* __restrict__ wn,
                  __nv_bfloat16* __restrict__ z_masked, uint8_t* __restrict__ selected, int32_t* __restrict__ cand_count,
                  int rows, int F, int up_m, int gate_m, int product_m, int top_k) {
  extern __shared__ uint8_t sm_raw[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const size_t per_warp = (size_t)F * 4 + 256 * 4 + (size_t)F;
  uint32_t* keys = reinterpret_cast<uint32_t*>(sm_raw + warp * per_warp);
  uint32_t* hist = keys + F;
  uint8_t* flags = reinterpret_cast<uint8_t*>(hist + 256);
  const int row = blockIdx.x * SEL_WARPS + warp;
  if (row >= rows) return;
  const float* uh = hats + (size_t)row * 2 * F;
  const float* gh = uh + F;
  for (int i = lane; i < F; i += 32) flags[i] = 0;
  // --- three candidate lists
  for (int i = lane; i < F; i += 32) keys[i] = order_key(fabsf(uh[i]) * wn[i]);
  __syncwarp();
  warp_select_topk(keys, F, up_m, flags, 1, hist, lane);
  for (int i = lane; i < F; i += 32) keys[i] = order_key(fabsf(rte::silu_f(gh[i])) * wn[i]);
  __syncwarp();
  warp_select_topk(keys, F, gate_m, flags, 1, hist, lane);
  for (int i = lane; i < F; i += 32) keys[i] = order_key(fabsf(uh[i] * rte::silu_f(gh[i])) * wn[i]);
  __syncwarp();
  warp_select_topk(keys, F, product_m, flags, 1, hist, lane);
  // --- exact re-rank over the candidates
  const __nv_bfloat16* up = ug + (size_t)row * 2 * F;
  const __nv_bfloat16* gate = up + F;
  int n_cand = 0;
  for (int i = lane; i < F; i += 32) {
    const float z = __bfloat162float(up[i]) * rte::silu_f(__bfloat162float(gate[i]));
    const bool c = flags[i] & 1;
    n_cand += c;
    keys[i] = order_key(c ? fabsf(z) * wn[i] : -INFINITY);
  }
  __syncwarp();
  warp_select_topk(keys, F, top_k, flags, 2, hist, lane);
  n_cand = (int)rte::warp_sum((float)n_cand);
  if (cand_count && lane == 0) cand_count[row] = n_cand;
  for (int i = lane; i < F; i += 32) {
    const bool s = flags[i] & 2;
    const float z = __bfloat162float(up[i]) * rte::silu_f(__bfloat162float(gate[i]));
    z_masked[(size_t)row * F + i] = __float2bfloat16_rn(s ? z : 0.f);
    if (selected) selected[(size_t)row * F + i] = s ? 1 : 0;
  }
}

// dug = SwiGLU backward of dz over the selected neurons only (zeros elsewhere)
__global__ void __launch_bounds__(256)
svd_swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ ug, const __nv_bfloat16* __restrict__ dz, const uint8_t* __restrict__ selected,
                      __nv_bfloat16* __restrict__ dug, long long rows, int F) {
  const long long total = rows * F;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / F;
    const int j = int(i % F);
    float du = 0.f, dg = 0.f;
    if (selected[i]) {
      const float u = __bfloat162float(ug[r * 2 * F + j]), g = __bfloat162float(ug[r * 2 * F + F + j]);
      const float d = __bfloat162float(dz[i]), sg = rte::sigmoid_f(g);
      du = d * g * sg;
      dg = d * u * sg * (1.f + g * (1.f - sg));
    }
    dug[r * 2 * F + j] = __float2bfloat16_rn(du);
    dug[r * 2 * F + F + j] = __float2bfloat16_rn(dg);
  }
}

__global__ void row_norm_kernel(const float* __restrict__ w, float* __restrict__ out, int rows, int d) {
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (row >= rows) return;
  float s = 0.f;
  for (int c = lane; c < d; c += 32) { const float x = w[(size_t)row * d + c]; s += x * x; }
  s = rte::warp_sum(s);
  if (lane == 0) out[row] = sqrtf(s);
}

}  // namespace

#define ST(s) reinterpret_cast<cudaStream_t>(s)

extern "C" int rte_svd_ffn_select(const float* hats, const void* ug, const float* wd_norm, void* z_masked, uint8_t* selected,
                                  int32_t* cand_count, int32_t rows, int32_t F, int32_t up_m, int32_t gate_m, int32_t product_m,
                                  int32_t top_k, rte_stream_t stream) {
  RTE_CHECK_ARG(hats && ug && wd_norm && z_masked && rows > 0 && F > 0 && top_k > 0 && top_k <= F);
  RTE_CHECK_ARG(up_m >= 0 && gate_m >= 0 && product_m >= 0);
  // with fewer candidates than top_k the reference's result depends on an unspecified ordering of non-candidates
  if (up_m < top_k && gate_m < top_k && product_m < top_k) return RTE_ERR_UNSUPPORTED;
  const size_t smem = (size_t)SEL_WARPS * ((size_t)F * 5 + 1024);
  if (smem > 200 * 1024 || F % 4) return RTE_ERR_UNSUPPORTED;
  if (smem > 48 * 1024) {
    static bool set = false;
    if (!set) {
      if (cudaFuncSetAttribute(svd_select_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
        return RTE_ERR_LAUNCH;
      set = true;
    }
  }
  svd_select_kernel<<<rte::ceil_div(rows, SEL_WARPS), SEL_WARPS * 32, smem, ST(stream)>>>(
      hats, reinterpret_cast<const __nv_bfloat16*>(ug), wd_norm, reinterpret_cast<__nv_bfloat16*>(z_masked), selected, cand_count,
      rows, F, up_m, gate_m, product_m, top_k);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_svd_ffn_swiglu_bwd(const void* ug, const void* dz, const uint8_t* selected, void* dug, int64_t rows, int32_t F,
                                      rte_stream_t stream) {
  RTE_CHECK_ARG(ug && dz && selected && dug && rows > 0 && F > 0);
  long long g = (rows * F + 255) / 256;
  if (g > 148 * 16) g = 148 * 16;
  svd_swiglu_bwd_kernel<<<(int)g, 256, 0, ST(stream)>>>(reinterpret_cast<const __nv_bfloat16*>(ug), reinterpret_cast<const __nv_bfloat16*>(dz),
                                                        selected, reinterpret_cast<__nv_bfloat16*>(dug), rows, F);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}

extern "C" int rte_row_norm_f32(const float* w, float* out, int32_t rows, int32_t d, rte_stream_t stream) {
  RTE_CHECK_ARG(w && out && rows > 0 && d > 0);
  row_norm_kernel<<<rte::ceil_div(rows, 8), 256, 0, ST(stream)>>>(w, out, rows, d);
  RTE_LAUNCH_CHECK();
  return RTE_OK;
}
