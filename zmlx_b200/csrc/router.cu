// Router kernels: router linear, softmax-family top-k, sigmoid+bias top-k with
// group-limited selection.  One warp owns one token row; the row's E scores live
// in registers (E <= 1024), top-k runs as K rounds of a warp arg-max whose order
// is (score descending, expert id ascending).
#include <math_constants.h>

#include "common.cuh"
#include "layer_route.cuh"
#include "plan.cuh"
#include "router_rows.cuh"

namespace zmoe {


template <int VPL>
__global__ void __launch_bounds__(128) softmax_topk_kernel(const void* __restrict__ logits, int dtype, int T, int E,
                                                           int K, int flavour, const float* __restrict__ bias,
                                                           int renorm, float* __restrict__ weights,
                                                           uint32_t* __restrict__ indices) {
  pdl_wait();
  pdl_trigger();
  extern __shared__ float topk_sm[];
  const int lane = threadIdx.x & 31;
  const int row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (row >= T) return;
  softmax_topk_row<VPL>(logits, dtype, row, E, K, flavour, bias, renorm, weights, indices, lane,
                        topk_sm + (size_t)(threadIdx.x >> 5) * (E + 2 * kMaxK));
}


template <int VPL>
__global__ void __launch_bounds__(128) sigmoid_topk_kernel(const void* __restrict__ logits, int dtype, int T, int E,
                                                           int K, const float* __restrict__ bias, int n_group,
                                                           int topk_group, float scale, float* __restrict__ weights,
                                                           uint32_t* __restrict__ indices) {
  extern __shared__ float sm[];
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int row = blockIdx.x * (blockDim.x >> 5) + wid;
  if (row >= T) return;
  sigmoid_topk_row<VPL>(logits, dtype, row, E, K, bias, n_group, topk_group, scale, weights, indices, lane,
                        sm + (size_t)wid * (2 * E + 64 + 2 * kMaxK));
}

// Router linear.  One warp per (expert, token tile of 8): 16-byte loads of the expert's weight row, the
// token rows come from L1/L2.  The order of the sum is the segmented one of router_logit_warp, which the
// one-launch decode block shares: both give the same logit bit for bit.
__global__ void __launch_bounds__(128) router_logits_kernel(const __nv_bfloat16* __restrict__ x,
                                                            const __nv_bfloat16* __restrict__ wr, int T, int E,
                                                            int d, void* __restrict__ logits, int out_dtype) {
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int e = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
  if (e >= E) return;
  const int t0 = blockIdx.y * 8;
  const uint4* wrow = reinterpret_cast<const uint4*>(wr + (size_t)e * d);
  const int nvec = d >> 3;
  const uint4* xrow[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) xrow[j] = reinterpret_cast<const uint4*>(x + (size_t)min(t0 + j, T - 1) * d);
  float s[8];
  router_logit_warp_multi<8>(wrow, xrow, nvec, lane, s);
  if (lane < 8 && t0 + lane < T) {
    float mine = s[0];
#pragma unroll
    for (int j = 1; j < 8; ++j)
      if (lane == j) mine = s[j];
    const size_t o = (size_t)(t0 + lane) * E + e;
    if (out_dtype == ZMOE_F32)
      reinterpret_cast<float*>(logits)[o] = mine;
    else
      reinterpret_cast<__nv_bfloat16*>(logits)[o] = __float2bfloat16_rn(mine);
  }
}

// Fused router: router linear for all tokens, then -- in the CTA that finishes last -- the
// family's top-k for every token and the token-sorted expert plan.  One launch replaces the
// router matmul, the top-k kernel and the plan kernel.  `counter` is one int of device memory
// that is zero before the first launch; the last CTA leaves it zero again.
struct RouteParams {
  const __nv_bfloat16* x;
  const __nv_bfloat16* wr;
  int T, E, d, K;
  int family;  // 0: top-k of logits then softmax; 1: softmax then top-k; 2: sigmoid + bias
  const float* bias;
  int renorm, n_group, topk_group;
  float scale;
  __nv_bfloat16* logits;  // (T, E) scratch / output
  float* weights;
  uint32_t* indices;
  int* plan;
  int* counter;
};

template <int VPL>
__global__ void __launch_bounds__(128) route_fused_kernel(const RouteParams p) {
  extern __shared__ int route_sm[];
  pdl_wait();
  pdl_trigger();
  const int lane = threadIdx.x & 31;
  const int wid = threadIdx.x >> 5;
  const int T = p.T, E = p.E, d = p.d;
  // ---- phase 1: one warp per expert row (summation order of router_logit_warp)
  const int e = blockIdx.x * 4 + wid;
  if (e < E) {
    const uint4* wrow = reinterpret_cast<const uint4*>(p.wr + (size_t)e * d);
    const int nvec = d >> 3;
    for (int t = 0; t < T; ++t) {
      const float sres = router_logit_warp(wrow, reinterpret_cast<const uint4*>(p.x + (size_t)t * d), nvec, lane);
      if (lane == 0) p.logits[(size_t)t * E + e] = __float2bfloat16_rn(sres);
    }
  }
  // ---- last CTA done?
  __shared__ int is_last;
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) is_last = (atomicAdd(p.counter, 1) == (int)gridDim.x - 1);
  __syncthreads();
  if (!is_last) return;
  __threadfence();
  // ---- phase 2: top-k of every token row (one warp per row)
  float* scratch = reinterpret_cast<float*>(route_sm);
  for (int row = wid; row < T; row += 4) {
    if (p.family == 2)
      sigmoid_topk_row<VPL>(p.logits, ZMOE_BF16, row, E, p.K, p.bias, p.n_group, p.topk_group, p.scale, p.weights,
                            p.indices, lane, scratch + (size_t)wid * (2 * E + 64 + 2 * kMaxK));
    else
      softmax_topk_row<VPL>(p.logits, ZMOE_BF16, row, E, p.K,
                            p.family == 0 ? ZMOE_ROUTER_TOPK_THEN_SOFTMAX : ZMOE_ROUTER_SOFTMAX_THEN_TOPK, p.bias,
                            p.renorm, p.weights, p.indices, lane, scratch + (size_t)wid * (2 * E + 64 + 2 * kMaxK));
  }
  __syncthreads();
  // ---- phase 3: plan over the (token, slot) pairs; pair p reads token row p / K
  if (p.plan)
    build_plan_block<128>(nullptr, p.K, reinterpret_cast<const int*>(p.indices), T * p.K, 1, E, p.plan, route_sm);
  if (threadIdx.x == 0) *p.counter = 0;
}

template <typename F>
static int dispatch_vpl(int E, F&& f) {
  if (E <= 128) return f(std::integral_constant<int, 4>{});
  if (E <= 256) return f(std::integral_constant<int, 8>{});
  if (E <= 512) return f(std::integral_constant<int, 16>{});
  return f(std::integral_constant<int, 32>{});
}

}  // namespace zmoe

using namespace zmoe;

extern "C" {

int zmoe_router_softmax_topk(const void* logits, int logits_dtype, int T, int E, int K, int flavour,
                             const float* bias, int renorm, float* weights, uint32_t* indices, void* stream) {
  ZMOE_REQUIRE(logits && weights && indices, ZMOE_ERR_SHAPE, "zmoe_router_softmax_topk: null pointer");
  ZMOE_REQUIRE(T >= 0 && E >= 1 && K >= 1, ZMOE_ERR_SHAPE, "zmoe_router_softmax_topk: bad sizes T=%d E=%d K=%d", T,
               E, K);
  ZMOE_REQUIRE(K <= E, ZMOE_ERR_SHAPE, "zmoe_router_softmax_topk: k=%d exceeds last dimension D=%d", K, E);
  ZMOE_REQUIRE(E <= 32 * kMaxVPL && K <= kMaxK, ZMOE_ERR_UNSUPPORTED,
               "zmoe_router_softmax_topk: E=%d (max %d) or K=%d (max %d) unsupported", E, 32 * kMaxVPL, K, kMaxK);
  ZMOE_REQUIRE(logits_dtype == ZMOE_F32 || logits_dtype == ZMOE_BF16, ZMOE_ERR_DTYPE,
               "zmoe_router_softmax_topk: logits dtype %d", logits_dtype);
  ZMOE_REQUIRE(flavour == ZMOE_ROUTER_TOPK_THEN_SOFTMAX || flavour == ZMOE_ROUTER_SOFTMAX_THEN_TOPK,
               ZMOE_ERR_UNSUPPORTED, "zmoe_router_softmax_topk: flavour %d", flavour);
  ZMOE_REQUIRE(!(flavour == ZMOE_ROUTER_TOPK_THEN_SOFTMAX && bias), ZMOE_ERR_UNSUPPORTED,
               "zmoe_router_softmax_topk: bias needs the softmax-then-top-k flavour");
  if (T == 0) return ZMOE_OK;
  dim3 grid((T + 3) / 4), block(128);
  cudaStream_t st = (cudaStream_t)stream;
  dispatch_vpl(E, [&](auto vpl) {
    launch_pdl(softmax_topk_kernel<decltype(vpl)::value>, grid, block, 4 * (size_t)(E + 2 * kMaxK) * sizeof(float), st, logits, logits_dtype, T, E, K, flavour,
               bias, renorm, weights, indices);
    return 0;
  });
  return check_launch("zmoe_router_softmax_topk");
}

int zmoe_router_sigmoid_bias_topk(const void* logits, int logits_dtype, int T, int E, int K, const float* bias,
                                  int n_group, int topk_group, float scale, float* weights, uint32_t* indices,
                                  void* stream) {
  ZMOE_REQUIRE(logits && bias && weights && indices, ZMOE_ERR_SHAPE, "zmoe_router_sigmoid_bias_topk: null pointer");
  ZMOE_REQUIRE(T >= 0 && E >= 1, ZMOE_ERR_SHAPE, "zmoe_router_sigmoid_bias_topk: bad sizes T=%d E=%d", T, E);
  ZMOE_REQUIRE(K >= 1, ZMOE_ERR_SHAPE, "deepseek_router_topk_sigmoid: k must be > 0");
  ZMOE_REQUIRE(K <= E, ZMOE_ERR_SHAPE, "deepseek_router_topk_sigmoid: k=%d exceeds D=%d", K, E);
  ZMOE_REQUIRE(n_group >= 1, ZMOE_ERR_SHAPE, "deepseek_router_topk_sigmoid: n_group must be > 0");
  ZMOE_REQUIRE(topk_group >= 1 && topk_group <= n_group, ZMOE_ERR_SHAPE,
               "deepseek_router_topk_sigmoid: invalid topk_group");
  ZMOE_REQUIRE(E % n_group == 0, ZMOE_ERR_SHAPE, "deepseek_router_topk_sigmoid: n_group must divide D");
  ZMOE_REQUIRE(E <= 32 * kMaxVPL && K <= kMaxK && n_group <= 32, ZMOE_ERR_UNSUPPORTED,
               "zmoe_router_sigmoid_bias_topk: E=%d K=%d n_group=%d beyond limits (%d, %d, 32)", E, K, n_group,
               32 * kMaxVPL, kMaxK);
  ZMOE_REQUIRE(logits_dtype == ZMOE_F32 || logits_dtype == ZMOE_BF16, ZMOE_ERR_DTYPE,
               "zmoe_router_sigmoid_bias_topk: logits dtype %d", logits_dtype);
  if (T == 0) return ZMOE_OK;
  dim3 grid((T + 3) / 4), block(128);
  size_t smem = 4 * (size_t)(2 * E + 64 + 2 * kMaxK) * sizeof(float);
  cudaStream_t st = (cudaStream_t)stream;
  dispatch_vpl(E, [&](auto vpl) {
    launch_pdl(sigmoid_topk_kernel<decltype(vpl)::value>, grid, block, smem, st, logits, logits_dtype, T, E, K, bias,
               n_group, topk_group, scale, weights, indices);
    return 0;
  });
  return check_launch("zmoe_router_sigmoid_bias_topk");
}

int zmoe_router_logits(const void* x, const void* wr, int T, int E, int d, void* logits, int out_dtype,
                       void* stream) {
  ZMOE_REQUIRE(x && wr && logits, ZMOE_ERR_SHAPE, "zmoe_router_logits: null pointer");
  ZMOE_REQUIRE(T >= 0 && E >= 1 && d >= 8, ZMOE_ERR_SHAPE, "zmoe_router_logits: bad sizes T=%d E=%d d=%d", T, E, d);
  ZMOE_REQUIRE(d % 8 == 0, ZMOE_ERR_ALIGN, "zmoe_router_logits: d=%d must be a multiple of 8", d);
  ZMOE_REQUIRE(((uintptr_t)x % 16 == 0) && ((uintptr_t)wr % 16 == 0), ZMOE_ERR_ALIGN,
               "zmoe_router_logits: x and wr must be 16-byte aligned");
  ZMOE_REQUIRE(out_dtype == ZMOE_F32 || out_dtype == ZMOE_BF16, ZMOE_ERR_DTYPE, "zmoe_router_logits: out dtype %d",
               out_dtype);
  if (T == 0) return ZMOE_OK;
  dim3 grid((E + 3) / 4, (T + 7) / 8), block(128);
  launch_pdl(router_logits_kernel, grid, block, 0, (cudaStream_t)stream, (const __nv_bfloat16*)x,
             (const __nv_bfloat16*)wr, T, E, d, logits, out_dtype);
  return check_launch("zmoe_router_logits");
}

int zmoe_route(const void* x, const void* wr, int T, int E, int d, int K, int family, const float* bias, int renorm,
               int n_group, int topk_group, float scale, void* logits, float* weights, uint32_t* indices, void* plan,
               size_t plan_bytes, int* counter, void* stream) {
  ZMOE_REQUIRE(x && wr && logits && weights && indices && counter, ZMOE_ERR_SHAPE, "zmoe_route: null pointer");
  ZMOE_REQUIRE(T >= 0 && E >= 1 && d >= 8 && K >= 1 && K <= E, ZMOE_ERR_SHAPE,
               "zmoe_route: bad sizes T=%d E=%d d=%d K=%d", T, E, d, K);
  ZMOE_REQUIRE(d % 8 == 0 && ((uintptr_t)x % 16) == 0 && ((uintptr_t)wr % 16) == 0, ZMOE_ERR_ALIGN,
               "zmoe_route: x and wr rows must be 16-byte aligned");
  ZMOE_REQUIRE(E <= 32 * kMaxVPL && K <= kMaxK, ZMOE_ERR_UNSUPPORTED, "zmoe_route: E=%d or K=%d beyond limits", E, K);
  ZMOE_REQUIRE(family >= 0 && family <= 2, ZMOE_ERR_UNSUPPORTED, "zmoe_route: family %d", family);
  if (family == 2) {
    ZMOE_REQUIRE(bias != nullptr, ZMOE_ERR_SHAPE, "zmoe_route: the sigmoid router needs a bias");
    ZMOE_REQUIRE(n_group >= 1 && n_group <= 32 && topk_group >= 1 && topk_group <= n_group && E % n_group == 0,
                 ZMOE_ERR_SHAPE, "zmoe_route: invalid n_group=%d / topk_group=%d", n_group, topk_group);
  }
  if (plan) {
    ZMOE_REQUIRE(E <= 4096 && (long long)T * K < (1ll << 24), ZMOE_ERR_UNSUPPORTED, "zmoe_route: plan too large");
    ZMOE_REQUIRE(plan_bytes >= zmoe_plan_bytes(T * K, E), ZMOE_ERR_WORKSPACE,
                 "zmoe_route: plan buffer of %zu bytes, need %zu", plan_bytes, zmoe_plan_bytes(T * K, E));
  }
  if (T == 0) return ZMOE_OK;
  RouteParams p;
  p.x = (const __nv_bfloat16*)x;
  p.wr = (const __nv_bfloat16*)wr;
  p.T = T;
  p.E = E;
  p.d = d;
  p.K = K;
  p.family = family;
  p.bias = bias;
  p.renorm = renorm;
  p.n_group = n_group;
  p.topk_group = topk_group;
  p.scale = scale;
  p.logits = (__nv_bfloat16*)logits;
  p.weights = weights;
  p.indices = indices;
  p.plan = (int*)plan;
  p.counter = counter;
  size_t smem_plan = (size_t)(2 * E + 2 * 128 + 2) * sizeof(int);
  size_t smem_sig = 4 * (size_t)(2 * E + 64 + 2 * kMaxK) * sizeof(float);
  size_t smem = smem_plan > smem_sig ? smem_plan : smem_sig;
  dim3 grid((E + 3) / 4), block(128);
  cudaStream_t st = (cudaStream_t)stream;
  dispatch_vpl(E, [&](auto vpl) {
    launch_pdl(route_fused_kernel<decltype(vpl)::value>, grid, block, smem, st, p);
    return 0;
  });
  return check_launch("zmoe_route");
}

}  // extern "C"
