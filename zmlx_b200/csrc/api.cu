// Error state, ABI version and the token-sorted expert plan.
#include <cstring>

#include "common.cuh"
#include "plan.cuh"

namespace zmoe {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

int check_launch(const char* what) {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "%s: %s", what, cudaGetErrorString(e));
  return ZMOE_OK;
}

constexpr int kPlanThreads = 1024;

__global__ void __launch_bounds__(kPlanThreads) build_plan_kernel(const int* __restrict__ lhs, int lhs_div,
                                                                  const int* __restrict__ rhs, int P, int M, int E,
                                                                  int* plan_base) {
  extern __shared__ int sm[];
  pdl_wait();
  pdl_trigger();
  build_plan_block<kPlanThreads>(lhs, lhs_div, rhs, P, M, E, plan_base, sm);
}

}  // namespace zmoe

using namespace zmoe;

extern "C" {

int zmoe_abi_version(void) { return ZMOE_ABI_VERSION; }

const char* zmoe_last_error(void) { return g_err; }

size_t zmoe_plan_bytes(int rows, int E) {
  if (rows < 0 || E <= 0) return 0;
  return plan_words(rows, E) * sizeof(int);
}

int zmoe_ep_alloc(size_t bytes, void** ptr) {
  ZMOE_REQUIRE(ptr != nullptr && bytes > 0, ZMOE_ERR_SHAPE, "zmoe_ep_alloc: bad arguments");
  cudaError_t e = cudaMalloc(ptr, bytes);
  if (e == cudaSuccess) e = cudaMemset(*ptr, 0, bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_ep_alloc: %s", cudaGetErrorString(e));
  return ZMOE_OK;
}

int zmoe_ep_free(void* ptr) {
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_ep_free: %s", cudaGetErrorString(e));
  return ZMOE_OK;
}

int zmoe_ep_export(const void* ptr, void* handle64) {
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is 64 bytes");
  ZMOE_REQUIRE(ptr != nullptr && handle64 != nullptr, ZMOE_ERR_SHAPE, "zmoe_ep_export: null pointer");
  cudaError_t e = cudaIpcGetMemHandle(reinterpret_cast<cudaIpcMemHandle_t*>(handle64), const_cast<void*>(ptr));
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_ep_export: %s", cudaGetErrorString(e));
  return ZMOE_OK;
}

int zmoe_ep_import(const void* handle64, void** ptr) {
  ZMOE_REQUIRE(ptr != nullptr && handle64 != nullptr, ZMOE_ERR_SHAPE, "zmoe_ep_import: null pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, sizeof(h));
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_ep_import: %s", cudaGetErrorString(e));
  return ZMOE_OK;
}

int zmoe_ep_unmap(void* ptr) {
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_ep_unmap: %s", cudaGetErrorString(e));
  return ZMOE_OK;
}

int zmoe_build_plan(const int32_t* lhs, int lhs_div, const int32_t* rhs, int P, int M, int E, void* plan,
                    size_t plan_bytes, void* stream) {
  ZMOE_REQUIRE(rhs != nullptr && plan != nullptr, ZMOE_ERR_SHAPE, "zmoe_build_plan: null pointer");
  ZMOE_REQUIRE(P >= 0 && M >= 1 && E >= 1, ZMOE_ERR_SHAPE, "zmoe_build_plan: bad sizes P=%d M=%d E=%d", P, M, E);
  ZMOE_REQUIRE(E <= 4096, ZMOE_ERR_UNSUPPORTED, "zmoe_build_plan: E=%d exceeds 4096", E);
  ZMOE_REQUIRE(lhs != nullptr || lhs_div >= 1, ZMOE_ERR_SHAPE, "zmoe_build_plan: lhs_div must be >= 1");
  ZMOE_REQUIRE((long long)P * M < (1ll << 24), ZMOE_ERR_SHAPE, "zmoe_build_plan: too many rows (limit 2^24)");
  ZMOE_REQUIRE(plan_bytes >= zmoe_plan_bytes(P * M, E), ZMOE_ERR_WORKSPACE,
               "zmoe_build_plan: plan buffer of %zu bytes, need %zu", plan_bytes, zmoe_plan_bytes(P * M, E));
  size_t smem = (size_t)(2 * E + 2 * kPlanThreads + 2) * sizeof(int);
  launch_pdl(build_plan_kernel, dim3(1), dim3(kPlanThreads), smem, (cudaStream_t)stream, lhs, lhs_div, rhs, P, M, E,
             (int*)plan);
  return check_launch("zmoe_build_plan");
}

}  // extern "C"
