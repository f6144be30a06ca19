// Error state, ABI version and the token-sorted expert plan.
#include <cstring>

#include "common.cuh"

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

// One CTA groups `rows` (pair, m) rows by expert: histogram, exclusive scan,
// scatter.  The order of rows inside an expert's segment is arbitrary; every
// output row is computed from its own input row only, so results do not
// depend on it.
constexpr int kPlanThreads = 1024;

__global__ void __launch_bounds__(kPlanThreads) build_plan_kernel(const int* __restrict__ lhs, int lhs_div,
                                                                  const int* __restrict__ rhs, int P, int M, int E,
                                                                  int* plan_base) {
  extern __shared__ int sm[];
  int* count = sm;           // E
  int* cursor = sm + E;      // E
  int* scan_tmp = sm + 2 * E;  // kPlanThreads
  const int rows = P * M;
  PlanView pv = plan_view(plan_base, rows, E);
  const int tid = threadIdx.x;
  __shared__ int bad;
  if (tid == 0) bad = 0;
  for (int e = tid; e < E; e += kPlanThreads) count[e] = 0;
  __syncthreads();
  for (int p = tid; p < P; p += kPlanThreads) {
    int e = rhs[p];
    if (e >= 0 && e < E)
      atomicAdd(&count[e], M);
    else
      bad = 1;
  }
  __syncthreads();
  // exclusive scan over E (chunked by kPlanThreads), plus compaction of active experts
  int base = 0, abase = 0;
  for (int e0 = 0; e0 < E; e0 += kPlanThreads) {
    int e = e0 + tid;
    int c = (e < E) ? count[e] : 0;
    int flag = c > 0;
    // inclusive scan of (c, flag) packed: counts < 2^20 rows assumed? keep separate scans
    scan_tmp[tid] = c;
    __syncthreads();
    for (int o = 1; o < kPlanThreads; o <<= 1) {
      int v = (tid >= o) ? scan_tmp[tid - o] : 0;
      __syncthreads();
      scan_tmp[tid] += v;
      __syncthreads();
    }
    int incl = scan_tmp[tid];
    int total = scan_tmp[kPlanThreads - 1];
    __syncthreads();
    scan_tmp[tid] = flag;
    __syncthreads();
    for (int o = 1; o < kPlanThreads; o <<= 1) {
      int v = (tid >= o) ? scan_tmp[tid - o] : 0;
      __syncthreads();
      scan_tmp[tid] += v;
      __syncthreads();
    }
    int aincl = scan_tmp[tid];
    int atotal = scan_tmp[kPlanThreads - 1];
    __syncthreads();
    if (e < E) {
      int off = base + incl - c;
      pv.offset[e] = off;
      cursor[e] = off;
      if (flag) {
        const int a = abase + aincl - 1;
        pv.active[a] = e;
        reinterpret_cast<int4*>(pv.tasks)[a] = make_int4(e, off, c, 0);
      }
    }
    base += total;
    abase += atotal;
  }
  for (int a = abase + tid; a < E; a += kPlanThreads) reinterpret_cast<int4*>(pv.tasks)[a] = make_int4(0, 0, 0, 0);
  if (tid == 0) {
    pv.offset[E] = base;
    pv.hdr[0] = abase;
    pv.hdr[1] = rows;
    pv.hdr[3] = E;
  }
  __syncthreads();
  for (int p = tid; p < P; p += kPlanThreads) {
    int e = rhs[p];
    if (e < 0 || e >= E) continue;
    int pos = atomicAdd(&cursor[e], M);
    int src = (lhs ? lhs[p] : p / lhs_div) * M;
    for (int m = 0; m < M; ++m) {
      pv.row_src[pos + m] = src + m;
      pv.row_dst[pos + m] = p * M + m;
    }
  }
  __syncthreads();
  if (tid == 0) pv.hdr[2] = bad;
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

int zmoe_build_plan(const int32_t* lhs, int lhs_div, const int32_t* rhs, int P, int M, int E, void* plan,
                    size_t plan_bytes, void* stream) {
  ZMOE_REQUIRE(rhs != nullptr && plan != nullptr, ZMOE_ERR_SHAPE, "zmoe_build_plan: null pointer");
  ZMOE_REQUIRE(P >= 0 && M >= 1 && E >= 1, ZMOE_ERR_SHAPE, "zmoe_build_plan: bad sizes P=%d M=%d E=%d", P, M, E);
  ZMOE_REQUIRE(E <= 4096, ZMOE_ERR_UNSUPPORTED, "zmoe_build_plan: E=%d exceeds 4096", E);
  ZMOE_REQUIRE(lhs != nullptr || lhs_div >= 1, ZMOE_ERR_SHAPE, "zmoe_build_plan: lhs_div must be >= 1");
  ZMOE_REQUIRE((long long)P * M < (1ll << 30), ZMOE_ERR_SHAPE, "zmoe_build_plan: too many rows");
  ZMOE_REQUIRE(plan_bytes >= zmoe_plan_bytes(P * M, E), ZMOE_ERR_WORKSPACE,
               "zmoe_build_plan: plan buffer of %zu bytes, need %zu", plan_bytes, zmoe_plan_bytes(P * M, E));
  size_t smem = (size_t)(2 * E + kPlanThreads) * sizeof(int);
  build_plan_kernel<<<1, kPlanThreads, smem, (cudaStream_t)stream>>>(lhs, lhs_div, rhs, P, M, E, (int*)plan);
  return check_launch("zmoe_build_plan");
}

}  // extern "C"
