// Weighted combine over the K expert slots under the reference's rounding
// contracts, plus the fused down-projection + combine entry point.
#include <mutex>

#include "qmm_common.cuh"

namespace zmoe {

int qmm_launch(int nmat, const void* x, int x_rows, int ldx, const uint32_t* const* w, const void* const* s,
               const void* const* b, int E, int N, int K, int group_size, int qmode, const void* plan, int rows,
               int rows_hint, void* out, int epilogue, int x_by_dst, void* stream, const char* who);

__device__ __forceinline__ float load_as_float(const void* p, int dtype, size_t i) {
  if (dtype == ZMOE_F32) return reinterpret_cast<const float*>(p)[i];
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// Each thread owns two adjacent columns of one token and walks the slots in
// order 0..K-1, which is the summation order of every reference kernel.
template <int MODE>
__global__ void __launch_bounds__(256) combine_kernel(const void* __restrict__ y, int y_dtype,
                                                      const void* __restrict__ w, int w_dtype, int T, int K, int D,
                                                      void* __restrict__ out, int out_t,
                                                      const __nv_bfloat16* __restrict__ residual) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.y;
  const int d = (blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (d >= D) return;
  const bool two = (d + 1) < D;
  float a0 = 0.0f, a1 = 0.0f;
  for (int i = 0; i < K; ++i) {
    float wi = load_as_float(w, w_dtype, (size_t)t * K + i);
    if (out_t & 2) wi = round_bf16(wi);
    const size_t o = ((size_t)t * K + i) * D + d;
    float v0, v1 = 0.0f;
    if (y_dtype == ZMOE_BF16 && two && ((o & 1) == 0)) {
      const uint32_t pr = *reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(y) + o);
      v0 = bf16_bits_to_float(pr & 0xffffu);
      v1 = bf16_bits_to_float(pr >> 16);
    } else {
      v0 = load_as_float(y, y_dtype, o);
      if (two) v1 = load_as_float(y, y_dtype, o + 1);
    }
    if (MODE == ZMOE_COMBINE_FP32 || MODE == ZMOE_COMBINE_T) {
      a0 = fmaf(wi, v0, a0);
      a1 = fmaf(wi, v1, a1);
    } else if (MODE == ZMOE_COMBINE_FP32_NO_FMA || MODE == ZMOE_COMBINE_NO_FMA) {
      a0 = __fadd_rn(a0, __fmul_rn(wi, v0));
      a1 = __fadd_rn(a1, __fmul_rn(wi, v1));
    } else if (MODE == ZMOE_COMBINE_EXACT) {
      wi = round_bf16(wi);
      a0 = round_bf16(__fadd_rn(a0, round_bf16(__fmul_rn(wi, v0))));
      a1 = round_bf16(__fadd_rn(a1, round_bf16(__fmul_rn(wi, v1))));
    } else {  // ZMOE_COMBINE_STREAM_T
      a0 = round_bf16(__fadd_rn(a0, __fmul_rn(wi, v0)));
      a1 = round_bf16(__fadd_rn(a1, __fmul_rn(wi, v1)));
    }
  }
  const size_t oo = (size_t)t * D + d;
  const bool fp32_mode = (MODE == ZMOE_COMBINE_FP32 || MODE == ZMOE_COMBINE_FP32_NO_FMA);
  if (fp32_mode && !(out_t & 1)) {
    float* of = reinterpret_cast<float*>(out);
    of[oo] = a0;
    if (two) of[oo + 1] = a1;
    return;
  }
  a0 = round_bf16(a0);
  a1 = round_bf16(a1);
  if (residual) {
    a0 = __fadd_rn(a0, __bfloat162float(residual[oo]));
    if (two) a1 = __fadd_rn(a1, __bfloat162float(residual[oo + 1]));
  }
  __nv_bfloat16* ob = reinterpret_cast<__nv_bfloat16*>(out);
  ob[oo] = __float2bfloat16_rn(a0);
  if (two) ob[oo + 1] = __float2bfloat16_rn(a1);
}

int combine_launch(const void* y, int y_dtype, const void* w, int w_dtype, int T, int K, int D, int mode, void* out,
                   int out_t, const void* residual, void* stream, const char* who) {
  ZMOE_REQUIRE(y && w && out, ZMOE_ERR_SHAPE, "%s: null pointer", who);
  ZMOE_REQUIRE(T >= 0 && K >= 1 && D >= 1, ZMOE_ERR_SHAPE, "%s: bad sizes T=%d K=%d D=%d", who, T, K, D);
  ZMOE_REQUIRE((y_dtype == ZMOE_F32 || y_dtype == ZMOE_BF16) && (w_dtype == ZMOE_F32 || w_dtype == ZMOE_BF16),
               ZMOE_ERR_DTYPE, "%s: dtypes y=%d w=%d", who, y_dtype, w_dtype);
  ZMOE_REQUIRE(mode >= ZMOE_COMBINE_FP32 && mode <= ZMOE_COMBINE_STREAM_T, ZMOE_ERR_UNSUPPORTED,
               "%s: combine mode %d", who, mode);
  const bool fp32_mode = (mode == ZMOE_COMBINE_FP32 || mode == ZMOE_COMBINE_FP32_NO_FMA);
  ZMOE_REQUIRE(!(residual && fp32_mode && !(out_t & 1)), ZMOE_ERR_UNSUPPORTED,
               "%s: a residual needs an output in T", who);
  ZMOE_REQUIRE(T <= 65535, ZMOE_ERR_UNSUPPORTED, "%s: T=%d exceeds 65535 per call", who, T);
  ZMOE_REQUIRE(((uintptr_t)y % 4) == 0 && ((uintptr_t)out % 4) == 0, ZMOE_ERR_ALIGN,
               "%s: y and out must be 4-byte aligned", who);
  if (T == 0) return ZMOE_OK;
  dim3 block(256), grid(((D + 1) / 2 + 255) / 256, T);
  cudaStream_t st = (cudaStream_t)stream;
  const __nv_bfloat16* res = (const __nv_bfloat16*)residual;
#define ZMOE_LAUNCH(M) \
  launch_pdl(combine_kernel<M>, grid, block, 0, st, y, y_dtype, w, w_dtype, T, K, D, out, out_t, res)
  switch (mode) {
    case ZMOE_COMBINE_FP32: ZMOE_LAUNCH(ZMOE_COMBINE_FP32); break;
    case ZMOE_COMBINE_FP32_NO_FMA: ZMOE_LAUNCH(ZMOE_COMBINE_FP32_NO_FMA); break;
    case ZMOE_COMBINE_T: ZMOE_LAUNCH(ZMOE_COMBINE_T); break;
    case ZMOE_COMBINE_NO_FMA: ZMOE_LAUNCH(ZMOE_COMBINE_NO_FMA); break;
    case ZMOE_COMBINE_EXACT: ZMOE_LAUNCH(ZMOE_COMBINE_EXACT); break;
    default: ZMOE_LAUNCH(ZMOE_COMBINE_STREAM_T); break;
  }
#undef ZMOE_LAUNCH
  return check_launch(who);
}

// ---------------------------------------------------------------- elementwise SwiGLU
// out = silu(gate) * up on T tensors of n elements (two per thread), under the rounding contracts of the fused
// projection's epilogue.
__global__ void __launch_bounds__(256) swiglu_kernel(const __nv_bfloat16* __restrict__ gate,
                                                     const __nv_bfloat16* __restrict__ up, long long n, int mode,
                                                     __nv_bfloat16* __restrict__ out) {
  pdl_wait();
  pdl_trigger();
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 2;
  if (i >= n) return;
#pragma unroll
  for (int k = 0; k < 2; ++k) {
    if (i + k < n) {
      const float g = __bfloat162float(gate[i + k]), u = __bfloat162float(up[i + k]);
      out[i + k] = __float2bfloat16_rn(mode == ZMOE_SWIGLU_CPU ? swiglu_cpu_contract(g, u) : swiglu_per_op(g, u));
    }
  }
}

// ---------------------------------------------------------------- allocation-free variant
// Scratch for zmoe_gather_qmm_combine_noalloc: lives in the library image, one copy per GPU that
// loads the library, for the life of the process.
constexpr size_t kStaticScratchBytes = 4u << 20;  // 4 MiB = 2,097,152 projected values in T
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
static std::mutex g_scratch_mutex;
static void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the CURRENT device.  In host code the symbol itself is only a
// stand-in; the real address comes from cudaGetSymbolAddress, asked once per device.
static int static_scratch_for_current_device(void** out, cudaStream_t stream) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_gather_qmm_combine_noalloc: cudaGetDevice: %s",
                                    cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(ZMOE_ERR_UNSUPPORTED, "zmoe_gather_qmm_combine_noalloc: device ordinal %d beyond %d", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_scratch_mutex);
  if (g_scratch_ptr[dev] == nullptr) {
    // the one-time address query is not a stream operation: inside a capture it would invalidate the capture,
    // so refuse instead and ask for a first call outside of it
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    e = cudaStreamIsCapturing(stream, &cap);
    if (e != cudaSuccess)
      return fail(ZMOE_ERR_CUDA, "zmoe_gather_qmm_combine_noalloc: cudaStreamIsCapturing: %s", cudaGetErrorString(e));
    if (cap != cudaStreamCaptureStatusNone)
      return fail(ZMOE_ERR_UNSUPPORTED,
                  "zmoe_gather_qmm_combine_noalloc: the first call on a device looks up the built-in scratch and "
                  "cannot run inside a stream capture; call it once outside the capture first");
    void* ptr = nullptr;
    e = cudaGetSymbolAddress(&ptr, g_static_scratch);
    if (e != cudaSuccess || ptr == nullptr)
      return fail(ZMOE_ERR_CUDA, "zmoe_gather_qmm_combine_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_scratch_ptr[dev] = ptr;
  }
  *out = g_scratch_ptr[dev];
  return ZMOE_OK;
}

}  // namespace zmoe

using namespace zmoe;

extern "C" {

int zmoe_moe_combine(const void* y, int y_dtype, const void* w, int w_dtype, int T, int K, int D, int mode,
                     void* out, int out_t, const void* residual, void* stream) {
  return combine_launch(y, y_dtype, w, w_dtype, T, K, D, mode, out, out_t, residual, stream, "zmoe_moe_combine");
}

int zmoe_swiglu(const void* gate, const void* up, long long n, int swiglu_mode, void* out, void* stream) {
  ZMOE_REQUIRE(gate && up && out, ZMOE_ERR_SHAPE, "zmoe_swiglu: null pointer");
  ZMOE_REQUIRE(n >= 0, ZMOE_ERR_SHAPE, "zmoe_swiglu: n=%lld", n);
  ZMOE_REQUIRE(swiglu_mode == ZMOE_SWIGLU_CPU || swiglu_mode == ZMOE_SWIGLU_PER_OP, ZMOE_ERR_UNSUPPORTED,
               "zmoe_swiglu: swiglu_mode %d", swiglu_mode);
  if (n == 0) return ZMOE_OK;
  const long long blocks = (n + 511) / 512;
  ZMOE_REQUIRE(blocks <= 0x7fffffffLL, ZMOE_ERR_UNSUPPORTED, "zmoe_swiglu: n=%lld is too large for one call", n);
  launch_pdl(swiglu_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, (const __nv_bfloat16*)gate,
             (const __nv_bfloat16*)up, n, swiglu_mode, (__nv_bfloat16*)out);
  return check_launch("zmoe_swiglu");
}

int zmoe_gather_qmm_combine(const void* act, int ldx, const uint32_t* w_, const void* scales, const void* biases,
                            int E, int N, int Kin, int group_size, int qmode, const void* plan, int T, int K,
                            const void* gate, int gate_dtype, int mode, void* scratch, void* out, int out_t,
                            void* stream) {
  ZMOE_REQUIRE(scratch != nullptr, ZMOE_ERR_WORKSPACE, "zmoe_gather_qmm_combine: scratch is required");
  ZMOE_REQUIRE(T >= 0 && K >= 1, ZMOE_ERR_SHAPE, "zmoe_gather_qmm_combine: bad sizes T=%d K=%d", T, K);
  const uint32_t* w[2] = {w_, nullptr};
  const void* s[2] = {scales, nullptr};
  const void* b[2] = {biases, nullptr};
  // Pairs whose expert id the plan dropped (outside 0..E-1) get no projected row: they count as zero, as in the
  // allocation-free entry point, instead of whatever the caller's scratch held.
  if (T > 0) {
    cudaError_t e = cudaMemsetAsync(scratch, 0, (size_t)T * K * N * sizeof(__nv_bfloat16), (cudaStream_t)stream);
    if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_gather_qmm_combine: clearing the scratch: %s", cudaGetErrorString(e));
  }
  int rc = qmm_launch(1, act, T * K, ldx, w, s, b, E, N, Kin, group_size, qmode, plan, T * K, T, scratch, 0, 1, stream,
                      "zmoe_gather_qmm_combine");
  if (rc != ZMOE_OK) return rc;
  return combine_launch(scratch, ZMOE_BF16, gate, gate_dtype, T, K, N, mode, out, out_t, nullptr, stream,
                        "zmoe_gather_qmm_combine");
}

int zmoe_gather_qmm_combine_noalloc(const void* act, int ldx, const uint32_t* w_, const void* scales,
                                    const void* biases, int E, int N, int Kin, int group_size, int qmode,
                                    const void* plan, int T, int K, const void* gate, int gate_dtype, int mode,
                                    void* out, int out_t, void* stream) {
  ZMOE_REQUIRE(T >= 0 && K >= 1 && N >= 1, ZMOE_ERR_SHAPE, "zmoe_gather_qmm_combine_noalloc: bad sizes T=%d K=%d N=%d",
               T, K, N);
  const size_t need = (size_t)T * K * N * 2;
  ZMOE_REQUIRE(need <= kStaticScratchBytes, ZMOE_ERR_WORKSPACE,
               "zmoe_gather_qmm_combine_noalloc: T*K*N = %zu projected values need %zu bytes, the built-in scratch "
               "holds %zu (use zmoe_gather_qmm_combine with caller scratch for larger calls)",
               (size_t)T * K * N, need, (size_t)kStaticScratchBytes);
  void* scratch = nullptr;
  int rc = static_scratch_for_current_device(&scratch, (cudaStream_t)stream);
  if (rc != ZMOE_OK) return rc;
  if (T == 0) return ZMOE_OK;
  // the array keeps the previous call's rows: rows whose expert id the plan dropped are never written by the
  // projection, so start the used part from zero
  cudaError_t e = cudaMemsetAsync(scratch, 0, need, (cudaStream_t)stream);
  if (e != cudaSuccess)
    return fail(ZMOE_ERR_CUDA, "zmoe_gather_qmm_combine_noalloc: cudaMemsetAsync: %s", cudaGetErrorString(e));
  return zmoe_gather_qmm_combine(act, ldx, w_, scales, biases, E, N, Kin, group_size, qmode, plan, T, K, gate,
                                 gate_dtype, mode, scratch, out, out_t, stream);
}

}  // extern "C"
