// Shared device/host helpers of libzmoe (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/zmoe.h"

namespace zmoe {

// ---------------------------------------------------------------- error state
void set_error(const char* fmt, ...);
int fail(int code, const char* fmt, ...);
int check_launch(const char* what);

#define ZMOE_REQUIRE(cond, code, ...)          \
  do {                                         \
    if (!(cond)) return ::zmoe::fail((code), __VA_ARGS__); \
  } while (0)

// --------------------------------------------------------------- plan layout
// int32 words: [0] n_active experts, [1] rows, [2] status (nonzero: a bad expert
// id was seen and its row dropped), [3] E; then tasks[E] (int4 {expert, offset,
// count, 0}, compact: entries past n_active have count 0), offset[E+1],
// active[E], row_src[rows], row_dst[rows].
struct PlanView {
  int* hdr;
  int* tasks;
  int* offset;
  int* active;
  int* row_src;
  int* row_dst;
};

__host__ __device__ inline PlanView plan_view(void* base, int rows, int E) {
  PlanView v;
  int* p = reinterpret_cast<int*>(base);
  v.hdr = p;
  v.tasks = p + 4;
  v.offset = v.tasks + 4 * (size_t)E;
  v.active = v.offset + (E + 1);
  v.row_src = v.active + E;
  v.row_dst = v.row_src + rows;
  return v;
}

inline size_t plan_words(int rows, int E) {
  return 4 + 4 * (size_t)E + (size_t)(E + 1) + (size_t)E + 2 * (size_t)rows;
}

// ------------------------------------------------- programmatic dependent launch
// Every libzmoe kernel is launched with the programmatic-stream-serialization attribute:
// its CTAs may start while the previous kernel of the stream drains, and it calls
// pdl_wait() before it touches anything that kernel may have written.  pdl_trigger()
// lets the next kernel of the stream start in the same way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                              Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}

// ------------------------------------------------------------- device helpers
__device__ __forceinline__ float bf16_bits_to_float(uint32_t h) { return __uint_as_float(h << 16); }

__device__ __forceinline__ float round_bf16(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ uint16_t float_to_bf16_bits(float v) {
  return __bfloat16_as_ushort(__float2bfloat16_rn(v));
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// y = 1/(1+exp|x|); x < 0 ? y : 1 - y   (the reference's stable sigmoid, src/zmlx/msl.py:20-24)
__device__ __forceinline__ float sigmoid_stable(float x) {
  float y = 1.0f / (1.0f + expf(fabsf(x)));
  return (x < 0.0f) ? y : 1.0f - y;
}

}  // namespace zmoe
