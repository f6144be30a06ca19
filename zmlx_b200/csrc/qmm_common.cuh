// Pieces shared by the quantised expert matmul kernels.
#pragma once

#include "common.cuh"

namespace zmoe {

struct QmmParams {
  const __nv_bfloat16* x;  // (x_rows, K) token rows, row stride ldx elements
  int ldx;
  const uint32_t* w[2];       // (E, N, K/8)
  const __nv_bfloat16* s[2];  // (E, N, K/64)
  const __nv_bfloat16* b[2];
  const int* plan;
  int rows, E;
  __nv_bfloat16* out;  // (rows, N)
  int ldo;
  int N, K, ngroups;
  int rs;        // token rows staged per pass (<= TT*NT)
  int epilogue;  // 0: store T; 1: SwiGLU CPU contract; 2: SwiGLU per-op contract
  int x_by_dst;  // token row r of the output reads x row r instead of the plan's source row
  int late_wait;  // the plan predates the previous kernel: stream the first weights before the dependency wait
};

__device__ __forceinline__ void mma_bf16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// codes at bits [sh, sh+4) and [sh+16, sh+20) -> bf16x2 (128+q_lo, 128+q_hi)
// The mask and the magic constant are passed in registers so that the and-or is a
// single three-register LOP3.
template <int SH>
__device__ __forceinline__ uint32_t deq_pair(uint32_t word, uint32_t mask, uint32_t magic) {
  uint32_t r;
  if (SH == 0) {
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(r) : "r"(word), "r"(mask), "r"(magic));
  } else {
    asm("{ .reg .b32 t; shr.b32 t, %1, %4; lop3.b32 %0, t, %2, %3, 0xEA; }"
        : "=r"(r)
        : "r"(word), "r"(mask), "r"(magic), "n"(SH));
  }
  return r;
}

__host__ __device__ inline int qmm_xs_stride(int K) { return K * 2 + 16; }
__host__ __device__ inline int qmm_sc_stride(int ngroups) { return ((ngroups + 3) & ~3) * 2 + 8; }

// 8-byte streaming load at a compile-time byte offset from a register base: the offset
// lives in the instruction, so a quad of groups costs no address arithmetic.
template <int OFF>
__device__ __forceinline__ uint2 ldg_stream_u2(const uint32_t* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2+%3];"
               : "=r"(v.x), "=r"(v.y)
               : "l"(p), "n"(OFF));
  return v;
}

__device__ __forceinline__ void cp_async_8(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// codes at bits [sh, sh+4) and [sh+16, sh+20) -> bf16x2 (128+q_lo, 128+q_hi)
template <int SH>
__device__ __forceinline__ uint32_t deq_imm(uint32_t word) {
  uint32_t r;
  if (SH == 0) {
    asm("lop3.b32 %0, %1, 0x000F000F, 0x43004300, 0xEA;" : "=r"(r) : "r"(word));
  } else {
    asm("{ .reg .b32 t; shr.b32 t, %1, %2; lop3.b32 %0, t, 0x000F000F, 0x43004300, 0xEA; }"
        : "=r"(r)
        : "r"(word), "n"(SH));
  }
  return r;
}

__device__ __forceinline__ float swiglu_cpu_contract(float g, float u) {
  g = round_bf16(g);
  u = round_bf16(u);
  float sig = 1.0f / (1.0f + expf(-g));
  return g * sig * u;
}

__device__ __forceinline__ float swiglu_per_op(float g, float u) {
  g = round_bf16(g);
  u = round_bf16(u);
  float e = round_bf16(expf(round_bf16(fabsf(g))));
  float y = round_bf16(1.0f / round_bf16(1.0f + e));
  float sig = (g < 0.0f) ? y : round_bf16(1.0f - y);
  return round_bf16(g * sig) * u;
}

// gate and up stay in float (the reference's dense fused GEMV, src/zmlx/kernels/quant.py:103-124)
__device__ __forceinline__ float swiglu_fp32(float g, float u) {
  const float y = 1.0f / (1.0f + expf(fabsf(g)));
  const float sig = (g < 0.0f) ? y : 1.0f - y;
  return (g * sig) * u;
}

__device__ __forceinline__ float swiglu_epilogue(int epilogue, float g, float u) {
  return epilogue == 2 ? swiglu_per_op(g, u) : (epilogue == 3 ? swiglu_fp32(g, u) : swiglu_cpu_contract(g, u));
}

// Warp wk owns the quads (4 consecutive groups) wk, wk+WK, ...; item gi of its
// stream is group (wk + (gi/4)*WK)*4 + gi%4.
template <int WK>
__device__ __forceinline__ int stream_group(int wk, int gi) {
  return (wk + (gi >> 2) * WK) * 4 + (gi & 3);
}

// Applies scale, bias and the 128 offset to a block of 8/TT multiplexed groups whose first
// item in the warp's stream is gi0.  Lane (g, tig) owns columns 2*tig and 2*tig+1.
// srow points at the lane's scale row (row g of the warp's 16), brow at its bias row;
// the rows of g+8 sit 8 * sc_stride bytes further.
template <int NT, int TT, int WK, bool FULLQ>
__device__ __forceinline__ void fixup_block(float (&acc)[NT][4], const float (&dg)[NT][4], const float* xsum,
                                            const unsigned char* srow, const unsigned char* brow, int sc_stride,
                                            int wk, int tig, int gi0, int nq_w, int ngroups) {
  constexpr int RC = 8 * NT;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col = 2 * tig + c;
    const int gi_c = gi0 + ((TT == 8) ? 0 : col / TT);
    const int G_c = (wk + (gi_c >> 2) * WK) * 4 + (gi_c & 3);
    if ((gi_c >> 2) < nq_w && (FULLQ || G_c < ngroups)) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float sv = __bfloat162float(
            *reinterpret_cast<const __nv_bfloat16*>(srow + h * 8 * sc_stride + G_c * 2));
        const float bv = __bfloat162float(
            *reinterpret_cast<const __nv_bfloat16*>(brow + h * 8 * sc_stride + G_c * 2));
        const float cv = fmaf(-128.0f, sv, bv);
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const float X = xsum[G_c * RC + ((TT == 8) ? nt * 8 + col : col % TT)];
          acc[nt][h * 2 + c] = fmaf(sv, dg[nt][h * 2 + c], fmaf(cv, X, acc[nt][h * 2 + c]));
        }
      }
    }
  }
}

}  // namespace zmoe
