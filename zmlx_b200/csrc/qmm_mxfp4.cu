// Token-grouped expert matmul for mxfp4 weights (e2m1 codes, one e8m0 scale per 32 along K).
//
// Same work decomposition as qmm.cu (task record x 16*WM-row tile, weights streamed once into
// registers two quads ahead, token rows in shared memory, column-multiplexed groups, fixed-order
// reductions).  The contraction runs on the FP8 tensor-core path: every e2m1 magnitude is exactly
// an e4m3 number, so four codes become four A bytes with ONE byte-permute lookup
// (prmt over the 8-entry table {0, .5, 1, 1.5, 2, 3, 4, 6}) plus a second prmt for the signs; the
// bf16 activations are split exactly into two e4m3 pieces after a per-token power-of-two scale.
// One mma.sync.m16n8k32 spans exactly one 32-wide scale group (4 lanes x 8 codes), so the group's
// power-of-two scale is applied to the fp32 group sum, not to the operands: the result is exact up to
// fp32 accumulation.  The reference has no mxfp4 kernel of its own (its fused op rejects the mode,
// gather_qmm_swiglu.patch:714-718); the arithmetic follows the OCP microscaling definition.
#include "qmm_common.cuh"

namespace zmoe {

__host__ __device__ inline int mx_xs_stride(int K) { return K * 2 + 16; }
__host__ __device__ inline int mx_sc_stride(int K) { return K / 32 + 8; }

struct MxSmem {
  int xs, sc, dscale, amax, zero, total;
};
__host__ __device__ inline MxSmem mx_smem(int K, int rs, int nmat, int wm, int wk, int nt) {
  MxSmem m;
  const int nwarps = wk * wm;
  int xs_bytes = rs * mx_xs_stride(K);
  int red_bytes = (wk > 1) ? wk * wm * 32 * nmat * nt * 4 * (int)sizeof(float) : 0;
  int a = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  m.xs = 0;
  a = (a + 15) & ~15;
  m.sc = a;
  a += nmat * 16 * wm * mx_sc_stride(K);
  a = (a + 15) & ~15;
  m.dscale = a;
  a += 8 * nt * 4;
  m.amax = a;
  a += nwarps * 8 * nt * 4;
  a = (a + 15) & ~15;
  m.zero = a;
  a += 32;
  m.total = a;
  return m;
}

template <int OFF>
__device__ __forceinline__ uint32_t ldg_stream_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.global.nc.u32 %0, [%1+%2];" : "=r"(v) : "l"(p), "n"(OFF));
  return v;
}

__device__ __forceinline__ void cp_async_8b(void* smem_dst, const void* gmem_src) {
  const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(d), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ uint32_t mx_pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ void mx_unpack_e4m3x4(uint32_t v, float (&out)[4]) {
  uint32_t h01, h23;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)(v & 0xffffu)));
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(v >> 16)));
  out[0] = __half2float(__ushort_as_half((unsigned short)(h01 & 0xffffu)));
  out[1] = __half2float(__ushort_as_half((unsigned short)(h01 >> 16)));
  out[2] = __half2float(__ushort_as_half((unsigned short)(h23 & 0xffffu)));
  out[3] = __half2float(__ushort_as_half((unsigned short)(h23 >> 16)));
}
__device__ __forceinline__ void mma_e4m3(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                         uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// eight e2m1 codes of a packed word -> two registers of four e4m3 bytes (codes 0-3, codes 4-7)
__device__ __forceinline__ void e2m1x8_to_e4m3(uint32_t w, uint32_t& lo, uint32_t& hi) {
  const uint32_t lut_a = 0x3C383000u, lut_b = 0x4C484440u;  // 0, .5, 1, 1.5 | 2, 3, 4, 6 as e4m3
  const uint32_t mag = w & 0x77777777u;
  const uint32_t sgn = (w >> 3) & 0x11111111u;  // selector 0 -> 0x00, 1 -> 0x80
  lo = __byte_perm(lut_a, lut_b, mag) | __byte_perm(0x00008000u, 0u, sgn);
  hi = __byte_perm(lut_a, lut_b, mag >> 16) | __byte_perm(0x00008000u, 0u, sgn >> 16);
}

template <int NMAT, int NT, int TT, int WK, int WM>
__global__ void __launch_bounds__(32 * WK * WM, (NT == 1) ? 512 / (32 * WK * WM) : 1)
    qmm_mxfp4_kernel(const QmmParams p) {
  static_assert(NT == 1 || TT == 8, "token tiles beyond the first are full");
  constexpr int GPB = 8 / TT;  // 32-wide groups multiplexed into one accumulator
  constexpr int NTH = 32 * WK * WM;
  constexpr int NW = WK * WM;
  constexpr int RC = 8 * NT;
  extern __shared__ __align__(16) unsigned char smem[];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;
  const int wk = wid % WK;
  const int wm = wid / WK;
  const int g = lane >> 2;
  const int tig = lane & 3;
  const int slot_g = g / TT;
  const int tok_g = g % TT;

  const int K = p.K, N = p.N;
  const int K8 = K >> 3;
  const int xs_stride = mx_xs_stride(K);
  const int sc_stride = mx_sc_stride(K);
  const MxSmem lay = mx_smem(K, p.rs, NMAT, WM, WK, NT);
  unsigned char* xs = smem + lay.xs;
  unsigned char* sraw = smem + lay.sc;
  float* dscale = reinterpret_cast<float*>(smem + lay.dscale);
  int* amax_s = reinterpret_cast<int*>(smem + lay.amax);
  float* red = reinterpret_cast<float*>(smem + lay.xs);

  if (!p.late_wait) pdl_wait();
  pdl_trigger();
  bool waited = !p.late_wait;
  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  const int nq = K >> 8;  // quads of four 64-code units (K % 256 == 0)
  const int nq_w = (nq > wk) ? (nq - wk + WK - 1) / WK : 0;
  bool first_pass = true;

  for (int a = blockIdx.y; a < p.E; a += gridDim.y) {
    const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + a);
    const int e = task.x, off = task.y, cnt = task.z;
    if (cnt == 0) break;
    const int n_cta = blockIdx.x * 16 * WM;
    const int n_lo = min(n_cta + wm * 16 + g, N - 1);
    const int n_hi = min(n_cta + wm * 16 + g + 8, N - 1);

    const uint32_t* wrow[NMAT][2];
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const uint32_t* we = p.w[m] + (size_t)e * N * K8;
      wrow[m][0] = we + (size_t)n_lo * K8 + tig + wk * 32;
      wrow[m][1] = we + (size_t)n_hi * K8 + tig + wk * 32;
    }

    for (int rc = 0; rc < cnt; rc += p.rs) {
      const int nrow = min(p.rs, cnt - rc);
      if (!first_pass) __syncthreads();
      first_pass = false;

      // ---- (1) prefetch two quads: per 64-code unit the lane's word of each of the two 32-wide groups
      const uint32_t* wp[NMAT][2];
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        wp[m][0] = wrow[m][0];
        wp[m][1] = wrow[m][1];
      }
      uint2 wbuf[2][4][NMAT][2];
      auto load_quad = [&](uint2 (&buf)[4][NMAT][2]) {
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            buf[0][m][h] = make_uint2(ldg_stream_u32<0>(wp[m][h]), ldg_stream_u32<16>(wp[m][h]));
            buf[1][m][h] = make_uint2(ldg_stream_u32<32>(wp[m][h]), ldg_stream_u32<48>(wp[m][h]));
            buf[2][m][h] = make_uint2(ldg_stream_u32<64>(wp[m][h]), ldg_stream_u32<80>(wp[m][h]));
            buf[3][m][h] = make_uint2(ldg_stream_u32<96>(wp[m][h]), ldg_stream_u32<112>(wp[m][h]));
            wp[m][h] += WK * 32;
          }
        }
      };
#pragma unroll
      for (int bq = 0; bq < 2; ++bq)
        if (bq < nq_w) load_quad(wbuf[bq]);

      // ---- (2) e8m0 scales of this CTA's rows
      if (rc == 0) {
        constexpr int ROWS = 16 * WM;
        const int cpr = K >> 8;  // 8-byte chunks per row
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const unsigned char* base = reinterpret_cast<const unsigned char*>(p.s[m]) + (size_t)e * N * (K >> 5);
          unsigned char* dst = sraw + m * ROWS * sc_stride;
          for (int i = tid; i < ROWS * cpr; i += NTH) {
            const int r = i / cpr;
            const int c = i - r * cpr;
            const int n = min(n_cta + r, N - 1);
            cp_async_8b(dst + r * sc_stride + c * 8, base + (size_t)n * (K >> 5) + c * 8);
          }
        }
      }

      if (!waited) {
        pdl_wait();
        waited = true;
      }
      // ---- (3) token rows: |x|max per row, then two e4m3 pieces per 8-block {hi 0-3, hi 4-7, lo 0-3, lo 4-7}
      if (tid < 8) reinterpret_cast<uint32_t*>(smem + lay.zero)[tid] = 0u;
      for (int t = 0; t < nrow; ++t) {
        const int src = p.x_by_dst ? pv.row_dst[off + rc + t] : pv.row_src[off + rc + t];
        const uint4* xrow = reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx);
        uint32_t mx = 0;
        for (int blk = tid; blk < K8; blk += NTH) {
          const uint4 v = __ldg(xrow + blk);
          *reinterpret_cast<uint4*>(xs + t * xs_stride + blk * 16) = v;
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            mx = max(mx, w4[i] & 0x7fffu);
            mx = max(mx, (w4[i] >> 16) & 0x7fffu);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        if (lane == 0) amax_s[wid * RC + t] = (int)mx;
      }
      __syncthreads();
      for (int t = 0; t < nrow; ++t) {
        uint32_t mx = 0;
#pragma unroll
        for (int w8 = 0; w8 < NW; ++w8) mx = max(mx, (uint32_t)amax_s[w8 * RC + t]);
        int ef = 261 - (int)(mx >> 7);  // scale = 2^(7 - floor(log2 |x|max)) puts |x|max in [128, 256)
        ef = (mx == 0) ? 127 : min(max(ef, 2), 252);
        const float scale = __uint_as_float((uint32_t)ef << 23);
        if (tid == 0) dscale[t] = __uint_as_float((uint32_t)(254 - ef) << 23);
        for (int blk = tid; blk < K8; blk += NTH) {
          uint4* px = reinterpret_cast<uint4*>(xs + t * xs_stride + blk * 16);
          const uint4 v = *px;  // written by this same thread above
          float f[8];
          f[0] = bf16_bits_to_float(v.x & 0xffffu) * scale;
          f[1] = bf16_bits_to_float(v.x >> 16) * scale;
          f[2] = bf16_bits_to_float(v.y & 0xffffu) * scale;
          f[3] = bf16_bits_to_float(v.y >> 16) * scale;
          f[4] = bf16_bits_to_float(v.z & 0xffffu) * scale;
          f[5] = bf16_bits_to_float(v.z >> 16) * scale;
          f[6] = bf16_bits_to_float(v.w & 0xffffu) * scale;
          f[7] = bf16_bits_to_float(v.w >> 16) * scale;
          uint4 o;
          o.x = mx_pack_e4m3x4(f[0], f[1], f[2], f[3]);
          o.y = mx_pack_e4m3x4(f[4], f[5], f[6], f[7]);
          float h0[4], h1[4];
          mx_unpack_e4m3x4(o.x, h0);
          mx_unpack_e4m3x4(o.y, h1);
          o.z = mx_pack_e4m3x4(f[0] - h0[0], f[1] - h0[1], f[2] - h0[2], f[3] - h0[3]);
          o.w = mx_pack_e4m3x4(f[4] - h1[0], f[5] - h1[1], f[6] - h1[2], f[7] - h1[3]);
          *px = o;
        }
      }
      asm volatile("cp.async.wait_all;" ::: "memory");
      __syncthreads();

      // ---- (4) main loop
      float acc[NMAT][NT][4];
      float dg[NMAT][NT][4];
#pragma unroll
      for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[m][nt][j] = 0.0f;
            dg[m][nt][j] = 0.0f;
          }
      const int xlane = lay.xs + ((TT == 8) ? g : tok_g) * xs_stride + tig * 16;
      const bool tok_ok = ((TT == 8) ? g : tok_g) < nrow;

      // fix-up of a block of GPB multiplexed 32-wide groups whose first stream item is mi0
      auto fixup = [&](int mi0) {
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int col = 2 * tig + c;
          const int mi_c = mi0 + ((TT == 8) ? 0 : col / TT);
          const int gi_c = mi_c >> 1;
          const int MX_c = ((wk + (gi_c >> 2) * WK) * 4 + (gi_c & 3)) * 2 + (mi_c & 1);
          if ((gi_c >> 2) < nq_w) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                const int r = wm * 16 + g + 8 * h;
                const uint32_t eb = sraw[(m * 16 * WM + r) * sc_stride + MX_c];
                const float sv = __uint_as_float(eb << 23);  // 2^(e - 127)
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  const int tok = (TT == 8) ? nt * 8 + col : col % TT;
                  acc[m][nt][h * 2 + c] = fmaf(sv * dscale[tok], dg[m][nt][h * 2 + c], acc[m][nt][h * 2 + c]);
                }
              }
            }
          }
        }
      };

      for (int qi = 0; qi < nq_w; qi += 2) {
#pragma unroll
        for (int bq = 0; bq < 2; ++bq) {
          const int quad = wk + (qi + bq) * WK;
          if (qi + bq < nq_w) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
#pragma unroll
              for (int mxh = 0; mxh < 2; ++mxh) {
                const int s2 = j * 2 + mxh;
                const int slot = s2 % GPB;
                if (slot == 0) {
#pragma unroll
                  for (int m = 0; m < NMAT; ++m)
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                      for (int jj = 0; jj < 4; ++jj) dg[m][nt][jj] = 0.0f;
                }
                uint4 xb[NT];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  const bool mine = (TT == 8) ? (nt * 8 + g < nrow) : (tok_ok && slot_g == slot);
                  const int xo = mine ? (xlane + nt * 8 * xs_stride + quad * 512 + j * 128 + mxh * 64) : lay.zero;
                  xb[nt] = *reinterpret_cast<const uint4*>(smem + xo);
                }
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                  const uint32_t wa = mxh ? wbuf[bq][j][m][0].y : wbuf[bq][j][m][0].x;
                  const uint32_t wb = mxh ? wbuf[bq][j][m][1].y : wbuf[bq][j][m][1].x;
                  uint32_t a0, a1, a2, a3;
                  e2m1x8_to_e4m3(wa, a0, a2);
                  e2m1x8_to_e4m3(wb, a1, a3);
#pragma unroll
                  for (int nt = 0; nt < NT; ++nt) {
                    mma_e4m3(dg[m][nt], a0, a1, a2, a3, xb[nt].x, xb[nt].y);
                    mma_e4m3(dg[m][nt], a0, a1, a2, a3, xb[nt].z, xb[nt].w);
                  }
                }
                if (slot == GPB - 1) fixup(((qi + bq) * 4 + j) * 2 + mxh - (GPB - 1));
              }
            }
            if (qi + bq + 2 < nq_w) load_quad(wbuf[bq]);
          }
        }
      }

      // ---- (5) reduce the K split across warps (fixed order), fold multiplexed columns, epilogue
      if (WK > 1) {
        __syncthreads();
        float* mine = red + ((wm * WK + wk) * 32 + lane) * (NMAT * NT * 4);
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
          for (int nt = 0; nt < NT; ++nt)
#pragma unroll
            for (int j = 0; j < 4; ++j) mine[(m * NT + nt) * 4 + j] = acc[m][nt][j];
        __syncthreads();
        if (wk == 0) {
#pragma unroll
          for (int o = 1; o < WK; ++o) {
            const float* other = red + ((wm * WK + o) * 32 + lane) * (NMAT * NT * 4);
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
              for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[m][nt][j] += other[(m * NT + nt) * 4 + j];
          }
        }
      }
      if (wk == 0) {
        if (TT < 8) {
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              if (TT == 1) {
                acc[m][0][h * 2] += acc[m][0][h * 2 + 1];
                acc[m][0][h * 2 + 1] = 0.0f;
              }
#pragma unroll
              for (int c = 0; c < 2; ++c) {
                float v = acc[m][0][h * 2 + c];
                if (TT <= 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                acc[m][0][h * 2 + c] = v;
              }
            }
          }
        }
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int col = 2 * tig + (j & 1);
            const int t = (TT == 8) ? nt * 8 + col : col;
            const int n = n_cta + wm * 16 + g + ((j >> 1) ? 8 : 0);
            const bool writer = (TT == 8) || (col < TT);
            if (writer && t < nrow && n < N) {
              float v;
              if (NMAT == 2) {
                v = (p.epilogue == 2) ? swiglu_per_op(acc[0][nt][j], acc[NMAT - 1][nt][j])
                                      : swiglu_cpu_contract(acc[0][nt][j], acc[NMAT - 1][nt][j]);
              } else {
                v = acc[0][nt][j];
              }
              const int dst = pv.row_dst[off + rc + t];
              p.out[(size_t)dst * p.ldo + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    }
  }
}

// ------------------------------------------------------------------ host side

template <int NMAT, int NT, int TT, int WK, int WM>
static int launch_mx(const QmmParams& p, int max_groups, cudaStream_t st) {
  auto kern = qmm_mxfp4_kernel<NMAT, NT, TT, WK, WM>;
  MxSmem lay = mx_smem(p.K, p.rs, NMAT, WM, WK, NT);
  if (lay.total > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lay.total);
    if (e != cudaSuccess)
      return fail(ZMOE_ERR_CUDA, "qmm_mxfp4: shared memory of %d bytes refused: %s", lay.total, cudaGetErrorString(e));
  }
  dim3 grid((p.N + 16 * WM - 1) / (16 * WM), max_groups);
  launch_pdl(kern, grid, dim3(32 * WK * WM), (size_t)lay.total, st, p);
  return check_launch("qmm_mxfp4_kernel");
}

template <int NMAT, int WK, int WM>
static int launch_mx_tokens(const QmmParams& p, int nt, int tt, int max_groups, cudaStream_t st) {
  if (nt == 1) {
    switch (tt) {
      case 1: return launch_mx<NMAT, 1, 1, WK, WM>(p, max_groups, st);
      case 2: return launch_mx<NMAT, 1, 2, WK, WM>(p, max_groups, st);
      case 4: return launch_mx<NMAT, 1, 4, WK, WM>(p, max_groups, st);
      default: return launch_mx<NMAT, 1, 8, WK, WM>(p, max_groups, st);
    }
  }
  if (nt == 2) return launch_mx<NMAT, 2, 8, WK, WM>(p, max_groups, st);
  return launch_mx<NMAT, 4, 8, WK, WM>(p, max_groups, st);
}

// Called by qmm_launch for ZMOE_Q_MXFP4 (p filled except rs).
int qmm_mxfp4_launch(QmmParams p, int nmat, int rows_hint, int max_groups, cudaStream_t st, const char* who) {
  ZMOE_REQUIRE(p.K % 256 == 0, ZMOE_ERR_UNSUPPORTED, "%s: mxfp4 needs K %% 256 == 0 (K=%d)", who, p.K);
  int nt = rows_hint <= 8 ? 1 : (rows_hint <= 16 ? 2 : 4);
  int tt = rows_hint <= 1 ? 1 : (rows_hint <= 2 ? 2 : (rows_hint <= 4 ? 4 : 8));
  int rs = (nt == 1) ? tt : 8 * nt;
  while (rs > 1 && (size_t)rs * mx_xs_stride(p.K) > 96 * 1024) rs /= 2;
  if (rs < 8) {
    nt = 1;
    tt = rs >= 4 ? 4 : (rs >= 2 ? 2 : 1);
    rs = tt;
  } else {
    tt = 8;
    nt = rs >= 32 ? 4 : (rs >= 16 ? 2 : 1);
    rs = 8 * nt;
  }
  p.rs = rs;
  const int nq = p.K >> 8;
  if (nq >= 8) return nmat == 2 ? launch_mx_tokens<2, 4, 1>(p, nt, tt, max_groups, st)
                                : launch_mx_tokens<1, 4, 1>(p, nt, tt, max_groups, st);
  if (nq >= 4) return nmat == 2 ? launch_mx_tokens<2, 2, 2>(p, nt, tt, max_groups, st)
                                : launch_mx_tokens<1, 2, 2>(p, nt, tt, max_groups, st);
  return nmat == 2 ? launch_mx_tokens<2, 1, 4>(p, nt, tt, max_groups, st)
                   : launch_mx_tokens<1, 1, 4>(p, nt, tt, max_groups, st);
}

}  // namespace zmoe
