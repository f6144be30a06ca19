// Token-grouped 4-bit quantised expert matmul (gate/up + SwiGLU, and down).
//
// Work unit: one expert (from the plan's list of experts that own rows) times a
// tile of 16*WM weight rows.  The expert's packed weights are streamed from HBM
// exactly once per CTA with 8-byte loads straight into registers, software
// pipelined PD groups deep; the expert's token rows (a handful at decode) sit in
// shared memory.  Codes are turned into bf16 in registers with one shift and one
// lop3 per pair -- code q becomes the bf16 value 128+q -- and contracted on the
// tensor cores (mma.sync m16n8k16, fp32 accumulate; weights are the 16-row A
// operand, tokens the 8-column B operand).  The 128 offset, the group scale and
// the group bias are applied in fp32 once per 64-wide group:
//     sum_k x_k (q_k s + b) = s * sum_k x_k (128 + q_k) + (b - 128 s) * sum_k x_k.
// A group of 64 codes of one row is held by the 4 lanes of a quad (16 codes
// each), so every mma accumulates inside one group and the scale factors out.
//
// The kernel is HBM-bound by design: per weight it issues ~0.9 integer ops and
// 1/256 of an mma, independent of the number of tokens (up to 8*NT per pass).
#include "common.cuh"

namespace zmoe {

struct QmmParams {
  const __nv_bfloat16* x;  // (x_rows, K) token rows, row stride ldx elements
  int ldx;
  const uint32_t* w[2];  // (E, N, K/8)
  const __nv_bfloat16* s[2];  // (E, N, K/64)
  const __nv_bfloat16* b[2];
  const int* plan;
  int rows, E;
  __nv_bfloat16* out;  // (rows, N)
  int ldo;
  int N, K, ngroups;
  int rs;        // token rows staged per pass (<= 8*NT)
  int epilogue;  // 0: store T; 1: SwiGLU CPU contract; 2: SwiGLU per-op contract
  int x_by_dst;  // token row r of the output reads x row r instead of the plan's source row
};

__host__ __device__ inline size_t qmm_xs_stride(int K) { return (size_t)K * 2 + 16; }

// Shared-memory carve-up, identical on host and device.
struct QmmSmem {
  size_t xs, xsum, sc, total;
};
__host__ __device__ inline QmmSmem qmm_smem(int K, int ngroups, int rs, int rc, int nmat, int wm, int wk, int nt) {
  QmmSmem m;
  size_t xs_bytes = (size_t)rs * qmm_xs_stride(K);
  size_t red_bytes = (wk > 1) ? (size_t)wk * wm * 32 * nmat * nt * 4 * sizeof(float) : 0;
  m.xs = 0;
  size_t a = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  a = (a + 15) & ~(size_t)15;
  m.xsum = a;
  a += (size_t)ngroups * rc * sizeof(float);
  a = (a + 15) & ~(size_t)15;
  m.sc = a;
  a += (size_t)nmat * 16 * wm * (ngroups + 1) * sizeof(float2);
  m.total = a;
  return m;
}

__device__ __forceinline__ uint2 ldg_stream_u2(const uint32_t* p) {
  uint2 v;
  asm volatile("ld.global.nc.L1::no_allocate.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
  return v;
}

__device__ __forceinline__ void mma_bf16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// codes at bits [sh, sh+4) and [sh+16, sh+20) -> bf16x2 (128+q_lo, 128+q_hi)
__device__ __forceinline__ uint32_t deq_pair(uint32_t word, int sh) {
  return ((word >> sh) & 0x000F000Fu) | 0x43004300u;
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

template <int NMAT, int NT, int WK, int WM, int PD>
__global__ void __launch_bounds__(32 * WK * WM) qmm_affine_kernel(const QmmParams p) {
  constexpr int NTH = 32 * WK * WM;
  constexpr int RC = 8 * NT;
  extern __shared__ __align__(16) unsigned char smem[];

  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;
  const int wk = wid % WK;
  const int wm = wid / WK;
  const int g = lane >> 2;
  const int tig = lane & 3;

  const int K = p.K, N = p.N, ngroups = p.ngroups;
  const int K8 = K >> 3;
  const size_t xs_stride = qmm_xs_stride(K);
  const QmmSmem lay = qmm_smem(K, ngroups, p.rs, RC, NMAT, WM, WK, NT);
  unsigned char* xs = smem + lay.xs;
  float* xsum = reinterpret_cast<float*>(smem + lay.xsum);
  float2* scs = reinterpret_cast<float2*>(smem + lay.sc);
  float* red = reinterpret_cast<float*>(smem + lay.xs);

  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  const int n_active = pv.hdr[0];
  const int ng_w = (ngroups > wk) ? (ngroups - wk + WK - 1) / WK : 0;  // groups of this warp: wk, wk+WK, ...

  for (int a = blockIdx.y; a < n_active; a += gridDim.y) {
    const int e = pv.active[a];
    const int off = pv.offset[e];
    const int cnt = pv.offset[e + 1] - off;
    const int n_cta = blockIdx.x * 16 * WM;
    const int n_lo = min(n_cta + wm * 16 + g, N - 1);
    const int n_hi = min(n_cta + wm * 16 + g + 8, N - 1);

    const uint32_t* wrow[NMAT][2];
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      const uint32_t* we = p.w[m] + (size_t)e * N * K8;
      wrow[m][0] = we + (size_t)n_lo * K8 + tig * 2;
      wrow[m][1] = we + (size_t)n_hi * K8 + tig * 2;
    }

    for (int rc = 0; rc < cnt; rc += p.rs) {
      const int nrow = min(p.rs, cnt - rc);

      // ---- prefetch the first PD groups of packed weights into registers
      uint2 wbuf[PD][NMAT][2];
#pragma unroll
      for (int s = 0; s < PD; ++s) {
        if (s < ng_w) {
          const int G = wk + s * WK;
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            wbuf[s][m][0] = ldg_stream_u2(wrow[m][0] + G * 8);
            wbuf[s][m][1] = ldg_stream_u2(wrow[m][1] + G * 8);
          }
        }
      }

      if (rc > 0 || a != (int)blockIdx.y) __syncthreads();  // previous pass is done with shared memory

      // ---- stage the token rows: 8-element blocks permuted to (0,4,1,5,2,6,3,7), plus group sums
      {
        const int items = nrow * K8;
        for (int i0 = 0; i0 < items; i0 += NTH) {
          const int i = i0 + tid;
          float part = 0.0f;
          if (i < items) {
            const int t = i / K8;
            const int blk = i - t * K8;
            const int src = p.x_by_dst ? pv.row_dst[off + rc + t] : pv.row_src[off + rc + t];
            const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx) + blk);
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410);
            o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410);
            o.w = __byte_perm(v.y, v.w, 0x7632);
            *reinterpret_cast<uint4*>(xs + (size_t)t * xs_stride + (size_t)blk * 16) = o;
            part = ((bf16_bits_to_float(v.x & 0xffffu) + bf16_bits_to_float(v.x >> 16)) +
                    (bf16_bits_to_float(v.y & 0xffffu) + bf16_bits_to_float(v.y >> 16))) +
                   ((bf16_bits_to_float(v.z & 0xffffu) + bf16_bits_to_float(v.z >> 16)) +
                    (bf16_bits_to_float(v.w & 0xffffu) + bf16_bits_to_float(v.w >> 16)));
          }
          part += __shfl_xor_sync(0xffffffffu, part, 1);
          part += __shfl_xor_sync(0xffffffffu, part, 2);
          part += __shfl_xor_sync(0xffffffffu, part, 4);
          if (i < items && (lane & 7) == 0) {
            const int t = i / K8;
            const int blk = i - t * K8;
            xsum[(blk >> 3) * RC + t] = part;
          }
        }
        // token slots beyond nrow contribute nothing
        for (int i = tid; i < ngroups * RC; i += NTH) {
          if ((i % RC) >= nrow) xsum[i] = 0.0f;
        }
      }
      // ---- stage (scale, bias - 128*scale) of this CTA's rows, once per expert
      if (rc == 0) {
        const int per_mat = 16 * WM * ngroups;
        for (int i = tid; i < NMAT * per_mat; i += NTH) {
          const int m = i / per_mat;
          const int r = (i - m * per_mat) / ngroups;
          const int G = i - m * per_mat - r * ngroups;
          const int n = min(n_cta + r, N - 1);
          const size_t o = ((size_t)e * N + n) * ngroups + G;
          const __nv_bfloat16* sp = (NMAT == 2 && m) ? p.s[1] : p.s[0];
          const __nv_bfloat16* bp = (NMAT == 2 && m) ? p.b[1] : p.b[0];
          const float sv = __bfloat162float(sp[o]);
          const float bv = __bfloat162float(bp[o]);
          scs[(size_t)(m * 16 * WM + r) * (ngroups + 1) + G] = make_float2(sv, fmaf(-128.0f, sv, bv));
        }
      }
      __syncthreads();

      // ---- main loop over this warp's groups
      float acc[NMAT][NT][4];
#pragma unroll
      for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][nt][j] = 0.0f;

      for (int it = 0; it < ng_w; it += PD) {
#pragma unroll
        for (int s = 0; s < PD; ++s) {
          const int gi = it + s;
          if (gi < ng_w) {
            const int G = wk + gi * WK;
            uint4 xb[NT][2];
            float2 xs2[NT];
#pragma unroll
            for (int nt = 0; nt < NT; ++nt) {
              const int tb = nt * 8 + g;
              if (tb < nrow) {
                const unsigned char* xp = xs + (size_t)tb * xs_stride + ((size_t)G * 64 + tig * 16) * 2;
                xb[nt][0] = *reinterpret_cast<const uint4*>(xp);
                xb[nt][1] = *reinterpret_cast<const uint4*>(xp + 16);
              } else {
                xb[nt][0] = make_uint4(0, 0, 0, 0);
                xb[nt][1] = make_uint4(0, 0, 0, 0);
              }
              xs2[nt] = *reinterpret_cast<const float2*>(xsum + G * RC + nt * 8 + 2 * tig);
            }
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
              const uint2 wa = wbuf[s][m][0];
              const uint2 wb = wbuf[s][m][1];
              float dg[NT][4];
#pragma unroll
              for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                for (int j = 0; j < 4; ++j) dg[nt][j] = 0.0f;
              {
                const uint32_t a0 = deq_pair(wa.x, 0), a1 = deq_pair(wb.x, 0);
                const uint32_t a2 = deq_pair(wa.x, 4), a3 = deq_pair(wb.x, 4);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16_m16n8k16(dg[nt], a0, a1, a2, a3, xb[nt][0].x, xb[nt][0].y);
              }
              {
                const uint32_t a0 = deq_pair(wa.x, 8), a1 = deq_pair(wb.x, 8);
                const uint32_t a2 = deq_pair(wa.x, 12), a3 = deq_pair(wb.x, 12);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16_m16n8k16(dg[nt], a0, a1, a2, a3, xb[nt][0].z, xb[nt][0].w);
              }
              {
                const uint32_t a0 = deq_pair(wa.y, 0), a1 = deq_pair(wb.y, 0);
                const uint32_t a2 = deq_pair(wa.y, 4), a3 = deq_pair(wb.y, 4);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16_m16n8k16(dg[nt], a0, a1, a2, a3, xb[nt][1].x, xb[nt][1].y);
              }
              {
                const uint32_t a0 = deq_pair(wa.y, 8), a1 = deq_pair(wb.y, 8);
                const uint32_t a2 = deq_pair(wa.y, 12), a3 = deq_pair(wb.y, 12);
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) mma_bf16_m16n8k16(dg[nt], a0, a1, a2, a3, xb[nt][1].z, xb[nt][1].w);
              }
              const float2 s_lo = scs[(size_t)(m * 16 * WM + wm * 16 + g) * (ngroups + 1) + G];
              const float2 s_hi = scs[(size_t)(m * 16 * WM + wm * 16 + g + 8) * (ngroups + 1) + G];
#pragma unroll
              for (int nt = 0; nt < NT; ++nt) {
                acc[m][nt][0] = fmaf(s_lo.x, dg[nt][0], fmaf(s_lo.y, xs2[nt].x, acc[m][nt][0]));
                acc[m][nt][1] = fmaf(s_lo.x, dg[nt][1], fmaf(s_lo.y, xs2[nt].y, acc[m][nt][1]));
                acc[m][nt][2] = fmaf(s_hi.x, dg[nt][2], fmaf(s_hi.y, xs2[nt].x, acc[m][nt][2]));
                acc[m][nt][3] = fmaf(s_hi.x, dg[nt][3], fmaf(s_hi.y, xs2[nt].y, acc[m][nt][3]));
              }
            }
            // refill this pipeline slot
            const int gn = gi + PD;
            if (gn < ng_w) {
              const int Gn = wk + gn * WK;
#pragma unroll
              for (int m = 0; m < NMAT; ++m) {
                wbuf[s][m][0] = ldg_stream_u2(wrow[m][0] + Gn * 8);
                wbuf[s][m][1] = ldg_stream_u2(wrow[m][1] + Gn * 8);
              }
            }
          }
        }
      }

      // ---- reduce the K-split across warps (fixed order), then the epilogue
      if (WK > 1) {
        __syncthreads();  // every warp is done reading the staged rows; reuse their space
        float* mine = red + ((size_t)(wm * WK + wk) * 32 + lane) * (NMAT * NT * 4);
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
            const float* other = red + ((size_t)(wm * WK + o) * 32 + lane) * (NMAT * NT * 4);
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
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int t = nt * 8 + 2 * tig + (j & 1);
            const int n = n_cta + wm * 16 + g + ((j >> 1) ? 8 : 0);
            if (t < nrow && n < N) {
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

struct QmmChoice {
  int nt, wk, wm;
};

static QmmChoice choose_config(int ngroups, int rows_hint) {
  QmmChoice c;
  c.nt = rows_hint <= 8 ? 1 : (rows_hint <= 16 ? 2 : 4);
  if (ngroups >= 16) {
    c.wk = 4;
    c.wm = 1;
  } else if (ngroups >= 8) {
    c.wk = 2;
    c.wm = 2;
  } else {
    c.wk = 1;
    c.wm = 4;
  }
  return c;
}

template <int NMAT, int NT, int WK, int WM>
static int launch_cfg(const QmmParams& p, int max_groups, cudaStream_t st) {
  constexpr int PD = 8;
  auto kern = qmm_affine_kernel<NMAT, NT, WK, WM, PD>;
  QmmSmem lay = qmm_smem(p.K, p.ngroups, p.rs, 8 * NT, NMAT, WM, WK, NT);
  if (lay.total > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lay.total);
    if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "qmm: shared memory of %zu bytes refused: %s", lay.total,
                                      cudaGetErrorString(e));
  }
  dim3 grid((p.N + 16 * WM - 1) / (16 * WM), max_groups);
  kern<<<grid, 32 * WK * WM, lay.total, st>>>(p);
  return check_launch("qmm_affine_kernel");
}

template <int NMAT>
static int launch_nmat(const QmmParams& p, const QmmChoice& c, int max_groups, cudaStream_t st) {
#define ZMOE_CASE(NT_, WK_, WM_) \
  if (c.nt == NT_ && c.wk == WK_ && c.wm == WM_) return launch_cfg<NMAT, NT_, WK_, WM_>(p, max_groups, st);
  ZMOE_CASE(1, 4, 1)
  ZMOE_CASE(2, 4, 1)
  ZMOE_CASE(4, 4, 1)
  ZMOE_CASE(1, 2, 2)
  ZMOE_CASE(2, 2, 2)
  ZMOE_CASE(4, 2, 2)
  ZMOE_CASE(1, 1, 4)
  ZMOE_CASE(2, 1, 4)
  ZMOE_CASE(4, 1, 4)
#undef ZMOE_CASE
  return fail(ZMOE_ERR_UNSUPPORTED, "qmm: no kernel for nt=%d wk=%d wm=%d", c.nt, c.wk, c.wm);
}

int qmm_launch(int nmat, const void* x, int x_rows, int ldx, const uint32_t* const* w, const void* const* s,
               const void* const* b, int E, int N, int K, int group_size, int qmode, const void* plan, int rows,
               int rows_hint, void* out, int epilogue, int x_by_dst, void* stream, const char* who) {
  ZMOE_REQUIRE(x && plan && out, ZMOE_ERR_SHAPE, "%s: null pointer", who);
  for (int m = 0; m < nmat; ++m)
    ZMOE_REQUIRE(w[m] && s[m], ZMOE_ERR_SHAPE, "%s: null weight or scale pointer", who);
  ZMOE_REQUIRE(E >= 1 && N >= 1 && K >= 1 && rows >= 0 && x_rows >= 0, ZMOE_ERR_SHAPE,
               "%s: bad sizes E=%d N=%d K=%d rows=%d", who, E, N, K, rows);
  ZMOE_REQUIRE(qmode == ZMOE_Q_AFFINE4, ZMOE_ERR_UNSUPPORTED, "%s: quantisation mode %d is not supported", who,
               qmode);
  ZMOE_REQUIRE(group_size == 64, ZMOE_ERR_UNSUPPORTED, "%s: group_size=%d (only 64 is supported)", who, group_size);
  ZMOE_REQUIRE(K % 64 == 0, ZMOE_ERR_SHAPE, "%s: K=%d must be a multiple of 64", who, K);
  for (int m = 0; m < nmat; ++m) ZMOE_REQUIRE(b[m], ZMOE_ERR_SHAPE, "%s: affine mode needs biases", who);
  ZMOE_REQUIRE(ldx >= K && ldx % 8 == 0 && ((uintptr_t)x % 16) == 0, ZMOE_ERR_ALIGN,
               "%s: x rows must be 16-byte aligned (ldx=%d)", who, ldx);
  for (int m = 0; m < nmat; ++m)
    ZMOE_REQUIRE(((uintptr_t)w[m] % 8) == 0, ZMOE_ERR_ALIGN, "%s: packed weights must be 8-byte aligned", who);
  if (rows == 0) return ZMOE_OK;
  if (rows_hint <= 0 || rows_hint > rows) rows_hint = rows;

  QmmParams p;
  p.x = (const __nv_bfloat16*)x;
  p.ldx = ldx;
  for (int m = 0; m < 2; ++m) {
    int mm = m < nmat ? m : 0;
    p.w[m] = w[mm];
    p.s[m] = (const __nv_bfloat16*)s[mm];
    p.b[m] = (const __nv_bfloat16*)b[mm];
  }
  p.plan = (const int*)plan;
  p.rows = rows;
  p.E = E;
  p.out = (__nv_bfloat16*)out;
  p.ldo = N;
  p.N = N;
  p.K = K;
  p.ngroups = K / 64;
  p.epilogue = epilogue;
  p.x_by_dst = x_by_dst;

  QmmChoice c = choose_config(p.ngroups, rows_hint);
  // keep the staged token rows within ~96 KB so that several CTAs share an SM
  int rs = 8 * c.nt;
  if (rows_hint < rs) rs = rows_hint;
  while (rs > 1 && (size_t)rs * qmm_xs_stride(K) > 96 * 1024) rs = (rs + 1) / 2;
  while (c.nt > 1 && 8 * (c.nt / 2) >= rs) c.nt /= 2;
  p.rs = rs;
  int max_groups = rows < E ? rows : E;
  if (max_groups > 65535) max_groups = 65535;
  if (nmat == 2) return launch_nmat<2>(p, c, max_groups, (cudaStream_t)stream);
  return launch_nmat<1>(p, c, max_groups, (cudaStream_t)stream);
}

}  // namespace zmoe

using namespace zmoe;

extern "C" {

int zmoe_gather_qmm_swiglu(const void* x, int x_rows, int ldx, const uint32_t* gate_w, const void* gate_scales,
                           const void* gate_biases, const uint32_t* up_w, const void* up_scales,
                           const void* up_biases, int E, int N, int K, int group_size, int qmode,
                           const void* plan, int rows, int rows_hint, void* out, int swiglu_mode, void* stream) {
  ZMOE_REQUIRE(swiglu_mode == ZMOE_SWIGLU_CPU || swiglu_mode == ZMOE_SWIGLU_PER_OP, ZMOE_ERR_UNSUPPORTED,
               "zmoe_gather_qmm_swiglu: swiglu_mode %d", swiglu_mode);
  const uint32_t* w[2] = {gate_w, up_w};
  const void* s[2] = {gate_scales, up_scales};
  const void* b[2] = {gate_biases, up_biases};
  return qmm_launch(2, x, x_rows, ldx, w, s, b, E, N, K, group_size, qmode, plan, rows, rows_hint, out,
                    swiglu_mode == ZMOE_SWIGLU_CPU ? 1 : 2, 0, stream, "zmoe_gather_qmm_swiglu");
}

int zmoe_gather_qmm(const void* x, int x_rows, int ldx, const uint32_t* w_, const void* scales, const void* biases,
                    int E, int N, int K, int group_size, int qmode, const void* plan, int rows, int rows_hint,
                    int x_by_output_row, void* out, void* stream) {
  const uint32_t* w[2] = {w_, nullptr};
  const void* s[2] = {scales, nullptr};
  const void* b[2] = {biases, nullptr};
  return qmm_launch(1, x, x_rows, ldx, w, s, b, E, N, K, group_size, qmode, plan, rows, rows_hint, out, 0,
                    x_by_output_row != 0, stream, "zmoe_gather_qmm");
}

}  // extern "C"
