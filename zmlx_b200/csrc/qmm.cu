// Token-grouped 4-bit quantised expert matmul (gate/up + SwiGLU, and down).
//
// Work unit: one expert (a task record of the plan) times a tile of 16*WM weight
// rows.  The expert's packed weights are streamed from HBM exactly once per CTA
// with 8-byte loads straight into registers, software pipelined PD groups deep;
// the expert's token rows (a handful at decode) sit in shared memory.  Codes are
// turned into bf16 in registers with one shift and one lop3 per pair -- code q
// becomes the bf16 value 128+q -- and contracted on the tensor cores (mma.sync
// m16n8k16, fp32 accumulate; weights are the 16-row A operand, tokens the
// 8-column B operand).  The 128 offset, the group scale and the group bias are
// applied in fp32:
//     sum_k x_k (q_k s + b) = s * sum_k x_k (128 + q_k) + (b - 128 s) * sum_k x_k.
// A group of 64 codes of one row is held by the 4 lanes of a quad (16 codes
// each), so every mma accumulates inside one group and the scale factors out.
//
// Column multiplexing: the mma has 8 token columns but decode brings TT = 1, 2 or
// 4 tokens per expert.  The spare columns carry *other groups*: column n is
// (group slot n / TT, token n % TT), and the B fragment of slot j is zero except
// in its own columns.  8/TT consecutive groups then accumulate side by side in one
// accumulator and the per-group fix-up above runs once per 8/TT groups.
//
// The kernel is HBM-bound by design: per weight it issues ~0.9 integer ops and
// 1/256 of an mma, independent of the number of tokens (up to 8*NT per pass).
#include "qmm_common.cuh"

namespace zmoe {

// Many rows per expert: tcgen05 / tensor-memory kernel (qmm_tc.cu).
int qmm_tc_launch(const QmmParams& q, int nmat, int rows_hint, int max_groups, cudaStream_t st, const char* who);
// mxfp4 weights (qmm_mxfp4.cu).
int qmm_mxfp4_launch(QmmParams p, int nmat, int rows_hint, int max_groups, cudaStream_t st, const char* who);


// Shared-memory carve-up, identical on host and device.
struct QmmSmem {
  int xs, xsum, sc, zero, total;
};
__host__ __device__ inline QmmSmem qmm_smem(int K, int ngroups, int rs, int rc, int nmat, int wm, int wk, int nt) {
  QmmSmem m;
  int xs_bytes = rs * qmm_xs_stride(K);
  int red_bytes = (wk > 1) ? wk * wm * 32 * nmat * nt * 4 * (int)sizeof(float) : 0;
  m.xs = 0;
  int a = xs_bytes > red_bytes ? xs_bytes : red_bytes;
  a = (a + 15) & ~15;
  m.xsum = a;
  a += ngroups * rc * (int)sizeof(float);
  a = (a + 15) & ~15;
  m.sc = a;
  a += nmat * 2 * 16 * wm * qmm_sc_stride(ngroups);  // raw T scales and biases of the CTA's rows
  a = (a + 15) & ~15;
  m.zero = a;  // 32 zero bytes: the B fragment of columns that carry another group
  a += 32;
  m.total = a;
  return m;
}

// Loads one quad (4 consecutive groups: 32 bytes of each of the lane's rows) into registers.
template <int NMAT, bool FULLQ>
__device__ __forceinline__ void load_quad(uint2 (&buf)[4][NMAT][2], const uint32_t* (&wp)[NMAT][2], int G0,
                                          int ngroups) {
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      if (FULLQ || G0 + 0 < ngroups) buf[0][m][h] = ldg_stream_u2<0>(wp[m][h]);
      if (FULLQ || G0 + 1 < ngroups) buf[1][m][h] = ldg_stream_u2<32>(wp[m][h]);
      if (FULLQ || G0 + 2 < ngroups) buf[2][m][h] = ldg_stream_u2<64>(wp[m][h]);
      if (FULLQ || G0 + 3 < ngroups) buf[3][m][h] = ldg_stream_u2<96>(wp[m][h]);
    }
  }
}

// Applies scale, bias and the 128 offset to a block of 8/TT multiplexed groups whose first
// item in the warp's stream is gi0.  Lane (g, tig) owns columns 2*tig and 2*tig+1.
template <int NMAT, int NT, int TT, int WK, int WM, bool FULLQ>
__device__ __forceinline__ void fixup_multi(float (&acc)[NMAT][NT][4], const float (&dg)[NMAT][NT][4],
                                            const float* xsum, const unsigned char* sraw, int sc_stride, int wk,
                                            int wm, int g, int tig, int gi0, int nq_w, int ngroups) {
  constexpr int RC = 8 * NT;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col = 2 * tig + c;
    const int gi_c = gi0 + ((TT == 8) ? 0 : col / TT);
    const int G_c = (wk + (gi_c >> 2) * WK) * 4 + (gi_c & 3);
    if ((gi_c >> 2) < nq_w && (FULLQ || G_c < ngroups)) {
#pragma unroll
      for (int nt = 0; nt < NT; ++nt) {
        const float X = xsum[G_c * RC + ((TT == 8) ? nt * 8 + col : col % TT)];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int r = wm * 16 + g + 8 * h;
            const float sv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(
                sraw + ((m * 2 + 0) * 16 * WM + r) * sc_stride + G_c * 2));
            const float bv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(
                sraw + ((m * 2 + 1) * 16 * WM + r) * sc_stride + G_c * 2));
            const float cv = fmaf(-128.0f, sv, bv);
            acc[m][nt][h * 2 + c] = fmaf(sv, dg[m][nt][h * 2 + c], fmaf(cv, X, acc[m][nt][h * 2 + c]));
          }
        }
      }
    }
  }
}

template <int NMAT, int NT, int TT, int WK, int WM, bool FULLQ>
__global__ void __launch_bounds__(32 * WK * WM, (NT == 1) ? 512 / (32 * WK * WM) : 1)
    qmm_affine_kernel(const QmmParams p) {
  static_assert(NT == 1 || TT == 8, "token tiles beyond the first are full");
  constexpr int GPB = 8 / TT;  // groups multiplexed into one accumulator
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
  // column g of the B operand is (slot g / TT, token g % TT)
  const int slot_g = g / TT;
  const int tok_g = g % TT;

  const int K = p.K, N = p.N, ngroups = p.ngroups;
  const int K8 = K >> 3;
  const int xs_stride = qmm_xs_stride(K);
  const int sc_stride = qmm_sc_stride(ngroups);
  const QmmSmem lay = qmm_smem(K, ngroups, p.rs, RC, NMAT, WM, WK, NT);
  unsigned char* xs = smem + lay.xs;
  float* xsum = reinterpret_cast<float*>(smem + lay.xsum);
  unsigned char* sraw = smem + lay.sc;
  float* red = reinterpret_cast<float*>(smem + lay.xs);

  // With late_wait the caller vouches that the plan was written before the previous kernel started (so it is
  // complete whenever this grid runs) and only the token rows come from the previous kernel: the first weights
  // are then streamed before the dependency wait.
  if (!p.late_wait) pdl_wait();
  pdl_trigger();
  bool waited = !p.late_wait;
  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  const int nq = (ngroups + 3) >> 2;
  const int nq_w = (nq > wk) ? (nq - wk + WK - 1) / WK : 0;
  bool first_pass = true;

  for (int a = blockIdx.y; a < p.E; a += gridDim.y) {
    const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + a);  // {expert, offset, count, -}
    const int e = task.x, off = task.y, cnt = task.z;
    if (cnt == 0) break;  // tasks are compact: nothing beyond the first empty one
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

      if (!first_pass) __syncthreads();  // the previous pass is done with shared memory
      first_pass = false;

      // ---- (1) prefetch the first two quads (8 groups) of packed weights into registers
      const uint32_t* wp[NMAT][2];  // this warp's next quad to fetch, per matrix and row half
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        wp[m][0] = wrow[m][0] + wk * 32;
        wp[m][1] = wrow[m][1] + wk * 32;
      }
      uint2 wbuf[2][4][NMAT][2];
#pragma unroll
      for (int bq = 0; bq < 2; ++bq) {
        if (bq < nq_w) {
          load_quad<NMAT, FULLQ>(wbuf[bq], wp, (wk + bq * WK) * 4, ngroups);
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            wp[m][0] += WK * 32;
            wp[m][1] += WK * 32;
          }
        }
      }

      // ---- (2) scales and biases of this CTA's rows: asynchronous copies, raw T values
      if (rc == 0) {
        constexpr int ROWS = 16 * WM;
#pragma unroll
        for (int arr = 0; arr < NMAT * 2; ++arr) {
          const __nv_bfloat16* base = (arr & 1) ? p.b[arr >> 1] : p.s[arr >> 1];
          base += (size_t)e * N * ngroups;
          unsigned char* dst = sraw + arr * ROWS * sc_stride;
          if ((ngroups & 3) == 0) {
            const int cpr = ngroups >> 2;  // 8-byte chunks per row
            for (int i = tid; i < ROWS * cpr; i += NTH) {
              const int r = i / cpr;
              const int c = i - r * cpr;
              const int n = min(n_cta + r, N - 1);
              cp_async_8(dst + r * sc_stride + c * 8, base + (size_t)n * ngroups + c * 4);
            }
          } else {
            for (int i = tid; i < ROWS * ngroups; i += NTH) {
              const int r = i / ngroups;
              const int c = i - r * ngroups;
              const int n = min(n_cta + r, N - 1);
              reinterpret_cast<__nv_bfloat16*>(dst + r * sc_stride)[c] = base[(size_t)n * ngroups + c];
            }
          }
        }
      }

      if (!waited) {
        pdl_wait();
        waited = true;
      }
      // ---- (3) stage the token rows: 8-element blocks permuted to (0,4,1,5,2,6,3,7), plus group sums
      for (int t = 0; t < nrow; ++t) {
        const int src = p.x_by_dst ? pv.row_dst[off + rc + t] : pv.row_src[off + rc + t];
        const uint4* xrow = reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx);
        for (int b0 = wid * 32; b0 < K8; b0 += NTH) {  // warp-uniform trip count (K8 is a multiple of 8)
          const int blk = b0 + lane;
          uint4 v = make_uint4(0, 0, 0, 0);
          if (blk < K8) {
            v = __ldg(xrow + blk);
            uint4 o;
            o.x = __byte_perm(v.x, v.z, 0x5410);
            o.y = __byte_perm(v.x, v.z, 0x7632);
            o.z = __byte_perm(v.y, v.w, 0x5410);
            o.w = __byte_perm(v.y, v.w, 0x7632);
            *reinterpret_cast<uint4*>(xs + t * xs_stride + blk * 16) = o;
          }
          float part = ((bf16_bits_to_float(v.x & 0xffffu) + bf16_bits_to_float(v.x >> 16)) +
                        (bf16_bits_to_float(v.y & 0xffffu) + bf16_bits_to_float(v.y >> 16))) +
                       ((bf16_bits_to_float(v.z & 0xffffu) + bf16_bits_to_float(v.z >> 16)) +
                        (bf16_bits_to_float(v.w & 0xffffu) + bf16_bits_to_float(v.w >> 16)));
          part += __shfl_xor_sync(0xffffffffu, part, 1);
          part += __shfl_xor_sync(0xffffffffu, part, 2);
          part += __shfl_xor_sync(0xffffffffu, part, 4);
          if (blk < K8 && (lane & 7) == 0) xsum[(blk >> 3) * RC + t] = part;
        }
      }
      if (tid < 8) reinterpret_cast<uint32_t*>(smem + lay.zero)[tid] = 0u;
      if (nrow < RC) {  // token slots beyond nrow contribute nothing
        for (int i = tid; i < ngroups * RC; i += NTH) {
          if ((i % RC) >= nrow) xsum[i] = 0.0f;
        }
      }
      cp_async_wait_all();
      __syncthreads();

      // ---- (4) main loop over this warp's groups
      float acc[NMAT][NT][4];
      float dg[NMAT][NT][4];
#pragma unroll
      for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int nt = 0; nt < NT; ++nt)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][nt][j] = 0.0f;

      // per-lane shared-memory bases: token row (or the zero page) and the scale rows
      const int xlane = lay.xs + ((TT == 8) ? g : tok_g) * xs_stride + tig * 32;  // byte offsets into smem
      const int zpage = lay.zero;
      const bool tok_ok = ((TT == 8) ? g : tok_g) < nrow;

      for (int qi = 0; qi < nq_w; qi += 2) {
#pragma unroll
        for (int bq = 0; bq < 2; ++bq) {
          const int quad = wk + (qi + bq) * WK;
          if (qi + bq < nq_w) {  // warp-uniform
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int s = bq * 4 + j;
              const int slot = s % GPB;
              const int G = quad * 4 + j;
              if (slot == 0) {
#pragma unroll
                for (int m = 0; m < NMAT; ++m)
#pragma unroll
                  for (int nt = 0; nt < NT; ++nt)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) dg[m][nt][jj] = 0.0f;
              }
              if (FULLQ || G < ngroups) {
                uint4 xb[NT][2];
#pragma unroll
                for (int nt = 0; nt < NT; ++nt) {
                  const bool mine = (TT == 8) ? (nt * 8 + g < nrow) : (tok_ok && slot_g == slot);
                  const int xo = mine ? (xlane + nt * 8 * xs_stride + quad * 512 + j * 128) : zpage;
                  xb[nt][0] = *reinterpret_cast<const uint4*>(smem + xo);
                  xb[nt][1] = *reinterpret_cast<const uint4*>(smem + xo + 16);
                }
#pragma unroll
                for (int m = 0; m < NMAT; ++m) {
                  const uint2 wa = wbuf[bq][j][m][0];
                  const uint2 wb = wbuf[bq][j][m][1];
                  {
                    const uint32_t a0 = deq_imm<0>(wa.x), a1 = deq_imm<0>(wb.x);
                    const uint32_t a2 = deq_imm<4>(wa.x), a3 = deq_imm<4>(wb.x);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                      mma_bf16_m16n8k16(dg[m][nt], a0, a1, a2, a3, xb[nt][0].x, xb[nt][0].y);
                  }
                  {
                    const uint32_t a0 = deq_imm<8>(wa.x), a1 = deq_imm<8>(wb.x);
                    const uint32_t a2 = deq_imm<12>(wa.x), a3 = deq_imm<12>(wb.x);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                      mma_bf16_m16n8k16(dg[m][nt], a0, a1, a2, a3, xb[nt][0].z, xb[nt][0].w);
                  }
                  {
                    const uint32_t a0 = deq_imm<0>(wa.y), a1 = deq_imm<0>(wb.y);
                    const uint32_t a2 = deq_imm<4>(wa.y), a3 = deq_imm<4>(wb.y);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                      mma_bf16_m16n8k16(dg[m][nt], a0, a1, a2, a3, xb[nt][1].x, xb[nt][1].y);
                  }
                  {
                    const uint32_t a0 = deq_imm<8>(wa.y), a1 = deq_imm<8>(wb.y);
                    const uint32_t a2 = deq_imm<12>(wa.y), a3 = deq_imm<12>(wb.y);
#pragma unroll
                    for (int nt = 0; nt < NT; ++nt)
                      mma_bf16_m16n8k16(dg[m][nt], a0, a1, a2, a3, xb[nt][1].z, xb[nt][1].w);
                  }
                }
              }
              if (GPB <= 4 && slot == GPB - 1)
                fixup_multi<NMAT, NT, TT, WK, WM, FULLQ>(acc, dg, xsum, sraw, sc_stride, wk, wm, g, tig,
                                                         (qi + bq) * 4 + j - (GPB - 1), nq_w, ngroups);
            }
            // refill this pipeline slot with the quad two steps ahead
            if (qi + bq + 2 < nq_w) {
              load_quad<NMAT, FULLQ>(wbuf[bq], wp, (quad + 2 * WK) * 4, ngroups);
#pragma unroll
              for (int m = 0; m < NMAT; ++m) {
                wp[m][0] += WK * 32;
                wp[m][1] += WK * 32;
              }
            }
          }
        }
        if (GPB == 8)
          fixup_multi<NMAT, NT, TT, WK, WM, FULLQ>(acc, dg, xsum, sraw, sc_stride, wk, wm, g, tig, qi * 4, nq_w,
                                                   ngroups);
      }

      // ---- (5) reduce the K-split across warps (fixed order)
      if (WK > 1) {
        __syncthreads();  // every warp is done reading the staged rows; reuse their space
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
        // ---- (6) fold the multiplexed columns back onto their tokens (fixed order), then the epilogue
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
                v = swiglu_epilogue(p.epilogue, acc[0][nt][j], acc[NMAT - 1][nt][j]);
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
  int nt, tt, wk, wm;
};

static QmmChoice choose_config(int ngroups, int rows_hint) {
  QmmChoice c;
  c.nt = rows_hint <= 8 ? 1 : (rows_hint <= 16 ? 2 : 4);
  c.tt = rows_hint <= 1 ? 1 : (rows_hint <= 2 ? 2 : (rows_hint <= 4 ? 4 : 8));
  const int nq = (ngroups + 3) / 4;
  if (nq >= 8) {
    c.wk = 4;
    c.wm = 1;
  } else if (nq >= 4) {
    c.wk = 2;
    c.wm = 2;
  } else {
    c.wk = 1;
    c.wm = 4;
  }
  return c;
}

template <int NMAT, int NT, int TT, int WK, int WM, bool FULLQ>
static int launch_full(const QmmParams& p, int max_groups, cudaStream_t st) {
  auto kern = qmm_affine_kernel<NMAT, NT, TT, WK, WM, FULLQ>;
  QmmSmem lay = qmm_smem(p.K, p.ngroups, p.rs, 8 * NT, NMAT, WM, WK, NT);
  if (lay.total > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, lay.total);
    if (e != cudaSuccess)
      return fail(ZMOE_ERR_CUDA, "qmm: shared memory of %d bytes refused: %s", lay.total, cudaGetErrorString(e));
  }
  dim3 grid((p.N + 16 * WM - 1) / (16 * WM), max_groups);
  launch_pdl(kern, grid, dim3(32 * WK * WM), (size_t)lay.total, st, p);
  return check_launch("qmm_affine_kernel");
}

template <int NMAT, int NT, int TT, int WK, int WM>
static int launch_cfg(const QmmParams& p, int max_groups, cudaStream_t st) {
  if ((p.ngroups & 3) == 0) return launch_full<NMAT, NT, TT, WK, WM, true>(p, max_groups, st);
  return launch_full<NMAT, NT, TT, WK, WM, false>(p, max_groups, st);
}

template <int NMAT, int WK, int WM>
static int launch_tokens(const QmmParams& p, const QmmChoice& c, int max_groups, cudaStream_t st) {
  if (c.nt == 1) {
    switch (c.tt) {
      case 1: return launch_cfg<NMAT, 1, 1, WK, WM>(p, max_groups, st);
      case 2: return launch_cfg<NMAT, 1, 2, WK, WM>(p, max_groups, st);
      case 4: return launch_cfg<NMAT, 1, 4, WK, WM>(p, max_groups, st);
      default: return launch_cfg<NMAT, 1, 8, WK, WM>(p, max_groups, st);
    }
  }
  if (c.nt == 2) return launch_cfg<NMAT, 2, 8, WK, WM>(p, max_groups, st);
  return launch_cfg<NMAT, 4, 8, WK, WM>(p, max_groups, st);
}

template <int NMAT>
static int launch_nmat(const QmmParams& p, const QmmChoice& c, int max_groups, cudaStream_t st) {
  if (c.wk == 4 && c.wm == 1) return launch_tokens<NMAT, 4, 1>(p, c, max_groups, st);
  if (c.wk == 2 && c.wm == 2) return launch_tokens<NMAT, 2, 2>(p, c, max_groups, st);
  if (c.wk == 1 && c.wm == 4) return launch_tokens<NMAT, 1, 4>(p, c, max_groups, st);
  return fail(ZMOE_ERR_UNSUPPORTED, "qmm: no kernel for wk=%d wm=%d", c.wk, c.wm);
}

int qmm_launch(int nmat, const void* x, int x_rows, int ldx, const uint32_t* const* w, const void* const* s,
               const void* const* b, int E, int N, int K, int group_size, int qmode, const void* plan, int rows,
               int rows_hint, void* out, int epilogue, int x_by_dst, void* stream, const char* who) {
  ZMOE_REQUIRE(x && plan && out, ZMOE_ERR_SHAPE, "%s: null pointer", who);
  for (int m = 0; m < nmat; ++m)
    ZMOE_REQUIRE(w[m] && s[m], ZMOE_ERR_SHAPE, "%s: null weight or scale pointer", who);
  ZMOE_REQUIRE(E >= 1 && N >= 1 && K >= 1 && rows >= 0 && x_rows >= 0, ZMOE_ERR_SHAPE,
               "%s: bad sizes E=%d N=%d K=%d rows=%d", who, E, N, K, rows);
  ZMOE_REQUIRE(qmode == ZMOE_Q_AFFINE4 || qmode == ZMOE_Q_MXFP4, ZMOE_ERR_UNSUPPORTED,
               "%s: quantisation mode %d is not supported", who, qmode);
  const bool mx = (qmode == ZMOE_Q_MXFP4);
  ZMOE_REQUIRE(group_size == (mx ? 32 : 64), ZMOE_ERR_UNSUPPORTED, "%s: group_size=%d (affine: 64, mxfp4: 32)", who,
               group_size);
  ZMOE_REQUIRE(K % 64 == 0, ZMOE_ERR_SHAPE, "%s: K=%d must be a multiple of 64", who, K);
  for (int m = 0; m < nmat; ++m) ZMOE_REQUIRE(mx || b[m], ZMOE_ERR_SHAPE, "%s: affine mode needs biases", who);
  ZMOE_REQUIRE(ldx >= K && ldx % 8 == 0 && ((uintptr_t)x % 16) == 0, ZMOE_ERR_ALIGN,
               "%s: x rows must be 16-byte aligned (ldx=%d)", who, ldx);
  for (int m = 0; m < nmat; ++m)
    ZMOE_REQUIRE(((uintptr_t)w[m] % 8) == 0 && ((uintptr_t)s[m] % 8) == 0 && (mx || ((uintptr_t)b[m] % 8) == 0),
                 ZMOE_ERR_ALIGN, "%s: packed weights, scales and biases must be 8-byte aligned", who);
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
  p.x_by_dst = x_by_dst & 1;
  p.late_wait = (x_by_dst & 2) ? 1 : 0;

  if (mx) {
    int mg = rows < E ? rows : E;
    if (mg > 65535) mg = 65535;
    return qmm_mxfp4_launch(p, nmat, rows_hint, mg, (cudaStream_t)stream, who);
  }
  // From about eight rows per expert on average the contraction is dense enough for the 5th-generation tensor
  // cores (tcgen05, accumulator in tensor memory): the expert's codes are expanded once per 128-row tile and
  // reused by up to 128 token rows.
  if ((long long)rows >= 8ll * E && rows_hint >= 16 && (p.ngroups & 3) == 0 && E <= 1024 && ((uintptr_t)w[0] % 16) == 0 &&
      (nmat == 1 || ((uintptr_t)w[1] % 16) == 0)) {
    int mg = rows < E ? rows : E;
    if (mg > 65535) mg = 65535;
    p.rs = 0;
    return qmm_tc_launch(p, nmat, rows_hint, mg, (cudaStream_t)stream, who);
  }
  // The token slots of a pass are sized for twice the average task, not for the largest possible one: with
  // top-k routing most experts see far fewer rows than there are tokens, and a task with more rows takes
  // another pass over its (L2-resident) weights.
  long long typical = (2ll * rows + E - 1) / E;
  if (typical > rows_hint) typical = rows_hint;
  if (typical < 1) typical = 1;
  QmmChoice c = choose_config(p.ngroups, (int)typical);
  // keep the staged token rows within ~96 KB so that several CTAs share an SM
  int rs = (c.nt == 1) ? c.tt : 8 * c.nt;
  while (rs > 1 && (size_t)rs * qmm_xs_stride(K) > 96 * 1024) rs = rs / 2;
  if (rs < 8) {
    c.nt = 1;
    c.tt = rs >= 4 ? 4 : (rs >= 2 ? 2 : 1);
    rs = c.tt;
  } else {
    c.tt = 8;
    c.nt = rs >= 32 ? 4 : (rs >= 16 ? 2 : 1);
    rs = 8 * c.nt;
  }
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
  ZMOE_REQUIRE(swiglu_mode == ZMOE_SWIGLU_CPU || swiglu_mode == ZMOE_SWIGLU_PER_OP ||
                   (swiglu_mode == ZMOE_SWIGLU_FP32 && qmode == ZMOE_Q_AFFINE4),
               ZMOE_ERR_UNSUPPORTED,
               "zmoe_gather_qmm_swiglu: swiglu_mode %d", swiglu_mode);
  const uint32_t* w[2] = {gate_w, up_w};
  const void* s[2] = {gate_scales, up_scales};
  const void* b[2] = {gate_biases, up_biases};
  return qmm_launch(2, x, x_rows, ldx, w, s, b, E, N, K, group_size, qmode, plan, rows, rows_hint, out,
                    swiglu_mode == ZMOE_SWIGLU_CPU ? 1 : (swiglu_mode == ZMOE_SWIGLU_PER_OP ? 2 : 3), 0, stream,
                    "zmoe_gather_qmm_swiglu");
}

int zmoe_gather_qmm(const void* x, int x_rows, int ldx, const uint32_t* w_, const void* scales, const void* biases,
                    int E, int N, int K, int group_size, int qmode, const void* plan, int rows, int rows_hint,
                    int x_by_output_row, void* out, void* stream) {
  const uint32_t* w[2] = {w_, nullptr};
  const void* s[2] = {scales, nullptr};
  const void* b[2] = {biases, nullptr};
  return qmm_launch(1, x, x_rows, ldx, w, s, b, E, N, K, group_size, qmode, plan, rows, rows_hint, out, 0,
                    x_by_output_row, stream, "zmoe_gather_qmm");
}

}  // extern "C"
