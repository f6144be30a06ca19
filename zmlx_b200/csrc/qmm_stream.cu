// Persistent, bulk-copy pipelined form of the token-grouped 4-bit expert matmul.
//
// Same result as qmm.cu (per-group fix-up in fp32, column-multiplexed groups for small
// token counts) with two changes: the codes go to the tensor cores as FP8 (see the FP8
// operand path below), and bytes reach the math through shared-memory rings.  Each CTA is persistent and owns a contiguous
// range of (expert task, 16-row tile) items.  One producer warp walks that range ahead
// of the math and feeds three shared-memory rings with cp.async.bulk copies that
// complete on mbarriers:
//   * weight stages: 32 row-chunks of up to 512 contiguous bytes (4 quads of groups)
//     each, one per lane, into rows padded to a bank-conflict-free stride;
//   * the scales and biases of an item (contiguous per tile);
//   * the token rows of an (expert, pass), which the consumer threads then permute in
//     place to the B-fragment order and reduce to per-group sums.
// Eight consumer warps (4-way K split x {gate, up} or x 2 row tiles) wait on "full"
// barriers, compute from shared memory and release stages through "empty" barriers.
// HBM therefore sees long sequential bursts with ~70 KB in flight per CTA, held by no
// registers, and the serial latency chain task -> row ids -> token rows -> weights is
// walked by the producer while the consumers work on earlier items.
//
// Every wait is bounded: after kSpinLimit failed polls a thread records the fact in a
// status word, sets a CTA-wide abort flag and stops waiting (results are then
// meaningless, but the kernel terminates and the context stays usable).
#include <cstdlib>

#include "qmm_common.cuh"

namespace zmoe {

constexpr int kMaxStages = 8;
constexpr int kCW = 8;                   // consumer warps
constexpr int kPW = 4;                   // producer warps: a warp's bulk copies are accepted one by one,
                                         // so several warps issue the stages round-robin
constexpr int kThreads = 32 * (kCW + kPW);
constexpr int kCQ = 4;                   // quads (of 4 groups) per weight stage: 512 bytes per row
constexpr int kRowStride = kCQ * 128 + 32;  // == 32 (mod 128): conflict-free 8-byte fragment loads
constexpr int kSpinLimit = 1 << 20;  // non-blocking polls (~20 ms) before a wait gives up

__device__ int g_stream_status = 0;

struct StreamSmem {
  int bars, abort_flag, stages, stage_bytes, sc, sc_bytes, x, x_bytes, xsum, xsum_bytes, red, zero, dscale, amax, total;
};

__host__ __device__ inline StreamSmem stream_smem(int K, int ngroups, int nmat, int rs, int nt, int nstages) {
  StreamSmem m;
  const int wm = (nmat == 2) ? 1 : 2;
  int a = 0;
  m.bars = a;
  a += (2 * kMaxStages + 8) * 8;
  m.abort_flag = a;
  a += 16;
  a = (a + 127) & ~127;
  m.stages = a;
  m.stage_bytes = nmat * wm * 16 * kRowStride;
  a += nstages * m.stage_bytes;
  m.sc = a;
  m.sc_bytes = (nmat * 2 * 16 * wm * ngroups * 2 + 15) & ~15;
  a += 2 * m.sc_bytes;
  m.x = a;
  m.x_bytes = (rs * (K * 2 + 16) + 15) & ~15;
  a += 2 * m.x_bytes;
  m.xsum = a;
  m.xsum_bytes = (ngroups * 8 * nt * 4 + 15) & ~15;
  a += 2 * m.xsum_bytes;
  m.red = a;
  a += kCW * 32 * nt * 4 * 4;
  m.zero = a;
  a += 32;
  m.dscale = a;  // per x buffer: 32 floats, 2^9 / (token scale)
  a += 2 * 32 * 4;
  m.amax = a;  // kCW x 32 partial maxima of |x| (as bf16 bit patterns)
  a += kCW * 32 * 4;
  m.total = a;
  return m;
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try(uint32_t bar, int parity) {
  uint32_t ok;
  asm volatile(
      "{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
      : "=r"(ok)
      : "r"(bar), "r"(parity)
      : "memory");
  return ok != 0;
}
// Bounded wait; gives up (and makes every later wait of the CTA return at once) after kSpinLimit polls.
__device__ __forceinline__ void mbar_wait(uint32_t bar, int parity, volatile int* abort_flag) {
  if (*abort_flag) return;
  for (int i = 0; i < kSpinLimit; ++i) {
    if (mbar_try(bar, parity)) return;
    if ((i & 1023) == 1023 && *abort_flag) return;
  }
  *abort_flag = 1;
  atomicExch(&g_stream_status, 1);
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, int bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCW * 32) : "memory"); }


// ---- FP8 operand path.  A 4-bit code q in the low nibble of a byte IS the e4m3 number q * 2^-9
// (0..7 are subnormals, 8..15 have exponent field 1 and the same spacing), so two ANDs and a
// shift turn a packed word into two A registers of mma.m16n8k32.e4m3 with no conversion at all.
// The bf16 activations are split exactly into two e4m3 pieces (hi + lo, 4 significant bits each)
// after a per-token power-of-two scale that puts |x|max in [128, 256); the tensor core
// accumulates both pieces in fp32.
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  uint16_t lo, hi;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(lo) : "f"(a), "f"(b));
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %2, %1;" : "=h"(hi) : "f"(c), "f"(d));
  return (uint32_t)lo | ((uint32_t)hi << 16);
}
__device__ __forceinline__ void unpack_e4m3x4(uint32_t v, float (&out)[4]) {
  uint32_t h01, h23;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h01) : "h"((uint16_t)(v & 0xffffu)));
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h23) : "h"((uint16_t)(v >> 16)));
  out[0] = __half2float(__ushort_as_half((unsigned short)(h01 & 0xffffu)));
  out[1] = __half2float(__ushort_as_half((unsigned short)(h01 >> 16)));
  out[2] = __half2float(__ushort_as_half((unsigned short)(h23 & 0xffffu)));
  out[3] = __half2float(__ushort_as_half((unsigned short)(h23 >> 16)));
}
__device__ __forceinline__ void mma_e4m3_m16n8k32(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                  uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k32.row.col.f32.e4m3.e4m3.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Fix-up of a block of 8/TT multiplexed groups for the FP8 path: acc += s * (D * dscale[token]) + b * sum(x).
template <int NT, int TT>
__device__ __forceinline__ void fixup_fp8(float (&acc)[NT][4], const float (&dg)[NT][4], const float* xsum,
                                          const float* dscale, const unsigned char* srow, const unsigned char* brow,
                                          int sc_stride, int wk, int tig, int gi0, int nq_w) {
  constexpr int RC = 8 * NT;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col = 2 * tig + c;
    const int gi_c = gi0 + ((TT == 8) ? 0 : col / TT);
    const int G_c = (wk + (gi_c >> 2) * 4) * 4 + (gi_c & 3);
    if ((gi_c >> 2) < nq_w) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const float sv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(srow + h * 8 * sc_stride + G_c * 2));
        const float bv = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(brow + h * 8 * sc_stride + G_c * 2));
#pragma unroll
        for (int nt = 0; nt < NT; ++nt) {
          const int tok = (TT == 8) ? nt * 8 + col : col % TT;
          const float X = xsum[G_c * RC + tok];
          acc[nt][h * 2 + c] = fmaf(sv * dscale[tok], dg[nt][h * 2 + c], fmaf(bv, X, acc[nt][h * 2 + c]));
        }
      }
    }
  }
}

template <int NMAT, int NT, int TT>
__global__ void __launch_bounds__(kThreads, 1) qmm_stream_kernel(const QmmParams p, int n_tiles, int nstages, int dbg) {
  static_assert(NT == 1 || TT == 8, "token tiles beyond the first are full");
  constexpr int WM = (NMAT == 2) ? 1 : 2;
  constexpr int GPB = 8 / TT;
  constexpr int RC = 8 * NT;
  constexpr int CT = kCW * 32;  // consumer threads
  constexpr int NCH = (NT == 1) ? 4 : 2;  // accumulation chains: hides the latency of dependent mmas
  extern __shared__ __align__(128) unsigned char smem[];

  pdl_wait();
  pdl_trigger();
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;
  const int K = p.K, N = p.N, ngroups = p.ngroups;
  const int K8 = K >> 3;
  const int nq = ngroups >> 2;  // the fast path has ngroups % 4 == 0
  const int nchunks = (nq + kCQ - 1) / kCQ;
  const int xs_stride = K * 2 + 16;
  const StreamSmem lay = stream_smem(K, ngroups, NMAT, p.rs, NT, nstages);
  const uint32_t bars = smem_u32(smem + lay.bars);
  // barrier slots: full[s] = s, empty[s] = kMaxStages + s, then scfull[2], scempty[2], xfull[2], xempty[2]
  const uint32_t bar_full = bars, bar_empty = bars + kMaxStages * 8;
  const uint32_t bar_scfull = bars + 2 * kMaxStages * 8, bar_scempty = bar_scfull + 16;
  const uint32_t bar_xfull = bar_scfull + 32, bar_xempty = bar_scfull + 48;
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem + lay.abort_flag);

  if (tid == 0) {
    for (int s = 0; s < nstages; ++s) {
      mbar_init(bar_full + s * 8, 1);
      mbar_init(bar_empty + s * 8, kCW);
    }
    for (int s = 0; s < 2; ++s) {
      mbar_init(bar_scfull + s * 8, 1);
      mbar_init(bar_scempty + s * 8, kCW);
      mbar_init(bar_xfull + s * 8, 1);
      mbar_init(bar_xempty + s * 8, kCW);
    }
    *abort_flag = 0;
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (tid < 8) reinterpret_cast<uint32_t*>(smem + lay.zero)[tid] = 0u;
  __syncthreads();

  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  const int n_active = pv.hdr[0];
  const int total = n_active * n_tiles;
  const int per = (total + gridDim.x - 1) / gridDim.x;
  const int it0 = blockIdx.x * per;
  const int it1 = min(total, it0 + per);
  if (it0 >= it1) return;
  const int a_first = it0 / n_tiles;

  int n_stage = 0, n_sc = 0, n_x = 0;  // running use counts of the three rings

  if (wid >= kCW) {
    // ------------------------------------------------------------------ producer warps
    const int pw = wid - kCW;
    for (int a = a_first; a * n_tiles < it1; ++a) {
      const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + a);
      const int e = task.x, off = task.y, cnt = task.z;
      const int nt_lo = max(it0, a * n_tiles) - a * n_tiles;
      const int nt_hi = min(it1, (a + 1) * n_tiles) - a * n_tiles;
      for (int rc = 0; rc < cnt; rc += p.rs) {
        const int nrow = min(p.rs, cnt - rc);
        if (pw == 0) {  // token rows of this (task, pass)
          const int xb = n_x & 1;
          if (n_x >= 2) mbar_wait(bar_xempty + xb * 8, ((n_x >> 1) - 1) & 1, abort_flag);
          if (lane == 0) mbar_expect_tx(bar_xfull + xb * 8, nrow * K * 2);
          __syncwarp();
          for (int t = lane; t < nrow; t += 32) {
            const int src = p.x_by_dst ? pv.row_dst[off + rc + t] : pv.row_src[off + rc + t];
            bulk_g2s(smem_u32(smem + lay.x + xb * lay.x_bytes + t * xs_stride), p.x + (size_t)src * p.ldx, K * 2,
                     bar_xfull + xb * 8);
          }
        }
        ++n_x;
        for (int nt = nt_lo; nt < nt_hi; ++nt) {
          if (pw == 0) {  // scales and biases of the item: one contiguous block per array
            const int sb = n_sc & 1;
            if (n_sc >= 2) mbar_wait(bar_scempty + sb * 8, ((n_sc >> 1) - 1) & 1, abort_flag);
            const int arr_bytes = 16 * WM * ngroups * 2;
            if (lane == 0) mbar_expect_tx(bar_scfull + sb * 8, NMAT * 2 * arr_bytes);
            __syncwarp();
            if (lane < NMAT * 2) {
              const __nv_bfloat16* base = (lane & 1) ? p.b[lane >> 1] : p.s[lane >> 1];
              bulk_g2s(smem_u32(smem + lay.sc + sb * lay.sc_bytes + lane * arr_bytes),
                       base + ((size_t)e * N + (size_t)nt * 16 * WM) * ngroups, arr_bytes, bar_scfull + sb * 8);
            }
          }
          ++n_sc;
          // weight stages: lane r copies row r of the 32-row stage
          const int rs_idx = lane >> 4;  // gate/up (NMAT == 2) or row tile (NMAT == 1)
          const uint32_t* wsrc = ((NMAT == 2 && rs_idx) ? p.w[1] : p.w[0]) +
                                 ((size_t)e * N + (size_t)nt * 16 * WM + (NMAT == 2 ? 0 : rs_idx * 16) + (lane & 15)) * K8;
          for (int ch = 0; ch < nchunks; ++ch, ++n_stage) {
            if ((n_stage % kPW) != pw) continue;
            const int s = n_stage % nstages;
            const int round = n_stage / nstages;
            if (round > 0) mbar_wait(bar_empty + s * 8, (round - 1) & 1, abort_flag);
            const int qn = min(kCQ, nq - ch * kCQ);
            if (lane == 0) mbar_expect_tx(bar_full + s * 8, 32 * qn * 128);
            __syncwarp();
            bulk_g2s(smem_u32(smem + lay.stages + s * lay.stage_bytes + lane * kRowStride), wsrc + ch * (kCQ * 32),
                     qn * 128, bar_full + s * 8);
          }
        }
      }
    }
    return;
  }

  // -------------------------------------------------------------------- consumer warps
  const int wk = wid & 3;
  const int rs_idx = wid >> 2;                     // stage row block: matrix (NMAT == 2) or row tile (NMAT == 1)
  const int mat = (NMAT == 2) ? rs_idx : 0;
  const int wm = (NMAT == 2) ? 0 : rs_idx;
  const int g = lane >> 2;
  const int tig = lane & 3;
  const int slot_g = g / TT;
  const int tok_g = g % TT;
  const int nq_w = (nq > wk) ? (nq - wk + 3) / 4 : 0;  // chunks in which this warp has a quad
  float* red = reinterpret_cast<float*>(smem + lay.red);
  const uint32_t kMask = 0x0F0F0F0Fu;

  for (int a = a_first; a * n_tiles < it1; ++a) {
    const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + a);
    const int off = task.y, cnt = task.z;
    const int nt_lo = max(it0, a * n_tiles) - a * n_tiles;
    const int nt_hi = min(it1, (a + 1) * n_tiles) - a * n_tiles;
    for (int rc = 0; rc < cnt; rc += p.rs) {
      const int nrow = min(p.rs, cnt - rc);
      // ---- token rows: wait for the copies, permute 8-element blocks to (0,4,1,5,2,6,3,7) in place, group sums
      const int xb = n_x & 1;
      unsigned char* xs = smem + lay.x + xb * lay.x_bytes;
      float* xsum = reinterpret_cast<float*>(smem + lay.xsum + xb * lay.xsum_bytes);
      mbar_wait(bar_xfull + xb * 8, (n_x >> 1) & 1, abort_flag);
      float* dscale = reinterpret_cast<float*>(smem + lay.dscale) + xb * 32;
      int* amax_s = reinterpret_cast<int*>(smem + lay.amax);
      // pass 1: |x|max of every token row (bf16 bit patterns compare like integers once the sign is cleared)
      for (int t = 0; t < nrow; ++t) {
        uint32_t m = 0;
        for (int blk = tid; blk < K8; blk += CT) {
          const uint4 v = *reinterpret_cast<const uint4*>(xs + t * xs_stride + blk * 16);
          const uint32_t w4[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            m = max(m, w4[i] & 0x7fffu);
            m = max(m, (w4[i] >> 16) & 0x7fffu);
          }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) m = max(m, __shfl_xor_sync(0xffffffffu, m, o));
        if (lane == 0) amax_s[wid * 32 + t] = (int)m;
      }
      consumer_sync();
      // pass 2: split into two e4m3 pieces in B-fragment order {even hi, odd hi, even lo, odd lo}, group sums
      for (int t = 0; t < nrow; ++t) {
        uint32_t m = 0;
#pragma unroll
        for (int w8 = 0; w8 < kCW; ++w8) m = max(m, (uint32_t)amax_s[w8 * 32 + t]);
        // scale = 2^(7 - floor(log2 amax)): exponent field 261 - E, kept inside the normal range
        int ef = 261 - (int)(m >> 7);
        ef = (m == 0) ? 127 : min(max(ef, 2), 252);
        const float scale = __uint_as_float((uint32_t)ef << 23);
        if (tid == 0) dscale[t] = 512.0f * __uint_as_float((uint32_t)(254 - ef) << 23);
        for (int b0 = wid * 32; b0 < K8; b0 += CT) {
          const int blk = b0 + lane;
          float f[8] = {0, 0, 0, 0, 0, 0, 0, 0};
          if (blk < K8) {
            uint4* px = reinterpret_cast<uint4*>(xs + t * xs_stride + blk * 16);
            const uint4 v = *px;
            f[0] = bf16_bits_to_float(v.x & 0xffffu);
            f[1] = bf16_bits_to_float(v.x >> 16);
            f[2] = bf16_bits_to_float(v.y & 0xffffu);
            f[3] = bf16_bits_to_float(v.y >> 16);
            f[4] = bf16_bits_to_float(v.z & 0xffffu);
            f[5] = bf16_bits_to_float(v.z >> 16);
            f[6] = bf16_bits_to_float(v.w & 0xffffu);
            f[7] = bf16_bits_to_float(v.w >> 16);
            uint4 o;
            o.x = pack_e4m3x4(f[0] * scale, f[2] * scale, f[4] * scale, f[6] * scale);
            o.y = pack_e4m3x4(f[1] * scale, f[3] * scale, f[5] * scale, f[7] * scale);
            float he[4], ho[4];
            unpack_e4m3x4(o.x, he);
            unpack_e4m3x4(o.y, ho);
            o.z = pack_e4m3x4(f[0] * scale - he[0], f[2] * scale - he[1], f[4] * scale - he[2], f[6] * scale - he[3]);
            o.w = pack_e4m3x4(f[1] * scale - ho[0], f[3] * scale - ho[1], f[5] * scale - ho[2], f[7] * scale - ho[3]);
            *px = o;
          }
          float part = ((f[0] + f[1]) + (f[2] + f[3])) + ((f[4] + f[5]) + (f[6] + f[7]));
          part += __shfl_xor_sync(0xffffffffu, part, 1);
          part += __shfl_xor_sync(0xffffffffu, part, 2);
          part += __shfl_xor_sync(0xffffffffu, part, 4);
          if (blk < K8 && (lane & 7) == 0) xsum[(blk >> 3) * RC + t] = part;
        }
      }
      if (nrow < RC) {
        for (int i = tid; i < ngroups * RC; i += CT)
          if ((i % RC) >= nrow) xsum[i] = 0.0f;
      }
      consumer_sync();
      ++n_x;

      const int xlane = lay.x + xb * lay.x_bytes + ((TT == 8) ? g : tok_g) * xs_stride + tig * 32;
      const bool tok_ok = ((TT == 8) ? g : tok_g) < nrow;

      for (int nt = nt_lo; nt < nt_hi; ++nt) {
        const int sb = n_sc & 1;
        mbar_wait(bar_scfull + sb * 8, (n_sc >> 1) & 1, abort_flag);
        const unsigned char* sc_base = smem + lay.sc + sb * lay.sc_bytes;
        const int arr_bytes = 16 * WM * ngroups * 2;
        const unsigned char* srow = sc_base + (mat * 2 + 0) * arr_bytes + (wm * 16 + g) * ngroups * 2;
        const unsigned char* brow = sc_base + (mat * 2 + 1) * arr_bytes + (wm * 16 + g) * ngroups * 2;

        float acc[NT][4];
        float dg[NT][4];
        float dgc[NCH][NT][4];  // independent mma accumulation chains, summed at the fix-up
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            acc[i][j] = 0.0f;
            dg[i][j] = 0.0f;
#pragma unroll
            for (int c = 0; c < NCH; ++c) dgc[c][i][j] = 0.0f;
          }

        for (int ch = 0; ch < nchunks; ++ch) {
          const int s = n_stage % nstages;
          mbar_wait(bar_full + s * 8, (n_stage / nstages) & 1, abort_flag);
          const int quad = ch * kCQ + wk;
          if (quad < nq && !(dbg & 1)) {
            const unsigned char* wlane =
                smem + lay.stages + s * lay.stage_bytes + (rs_idx * 16 + g) * kRowStride + wk * 128 + tig * 8;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              // position of this group in its fix-up block of GPB groups
              const int slot = (GPB == 8) ? ((ch & 1) * 4 + j) : (j % GPB);
              if ((GPB == 8) ? (slot == 0) : (j % GPB == 0)) {
#pragma unroll
                for (int c = 0; c < NCH; ++c)
#pragma unroll
                  for (int i = 0; i < NT; ++i)
#pragma unroll
                    for (int jj = 0; jj < 4; ++jj) dgc[c][i][jj] = 0.0f;
              }
              uint4 xbf[NT][2];
#pragma unroll
              for (int i = 0; i < NT; ++i) {
                const bool mine = (TT == 8) ? (i * 8 + g < nrow) : (tok_ok && slot_g == slot);
                const int xo = mine ? (xlane + i * 8 * xs_stride + quad * 512 + j * 128) : lay.zero;
                xbf[i][0] = *reinterpret_cast<const uint4*>(smem + xo);
                xbf[i][1] = *reinterpret_cast<const uint4*>(smem + xo + 16);
              }
              const uint2 wa = *reinterpret_cast<const uint2*>(wlane + j * 32);
              const uint2 wb = *reinterpret_cast<const uint2*>(wlane + 8 * kRowStride + j * 32);
              {
                const uint32_t a0 = wa.x & kMask, a1 = wb.x & kMask;
                const uint32_t a2 = (wa.x >> 4) & kMask, a3 = (wb.x >> 4) & kMask;
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                  mma_e4m3_m16n8k32(dgc[0][i], a0, a1, a2, a3, xbf[i][0].x, xbf[i][0].y);
                  mma_e4m3_m16n8k32(dgc[1][i], a0, a1, a2, a3, xbf[i][0].z, xbf[i][0].w);
                }
              }
              {
                const uint32_t a0 = wa.y & kMask, a1 = wb.y & kMask;
                const uint32_t a2 = (wa.y >> 4) & kMask, a3 = (wb.y >> 4) & kMask;
#pragma unroll
                for (int i = 0; i < NT; ++i) {
                  mma_e4m3_m16n8k32(dgc[NCH == 4 ? 2 : 0][i], a0, a1, a2, a3, xbf[i][1].x, xbf[i][1].y);
                  mma_e4m3_m16n8k32(dgc[NCH == 4 ? 3 : 1][i], a0, a1, a2, a3, xbf[i][1].z, xbf[i][1].w);
                }
              }
              if (GPB <= 4 && (j % GPB) == GPB - 1) {
#pragma unroll
                for (int i = 0; i < NT; ++i)
#pragma unroll
                  for (int jj = 0; jj < 4; ++jj)
                    dg[i][jj] = (NCH == 4) ? (dgc[0][i][jj] + dgc[1][i][jj]) + (dgc[2][i][jj] + dgc[3][i][jj])
                                           : dgc[0][i][jj] + dgc[1][i][jj];
                fixup_fp8<NT, TT>(acc, dg, xsum, dscale, srow, brow, ngroups * 2, wk, tig, ch * 4 + j - (GPB - 1),
                                  nq_w);
              }
            }
          }
          __syncwarp();
          if (lane == 0) mbar_arrive(bar_empty + s * 8);
          ++n_stage;
          // a block of 8 multiplexed groups spans two chunks
          if (GPB == 8 && ((ch & 1) == 1 || ch == nchunks - 1)) {
#pragma unroll
            for (int i = 0; i < NT; ++i)
#pragma unroll
              for (int jj = 0; jj < 4; ++jj)
                dg[i][jj] = (NCH == 4) ? (dgc[0][i][jj] + dgc[1][i][jj]) + (dgc[2][i][jj] + dgc[3][i][jj])
                                       : dgc[0][i][jj] + dgc[1][i][jj];
            fixup_fp8<NT, TT>(acc, dg, xsum, dscale, srow, brow, ngroups * 2, wk, tig, (ch & ~1) * 4, nq_w);
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(bar_scempty + sb * 8);
        ++n_sc;

        if (dbg & 4) continue;
        // ---- gather the K split (and the second matrix) in the first warp of each row block, fixed order
        consumer_sync();  // the previous item's readers are done with the buffer
        float* mine_red = red + (wid * 32 + lane) * (NT * 4);
#pragma unroll
        for (int i = 0; i < NT; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) mine_red[i * 4 + j] = acc[i][j];
        consumer_sync();
        const bool leader = (wk == 0) && (NMAT == 1 || mat == 0);
        if (leader) {
          float accu[NT][4];
#pragma unroll
          for (int i = 0; i < NT; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j) accu[i][j] = 0.0f;
#pragma unroll
          for (int mm = 0; mm < NMAT; ++mm) {
#pragma unroll
            for (int o = 0; o < 4; ++o) {
              if (mm == 0 && o == 0) continue;
              const int ow = (NMAT == 2) ? (mm * 4 + o) : (wm * 4 + o);
              const float* other = red + (ow * 32 + lane) * (NT * 4);
#pragma unroll
              for (int i = 0; i < NT; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                  if (mm == 0)
                    acc[i][j] += other[i * 4 + j];
                  else
                    accu[i][j] += other[i * 4 + j];
                }
            }
          }
          if (TT < 8) {  // fold the multiplexed columns back onto their tokens
#pragma unroll
            for (int mm = 0; mm < NMAT; ++mm) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                float v0 = mm ? accu[0][h * 2] : acc[0][h * 2];
                float v1 = mm ? accu[0][h * 2 + 1] : acc[0][h * 2 + 1];
                if (TT == 1) {
                  v0 += v1;
                  v1 = 0.0f;
                }
                if (TT <= 2) v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
                v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
                if (TT > 1) {
                  if (TT <= 2) v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
                  v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
                }
                if (mm) {
                  accu[0][h * 2] = v0;
                  accu[0][h * 2 + 1] = v1;
                } else {
                  acc[0][h * 2] = v0;
                  acc[0][h * 2 + 1] = v1;
                }
              }
            }
          }
#pragma unroll
          for (int i = 0; i < NT; ++i) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = 2 * tig + (j & 1);
              const int t = (TT == 8) ? i * 8 + col : col;
              const int n = nt * 16 * WM + wm * 16 + g + ((j >> 1) ? 8 : 0);
              const bool writer = (TT == 8) || (col < TT);
              if (writer && t < nrow) {
                float v;
                if (NMAT == 2) {
                  v = (p.epilogue == 2) ? swiglu_per_op(acc[i][j], accu[i][j]) : swiglu_cpu_contract(acc[i][j], accu[i][j]);
                } else {
                  v = acc[i][j];
                }
                const int dst = pv.row_dst[task.y + rc + t];
                p.out[(size_t)dst * p.ldo + n] = __float2bfloat16_rn(v);
              }
            }
          }
        }
      }
      // this (task, pass) is done with its token rows: order the in-place writes before the next bulk copy
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
      __syncwarp();
      if (lane == 0) mbar_arrive(bar_xempty + xb * 8);
    }
    (void)off;
  }
}

// ------------------------------------------------------------------ host side

template <int NMAT, int NT, int TT>
static int launch_stream(const QmmParams& p, int n_tiles, int max_items, int nstages, int smem_bytes, cudaStream_t st) {
  auto kern = qmm_stream_kernel<NMAT, NT, TT>;
  static int sms = 0;
  if (sms == 0) {
    int dev = 0;
    cudaGetDevice(&dev);
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
  }
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes);
  if (e != cudaSuccess)
    return fail(ZMOE_ERR_CUDA, "qmm_stream: shared memory of %d bytes refused: %s", smem_bytes, cudaGetErrorString(e));
  const int per_sm = 1;
  int grid = sms * per_sm;
  if (grid > max_items) grid = max_items;
  static const int dbg = getenv("ZMOE_STREAM_DBG") ? atoi(getenv("ZMOE_STREAM_DBG")) : 0;
  launch_pdl(kern, dim3(grid), dim3(kThreads), (size_t)smem_bytes, st, p, n_tiles, nstages, dbg);
  return check_launch("qmm_stream_kernel");
}

int qmm_stream_launch(const QmmParams& p_in, int nmat, int rows_hint, cudaStream_t st) {
  QmmParams p = p_in;
  const int wm = (nmat == 2) ? 1 : 2;
  if ((p.ngroups & 3) != 0 || (p.N % (16 * wm)) != 0) return 1;   // outside the fast path
  // Only the one-row-per-expert form is covered by the test suite.  With eight rows per expert this kernel once
  // ended in a launch failure (cause not found by reading); it declines such calls and the default kernel runs.
  if (rows_hint > 1) return 1;
  if (((uintptr_t)p.x % 16) != 0 || (p.ldx % 8) != 0) return 1;
  for (int m = 0; m < nmat; ++m)
    if (((uintptr_t)p.w[m] % 16) != 0 || ((uintptr_t)p.s[m] % 16) != 0 || ((uintptr_t)p.b[m] % 16) != 0) return 1;
  // token rows per pass: the largest of 32/16/8/4/2/1 that the hint needs and shared memory allows
  int rs = rows_hint <= 1 ? 1 : rows_hint <= 2 ? 2 : rows_hint <= 4 ? 4 : rows_hint <= 8 ? 8 : rows_hint <= 16 ? 16 : 32;
  int nstages = 4;
  StreamSmem lay;
  const int two_per_sm = 113 * 1024;  // two CTAs share the 227 KB of an SM
  for (;;) {
    const int nt = rs >= 8 ? rs / 8 : 1;
    nstages = 4;
    lay = stream_smem(p.K, p.ngroups, nmat, rs, nt, nstages);
    if (lay.total <= two_per_sm) break;
    nstages = 3;
    lay = stream_smem(p.K, p.ngroups, nmat, rs, nt, nstages);
    if (lay.total <= two_per_sm) break;
    if (rs > 1) {
      rs >>= 1;
      continue;
    }
    // a single token row does not fit twice: one CTA per SM, and use the room for a deeper weight ring
    nstages = 4;
    if (stream_smem(p.K, p.ngroups, nmat, 1, 1, nstages).total > 220 * 1024) return 1;
    while (nstages < kMaxStages && stream_smem(p.K, p.ngroups, nmat, 1, 1, nstages + 1).total <= 200 * 1024) ++nstages;
    lay = stream_smem(p.K, p.ngroups, nmat, 1, 1, nstages);
    break;
  }
  p.rs = rs;
  const int n_tiles = p.N / (16 * wm);
  long long max_items = (long long)(p.rows < p.E ? p.rows : p.E) * n_tiles;
  if (max_items > (1 << 30)) max_items = 1 << 30;
  const int nt = rs >= 8 ? rs / 8 : 1;
  const int tt = rs >= 8 ? 8 : rs;
#define ZMOE_STREAM_CASE(NT_, TT_)                                                                        \
  if (nt == NT_ && tt == TT_)                                                                             \
    return nmat == 2 ? launch_stream<2, NT_, TT_>(p, n_tiles, (int)max_items, nstages, lay.total, st)     \
                     : launch_stream<1, NT_, TT_>(p, n_tiles, (int)max_items, nstages, lay.total, st);
  ZMOE_STREAM_CASE(1, 1)
  ZMOE_STREAM_CASE(1, 2)
  ZMOE_STREAM_CASE(1, 4)
  ZMOE_STREAM_CASE(1, 8)
  ZMOE_STREAM_CASE(2, 8)
  ZMOE_STREAM_CASE(4, 8)
#undef ZMOE_STREAM_CASE
  return 1;
}

int stream_status_reset() {
  int v = 0, zero = 0;
  if (cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)) != cudaSuccess) return -1;
  cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int));
  return v;
}

}  // namespace zmoe
