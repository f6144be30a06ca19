// Token-grouped 4-bit expert matmul for MANY rows per expert (prefill, large decode batches) on the 5th-generation
// tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
// With r rows per expert visit the contraction has 3.6 r flop per weight byte: from r ~ 16 the CUDA-core and
// mma.sync forms of qmm.cu stop being HBM-bound.  Here a CTA owns (expert task, 128 weight rows, a block of up
// to 128 of the task's token rows) and walks K one quantisation group (64 codes) at a time:
//
//   * the packed codes of the CTA's 128 rows arrive by plain 32-byte loads, one group ahead, in registers
//     (thread = weight row); scales and biases of the group come with them;
//   * the group is expanded ONCE into an fp16 tile in shared memory, K-major with the 128-byte swizzle that
//     tcgen05 reads: code pair -> half2 (1024 + q) by shift + or, minus 1032 (exact), then one fp16 FMA
//     (q - 8) * s + (b + 8 s).  b + 8 s is the middle of the group's range, small, so rounding it to fp16 costs
//     nothing; the FMA rounds once: the tile holds fp16(q s + b), 11 significant bits (a bf16 tile, 8 bits,
//     measurably widens the error of the SwiGLU output);
//   * the token rows of the block (gathered through the plan) are fetched one group ahead, converted to fp16 and
//     written into a second swizzled tile;
//   * one thread issues four tcgen05.mma (M 128 x N tokens x K 16, kind::f16, fp16 x fp16 -> fp32) per matrix
//     and group, accumulating in tensor memory (gate and up side by side: 2 x N columns), then
//     tcgen05.commit onto an mbarrier; tiles are double-buffered, so expanding group g+1 overlaps the MMAs of g;
//   * the epilogue reads the accumulators with tcgen05.ld (thread = weight row, 16 token columns at a time),
//     applies the SwiGLU contract and stores bf16 rows through the plan's destination list.
//
// Weights are the M side (128 rows fill the tensor-core tile whatever the token count), tokens the N side
// (16..128 per block).  Every wait on an mbarrier is bounded; a wait that runs out sets the error word, and the
// CTA frees its tensor memory and returns.
#include <cuda_fp16.h>

#include "qmm_common.cuh"

namespace zmoe {

constexpr int kTcThreads = 128;       // thread = weight row of the tile
constexpr int kTcRows = 128;          // weight rows per CTA (MMA M)
constexpr int kTcMaxTok = 128;        // token rows per CTA (MMA N) at most
constexpr int kTcATile = kTcRows * 128;    // bytes of one expanded weight tile: 128 rows x 64 bf16
constexpr int kTcBTile = kTcMaxTok * 128;  // bytes of one token tile
constexpr int kTcSpin = 1 << 22;

struct TcParams {
  QmmParams q;
  int nmat;
  int tok_block;  // token rows per CTA (multiple of 16)
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ bool tc_mbar_wait(uint32_t bar, int parity) {
  for (int i = 0; i < kTcSpin; ++i) {
    uint32_t ok;
    asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
                 : "=r"(ok)
                 : "r"(bar), "r"(parity)
                 : "memory");
    if (ok) return true;
  }
  return false;
}

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 128 bytes, eight rows per
// 1024-byte atom (stride between atoms = 1024 bytes), descriptor version 1.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: D fp32, A and B fp16, both K-major, M = 128, N = n.
__device__ __forceinline__ uint32_t tc_idesc(int n) {
  return (1u << 4) | (0u << 7) | (0u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(kTcRows >> 4) << 24);
}
__device__ __forceinline__ void tc_mma(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  asm volatile(
      "{ .reg .pred p; setp.ne.b32 p, %4, 0; tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p; }" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"((uint32_t)accumulate)
      : "memory");
}
__device__ __forceinline__ void tc_commit(uint32_t bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tc_ld16(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}

// Eight codes of a packed word -> four half2 (q0 s + b, q1 s + b), ... in K order.
__device__ __forceinline__ void tc_expand_word(uint32_t w, __half2 s2, __half2 b2, uint32_t (&out)[4]) {
  const __half2 k1032 = __floats2half2_rn(1032.0f, 1032.0f);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    // codes 2i (bits 8i..8i+3) and 2i+1 (bits 8i+4..8i+7) -> low / high half of a half2 = (1024 + q)
    const uint32_t lo = (w >> (8 * i)) & 0xFu, hi = (w >> (8 * i + 4)) & 0xFu;
    const uint32_t pair = 0x64006400u | lo | (hi << 16);
    __half2 v = *reinterpret_cast<const __half2*>(&pair);
    v = __hfma2(__hsub2(v, k1032), s2, b2);  // (q - 8) s + (b + 8 s), one rounding
    out[i] = *reinterpret_cast<const uint32_t*>(&v);
  }
}

template <int NMAT>
__global__ void __launch_bounds__(kTcThreads, 1) qmm_tc_kernel(const TcParams tp) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  __shared__ uint32_t tmem_base_s;
  __shared__ __align__(8) unsigned long long bars_s[2];  // one per tile buffer: its MMAs are done
  __shared__ int abort_s;

  const QmmParams& p = tp.q;
  const int tid = threadIdx.x, wid = tid >> 5;
  const int K = p.K, N = p.N, ngroups = p.ngroups, K8 = K >> 3;
  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  // 1024-byte aligned tiles: [buffer][matrix] weight tiles, then [buffer] token tiles
  unsigned char* a_tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem) + 1023) & ~(uintptr_t)1023);
  unsigned char* b_tiles = a_tiles + 2 * NMAT * kTcATile;
  const uint32_t bars = tc_smem_u32(bars_s);

  pdl_wait();
  pdl_trigger();
  const int NB = tp.tok_block;
  constexpr int kCols = 256;  // tensor-memory columns of the CTA: NMAT accumulators of up to 128 columns
  if (tid == 0) {
    tc_mbar_init(bars, 1);
    tc_mbar_init(bars + 8, 1);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (wid == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_base_s)),
                 "r"(kCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t idesc = tc_idesc(NB);
  int uses[2] = {0, 0};  // MMA batches committed on each buffer so far (parity of the next wait)

  for (int a = blockIdx.y; a < p.E; a += gridDim.y) {
    const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + a);  // {expert, offset, count, -}
    const int e = task.x, off = task.y, cnt = task.z;
    if (cnt == 0) break;  // tasks are compact
    const int n0 = blockIdx.x * kTcRows;
    const int row = min(n0 + tid, N - 1);  // this thread's weight row (clamped rows are computed, not stored)
    const uint32_t* wrow[NMAT];
    const __nv_bfloat16* srow[NMAT];
    const __nv_bfloat16* brow[NMAT];
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
      wrow[m] = p.w[m] + ((size_t)e * N + row) * K8;
      srow[m] = p.s[m] + ((size_t)e * N + row) * ngroups;
      brow[m] = p.b[m] + ((size_t)e * N + row) * ngroups;
    }
    for (int t0 = 0; t0 < cnt; t0 += NB) {
      const int nt = min(NB, cnt - t0);
      // ---- group 0 of the packed rows, into registers
      uint4 wq[NMAT][2];
      __nv_bfloat16 sv[NMAT], bv[NMAT];
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        wq[m][0] = __ldg(reinterpret_cast<const uint4*>(wrow[m]));
        wq[m][1] = __ldg(reinterpret_cast<const uint4*>(wrow[m]) + 1);
        sv[m] = srow[m][0];
        bv[m] = brow[m][0];
      }
      // Token tile of group g: token t's 64 values at row t of the tile, 16-byte piece c at position c ^ (t % 8),
      // as fp16 (tcgen05 wants both operands of one 16-bit type; fp16 keeps every bit of a bfloat16 inside
      // +-65504, beyond which the value is clamped -- normalised activations are orders of magnitude below).
      // The pieces are fetched into registers one group ahead and converted when the tile is free.
      constexpr int kXr = kTcMaxTok * 8 / kTcThreads;  // pieces per thread at most
      uint4 xr[kXr];
      auto load_tokens = [&](int g) {
#pragma unroll
        for (int u = 0; u < kXr; ++u) {
          const int i = tid + u * kTcThreads;
          const int t = i >> 3, c = i & 7;
          xr[u] = make_uint4(0u, 0u, 0u, 0u);
          if (i < NB * 8 && t < nt) {
            const int src = p.x_by_dst ? pv.row_dst[off + t0 + t] : pv.row_src[off + t0 + t];
            xr[u] = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)src * p.ldx + g * 64) + c);
          }
        }
      };
      auto store_tokens = [&](int buf) {
        unsigned char* bt = b_tiles + buf * kTcBTile;
#pragma unroll
        for (int u = 0; u < kXr; ++u) {
          const int i = tid + u * kTcThreads;
          const int t = i >> 3, c = i & 7;
          if (i < NB * 8) {
            const uint32_t q[4] = {xr[u].x, xr[u].y, xr[u].z, xr[u].w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
              const float lo = fminf(fmaxf(bf16_bits_to_float(q[k] & 0xffffu), -65504.0f), 65504.0f);
              const float hi = fminf(fmaxf(bf16_bits_to_float(q[k] >> 16), -65504.0f), 65504.0f);
              const __half2 h = __floats2half2_rn(lo, hi);
              o[k] = *reinterpret_cast<const uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(bt + (t >> 3) * 1024 + (t & 7) * 128 + ((c ^ (t & 7)) << 4)) =
                make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
      };
      load_tokens(0);
      store_tokens(0);

      bool ok = true;
      for (int g = 0; g < ngroups; ++g) {
        const int buf = g & 1;
        // the MMAs that read this buffer two groups ago must be done before it is overwritten
        if (uses[buf] > 0 && g >= 2 && ok) ok = tc_mbar_wait(bars + buf * 8, (uses[buf] - 1) & 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (g + 1 < ngroups) load_tokens(g + 1);  // lands while the weights are expanded
        // ---- expand this thread's row of the group into the weight tile(s)
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          unsigned char* at = a_tiles + (buf * NMAT + m) * kTcATile + (tid >> 3) * 1024 + (tid & 7) * 128;
          const float sf = __bfloat162float(sv[m]), bf = __bfloat162float(bv[m]);
          const __half2 s2 = __float2half2_rn(sf);  // a bfloat16 scale is exact in fp16 (inside its normal range)
          const __half2 b2 = __float2half2_rn(fmaf(8.0f, sf, bf));
          const uint32_t words[8] = {wq[m][0].x, wq[m][0].y, wq[m][0].z, wq[m][0].w,
                                     wq[m][1].x, wq[m][1].y, wq[m][1].z, wq[m][1].w};
#pragma unroll
          for (int c = 0; c < 8; ++c) {  // word c = codes 8c .. 8c+7 = 16 bytes of bf16
            uint32_t o[4];
            tc_expand_word(words[c], s2, b2, o);
            *reinterpret_cast<uint4*>(at + ((c ^ (tid & 7)) << 4)) = make_uint4(o[0], o[1], o[2], o[3]);
          }
        }
        // ---- the next group's packed codes and token rows are requested now
        if (g + 1 < ngroups) {
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            wq[m][0] = __ldg(reinterpret_cast<const uint4*>(wrow[m] + (g + 1) * 8));
            wq[m][1] = __ldg(reinterpret_cast<const uint4*>(wrow[m] + (g + 1) * 8) + 1);
            sv[m] = srow[m][g + 1];
            bv[m] = brow[m][g + 1];
          }
        }
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0 && ok) {
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          const uint64_t bdesc = tc_desc(tc_smem_u32(b_tiles + buf * kTcBTile));
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            const uint64_t adesc = tc_desc(tc_smem_u32(a_tiles + (buf * NMAT + m) * kTcATile));
#pragma unroll
            for (int k = 0; k < 4; ++k)  // 16 bf16 = 32 bytes further along K inside the swizzled row
              tc_mma(tmem_base + m * kTcMaxTok, adesc + 2 * k, bdesc + 2 * k, idesc, (g > 0) || (k > 0));
          }
          tc_commit(bars + buf * 8);
        }
        if (g + 1 < ngroups) {
          // the other token buffer is free once the MMAs of group g-1 are done
          if (uses[buf ^ 1] > 0 && g >= 1 && ok) ok = tc_mbar_wait(bars + (buf ^ 1) * 8, (uses[buf ^ 1] - 1) & 1);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          store_tokens(buf ^ 1);
        }
        ++uses[buf];
      }
      // ---- all groups issued: wait for the last batch (it orders after all earlier ones)
      const int last = (ngroups - 1) & 1;
      if (ok) ok = tc_mbar_wait(bars + last * 8, (uses[last] - 1) & 1);
      if (ngroups > 1 && ok) ok = tc_mbar_wait(bars + (last ^ 1) * 8, (uses[last ^ 1] - 1) & 1);
      if (!ok) abort_s = 1;
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      __syncthreads();
      if (abort_s) break;
      // ---- epilogue: thread = weight row (tensor-memory lane), 16 token columns per read
      const int n = n0 + tid;
      for (int c0 = 0; c0 < nt; c0 += 16) {
        uint32_t acc[NMAT][16];
        const uint32_t taddr = tmem_base + ((uint32_t)(wid * 32) << 16) + c0;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) tc_ld16(taddr + m * kTcMaxTok, acc[m]);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          if (c0 + j < nt && n < N) {
            float v;
            if (NMAT == 2) {
              const float gv = __uint_as_float(acc[0][j]), uv = __uint_as_float(acc[NMAT - 1][j]);
              v = (p.epilogue == 2) ? swiglu_per_op(gv, uv) : swiglu_cpu_contract(gv, uv);
            } else {
              v = __uint_as_float(acc[0][j]);
            }
            const int dst = pv.row_dst[off + t0 + c0 + j];
            p.out[(size_t)dst * p.ldo + n] = __float2bfloat16_rn(v);
          }
        }
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncthreads();  // the accumulators are free for the next block
    }
    if (abort_s) break;
  }
  if (abort_s && tid == 0) atomicExch(pv.hdr + 2, 2);  // the plan's status word: a bounded wait ran out
  __syncthreads();
  if (wid == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kCols) : "memory");
  }
}

// Host side: called by qmm_launch for affine banks when an expert visit has many rows.

int qmm_tc_launch(const QmmParams& q, int nmat, int rows_hint, int max_groups, cudaStream_t st, const char* who) {
  TcParams tp;
  tp.q = q;
  tp.nmat = nmat;
  int nb = (rows_hint + 15) & ~15;
  if (nb > kTcMaxTok) nb = kTcMaxTok;
  if (nb < 16) nb = 16;
  tp.tok_block = nb;
  const size_t smem = 1024 + (size_t)2 * nmat * kTcATile + 2 * kTcBTile;
  dim3 grid((q.N + kTcRows - 1) / kTcRows, max_groups);
  cudaError_t e;
  if (nmat == 2) {
    e = cudaFuncSetAttribute(qmm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = launch_pdl(qmm_tc_kernel<2>, grid, dim3(kTcThreads), smem, st, tp);
  } else {
    e = cudaFuncSetAttribute(qmm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = launch_pdl(qmm_tc_kernel<1>, grid, dim3(kTcThreads), smem, st, tp);
  }
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "%s: tensor-memory kernel launch failed: %s", who, cudaGetErrorString(e));
  return check_launch("qmm_tc_kernel");
}

}  // namespace zmoe
