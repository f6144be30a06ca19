// Token-grouped 4-bit expert matmul for MANY rows per expert (prefill, large decode batches) on the 5th-generation
// tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
// With r rows per expert visit the contraction has 3.6 r flop per weight byte: from r ~ 16 the CUDA-core and
// mma.sync forms of qmm.cu stop being HBM-bound.  Here a CTA owns (expert task, 128 weight rows, a block of up
// to 32 of the task's token rows) and walks K one quantisation group (64 codes) at a time.  Its 8 warps split
// into two roles of 128 threads, thread = weight row in both:
//
//   expanders  fetch the row's 32 packed bytes of the next group (plain loads, one group ahead) and write them
//              ONCE into an fp16 tile in shared memory as the exact integers q - 8 (four lop3, one shift and four
//              exact fp16 operations per packed word; K-major, 128-byte swizzle).  They also fetch the block's
//              token rows through the plan, convert them to fp16 (exact inside +-65504, clamped beyond), write
//              the token tile in the same K order and leave each token's group sum in shared memory.  One of
//              them then issues four tcgen05.mma (M 128 x N 32 x K 16, kind::f16, fp32 accumulate) per matrix
//              into a FRESH tensor-memory accumulator and commits them onto an mbarrier;
//   finishers  wait for that mbarrier, read the group's sums D = sum_k x_k (q_k - 8) from tensor memory
//              (tcgen05.ld, 16 token columns at a time) and apply the group's scale and bias in fp32,
//                  acc += s * D + (b + 8 s) * sum_k x_k,
//              the per-group arithmetic of the decode kernels: no weight is rounded before the fp32 sum.
//              At the end of the block they apply the SwiGLU contract and store bf16 rows through the plan.
//
// Tiles and accumulators are double-buffered: group g+1 is expanded while the tensor core works on g and the
// finishers fold g-1.  Weights are the M side (128 rows fill the tensor-core tile whatever the token count),
// tokens the N side.  Every wait on an mbarrier is bounded; a wait that runs out sets the plan's status word, the
// thread stops waiting (it still walks its loops, so that no barrier is left short), and the CTA frees its tensor
// memory and returns.
#include <cuda_fp16.h>

#include "qmm_common.cuh"

namespace zmoe {

constexpr int kTcRole = 128;  // threads per role; thread = weight row of the tile
constexpr int kTcThreads = 2 * kTcRole;
constexpr int kTcRows = 128;             // weight rows per CTA (MMA M)
constexpr int kTcTok = 32;               // token rows per CTA (MMA N)
constexpr int kTcATile = kTcRows * 128;  // bytes of one expanded weight tile: 128 rows x 64 fp16
constexpr int kTcBTile = kTcTok * 128;   // bytes of one token tile
constexpr int kTcCols = 128;             // tensor-memory columns: 2 buffers x 2 accumulators x 32 token columns
constexpr int kTcRing = 2;               // groups of packed rows and token pieces in flight per thread (cp.async)
constexpr int kTcRawW = kTcRows * 32;    // bytes of one matrix's packed group: 128 rows x 32 bytes
constexpr int kTcRawX = kTcTok * 128;    // bytes of the block's token rows of one group (bf16)
constexpr int kTcScArr = kTcRows * 8;    // bytes of one array (scales or biases) of a matrix for four groups
constexpr int kTcSpin = 1 << 22;

struct TcParams {
  QmmParams q;
  int nmat;
};

__device__ __forceinline__ uint32_t tc_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void tc_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void tc_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
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
// 16-byte asynchronous copy global -> shared; src_bytes = 0 writes zeros
__device__ __forceinline__ void tc_cp16(void* dst, const void* src, int src_bytes) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(tc_smem_u32(dst)), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void tc_cp8(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(tc_smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void tc_cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void tc_cp_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
// barrier of the 128 expander threads
__device__ __forceinline__ void tc_expander_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kTcRole) : "memory"); }

// Shared-memory matrix descriptor of a K-major tile with the 128-byte swizzle: rows of 128 bytes, eight rows per
// 1024-byte atom (stride between atoms = 1024 bytes), descriptor version 1.
__device__ __forceinline__ uint64_t tc_desc(uint32_t smem_addr) {
  return (uint64_t)((smem_addr & 0x3FFFFu) >> 4) | (1ull << 16) | ((uint64_t)(1024 >> 4) << 32) | (1ull << 46) |
         (2ull << 61);
}
// Instruction descriptor: D fp32, A and B fp16 (tcgen05 wants both operands of one 16-bit type), both K-major,
// M = 128, N = n.
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
__device__ __forceinline__ void tc_ld16(uint32_t taddr, float (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=f"(r[0]), "=f"(r[1]), "=f"(r[2]), "=f"(r[3]), "=f"(r[4]), "=f"(r[5]), "=f"(r[6]), "=f"(r[7]), "=f"(r[8]),
        "=f"(r[9]), "=f"(r[10]), "=f"(r[11]), "=f"(r[12]), "=f"(r[13]), "=f"(r[14]), "=f"(r[15])
      : "r"(taddr)
      : "memory");
}

// Eight codes of a packed word -> the exact integers q - 8 as four half2, in the order (q0,q4) (q1,q5) (q2,q6)
// (q3,q7): (w & 0x000F000F) | 0x64006400 is the half2 (1024 + q0, 1024 + q4) and (w & 0x00F000F0) | 0x64006400
// is (1024 + 16 q1, 1024 + 16 q5); the same on w >> 8.  The token tile uses the same order inside every eight.
__device__ __forceinline__ uint4 tc_expand_word(uint32_t w) {
  const __half2 k1032 = __floats2half2_rn(1032.0f, 1032.0f);
  const __half2 k16th = __floats2half2_rn(0.0625f, 0.0625f);
  const __half2 km72 = __floats2half2_rn(-72.0f, -72.0f);
  uint32_t p0, p1, p2, p3;
  const uint32_t w8 = w >> 8;
  asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(p0) : "r"(w));
  asm("lop3.b32 %0, %1, 0x00F000F0, 0x64006400, 0xEA;" : "=r"(p1) : "r"(w));
  asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(p2) : "r"(w8));
  asm("lop3.b32 %0, %1, 0x00F000F0, 0x64006400, 0xEA;" : "=r"(p3) : "r"(w8));
  // (1024 + q) - 1032 = q - 8;  (1024 + 16 q) / 16 - 72 = q - 8: both exact in fp16
  const __half2 a0 = __hsub2(*reinterpret_cast<__half2*>(&p0), k1032);
  const __half2 a1 = __hfma2(*reinterpret_cast<__half2*>(&p1), k16th, km72);
  const __half2 a2 = __hsub2(*reinterpret_cast<__half2*>(&p2), k1032);
  const __half2 a3 = __hfma2(*reinterpret_cast<__half2*>(&p3), k16th, km72);
  return make_uint4(*reinterpret_cast<const uint32_t*>(&a0), *reinterpret_cast<const uint32_t*>(&a1),
                    *reinterpret_cast<const uint32_t*>(&a2), *reinterpret_cast<const uint32_t*>(&a3));
}

template <int NMAT>
__global__ void __launch_bounds__(kTcThreads, 2) qmm_tc_kernel(const TcParams tp) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  __shared__ uint32_t tmem_base_s;
  // [0..1] a buffer's MMAs are done (tcgen05.commit); [2..3] the finishers have folded the buffer's accumulator
  // and read its token sums
  __shared__ __align__(8) unsigned long long bars_s[4];
  __shared__ float xsum_s[2][kTcTok];
  __shared__ int abort_s;

  const QmmParams& p = tp.q;
  const int tid = threadIdx.x, wid = tid >> 5;
  const bool expander = tid < kTcRole;
  const int r = expander ? tid : tid - kTcRole;  // weight row of the tile (= tensor-memory lane)
  const int K = p.K, N = p.N, ngroups = p.ngroups, K8 = K >> 3;
  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  // 1024-byte aligned tiles: [buffer][matrix] weight tiles, then [buffer] token tiles
  unsigned char* a_tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem) + 1023) & ~(uintptr_t)1023);
  unsigned char* b_tiles = a_tiles + 2 * NMAT * kTcATile;
  // ring of raw groups: [slot][matrix][row][32 bytes], then [slot][piece][16 bytes]; a thread reads back only
  // what it copied itself, so its own cp.async.wait_group is all the synchronisation the ring needs
  unsigned char* raw_w = b_tiles + 2 * kTcBTile;
  unsigned char* raw_x = raw_w + kTcRing * NMAT * kTcRawW;
  // scales and biases of four groups at a time: [chunk parity][matrix][scale | bias][row][4 bf16], copied by the
  // expander of the row two groups before the chunk's first group and read by the row's finisher
  unsigned char* sc_tiles = raw_x + kTcRing * kTcRawX;
  const uint32_t bars = tc_smem_u32(bars_s);

  pdl_wait();
  pdl_trigger();
  {  // a CTA whose token blocks lie beyond the end of its tasks leaves before it takes any tensor memory
    bool any = false;
    for (int a = blockIdx.y; a < p.E; a += gridDim.y) {
      const int cnt = __ldg(pv.tasks + 4 * a + 2);
      if (cnt == 0) break;
      any = any || (int)(blockIdx.z * kTcTok) < cnt;
    }
    if (!any) return;
  }
  if (tid == 0) {
    tc_mbar_init(bars, 1);
    tc_mbar_init(bars + 8, 1);
    tc_mbar_init(bars + 16, kTcRole);
    tc_mbar_init(bars + 24, kTcRole);
    abort_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  if (wid == 0) {
    __syncwarp();
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tc_smem_u32(&tmem_base_s)),
                 "r"(kTcCols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  const uint32_t tmem_base = tmem_base_s;
  const uint32_t idesc = tc_idesc(kTcTok);
  int n_done[2] = {0, 0};  // groups this thread's role has taken through each buffer (parities of the waits)
  bool ok = true;

  for (int a = blockIdx.y; a < p.E; a += gridDim.y) {
    const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + a);  // {expert, offset, count, -}
    const int e = task.x, off = task.y, cnt = task.z;
    if (cnt == 0) break;  // tasks are compact
    const int n0 = blockIdx.x * kTcRows;
    const int row = min(n0 + r, N - 1);  // clamped rows are computed, not stored
    for (int t0 = blockIdx.z * kTcTok; t0 < cnt; t0 += gridDim.z * kTcTok) {
      const int nt = min(kTcTok, cnt - t0);
      if (expander) {
        // ================================================================ expanders
        const uint32_t* wrow[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) wrow[m] = p.w[m] + ((size_t)e * N + row) * K8;
        // each thread brings two 16-byte pieces of the token tile: piece i = token i / 8, values 8 (i % 8) ..
        int xsrc[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int t = (tid + u * kTcRole) >> 3;
          xsrc[u] = -1;
          if (t < nt) xsrc[u] = p.x_by_dst ? pv.row_dst[off + t0 + t] : pv.row_src[off + t0 + t];
        }
        const unsigned char* xrow[2];
#pragma unroll
        for (int u = 0; u < 2; ++u)
          xrow[u] = reinterpret_cast<const unsigned char*>(p.x + (size_t)max(xsrc[u], 0) * p.ldx) + (tid & 7) * 16;
        const __nv_bfloat16* srow[NMAT];
        const __nv_bfloat16* brow[NMAT];
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          srow[m] = p.s[m] + ((size_t)e * N + row) * ngroups;
          brow[m] = p.b[m] + ((size_t)e * N + row) * ngroups;
        }
        auto fetch_scales = [&](int c) {  // this row's scales and biases of groups 4c .. 4c+3
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            unsigned char* dst = sc_tiles + ((c & 1) * NMAT + m) * 2 * kTcScArr + tid * 8;
            tc_cp8(dst, srow[m] + 4 * c);
            tc_cp8(dst + kTcScArr, brow[m] + 4 * c);
          }
        };
        auto fetch = [&](int g) {  // this thread's 32 packed bytes per matrix and two token pieces of group g
          const int slot = g % kTcRing;
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            unsigned char* dst = raw_w + (slot * NMAT + m) * kTcRawW + tid * 32;
            tc_cp16(dst, wrow[m] + g * 8, 16);
            tc_cp16(dst + 16, wrow[m] + g * 8 + 4, 16);
          }
#pragma unroll
          for (int u = 0; u < 2; ++u)
            tc_cp16(raw_x + slot * kTcRawX + (tid + u * kTcRole) * 16, xrow[u] + (size_t)g * 128, xsrc[u] >= 0 ? 16 : 0);
        };
        // The previous block must be folded completely before its last scales are overwritten.
#pragma unroll
        for (int b2 = 0; b2 < 2; ++b2)
          if (n_done[b2] > 0 && ok) ok = tc_mbar_wait(bars + 16 + b2 * 8, (n_done[b2] - 1) & 1);
        fetch_scales(0);
#pragma unroll
        for (int g = 0; g < kTcRing - 1; ++g) {
          if (g < ngroups) fetch(g);
          tc_cp_commit();
        }
        for (int g = 0; g < ngroups; ++g) {
          const int buf = g & 1;
          // the buffer's previous group must be through the tensor core AND folded by the finishers
          if (n_done[buf] > 0 && ok) {
            ok = tc_mbar_wait(bars + buf * 8, (n_done[buf] - 1) & 1) &&
                 tc_mbar_wait(bars + 16 + buf * 8, (n_done[buf] - 1) & 1);
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          }
          tc_cp_wait<kTcRing - 2>();  // this thread's copies of group g have landed
          const int slot = g % kTcRing;
          // ---- weight tile(s): this thread's row; word c = codes 8c .. 8c+7 -> 16 bytes at piece c ^ (row % 8)
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            unsigned char* at = a_tiles + (buf * NMAT + m) * kTcATile + (tid >> 3) * 1024 + (tid & 7) * 128;
            const uint4 w0 = *reinterpret_cast<const uint4*>(raw_w + (slot * NMAT + m) * kTcRawW + tid * 32);
            const uint4 w1 = *reinterpret_cast<const uint4*>(raw_w + (slot * NMAT + m) * kTcRawW + tid * 32 + 16);
            const uint32_t words[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
#pragma unroll
            for (int c = 0; c < 8; ++c)
              *reinterpret_cast<uint4*>(at + ((c ^ (tid & 7)) << 4)) = tc_expand_word(words[c]);
          }
          // ---- token tile: fp16, every eight values in the order (0,4) (1,5) (2,6) (3,7); sums of the group
#pragma unroll
          for (int u = 0; u < 2; ++u) {
            const int i = tid + u * kTcRole;
            const int t = i >> 3, c = i & 7;
            const uint4 xq = *reinterpret_cast<const uint4*>(raw_x + slot * kTcRawX + i * 16);
            const uint32_t q[4] = {xq.x, xq.y, xq.z, xq.w};
            float v[8];
            const __nv_bfloat162 lim = __floats2bfloat162_rn(65280.0f, 65280.0f);  // largest bfloat16 below 65504
#pragma unroll
            for (int k = 0; k < 4; ++k) {  // clamp two values at a time (NaN stays NaN), then widen
              __nv_bfloat162 h = *reinterpret_cast<const __nv_bfloat162*>(&q[k]);
              h = __hmax2_nan(__hmin2_nan(h, lim), __hneg2(lim));
              const uint32_t hb = *reinterpret_cast<const uint32_t*>(&h);
              v[2 * k] = __uint_as_float(hb << 16);
              v[2 * k + 1] = __uint_as_float(hb & 0xffff0000u);
            }
            auto pack = [&](int i0, int i1) {
              const __half2 h = __floats2half2_rn(v[i0], v[i1]);
              return *reinterpret_cast<const uint32_t*>(&h);
            };
            *reinterpret_cast<uint4*>(b_tiles + buf * kTcBTile + (t >> 3) * 1024 + (t & 7) * 128 + ((c ^ (t & 7)) << 4)) =
                make_uint4(pack(0, 4), pack(1, 5), pack(2, 6), pack(3, 7));
            float part = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            part += __shfl_xor_sync(0xffffffffu, part, 1);
            part += __shfl_xor_sync(0xffffffffu, part, 2);
            part += __shfl_xor_sync(0xffffffffu, part, 4);
            if (c == 0) xsum_s[buf][t] = part;
          }
          if (g + kTcRing - 1 < ngroups) fetch(g + kTcRing - 1);  // into the slot this thread emptied last time
          if ((g & 3) == 2 && g + 2 < ngroups) fetch_scales((g + 2) >> 2);
          tc_cp_commit();
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          tc_expander_sync();
          if (tid == 0 && ok) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t bdesc = tc_desc(tc_smem_u32(b_tiles + buf * kTcBTile));
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
              const uint64_t adesc = tc_desc(tc_smem_u32(a_tiles + (buf * NMAT + m) * kTcATile));
#pragma unroll
              for (int k = 0; k < 4; ++k)  // 16 values = 32 bytes further along K inside the swizzled row
                tc_mma(tmem_base + (buf * NMAT + m) * kTcTok, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0);
            }
            tc_commit(bars + buf * 8);  // the token sums of the buffer were written before the expanders' barrier
          }
          ++n_done[buf];
        }
      } else {
        // ================================================================ finishers
        float acc[NMAT][kTcTok];
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
          for (int j = 0; j < kTcTok; ++j) acc[m][j] = 0.0f;
        for (int g = 0; g < ngroups; ++g) {
          const int buf = g & 1;
          if (ok) ok = tc_mbar_wait(bars + buf * 8, n_done[buf] & 1);
          asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
          if (ok) {
            float sv[NMAT], cv[NMAT];  // the group's scale and b + 8 s, staged by the row's expander
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
              const unsigned char* src = sc_tiles + (((g >> 2) & 1) * NMAT + m) * 2 * kTcScArr + r * 8 + (g & 3) * 2;
              sv[m] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src));
              cv[m] = fmaf(8.0f, sv[m], __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src + kTcScArr)));
            }
#pragma unroll
            for (int c0 = 0; c0 < kTcTok; c0 += 16) {
              float dreg[NMAT][16];
              const uint32_t taddr = tmem_base + ((uint32_t)((wid & 3) * 32) << 16) + buf * NMAT * kTcTok + c0;
#pragma unroll
              for (int m = 0; m < NMAT; ++m) tc_ld16(taddr + m * kTcTok, dreg[m]);
              asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
              for (int j = 0; j < 16; ++j) {
                const float xs = xsum_s[buf][c0 + j];
#pragma unroll
                for (int m = 0; m < NMAT; ++m) acc[m][c0 + j] = fmaf(sv[m], dreg[m][j], fmaf(cv[m], xs, acc[m][c0 + j]));
              }
            }
          }
          asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
          tc_mbar_arrive(bars + 16 + buf * 8);  // the buffer's accumulator and token sums are free
          ++n_done[buf];
        }
        // ---- end of the block: SwiGLU contract and bf16 stores, thread = weight row
        const int n = n0 + r;
        if (ok && n < N) {
#pragma unroll
          for (int j = 0; j < kTcTok; ++j) {
            if (j < nt) {
              float v;
              if (NMAT == 2)
                v = (p.epilogue == 2) ? swiglu_per_op(acc[0][j], acc[NMAT - 1][j])
                                      : swiglu_cpu_contract(acc[0][j], acc[NMAT - 1][j]);
              else
                v = acc[0][j];
              const int dst = pv.row_dst[off + t0 + j];
              p.out[(size_t)dst * p.ldo + n] = __float2bfloat16_rn(v);
            }
          }
        }
      }
    }
  }
  if (!ok) abort_s = 1;
  asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
  __syncthreads();
  asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
  if (abort_s && tid == 0) atomicExch(pv.hdr + 2, 2);  // the plan's status word: a bounded wait ran out
  if (wid == 0) {
    __syncwarp();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTcCols) : "memory");
  }
}

// Host side: called by qmm_launch for affine banks when an expert visit has many rows.
int qmm_tc_launch(const QmmParams& q, int nmat, int rows_hint, int max_groups, cudaStream_t st, const char* who) {
  TcParams tp;
  tp.q = q;
  tp.nmat = nmat;
  const size_t smem = 1024 + (size_t)2 * nmat * kTcATile + 2 * kTcBTile + (size_t)kTcRing * (nmat * kTcRawW + kTcRawX) +
                      (size_t)2 * nmat * 2 * kTcScArr;
  // token blocks of one task are dealt over grid.z: enough for twice the average task, never more than the
  // largest possible task needs; a CTA strides over the blocks beyond that
  const int avg = (q.rows + q.E - 1) / q.E;
  int zs = (2 * avg + kTcTok - 1) / kTcTok;
  const int zmax = (rows_hint + kTcTok - 1) / kTcTok;
  if (zs > zmax) zs = zmax;
  if (zs > 64) zs = 64;
  if (zs < 1) zs = 1;
  dim3 grid((q.N + kTcRows - 1) / kTcRows, max_groups, zs);
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
