// Token-grouped 4-bit expert matmul for MANY rows per expert (prefill, large decode batches) on the 5th-generation
// tensor cores: tcgen05.mma with the accumulator in tensor memory.
//
// With r rows per expert visit the contraction has 3.6 r flop per weight byte: from r ~ 16 the CUDA-core and
// mma.sync forms of qmm.cu stop being HBM-bound.  Here the work is cut into items (expert task, 128 weight rows,
// a block of up to 32 of the task's token rows); a persistent grid of one CTA per SM deals the items round-robin,
// same-weights items next to each other so that they run at the same time on different SMs and share the weights
// through L2.  A CTA walks its items one quantisation group (64 codes) at a time, as one unbroken stream of steps:
// copies for step s+7 are issued while step s is expanded, across item boundaries.  Sixteen of its 17 warps split
// into two roles of 256 threads; the first lane of the 17th issues the MMAs:
//
//   expanders  (thread = weight row x half of the group) keep a ring of raw packed bytes, token pieces and
//              scale/bias chunks filled with cp.async; a thread reads back only what it copied itself, so its own
//              cp.async.wait_group is all the ring needs.  Per step they write the group ONCE into an fp16 tile in
//              shared memory as the exact integers q - 8 (four lop3, one shift and four exact fp16 operations per
//              packed word; K-major, 128-byte swizzle), convert the block's token rows to fp16 (exact inside
//              +-65280, clamped beyond), write the token tile in the same K order and leave each token's group
//              sum in shared memory; each warp then arrives on the step's "tiles full" mbarrier and moves on;
//   issuer     waits for that mbarrier, issues four tcgen05.mma (M 128 x N 32 x K 16, kind::f16, fp32
//              accumulate) per matrix into a FRESH tensor-memory accumulator and commits them onto an mbarrier;
//   finishers  (thread = weight row x 16 token columns) wait for that mbarrier, read the group's sums
//              D = sum_k x_k (q_k - 8) from tensor memory (tcgen05.ld) and apply the group's scale and bias in
//              fp32, acc += s * D + (b + 8 s) * sum_k x_k: the per-group arithmetic of the decode kernels, no
//              weight is rounded before the fp32 sum.  At the end of an item they apply the SwiGLU contract and
//              store bf16 rows through the plan.
//
// Tiles and accumulators are double-buffered: group g+1 is expanded while the tensor core works on g and the
// finishers fold g-1.  Weights are the M side (128 rows fill the tensor-core tile whatever the token count),
// tokens the N side.  Every wait on an mbarrier is bounded; a wait that runs out sets the plan's status word, the
// thread stops waiting (it still walks its steps, so that no barrier is left short), and the CTA frees its tensor
// memory and returns.
#include <cuda_fp16.h>

#include "qmm_common.cuh"

namespace zmoe {

constexpr int kTcRole = 256;  // threads per role
constexpr int kTcThreads = 2 * kTcRole + 32;  // + the warp whose first lane issues the MMAs
constexpr int kTcRows = 128;             // weight rows per item (MMA M)
constexpr int kTcTok = 32;               // token rows per item (MMA N)
constexpr int kTcATile = kTcRows * 128;  // bytes of one expanded weight tile: 128 rows x 64 fp16
constexpr int kTcBTile = kTcTok * 128;   // bytes of one token tile
constexpr int kTcCols = 128;             // tensor-memory columns: 2 buffers x 2 accumulators x 32 token columns
constexpr int kTcRing = 8;               // steps of raw bytes in flight per thread (cp.async)
constexpr int kTcRawW = kTcRows * 32;    // bytes of one matrix's packed group: 128 rows x 32 bytes
constexpr int kTcRawX = kTcTok * 128;    // bytes of the item's token rows of one group (bf16)
constexpr int kTcScArr = kTcRows * 8;    // bytes of one array (scales or biases) of a matrix for four groups
constexpr int kTcScSlots = 4;            // chunks of four groups of scales and biases in the ring
constexpr int kTcMaxTasks = 1024;        // experts with rows, at most (prefix sums live in shared memory)
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
  uint32_t done;
  asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(done)
               : "r"(bar), "r"(parity)
               : "memory");
  if (done) return true;
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

// One item of the persistent grid's work list.
struct TcItem {
  int e, off, t0, nt, n0;
};

// Items are numbered task-major; inside a task the token blocks of one row tile are neighbours.  prefix[a] =
// token blocks of the tasks before a.
__device__ __forceinline__ TcItem tc_item(const PlanView& pv, const int* prefix, int ntasks, int ntiles, int w) {
  int lo = 0, hi = ntasks - 1;
  while (lo < hi) {  // the last task whose first item is <= w
    const int mid = (lo + hi + 1) >> 1;
    if (ntiles * prefix[mid] <= w) lo = mid; else hi = mid - 1;
  }
  const int local = w - ntiles * prefix[lo];
  const int nblk = prefix[lo + 1] - prefix[lo];
  const int tile = local / nblk, blk = local - tile * nblk;
  const int4 task = __ldg(reinterpret_cast<const int4*>(pv.tasks) + lo);  // {expert, offset, count, -}
  TcItem it;
  it.e = task.x;
  it.off = task.y;
  it.t0 = blk * kTcTok;
  it.nt = min(kTcTok, task.z - it.t0);
  it.n0 = tile * kTcRows;
  return it;
}

template <int NMAT>
__global__ void __launch_bounds__(kTcThreads, 1) qmm_tc_kernel(const TcParams tp) {
  extern __shared__ __align__(1024) unsigned char tc_smem[];
  __shared__ uint32_t tmem_base_s;
  // [0..1] a buffer's MMAs are done (tcgen05.commit); [2..3] the finishers have folded the buffer's accumulator
  // and read its token sums; [4..5] the expanders have filled the buffer's tiles (one arrival per warp)
  __shared__ __align__(8) unsigned long long bars_s[6];
  __shared__ __align__(16) float xsum_s[2][kTcTok];
  __shared__ int abort_s;
  __shared__ int prefix_s[kTcMaxTasks + 1];

  const QmmParams& p = tp.q;
  const int tid = threadIdx.x, wid = tid >> 5, lane = tid & 31;
  const bool expander = tid < kTcRole, finisher = !expander && tid < 2 * kTcRole;
  const int N = p.N, ngroups = p.ngroups, K8 = p.K >> 3;
  const PlanView pv = plan_view(const_cast<int*>(p.plan), p.rows, p.E);
  // 1024-byte aligned tiles: [buffer][matrix] weight tiles, [buffer] token tiles, then the rings of raw bytes:
  // [slot][matrix][row][32 bytes] packed codes, [slot][piece][16 bytes] token pieces, and
  // [chunk slot][matrix][scale | bias][row][4 bf16] for four groups at a time
  unsigned char* a_tiles = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(tc_smem) + 1023) & ~(uintptr_t)1023);
  unsigned char* b_tiles = a_tiles + 2 * NMAT * kTcATile;
  unsigned char* raw_w = b_tiles + 2 * kTcBTile;
  unsigned char* raw_x = raw_w + kTcRing * NMAT * kTcRawW;
  unsigned char* sc_tiles = raw_x + kTcRing * kTcRawX;
  const uint32_t bars = tc_smem_u32(bars_s);

  pdl_wait();
  pdl_trigger();
  // ---- token blocks per task, prefix-summed by warp 0 (lane = a contiguous run of tasks)
  const int ntasks = min(pv.hdr[0], kTcMaxTasks);
  if (wid == 0) {
    const int per = (ntasks + 31) >> 5;
    int sum = 0;
    for (int i = lane * per; i < min(ntasks, (lane + 1) * per); ++i)
      sum += (__ldg(pv.tasks + 4 * i + 2) + kTcTok - 1) / kTcTok;
    int incl = sum;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const int v = __shfl_up_sync(0xffffffffu, incl, o);
      if (lane >= o) incl += v;
    }
    int run = incl - sum;
    for (int i = lane * per; i < min(ntasks, (lane + 1) * per); ++i) {
      prefix_s[i] = run;
      run += (__ldg(pv.tasks + 4 * i + 2) + kTcTok - 1) / kTcTok;
    }
    if (lane == 31) prefix_s[ntasks] = incl;
  }
  __syncthreads();
  const int ntiles = (N + kTcRows - 1) / kTcRows;
  const int total = ntiles * prefix_s[ntasks];
  if ((int)blockIdx.x >= total) return;  // nothing for this CTA: it leaves before it takes any tensor memory
  const int n_items = (total - (int)blockIdx.x + (int)gridDim.x - 1) / (int)gridDim.x;
  const int n_steps = n_items * ngroups;

  if (tid == 0) {
    tc_mbar_init(bars, 1);
    tc_mbar_init(bars + 8, 1);
    tc_mbar_init(bars + 16, kTcRole / 32);  // one arrival per finisher warp
    tc_mbar_init(bars + 24, kTcRole / 32);
    tc_mbar_init(bars + 32, kTcRole / 32);  // one arrival per expander warp
    tc_mbar_init(bars + 40, kTcRole / 32);
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
  bool ok = true;

  if (expander) {
    // ================================================================== expanders
    const int r = tid & 127, half = tid >> 7;  // weight row of the tile; which four packed words of the group
    // ---- the copy cursor runs kTcRing - 1 steps ahead of the step being expanded, across items
    int f_item = -1, f_g = ngroups;
    const unsigned char* f_w[NMAT];
    const unsigned char* f_s[NMAT];
    const unsigned char* f_b[NMAT];
    const unsigned char* f_x = nullptr;
    int f_xbytes = 0;
    auto fetch = [&](int sf) {
      if (sf >= n_steps) return;
      if (f_g == ngroups) {
        ++f_item;
        f_g = 0;
        const TcItem it = tc_item(pv, prefix_s, ntasks, ntiles, (int)blockIdx.x + f_item * (int)gridDim.x);
        const int row = min(it.n0 + r, N - 1);  // clamped rows are computed, not stored
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          f_w[m] = reinterpret_cast<const unsigned char*>(p.w[m] + ((size_t)it.e * N + row) * K8 + half * 4);
          f_s[m] = reinterpret_cast<const unsigned char*>(p.s[m] + ((size_t)it.e * N + row) * ngroups);
          f_b[m] = reinterpret_cast<const unsigned char*>(p.b[m] + ((size_t)it.e * N + row) * ngroups);
        }
        const int t = tid >> 3;  // this thread's token piece: token t, values 8 (tid % 8) ..
        f_x = reinterpret_cast<const unsigned char*>(p.x);
        f_xbytes = 0;
        if (t < it.nt) {
          const int src = p.x_by_dst ? pv.row_dst[it.off + it.t0 + t] : pv.row_src[it.off + it.t0 + t];
          f_x = reinterpret_cast<const unsigned char*>(p.x + (size_t)src * p.ldx + (tid & 7) * 8);
          f_xbytes = 16;
        }
      }
      const int slot = sf % kTcRing;
#pragma unroll
      for (int m = 0; m < NMAT; ++m)
        tc_cp16(raw_w + (slot * NMAT + m) * kTcRawW + r * 32 + half * 16, f_w[m] + (size_t)f_g * 32, 16);
      tc_cp16(raw_x + slot * kTcRawX + tid * 16, f_x + (size_t)f_g * 128 * (f_xbytes >> 4), f_xbytes);
      if ((f_g & 3) == 0 && half == 0) {  // the row's scales and biases of this and the next three groups
        const int cslot = (sf >> 2) % kTcScSlots;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          unsigned char* dst = sc_tiles + (cslot * NMAT + m) * 2 * kTcScArr + r * 8;
          tc_cp8(dst, f_s[m] + f_g * 2);
          tc_cp8(dst + kTcScArr, f_b[m] + f_g * 2);
        }
      }
      ++f_g;
    };
#pragma unroll 1
    for (int sf = 0; sf < kTcRing - 1; ++sf) {
      fetch(sf);
      tc_cp_commit();
    }
#pragma unroll 1
    for (int s = 0; s < n_steps; ++s) {
      const int buf = s & 1;
      // the buffer's previous group must be folded by the finishers, who had waited for its MMAs before that
      if (s >= 2 && ok) {
        ok = tc_mbar_wait(bars + 16 + buf * 8, ((s >> 1) - 1) & 1);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      }
      tc_cp_wait<kTcRing - 2>();  // this thread's copies of step s have landed
      const int slot = s % kTcRing;
      // ---- weight tile(s): word c = codes 8c .. 8c+7 of the row -> 16 bytes at piece c ^ (row % 8)
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        unsigned char* at = a_tiles + (buf * NMAT + m) * kTcATile + (r >> 3) * 1024 + (r & 7) * 128;
        const uint4 w4 = *reinterpret_cast<const uint4*>(raw_w + (slot * NMAT + m) * kTcRawW + r * 32 + half * 16);
        const uint32_t words[4] = {w4.x, w4.y, w4.z, w4.w};
#pragma unroll
        for (int c4 = 0; c4 < 4; ++c4)
          *reinterpret_cast<uint4*>(at + (((half * 4 + c4) ^ (r & 7)) << 4)) = tc_expand_word(words[c4]);
      }
      // ---- token tile: fp16, every eight values in the order (0,4) (1,5) (2,6) (3,7); sums of the group
      {
        const int t = tid >> 3, c = tid & 7;
        const uint4 xq = *reinterpret_cast<const uint4*>(raw_x + slot * kTcRawX + tid * 16);
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
      fetch(s + kTcRing - 1);  // into the slot this thread emptied at the step before
      tc_cp_commit();
      asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic-proxy writes -> visible to the MMA
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(bars + 32 + buf * 8);  // this warp's part of the step's tiles is written
    }
    tc_cp_wait<0>();
  } else if (finisher) {
    // ================================================================== finishers
    const int y = tid - kTcRole;
    const int r = y & 127, ch = y >> 7;  // weight row (= tensor-memory lane); which 16 token columns
    float acc[NMAT][16];
    TcItem it;
    int item = 0, g = 0;
#pragma unroll 1
    for (int s = 0; s < n_steps; ++s) {
      const int buf = s & 1;
      if (g == 0) {
        it = tc_item(pv, prefix_s, ntasks, ntiles, (int)blockIdx.x + item * (int)gridDim.x);
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
          for (int j = 0; j < 16; ++j) acc[m][j] = 0.0f;
      }
      if (ok) ok = tc_mbar_wait(bars + buf * 8, (s >> 1) & 1);
      asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
      if (ok) {
        float sv[NMAT], cv[NMAT];  // the group's scale and b + 8 s, staged by the row's expander
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const unsigned char* src = sc_tiles + (((s >> 2) % kTcScSlots) * NMAT + m) * 2 * kTcScArr + r * 8 + (s & 3) * 2;
          sv[m] = __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src));
          cv[m] = fmaf(8.0f, sv[m], __bfloat162float(*reinterpret_cast<const __nv_bfloat16*>(src + kTcScArr)));
        }
        float dreg[NMAT][16];
        const uint32_t taddr = tmem_base + ((uint32_t)((wid & 3) * 32) << 16) + buf * NMAT * kTcTok + ch * 16;
#pragma unroll
        for (int m = 0; m < NMAT; ++m) tc_ld16(taddr + m * kTcTok, dreg[m]);
        float xs[16];
#pragma unroll
        for (int j4 = 0; j4 < 4; ++j4) {
          const float4 t4 = *reinterpret_cast<const float4*>(&xsum_s[buf][ch * 16 + 4 * j4]);
          xs[4 * j4] = t4.x, xs[4 * j4 + 1] = t4.y, xs[4 * j4 + 2] = t4.z, xs[4 * j4 + 3] = t4.w;
        }
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
        for (int j = 0; j < 16; ++j)
#pragma unroll
          for (int m = 0; m < NMAT; ++m) acc[m][j] = fmaf(sv[m], dreg[m][j], fmaf(cv[m], xs[j], acc[m][j]));
      }
      asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
      __syncwarp();
      if (lane == 0) tc_mbar_arrive(bars + 16 + buf * 8);  // the buffer's accumulator and token sums are free
      if (++g == ngroups) {
        // ---- end of the item: SwiGLU contract and bf16 stores
        const int n = it.n0 + r;
        if (ok && n < N) {
#pragma unroll
          for (int j = 0; j < 16; ++j) {
            const int tok = ch * 16 + j;
            if (tok < it.nt) {
              float v;
              if (NMAT == 2)
                v = swiglu_epilogue(p.epilogue, acc[0][j], acc[NMAT - 1][j]);
              else
                v = acc[0][j];
              const int dst = pv.row_dst[it.off + it.t0 + tok];
              p.out[(size_t)dst * p.ldo + n] = __float2bfloat16_rn(v);
            }
          }
        }
        g = 0;
        ++item;
      }
    }
  }
  else if (lane == 0) {
    // ================================================================== the thread that issues the MMAs
#pragma unroll 1
    for (int s = 0; s < n_steps; ++s) {
      const int buf = s & 1;
      if (ok) ok = tc_mbar_wait(bars + 32 + buf * 8, (s >> 1) & 1);  // tiles, token sums, scales of the step
      if (ok) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint64_t bdesc = tc_desc(tc_smem_u32(b_tiles + buf * kTcBTile));
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const uint64_t adesc = tc_desc(tc_smem_u32(a_tiles + (buf * NMAT + m) * kTcATile));
#pragma unroll
          for (int k = 0; k < 4; ++k)  // 16 values = 32 bytes further along K inside the swizzled row
            tc_mma(tmem_base + (buf * NMAT + m) * kTcTok, adesc + 2 * k, bdesc + 2 * k, idesc, k > 0);
        }
        tc_commit(bars + buf * 8);
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
  (void)rows_hint;
  TcParams tp;
  tp.q = q;
  tp.nmat = nmat;
  const size_t smem = 1024 + (size_t)2 * nmat * kTcATile + 2 * kTcBTile + (size_t)kTcRing * (nmat * kTcRawW + kTcRawX) +
                      (size_t)kTcScSlots * nmat * 2 * kTcScArr;
  int sms = 0, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess ||
      cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
    return fail(ZMOE_ERR_CUDA, "%s: SM count query failed", who);
  // one CTA per SM, fewer when the work list is shorter: token blocks <= rows / 32 + tasks
  const long long ntiles = (q.N + kTcRows - 1) / kTcRows;
  const long long items = ntiles * ((long long)q.rows / kTcTok + max_groups);
  const int grid = (int)(items < sms ? items : sms);
  cudaError_t e;
  if (nmat == 2) {
    e = cudaFuncSetAttribute(qmm_tc_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = launch_pdl(qmm_tc_kernel<2>, dim3(grid), dim3(kTcThreads), smem, st, tp);
  } else {
    e = cudaFuncSetAttribute(qmm_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess) e = launch_pdl(qmm_tc_kernel<1>, dim3(grid), dim3(kTcThreads), smem, st, tp);
  }
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "%s: tensor-memory kernel launch failed: %s", who, cudaGetErrorString(e));
  return check_launch("qmm_tc_kernel");
}

}  // namespace zmoe
