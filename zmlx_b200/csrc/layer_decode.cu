// One MoE block for a handful of decode tokens in ONE launch: router linear, top-k, fused gate/up + SwiGLU,
// down projection, ordered weighted combine, shared expert.
//
// A persistent grid of one CTA per SM.  Each CTA is 16 consumer warps (four teams of four) plus one PRODUCER
// warp per team that does nothing but issue asynchronous copies (cp.async) of packed expert weights into a ring of shared-memory
// stages (one mbarrier pair per stage).  The producer runs ahead of the math: it starts with the shared
// expert's first tiles before the routing is known, follows the routed gate/up tiles with the down-projection
// tiles without a pause, and so keeps >100 KB per SM in flight across every phase boundary.  There is no
// grid-wide barrier: what one CTA produces for the others travels as tagged 32-bit "hand-over words" that a
// consumer re-reads until they carry the current launch's tag.
//
//   routing   the router linear is spread over the grid (one expert row per CTA at a time, its 16 warps take
//             one segment of the row each); logits are published as hand-over words; every CTA waits for
//             them and repeats the top-k of the T rows (cheap, and it spares a second exchange);
//   gate/up   items (task, 16 weight rows of gate and of up) are dealt round-robin over the grid, the shared
//             expert's first; a team owns an item, its four warps split K; h = SwiGLU is published as
//             hand-over words;
//   down      items (task, 32 output columns) are cut into contiguous, equally long ranges per CTA (so a CTA
//             needs the h rows of one or two tasks only); projected rows y are published as hand-over words;
//   combine   64 output elements per half-warp pair anywhere in the grid: wait for the K (+ shared) words of
//             an element, combine them in slot order under the block's rounding contract.
//
// The matmul core: a stage holds 32 row segments of up to 512 bytes (16 groups of 64 codes).  A lane reads
// 8 bytes of rows g and g+8 and turns each packed word into four half2 operands with four lop3, ONE shift and two
// exact fp16 subtractions:
//     (w & 0x000F000F) | 0x64006400 = (1024 + q0, 1024 + q4), minus 1024 = (q0, q4)
//     (w & 0x00F000F0) | 0x64006400 = (1024 + 16 q1, 1024 + 16 q5), and the same on w >> 8 for q2, q6, q3, q7
// (fp16 has ten mantissa bits, so a code at bit 4 still lands inside the mantissa of 1024).  The token rows are
// staged in shared memory as fp16 in the matching order, the odd positions pre-divided by 16, after a
// per-row power-of-two scale that puts the row maximum in [2^14, 2^15) (exact for every element within 2^-24
// of the maximum; bf16 has 8 significant bits, fp16 11).  Products are exact, accumulation is fp32
// (mma.sync m16n8k16).  The offset left on the odd positions, the group scale and the group bias are applied per
// group in fp32:
//     sum_k x_k (q_k s + b) = s * (D - C) + b * X,   D = the mma sum, C = 64 sum_odd x, X = sum x.
// Spare mma columns carry other groups (column multiplexing, see qmm.cu).  Scales and biases are read straight
// from L1/L2 into registers one block of groups ahead.
//
// Every wait on another warp, CTA or copy is bounded: when the limit is hit the warp records it in the status
// word and leaves; the producer then waits (bounded) for its copies in flight before the CTA ends.
#include <cuda_fp16.h>

#include <mutex>
#include <type_traits>

#include "layer_route.cuh"
#include "qmm_common.cuh"

namespace zmoe {

constexpr int kLdTeams = 4;                          // teams of consumer warps; a team owns one item at a time
#ifndef ZMOE_LD_SEG_BYTES
#define ZMOE_LD_SEG_BYTES 512
#endif
constexpr int kLdSegBytes = ZMOE_LD_SEG_BYTES;       // bytes of one weight row in one stage (256 or 512).  A team holds
                                                     // one stage while it computes, so smaller stages leave more of
                                                     // the ring in flight
constexpr int kLdSegGroups = kLdSegBytes / 32;       // groups of 64 codes of a row in one stage
constexpr int kLdGW = kLdSegGroups / 4;              // ... of which each warp of the team takes this many
constexpr int kLdSegStride = kLdSegBytes + 32;       // == 32 mod 128: the 8-byte fragment reads of a warp hit all banks once
constexpr int kLdScOff = 32 * kLdSegStride;          // after the 32 row segments of a stage: their scales and biases,
constexpr int kLdScRow = kLdSegGroups * 2;           // [scale | bias][matrix][row 0..15][groups of the stage] bfloat16
constexpr int kLdScBytes = 64 * kLdScRow;
constexpr int kLdSlotBytes = kLdScOff + kLdScBytes;  // one stage
static_assert(kLdSegBytes == 256 || kLdSegBytes == 512, "stage geometry");
constexpr int kLdMaxDepth = 8;                       // stages per team at most
constexpr int kLdSmemLimit = 227 * 1024;
constexpr int kLdMaxMine = 4;                        // router rows per CTA at most (E <= 4 * grid)
constexpr int kLdMaxRanks = 8;                       // GPUs of an expert-parallel group at most

struct LdBank {
  const uint32_t* w[2];
  const __nv_bfloat16* s[2];
  const __nv_bfloat16* b[2];
};

struct LdParams {
  const __nv_bfloat16* x;
  int ldx, T;
  const __nv_bfloat16* wr;
  const float* rbias;
  int family, renorm, n_group, topk_group;
  float scale;
  int E, d, f, K;
  LdBank gu, dn, sgu, sdn;  // routed gate/up, routed down, shared gate/up, shared down
  int n_shared;
  int epi, sepi;  // SwiGLU contract of routed / shared experts (1: CPU contract, 2: per-op)
  int combine_mode, out_flags;
  int withhold;  // test hook: expert 0's logit is never published, so every wait for it runs out
  int pdl;       // regular launch with programmatic dependent launch instead of a cooperative one
  int hrows;     // h rows a CTA stages at most for its share of the down projection
  int slots;     // ring stages of a CTA (dealt to the four teams)
  // expert parallel: this GPU holds experts e_lo .. e_lo + e_cnt - 1 (the banks' rows 0 ..), brings T of the
  // T * ep_world tokens and has an inbox in which every rank deposits token rows and projected rows
  int ep_world, ep_rank, e_lo, e_cnt;
  int use_inbox;             // token rows are read from the inbox (ep_world > 1, or the single-GPU test of that path)
  uint32_t* inbox[kLdMaxRanks];  // every rank's inbox: [2 launch parities][T * ep_world rows][d] token words, then
                                 // [2][T * K + T rows][d] projected-row words; NULL when there is none
  int* sync;         // {-, -, sign-in count, status, launch count}
  uint32_t* logits;  // (T, E) hand-over words, each repeated eight times (one 32-byte sector per logit)
  uint32_t* h;       // (rows, f) hand-over words
  uint32_t* y;       // (rows, d) hand-over words
  float* weights;
  uint32_t* indices;
  void* out;
  long long* stamps;  // debug: CTA 0 records its cycle counter at the phase boundaries (NULL: off)
};

struct LdMeta {
  int n_tasks, n_routed, n_h;
  int idx[kLdMaxRouted];
  float w[kLdMaxRouted];
  int rank[kLdMaxRouted];
  int task_expert[kLdMaxTasks];
  int task_cnt[kLdMaxTasks];
  unsigned char task_rows[kLdMaxTasks][kLdMaxT];
  unsigned char hlist[kLdMaxRouted + kLdMaxT];  // staged h row -> row of the (rows, f) buffer
  unsigned char hloc[kLdMaxRouted + kLdMaxT];   // and back
};

struct LdSmem {
  int xs, xsum, isig, rowmax, route, rbias, meta, red, flags, bars, zero, ring, total;
};

__host__ __device__ inline int ld_align16(int a) { return (a + 15) & ~15; }

// Shared-memory carve-up, identical on host and device.  hrows and slots come from the host (ld_plan).
__host__ __device__ inline LdSmem ld_smem(int T, int K, int E, int d, int f, int hrows, int slots) {
  LdSmem m;
  const int ngd = d / 64, ngf = f / 64;
  int a = 0;
  m.xs = a;  // token rows (gate/up), later the staged h rows (down): fp16, fragment order
  const int xs1 = T * qmm_xs_stride(d), xs2 = hrows * qmm_xs_stride(f);
  a += ld_align16(xs1 > xs2 ? xs1 : xs2);
  m.xsum = a;  // per (group, row): {sum x, 64 sum_odd x}
  const int su1 = ngd * T, su2 = ngf * hrows;
  a += ld_align16((su1 > su2 ? su1 : su2) * 8);
  const int nr = T > hrows ? T : hrows;
  m.isig = a;  // per staged row: 1 / its power-of-two scale
  a += ld_align16(nr * 4);
  m.rowmax = a;
  a += ld_align16(nr * 4);
  m.rbias = a;  // the router's selection bias (a constant: copied in before the dependency wait)
  a += ld_align16(E * 4);
  m.meta = a;
  a += ld_align16((int)sizeof(LdMeta));
  m.red = a;  // K-split partial sums of the teams (and the router's segment sums before that)
  a += kLdTeams * 3 * 32 * 8 * 4;
  m.flags = a;  // [0] a wait ran out; [1..4] items whose partial sums a team's first warp has read;
  a += 128;     // [8 + 3 team + w] items whose partial sums warp w+1 of the team has written
  m.bars = a;   // full[team][stage], empty[team][stage], routing done
  a += (2 * kLdTeams * kLdMaxDepth + 1) * 8 + 8;
  m.zero = a;  // 32 zero bytes: the B fragment of columns that carry another group
  a += 32;
  a = (a + 127) & ~127;
  m.ring = a;
  a += slots * kLdSlotBytes;
  m.total = a;
  // Routing scratch (per row: sort keys, scores, logits, group scratch, winners) lives in the stages of teams
  // 1..3: before the routing is known only team 0's producer copies anything (the shared expert's first tiles),
  // and the scratch is dead once the task list is published.
  m.route = m.ring + (slots / kLdTeams + (slots % kLdTeams ? 1 : 0)) * kLdSlotBytes;
  return m;
}

// ------------------------------------------------------------------ mbarriers and bulk copies
__device__ __forceinline__ uint32_t ld_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ld_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ld_mbar_arrive(uint32_t bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool ld_mbar_try(uint32_t bar, int parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
// The same test, but the hardware may suspend the warp inside it for a while (no issue slots burnt).
__device__ __forceinline__ bool ld_mbar_try_sleep(uint32_t bar, int parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
__device__ __forceinline__ unsigned long long ld_now_ns() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
constexpr unsigned long long kLdWaitNs = 1000000000ull;  // a wait that lasts a second has run out
// Bounded wait for a phase of an mbarrier; gives up early when another warp of the CTA has.
__device__ __forceinline__ bool ld_mbar_wait(uint32_t bar, int parity, const volatile int* flags) {
  if (ld_mbar_try(bar, parity)) return true;
  const unsigned long long t0 = ld_now_ns();
  for (;;) {
    if (ld_mbar_try_sleep(bar, parity)) return true;
    if (flags[0] || ld_now_ns() - t0 > kLdWaitNs) return false;
  }
}
// 16-byte asynchronous copy global -> shared (L2 only), and the arrival that fires on an mbarrier once all of
// the thread's earlier copies have landed.
// The packed weights are read once: they are marked "evict first" in L2 so that they do not push out what is
// re-read there (token rows, router logits, the hand-over words).
__device__ __forceinline__ unsigned long long ld_policy_evict_first() {
  unsigned long long pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ void ld_cp16(uint32_t dst, const void* src, unsigned long long pol) {
  asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "l"(pol)
               : "memory");
}
__device__ __forceinline__ void ld_cp8(uint32_t dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ void ld_cp_arrive(uint32_t bar) {
  asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
// Bounded wait until a flag in shared memory reaches `want`.
__device__ __forceinline__ bool ld_flag_wait(const volatile int* flag, int want, const volatile int* flags) {
  for (int i = 0; i < kLdSpinLimit; ++i) {
    if (*flag >= want) return true;
    if ((i & 1023) == 1023 && flags[0]) return false;
  }
  return false;
}

__device__ __forceinline__ void mma_f16_m16n8k16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                 uint32_t b0, uint32_t b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
// codes at bits [0,4) and [16,20) -> half2 (q, q'); codes at bits [4,8) and [20,24) -> half2
// (1024 + 16 q, 1024 + 16 q').  One LOP3 each, (w & mask) | 0x64006400, and one exact subtraction for the former.
__device__ __forceinline__ uint32_t deq_h_lo(uint32_t w) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x000F000F, 0x64006400, 0xEA;" : "=r"(r) : "r"(w));
  // (1024 + q) - 1024, exact: these codes reach the tensor core as the plain integers q.  Left as 1024 + q the
  // offset would ride through the fp32 accumulator as 1024 * sum(x) and cost the group sum several bits (measured:
  // six times more outputs beyond 1e-2 of the oracle, one of 143,360 beyond 2e-2); the other half of the codes
  // carries 64 * sum(x) only, like the bfloat16 form of the register-fed kernels.
  const __half2 k = __floats2half2_rn(1024.0f, 1024.0f);
  const __half2 v = __hsub2(*reinterpret_cast<__half2*>(&r), k);
  return *reinterpret_cast<const uint32_t*>(&v);
}
__device__ __forceinline__ uint32_t deq_h_hi(uint32_t w) {
  uint32_t r;
  asm("lop3.b32 %0, %1, 0x00F000F0, 0x64006400, 0xEA;" : "=r"(r) : "r"(w));
  return r;
}

template <int OFF>
__device__ __forceinline__ uint2 ld_lds64(uint32_t addr) {
  uint2 v;
  asm volatile("ld.shared.v2.u32 {%0,%1}, [%2+%3];" : "=r"(v.x), "=r"(v.y) : "r"(addr), "n"(OFF));
  return v;
}
template <int OFF>
__device__ __forceinline__ uint4 ld_lds128(uint32_t addr) {
  uint4 v;
  asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%5];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "r"(addr), "n"(OFF));
  return v;
}

// the same under a predicate: zeros, and no shared-memory access at all, where it is false
template <int OFF>
__device__ __forceinline__ uint4 ld_lds128_if(uint32_t addr, bool pred) {
  uint4 v = make_uint4(0u, 0u, 0u, 0u);
  asm volatile("{ .reg .pred p; setp.ne.b32 p, %5, 0; @p ld.shared.v4.u32 {%0,%1,%2,%3}, [%4+%6]; }"
               : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
               : "r"(addr), "r"((int)pred), "n"(OFF));
  return v;
}

#define LD_STAMP_NS(i)                                                                         \
  do {                                                                                         \
    if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.stamps[i] = (long long)ld_now_ns(); \
  } while (0)
#define LD_STAMP(i)                                                            \
  do {                                                                         \
    if (p.stamps != nullptr && blockIdx.x == 0 && threadIdx.x == 0) p.stamps[i] = clock64(); \
  } while (0)

// ------------------------------------------------------------------ staging of token rows
// nrows rows of K8 * 8 bfloat16 values go to shared memory as fp16 in fragment order, with the per-group sums
// the fix-up needs.  Pass 1 brings the raw rows in (TAGGED: the source holds hand-over words; a block of eight
// is re-read until its tags are the current launch's) and finds each row's largest magnitude; pass 2 scales
// by the row's power of two, converts and permutes in place.  Eight-element block k of a row (the codes of one
// packed word) becomes [x0, x4, x1/16, x5/16, x2, x6, x3/16, x7/16].  All consumer threads must call this;
// returns false when a wait ran out (every thread of the CTA sees flags[0] set after the last barrier).
// SYS: the words may have been written by another GPU (system-scope loads); words written on this GPU are read
// with device-scope loads, which are measurably cheaper.
// Pass 1: raw bfloat16 rows into shared memory (row t at xs + t * xs_stride, as stored) and each row's largest
// magnitude.
template <bool TAGGED, bool SYS = false>
__device__ __forceinline__ void ld_stage_pass1(unsigned char* xs, int xs_stride, int* rowmax, const void* src, int ld,
                                               const unsigned char* rowlist, int nrows, int K8, uint32_t tag,
                                               volatile int* flags, int* status) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int total = nrows * K8;
  if (tid < nrows) rowmax[tid] = 0;
  ld_csync();
#pragma unroll 1
  for (int base = (int)(tid & ~31u); base < total; base += kLdConsumers) {
    const int i = base + lane;
    int t = -1;
    uint32_t m = 0;
    if (i < total) {
      t = i / K8;
      const int blk = i - t * K8;
      uint4 v;
      if (TAGGED) {
        const uint32_t* w32 = reinterpret_cast<const uint32_t*>(src) + (size_t)(rowlist ? rowlist[t] : t) * ld + blk * 8;
        uint4 a, b;
        int spins = 0;
        for (;;) {
          a = SYS ? ld_relaxed_sys_v4(w32) : ld_relaxed_v4(w32);
          b = SYS ? ld_relaxed_sys_v4(w32 + 4) : ld_relaxed_v4(w32 + 4);
          const uint32_t bad = ((a.x ^ tag) | (a.y ^ tag) | (a.z ^ tag) | (a.w ^ tag) | (b.x ^ tag) | (b.y ^ tag) |
                                (b.z ^ tag) | (b.w ^ tag)) & 0xffff0000u;
          if (bad == 0u) break;
          ++spins;
          if (spins >= kLdSpinLimit || ((spins & 1023) == 1023 && flags[0])) {
            flags[0] = 1;
            atomicExch(status, 1);
            a = b = make_uint4(0u, 0u, 0u, 0u);
            break;
          }
        }
        v.x = (a.x & 0xffffu) | (a.y << 16);
        v.y = (a.z & 0xffffu) | (a.w << 16);
        v.z = (b.x & 0xffffu) | (b.y << 16);
        v.w = (b.z & 0xffffu) | (b.w << 16);
      } else {
        v = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(src) + (size_t)t * ld) + blk);
      }
      *reinterpret_cast<uint4*>(xs + t * xs_stride + blk * 16) = v;
      // magnitudes of bfloat16 order like their low 15 bits
      const uint32_t q[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int k = 0; k < 4; ++k) m = max(m, max(q[k] & 0x7fffu, (q[k] >> 16) & 0x7fffu));
    }
    // one shared-memory atomic per warp when the warp sits inside one row (the common case), else one per lane
    const int t0 = __shfl_sync(0xffffffffu, t, 0);
    if (__all_sync(0xffffffffu, t == t0 || t < 0)) {
      m = __reduce_max_sync(0xffffffffu, m);
      if (lane == 0 && t0 >= 0) atomicMax(rowmax + t0, (int)m);
    } else if (t >= 0) {
      atomicMax(rowmax + t, (int)m);
    }
  }
  ld_csync();
}

// Pass 2: scale by the row's power of two, convert, permute in place; group sums.
__device__ __forceinline__ void ld_stage_pass2(unsigned char* xs, int xs_stride, float2* xsum, int rs, float* isig,
                                               const int* rowmax, int nrows, int K8) {
  const int tid = threadIdx.x, lane = tid & 31;
  const int total = nrows * K8;
#pragma unroll 1
  for (int base = (int)(tid & ~31u); base < total; base += kLdConsumers) {
    const int i = base + lane;
    const bool ok = i < total;
    int t = 0, blk = 0;
    float se = 0.0f, so = 0.0f;
    if (ok) {
      t = i / K8;
      blk = i - t * K8;
      const int m = rowmax[t];
      const int e8 = m >> 7;  // biased exponent of the largest magnitude
      int sexp = (m == 0 || e8 == 255) ? 0 : 14 - (e8 - 127);
      sexp = max(-100, min(100, sexp));
      const float sigma = __uint_as_float((uint32_t)(sexp + 127) << 23);
      uint4* slot = reinterpret_cast<uint4*>(xs + t * xs_stride + blk * 16);
      const uint4 v = *slot;
      const uint32_t q[4] = {v.x, v.y, v.z, v.w};
      __half hv[8];
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const float lo = bf16_bits_to_float(q[k] & 0xffffu) * sigma;            // element 2k (even position)
        const float hi = bf16_bits_to_float(q[k] >> 16) * sigma * 0.0625f;      // element 2k+1 (odd position)
        hv[2 * k] = __float2half_rn(lo);
        hv[2 * k + 1] = __float2half_rn(hi);
        se += __half2float(hv[2 * k]);
        so += __half2float(hv[2 * k + 1]);
      }
      auto pack = [&](int a, int b) {
        return (uint32_t)__half_as_ushort(hv[a]) | ((uint32_t)__half_as_ushort(hv[b]) << 16);
      };
      uint4 o;
      o.x = pack(0, 4);
      o.y = pack(1, 5);
      o.z = pack(2, 6);
      o.w = pack(3, 7);
      *slot = o;
      if (blk == 0) isig[t] = __uint_as_float((uint32_t)(127 - sexp) << 23);
    }
    se += __shfl_xor_sync(0xffffffffu, se, 1);
    so += __shfl_xor_sync(0xffffffffu, so, 1);
    se += __shfl_xor_sync(0xffffffffu, se, 2);
    so += __shfl_xor_sync(0xffffffffu, so, 2);
    se += __shfl_xor_sync(0xffffffffu, se, 4);
    so += __shfl_xor_sync(0xffffffffu, so, 4);
    if (ok && (lane & 7) == 0) xsum[(blk >> 3) * rs + t] = make_float2(fmaf(16.0f, so, se), 1024.0f * so);
  }
  ld_csync();
}

template <bool TAGGED, bool SYS = false>
__device__ __forceinline__ void ld_stage_rows(unsigned char* xs, int xs_stride, float2* xsum, int rs, float* isig,
                                              int* rowmax, const void* src, int ld, const unsigned char* rowlist,
                                              int nrows, int K8, uint32_t tag, volatile int* flags, int* status) {
  ld_stage_pass1<TAGGED, SYS>(xs, xs_stride, rowmax, src, ld, rowlist, nrows, K8, tag, flags, status);
  ld_stage_pass2(xs, xs_stride, xsum, rs, isig, rowmax, nrows, K8);
}

// ------------------------------------------------------------------ what a consumer warp carries around
struct LdCtx {
  unsigned char* smem;
  LdMeta* meta;
  volatile int* flags;
  float* red;
  uint32_t bars, ring;  // shared-space addresses
  uint32_t tag;
  int team, wk, lane, g, tig;
  int depth, slot0;  // this team's stages: slot0 .. slot0 + depth - 1 of the ring
  int use, slot;     // position in the team's stage sequence: uses of the current slot so far, the slot
  int itn;           // items the team has finished
  bool alive;
};

__device__ __forceinline__ uint32_t ld_full_bar(uint32_t bars, int team, int s) {
  return bars + (team * kLdMaxDepth + s) * 8;
}
__device__ __forceinline__ uint32_t ld_empty_bar(uint32_t bars, int team, int s) {
  return bars + ((kLdTeams + team) * kLdMaxDepth + s) * 8;
}
__device__ __forceinline__ uint32_t ld_route_bar(uint32_t bars) { return bars + 2 * kLdTeams * kLdMaxDepth * 8; }

// Stream position p of a warp (kLdGW groups per chunk) -> group of the row: chunk p / kLdGW holds groups
// kLdSegGroups * chunk .., warp wk owns kLdGW consecutive ones of them.
__device__ __forceinline__ int ld_group_of(int p, int wk) {
  return (p / kLdGW) * kLdSegGroups + wk * kLdGW + (p % kLdGW);
}

// Scales and biases of a lane's column(s) from the stage's copy: sb[m][h][0] scale, [1] bias of row g + 8h of
// matrix m, for local group `gl` of the chunk.  With one token a lane's two columns are two adjacent
// groups (one 32-bit read brings both); otherwise both columns are the same group.
template <int TT>
__device__ __forceinline__ void ld_load_sb(uint32_t (&sb)[2][2][2], uint32_t sc, int g, int gl) {
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int h = 0; h < 2; ++h)
#pragma unroll
      for (int arr = 0; arr < 2; ++arr) {
        const uint32_t addr = sc + (uint32_t)(((arr * 2 + m) * 16 + g + 8 * h) * kLdScRow + gl * 2);
        if (TT == 1)
          asm volatile("ld.shared.u32 %0, [%1];" : "=r"(sb[m][h][arr]) : "r"(addr));
        else
          asm volatile("ld.shared.u16 %0, [%1];" : "=r"(sb[m][h][arr]) : "r"(addr));
      }
}

// Scale, bias and the offsets for the block of 8 / TT multiplexed groups that starts at stream position p0.
// Lane (g, tig) owns columns 2*tig and 2*tig+1; srow_c[c] is the staged row of column c's token (-1: none).
template <int TT>
__device__ __forceinline__ void ld_fixup(float (&acc)[2][4], const float (&dg)[2][2][4], const uint32_t (&sb)[2][2][2],
                                         const float2* xsum, int rs, const int (&srow_c)[2], int ng, int p0, int wk,
                                         int tig) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int G = ld_group_of(p0 + ((TT == 8) ? 0 : (2 * tig + c) / TT), wk);
    float2 xc = make_float2(0.0f, 0.0f);
    if (G < ng && srow_c[c] >= 0) xc = xsum[G * rs + srow_c[c]];
#pragma unroll
    for (int m = 0; m < 2; ++m)
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        const uint32_t sraw = sb[m][h][0], braw = sb[m][h][1];
        const float sv = __uint_as_float((TT == 1 && c == 1) ? (sraw & 0xffff0000u) : (sraw << 16));
        const float bv = __uint_as_float((TT == 1 && c == 1) ? (braw & 0xffff0000u) : (braw << 16));
        const float dsum = dg[m][0][h * 2 + c] + dg[m][1][h * 2 + c];
        acc[m][h * 2 + c] = fmaf(sv, dsum - xc.y, fmaf(bv, xc.x, acc[m][h * 2 + c]));
      }
  }
}

// One (task, tile) item of a team: every warp walks its quad of each chunk as the producer's copies land.
// DN = false: gate/up, matrices m = gate, up of rows n0 .. n0+15; DN = true: down, m = rows n0 + 16 m ..
// Leaves the K-split total of the team in the first warp's acc, columns folded back onto their tokens.
template <int TT, bool DN>
__device__ __forceinline__ void ld_item(LdCtx& c, float (&acc)[2][4], int K8, uint32_t xaddr, uint32_t zaddr,
                                        bool tok_ok, int slot_g, const float2* xsum, int rs,
                                        const int (&srow_c)[2]) {
  constexpr int GPB = 8 / TT;  // groups multiplexed into one accumulator
  (void)zaddr;
  const int ng = K8 >> 3;
  const int rb = K8 << 2;  // bytes of a weight row
  const int nch = (rb + kLdSegBytes - 1) / kLdSegBytes;
  const int wk = c.wk, g = c.g, tig = c.tig;
  float dg[2][2][4];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[m][j] = 0.0f;
      dg[m][0][j] = 0.0f;
      dg[m][1][j] = 0.0f;
    }
  uint32_t sb[2][2][2];
#pragma unroll
  for (int m = 0; m < 2; ++m)
#pragma unroll
    for (int h = 0; h < 2; ++h) sb[m][h][0] = sb[m][h][1] = 0u;
  int open_p0 = -1;  // first stream position of a block of multiplexed groups that still awaits its fix-up

#pragma unroll 1
  for (int ch = 0; ch < nch; ++ch) {
    // ---- wait for the stage (every lane polls: the data was written by the copy engine)
    const uint32_t full = ld_full_bar(c.bars, c.team, c.slot);
    if (c.alive && !ld_mbar_wait(full, c.use & 1, c.flags)) {
      c.alive = false;
      c.flags[0] = 1;
    }
    const bool have = c.alive && ((ch * kLdSegGroups + wk * kLdGW) * 32 < rb);  // the warp's groups exist in this row
    if (have) {
      const uint32_t stage = c.ring + (uint32_t)(c.slot0 + c.slot) * kLdSlotBytes;
      const uint32_t wbase = stage + g * kLdSegStride + wk * (kLdGW * 32) + tig * 8;
      const uint32_t xchunk = xaddr + (uint32_t)(ch * kLdSegGroups + wk * kLdGW) * 128;
      // slot (position inside the block of GPB multiplexed groups) of the chunk's first group
      const int slot0 = (GPB > kLdGW) ? (ch % (GPB / kLdGW > 0 ? GPB / kLdGW : 1)) * kLdGW : 0;
      // the slot of the lane's own column(s): its scales and biases are read while that group's stage is held
      const int qlane = (TT == 1) ? 2 * tig : ((TT == 8) ? 0 : (2 * tig) / TT);
      auto group = [&](auto jc) {
        constexpr int j = decltype(jc)::value;
        const int slot = (GPB > kLdGW) ? slot0 + j : (j % GPB);
        const int pos = ch * kLdGW + j;
        if (slot == qlane) ld_load_sb<TT>(sb, stage + kLdScOff, g, wk * kLdGW + j);
        // lanes whose column carries another group (or no token) feed zeros and skip the load
        const bool mine = tok_ok && (TT == 8 || slot_g == slot);
        const uint32_t xa = xchunk + j * 128;
        const uint4 xb0 = ld_lds128_if<0>(xa, mine);
        const uint4 xb1 = ld_lds128_if<16>(xa, mine);
#pragma unroll
        for (int m = 0; m < 2; ++m) {
          const uint2 wa = (m == 0) ? ld_lds64<j * 32>(wbase) : ld_lds64<16 * kLdSegStride + j * 32>(wbase);
          const uint2 wb = (m == 0) ? ld_lds64<8 * kLdSegStride + j * 32>(wbase)
                                    : ld_lds64<24 * kLdSegStride + j * 32>(wbase);
          const uint32_t wa8 = wa.x >> 8, wb8 = wb.x >> 8;
          mma_f16_m16n8k16(dg[m][0], deq_h_lo(wa.x), deq_h_lo(wb.x), deq_h_hi(wa.x), deq_h_hi(wb.x), xb0.x, xb0.y);
          mma_f16_m16n8k16(dg[m][1], deq_h_lo(wa8), deq_h_lo(wb8), deq_h_hi(wa8), deq_h_hi(wb8), xb0.z, xb0.w);
          const uint32_t wc8 = wa.y >> 8, wd8 = wb.y >> 8;
          mma_f16_m16n8k16(dg[m][0], deq_h_lo(wa.y), deq_h_lo(wb.y), deq_h_hi(wa.y), deq_h_hi(wb.y), xb1.x, xb1.y);
          mma_f16_m16n8k16(dg[m][1], deq_h_lo(wc8), deq_h_lo(wd8), deq_h_hi(wc8), deq_h_hi(wd8), xb1.z, xb1.w);
        }
        if (slot == GPB - 1) {
          ld_fixup<TT>(acc, dg, sb, xsum, rs, srow_c, ng, pos - (GPB - 1), wk, tig);
#pragma unroll
          for (int m = 0; m < 2; ++m)
#pragma unroll
            for (int jj = 0; jj < 4; ++jj) {
              dg[m][0][jj] = 0.0f;
              dg[m][1][jj] = 0.0f;
            }
          open_p0 = -1;
        } else {
          open_p0 = pos - slot;
        }
      };
      group(std::integral_constant<int, 0>{});
      group(std::integral_constant<int, 1>{});
      if constexpr (kLdGW == 4) {
        group(std::integral_constant<int, 2>{});
        group(std::integral_constant<int, 3>{});
      }
    }
    // ---- hand the stage back to the producer
    __syncwarp();
    if (c.alive && c.lane == 0) ld_mbar_arrive(ld_empty_bar(c.bars, c.team, c.slot));
    if (++c.slot == c.depth) {
      c.slot = 0;
      ++c.use;
    }
  }
  // a warp whose groups end inside a block of multiplexed groups (rows that are not a multiple of the block, or
  // a last chunk that holds groups of the team's first warps only) still owes that block its fix-up
  if (open_p0 >= 0 && c.alive) ld_fixup<TT>(acc, dg, sb, xsum, rs, srow_c, ng, open_p0, wk, tig);

  // ---- K-split: the partial sums of warps 1..3 go to the team's first warp in warp order
  const int it = c.itn++;
  if (c.alive) {
    if (wk != 0) {
      // the first warp must have read the previous item's sums before they are overwritten
      if (it > 0 && !ld_flag_wait(c.flags + 1 + c.team, it, c.flags)) {
        c.alive = false;
        c.flags[0] = 1;
      }
      float* mine = c.red + ((c.team * 3 + wk - 1) * 32 + c.lane) * 8;
#pragma unroll
      for (int m = 0; m < 2; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[m * 4 + j] = acc[m][j];
      __threadfence_block();
      __syncwarp();
      if (c.lane == 0) c.flags[8 + c.team * 3 + wk - 1] = it + 1;
    } else {
#pragma unroll 1
      for (int o = 1; o < 4; ++o) {
        if (c.alive && !ld_flag_wait(c.flags + 8 + c.team * 3 + o - 1, it + 1, c.flags)) {
          c.alive = false;
          c.flags[0] = 1;
        }
        __threadfence_block();
        const float* other = c.red + ((c.team * 3 + o - 1) * 32 + c.lane) * 8;
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][j] += other[m * 4 + j];
      }
      __threadfence_block();
      __syncwarp();
      if (c.lane == 0) c.flags[1 + c.team] = it + 1;
      // fold the multiplexed columns back onto their tokens: afterwards column col < TT holds token col
      if (TT < 8) {
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            if (TT == 1) {
              acc[m][h * 2] += acc[m][h * 2 + 1];
              acc[m][h * 2 + 1] = 0.0f;
            }
#pragma unroll
            for (int cc = 0; cc < 2; ++cc) {
              float v = acc[m][h * 2 + cc];
              if (TT <= 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
              v += __shfl_xor_sync(0xffffffffu, v, 2);
              acc[m][h * 2 + cc] = v;
            }
          }
      }
    }
  }
}

// ------------------------------------------------------------------ the kernel
// EP: the token rows come from, and the projected rows go to, the ranks' inboxes (expert parallel, or the one-GPU
// test of that data path).  The plain instance carries none of that code: the kernel is sensitive to its size.
template <int TT, bool EP>
__global__ void __launch_bounds__(kLdThreads, 1) layer_decode_kernel(const LdParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;
  // To tokens are this rank's own; T = To * ranks are routed here (expert parallel: every rank routes every token
  // and computes the (token, slot) rows whose expert it holds); tok0 is the first own token
  const int To = p.T, T = EP ? p.T * p.ep_world : p.T, tok0 = EP ? p.ep_rank * p.T : 0;
  const int K = p.K, E = p.E, d = p.d, f = p.f;
  const int R = T * K;
  const int nblocks = gridDim.x;
  const LdSmem lay = ld_smem(T, K, E, d, f, p.hrows, p.slots);
  volatile int* flags = reinterpret_cast<volatile int*>(smem + lay.flags);
  LdMeta* meta = reinterpret_cast<LdMeta*>(smem + lay.meta);
  const uint32_t bars = ld_smem_u32(smem + lay.bars);
  const uint32_t ring = ld_smem_u32(smem + lay.ring);
  const uint32_t smem_base = ld_smem_u32(smem);
  const int ntf = f >> 4;  // gate/up tiles of 16 rows per task
  const int ntd = d >> 5;  // down tiles of 32 rows per task
  const int nch_gu = ((d >> 1) + kLdSegBytes - 1) / kLdSegBytes;
  const int nch_dn = ((f >> 1) + kLdSegBytes - 1) / kLdSegBytes;
  // stages of team t: depth_of(t) consecutive slots from slot0_of(t)
  const int dbase = p.slots / kLdTeams, dextra = p.slots % kLdTeams;

  LD_STAMP_NS(10);
  // Router rows are constants: a consumer warp's pieces of the CTA's first two rows are requested before anything
  // that depends on the previous kernel of the stream, so that with programmatic dependent launch their HBM
  // latency hides behind that kernel.
  const int nvec = d >> 3;
  uint4 wpre[2][2];
  if (wid < kLdWarps) {
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        const int e = blockIdx.x + nblocks * k;
        const int i = wid * 32 + lane + 32 * kRouterSegs * r;
        wpre[k][r] = (e < E && i < nvec) ? __ldg(reinterpret_cast<const uint4*>(p.wr + (size_t)e * d) + i)
                                         : make_uint4(0u, 0u, 0u, 0u);
      }
  }
  if (tid == 0) {
    for (int t = 0; t < kLdTeams; ++t)
      for (int s = 0; s < kLdMaxDepth; ++s) {
        ld_mbar_init(ld_full_bar(bars, t, s), 32);  // one arrival per producer lane, when its copies have landed
        ld_mbar_init(ld_empty_bar(bars, t, s), 4);
      }
    ld_mbar_init(ld_route_bar(bars), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }
  if (tid < 32) flags[tid] = 0;
  if (tid < 8) reinterpret_cast<uint32_t*>(smem + lay.zero)[tid] = 0u;
  if (p.rbias != nullptr)
    for (int i = tid; i < E; i += kLdThreads) reinterpret_cast<float*>(smem + lay.rbias)[i] = __ldg(p.rbias + i);
  for (int i = tid; i < kLdMaxTasks; i += kLdThreads) meta->task_cnt[i] = 0;
  __syncthreads();
  if (p.pdl) pdl_trigger();  // the next kernel of the stream may be set up now; it waits for this one to finish

  // =================================================================== producer warp
  if (wid >= kLdWarps) {
    // producer warp of team t: walks the team's stage sequence (its gate/up items chunk by chunk, then its
    // down-projection items) and fills a stage as soon as the team has handed it back
    const int t = wid - kLdWarps;
    const int depth = dbase + (t < dextra ? 1 : 0);
    const int slot0 = t * dbase + min(t, dextra);
    const int K8g = d >> 3, K8d = f >> 3;
    const unsigned long long pol = ld_policy_evict_first();
    // The shared expert's tiles come first in the gate/up order and do not depend on the routing: when this
    // CTA's first item is one of them, team 0's producer copies its chunks before the routing is known.
    int total = (t == 0 && p.n_shared && (int)blockIdx.x < ntf) ? nch_gu : 0;
    const int free_jobs = total;  // stages that need no task list
    int ngu = 1, n_routed = 0, dn_lo = 0;
    bool ok = true;
    int j = 0;
    for (;; ++j) {
      if (j == free_jobs) {
        // from here on the task list is needed
        ok = ld_mbar_wait(ld_route_bar(bars), 0, flags) && flags[0] == 0;
        if (!ok) break;
        const int n_tasks = meta->n_tasks;
        n_routed = meta->n_routed;
        const int items_gu = n_tasks * ntf;
        const int nq_gu = (items_gu > (int)blockIdx.x) ? (items_gu - 1 - (int)blockIdx.x) / nblocks + 1 : 0;
        const long long items_dn = (long long)n_tasks * ntd;
        dn_lo = (int)(items_dn * blockIdx.x / nblocks);
        const int nq_dn = (int)(items_dn * (blockIdx.x + 1) / nblocks) - dn_lo;
        ngu = (nq_gu > t) ? (nq_gu - 1 - t) / kLdTeams + 1 : 0;
        const int ndn = (nq_dn > t) ? (nq_dn - 1 - t) / kLdTeams + 1 : 0;
        total = ngu * nch_gu + ndn * nch_dn;
      }
      if (j >= total) break;
      const int s = j % depth, use = j / depth;
      ok = ld_mbar_wait(ld_empty_bar(bars, t, s), (use & 1) ^ 1, flags);
      if (!ok) break;
      // ---- which chunk of which item
      const bool dn = j >= ngu * nch_gu;
      int ch, e, n0;
      bool sh;
      if (!dn) {
        const int qi = j / nch_gu;
        ch = j - qi * nch_gu;
        const int i = (int)blockIdx.x + (t + kLdTeams * qi) * nblocks;
        const int ao = i / ntf;
        sh = p.n_shared && ao == 0;
        e = sh ? 0 : meta->task_expert[ao - (p.n_shared ? 1 : 0)];
        n0 = (i - ao * ntf) << 4;
      } else {
        const int jj = j - ngu * nch_gu;
        const int qi = jj / nch_dn;
        ch = jj - qi * nch_dn;
        const int i = dn_lo + t + kLdTeams * qi;
        const int a = i / ntd;
        sh = a >= n_routed;
        e = meta->task_expert[a];
        n0 = (i - a * ntd) << 5;
      }
      // ---- the copies: one instruction moves one 512-byte row segment (16 bytes per lane), eight more move the
      // rows' scales and biases (8 bytes per lane); the stage's barrier gets one arrival per lane when that
      // lane's copies have landed
      const LdBank& bank = dn ? (sh ? p.sdn : p.dn) : (sh ? p.sgu : p.gu);
      const int K8 = dn ? K8d : K8g;
      const int N = dn ? d : f;
      const int rb = K8 << 2, ng = K8 >> 3;
      const int bytes = min(kLdSegBytes, rb - ch * kLdSegBytes);
      const uint32_t stage = ring + (uint32_t)(slot0 + s) * kLdSlotBytes;
      const size_t row0 = (size_t)e * N + n0;
      {
        // weights: 16 bytes per lane; kLdSegBytes / 16 lanes cover one row segment
        constexpr int LPS = kLdSegBytes / 16, SPI = 32 / LPS;  // lanes per segment, segments per instruction
        const int piece = lane % LPS, sub = lane / LPS;
        const uint32_t dst = stage + sub * kLdSegStride + piece * 16;
        const size_t off = row0 * rb + (size_t)ch * kLdSegBytes + (size_t)sub * rb + piece * 16;
        const unsigned char* src0 = reinterpret_cast<const unsigned char*>(bank.w[0]) + off;
        const unsigned char* src1 =
            dn ? src0 + (size_t)16 * rb : reinterpret_cast<const unsigned char*>(bank.w[1]) + off;
        if (piece * 16 < bytes) {
#pragma unroll
          for (int r = 0; r < 16; r += SPI) ld_cp16(dst + r * kLdSegStride, src0 + (size_t)r * rb, pol);
#pragma unroll
          for (int r = 0; r < 16; r += SPI) ld_cp16(dst + (16 + r) * kLdSegStride, src1 + (size_t)r * rb, pol);
        }
      }
      {
        // scales and biases: 8 bytes per lane; kLdScRow / 8 lanes cover the groups of one row of one tensor
        constexpr int PPP = kLdScRow / 8, RPI = 32 / PPP;  // parts per piece, rows per instruction
        const int part = lane % PPP, srow = lane / PPP;
        if (part * 4 < (bytes >> 5)) {
          const uint32_t dst = stage + kLdScOff + srow * kLdScRow + part * 8;
          const size_t off = (row0 + srow) * ng + ch * kLdSegGroups + part * 4;  // elements
#pragma unroll
          for (int it = 0; it < 64 / RPI; ++it) {
            const int am = (it * RPI) >> 4, r0 = (it * RPI) & 15;  // tensor (scale | bias, matrix), first row
            const int m = am & 1;
            const __nv_bfloat16* base = ((am >> 1) ? bank.b : bank.s)[dn ? 0 : m];
            ld_cp8(dst + (am * 16 + r0) * kLdScRow, base + off + (size_t)((dn ? m * 16 : 0) + r0) * ng);
          }
        }
      }
      ld_cp_arrive(ld_full_bar(bars, t, s));
    }
    if (!ok && lane == 0) {
      flags[0] = 1;
      atomicExch(p.sync + 3, 1);
    }
    // copies still in flight must have landed before the CTA's shared memory goes away
    for (int k = max(0, j - depth); k < j; ++k) {
      const uint32_t bar = ld_full_bar(bars, t, k % depth);
      const int par = (k / depth) & 1;
      for (int i = 0; i < kLdSpinLimit && !ld_mbar_try(bar, par); ++i) {
      }
    }
    return;
  }

  // =================================================================== consumer warps
  const int g = lane >> 2;
  const int tig = lane & 3;
  const int slot_g = g / TT;
  const int tok_g = g % TT;
  unsigned char* xs = smem + lay.xs;
  float2* xsum = reinterpret_cast<float2*>(smem + lay.xsum);
  float* isig = reinterpret_cast<float*>(smem + lay.isig);
  int* rowmax = reinterpret_cast<int*>(smem + lay.rowmax);
  float* red = reinterpret_cast<float*>(smem + lay.red);
  uint2* keys = reinterpret_cast<uint2*>(smem + lay.route);  // 8-byte aligned: the region starts 16-byte aligned
  float* vals = reinterpret_cast<float*>(keys + T * E);
  float* lgs = vals + T * E;
  float* gsc = lgs + T * E;
  int* sel_idx = reinterpret_cast<int*>(gsc + T * 64);
  const float* rbias = p.rbias != nullptr ? reinterpret_cast<const float*>(smem + lay.rbias) : nullptr;

  if (p.pdl) pdl_wait();  // nothing below may run before the previous kernel has finished and flushed
  // launch count: every consumer thread reads it here; the last CTA to sign in (below) bumps it for the next
  // launch; tag of this launch's words
  LD_STAMP_NS(11);
  const int epoch = __ldcg(p.sync + 4);
  const uint32_t tag = (uint32_t)((epoch % 65535) + 1) << 16;

  LD_STAMP(0);
  // inbox regions of this launch (they alternate with the launch parity, so that a rank that is one launch ahead
  // never overwrites words a slower rank still reads)
  const size_t xwords = (size_t)T * d, ywords = (size_t)(To * K + To) * d;
  const size_t x_off = (size_t)(epoch & 1) * xwords, y_off = 2 * xwords + (size_t)(epoch & 1) * ywords;
  const uint32_t* xin = EP ? p.inbox[p.ep_rank] + x_off : nullptr;
  uint32_t* yown = EP ? p.inbox[p.ep_rank] + y_off : p.y;  // where this rank's projected rows arrive
  if (EP && (int)blockIdx.x < p.ep_world) {
    // ---- this rank's token rows go to rank blockIdx.x's inbox as tagged words (plain peer stores)
    uint32_t* dst = p.inbox[blockIdx.x] + x_off + (size_t)tok0 * d;
    for (int i = tid; i < To * nvec; i += kLdConsumers) {
      const int t = i / nvec, v = i - t * nvec;
      const uint4 xv = __ldg(reinterpret_cast<const uint4*>(p.x + (size_t)t * p.ldx) + v);
      uint32_t* o = dst + (size_t)t * d + v * 8;
      st_relaxed_sys_v4(o, make_uint4(tag | (xv.x & 0xffffu), tag | (xv.x >> 16), tag | (xv.y & 0xffffu), tag | (xv.y >> 16)));
      st_relaxed_sys_v4(o + 4, make_uint4(tag | (xv.z & 0xffffu), tag | (xv.z >> 16), tag | (xv.w & 0xffffu), tag | (xv.w >> 16)));
    }
  }
  // ---- token rows -> shared memory as stored (pass 1 of the staging; in the expert-parallel form this is where
  // the launch waits for the other ranks' rows); the router reads them from there
  if (EP)
    ld_stage_pass1<true, true>(xs, qmm_xs_stride(d), rowmax, xin, d, nullptr, T, d >> 3, tag, flags, p.sync + 3);
  else
    ld_stage_pass1<false>(xs, qmm_xs_stride(d), rowmax, p.x, p.ldx, nullptr, T, d >> 3, 0u, flags, p.sync + 3);
  const int xs_stride_x = qmm_xs_stride(d);
  auto x8 = [&](int t, int v) -> uint4 { return *reinterpret_cast<const uint4*>(xs + t * xs_stride_x + v * 16); };
  // ---- router linear: the CTA's rows blockIdx.x, blockIdx.x + grid, ...; warp w sums segment w of a row
  {
    int n_mine = 0;
    for (int k = 0; k < kLdMaxMine; ++k) n_mine += ((int)blockIdx.x + nblocks * k < E);
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      const int e = blockIdx.x + nblocks * k;
      if (e < E) {
        const uint4* wrow = reinterpret_cast<const uint4*>(p.wr + (size_t)e * d);
#pragma unroll 1
        for (int t = 0; t < T; ++t) {
          float acc = 0.0f;
#pragma unroll
          for (int r = 0; r < 2; ++r) {
            const int i = wid * 32 + lane + 32 * kRouterSegs * r;
            if (i < nvec) acc = router_fma8(wpre[k][r], x8(t, i), acc);
          }
          for (int i = wid * 32 + lane + 64 * kRouterSegs; i < nvec; i += 32 * kRouterSegs)
            acc = router_fma8(__ldg(wrow + i), x8(t, i), acc);
          acc = warp_sum(acc);
          if (lane == 0) red[(k * T + t) * kRouterSegs + wid] = acc;
        }
      }
    }
#pragma unroll 1
    for (int k = 2; k < n_mine; ++k) {
      const int e = blockIdx.x + nblocks * k;
      const uint4* wrow = reinterpret_cast<const uint4*>(p.wr + (size_t)e * d);
      for (int t = 0; t < T; ++t) {
        float acc = 0.0f;
        for (int i = wid * 32 + lane; i < nvec; i += 32 * kRouterSegs) acc = router_fma8(__ldg(wrow + i), x8(t, i), acc);
        acc = warp_sum(acc);
        if (lane == 0) red[(k * T + t) * kRouterSegs + wid] = acc;
      }
    }
    ld_csync();
    if (tid < n_mine * T) {
      const int k = tid / T, t = tid - k * T;
      const int e = blockIdx.x + nblocks * k;
      const int nseg = min(kRouterSegs, (nvec + 31) >> 5);
      float total = 0.0f;
      for (int s = 0; s < nseg; ++s) total += red[(k * T + t) * kRouterSegs + s];
      // eight copies = one full 32-byte sector: L2 holds it whole and never has to merge it with a stale copy
      // from HBM when the other CTAs read it
      if (!(p.withhold && e == 0)) {
        uint32_t* dst = p.logits + ((size_t)t * E + e) * 8;
        const uint32_t word = tag | float_to_bf16_bits(total);
        st_relaxed_v4(dst, word);
        st_relaxed_v4(dst + 4, word);
      }
    }
  }
  LD_STAMP(1);
  // Launch count for the next launch.  Every consumer thread of this CTA has read the count (they all passed
  // the barriers above), so the CTA can sign in; the last CTA of the grid to do so bumps the count (the tags of
  // THIS launch live in registers already) and clears the sign-in counter.
  if (tid == 0) {
    if (atomicAdd(p.sync + 2, 1) == nblocks - 1) {
      p.sync[4] = epoch + 1;
      p.sync[2] = 0;
    }
  }

  // ---- the staged rows become fp16 in fragment order with their group sums (pass 2), while the logits travel
  ld_stage_pass2(xs, qmm_xs_stride(d), xsum, T, isig, rowmax, T, d >> 3);
  LD_STAMP(2);
  // ---- routing of every row, repeated by every CTA (one warp per row); the logits arrive as hand-over words,
  // so this is also where the CTA waits for the router threads of the other CTAs
  // the sigmoid family with no groups, or with groups of 32 experts, is routed by one warp per row in registers
  const bool warp_route = p.family == 2 && E <= 256 && (p.n_group == 1 || E == 32 * p.n_group);
  if (wid < T) {
    const bool okr = ld_route_scores(p.logits + (size_t)wid * E * 8, tag, E, p.family, rbias, vals + wid * E,
                                     lgs + wid * E, keys + wid * E, lane);
    if (!okr && lane == 0) {
      flags[0] = 1;
      atomicExch(p.sync + 3, 1);
    }
    if (okr && warp_route) {
      __syncwarp();
      ld_sigmoid_route_warp(E, K, rbias, p.n_group, p.topk_group, lgs + wid * E, sel_idx + wid * K, lane);
    }
  }
  ld_csync();
  LD_STAMP(3);
  if (!warp_route) {
    if (p.family == 2) {
      ld_sigmoid_scores(T, E, rbias, p.n_group, p.topk_group, vals, lgs, keys, gsc);
      ld_csync();
    }
    if (T * E <= 128)  // uniform over the CTA
      ld_rank_select(keys, T, E, K, sel_idx);
    else
      ld_topk_select(keys, T, E, K, reinterpret_cast<uint32_t*>(red), reinterpret_cast<int*>(red) + T * 64, sel_idx);
    ld_csync();
  }
  LD_STAMP(4);
  if (wid < T && flags[0] == 0)
    ld_finish_row(vals + wid * E, lgs + wid * E, K, p.family, p.renorm, p.scale, sel_idx + wid * K, meta->w + wid * K,
                  meta->idx + wid * K, lane);
  if (T == 1) {
    // one token: its K experts are distinct, so slot a is task a
    if (tid < K) {  // lanes of warp 0: each reads back the slot it has just written itself
      meta->task_expert[tid] = meta->idx[tid];
      meta->task_cnt[tid] = 1;
      meta->task_rows[tid][0] = (unsigned char)tid;
    }
    if (tid == 0) {
      meta->n_routed = K;
      meta->n_tasks = K + (p.n_shared ? 1 : 0);
      if (p.n_shared) {
        meta->task_expert[K] = 0;
        meta->task_cnt[K] = 1;
        meta->task_rows[K][0] = (unsigned char)R;
      }
    }
  }
  ld_csync();
  if (T > 1 && flags[0] == 0) {
    // tasks = distinct experts THIS rank holds, in order of first use; a task's rows in row order.  Rows whose
    // expert lives on another rank are that rank's work (rank -1 marks them).
    const int e_hi = p.e_lo + p.e_cnt;
    if (tid < R) {
      const int e = meta->idx[tid];
      int rk = 0;
      for (int r = 0; r < tid; ++r) rk += (meta->idx[r] == e);
      meta->rank[tid] = (e >= p.e_lo && e < e_hi) ? rk : -1;
    }
    ld_csync();
    if (tid < R && meta->rank[tid] >= 0) {
      const int e = meta->idx[tid];
      int r0 = 0;
      while (meta->idx[r0] != e) ++r0;  // first row of this expert (r0 <= tid)
      int tk = 0;
      for (int r = 0; r < r0; ++r) tk += (meta->rank[r] == 0);
      const int rk = meta->rank[tid];
      if (rk == 0) meta->task_expert[tk] = e - p.e_lo;  // row of the rank's own banks
      if (rk < kLdMaxT) meta->task_rows[tk][rk] = (unsigned char)tid;
      atomicAdd(&meta->task_cnt[tk], 1);
    }
    if (tid == 0) {
      int n = 0;
      for (int r = 0; r < R; ++r) n += (meta->rank[r] == 0);
      meta->n_routed = n;
      meta->n_tasks = n + (p.n_shared ? 1 : 0);
      if (p.n_shared) {  // the shared expert runs for the rank's own tokens
        meta->task_expert[n] = 0;
        meta->task_cnt[n] = To;
        for (int t = 0; t < To; ++t) meta->task_rows[n][t] = (unsigned char)(R + t);
      }
    }
    ld_csync();
  } else if (T > 1) {
    ld_csync();
    ld_csync();
  }
  // the producer may read the task list now (it also looks at flags[0])
  if (tid == 0) ld_mbar_arrive(ld_route_bar(bars));
  LD_STAMP(5);

  LdCtx c;
  c.smem = smem;
  c.meta = meta;
  c.flags = flags;
  c.red = red;
  c.bars = bars;
  c.ring = ring;
  c.tag = tag;
  c.team = wid >> 2;
  c.wk = wid & 3;
  c.lane = lane;
  c.g = g;
  c.tig = tig;
  c.depth = dbase + (c.team < dextra ? 1 : 0);
  c.slot0 = c.team * dbase + min(c.team, dextra);
  c.use = 0;
  c.slot = 0;
  c.itn = 0;
  c.alive = (flags[0] == 0);
  const int n_tasks = c.alive ? meta->n_tasks : 0;
  const int n_routed = c.alive ? meta->n_routed : 0;
  if (c.alive && blockIdx.x == 0 && tid < To * K) {  // the routing of the rank's own tokens
    if (p.weights) p.weights[tid] = meta->w[tok0 * K + tid];
    if (p.indices) p.indices[tid] = (uint32_t)meta->idx[tok0 * K + tid];
  }

  // ---- gate/up + SwiGLU: item i = blockIdx.x + q * grid, the CTA's q-th item goes to team q % 4
  {
    const int items = n_tasks * ntf;
    const int nq = (items > (int)blockIdx.x) ? (items - 1 - (int)blockIdx.x) / nblocks + 1 : 0;
    const int xs_stride = qmm_xs_stride(d);
#pragma unroll 1
    for (int q = c.team; q < nq; q += kLdTeams) {
      const int i = (int)blockIdx.x + q * nblocks;
      const int ao = i / ntf, tile = i - ao * ntf;
      const int a = p.n_shared ? (ao == 0 ? n_routed : ao - 1) : ao;
      const bool is_sh = a >= n_routed;
      const int n0 = tile << 4;
      const int cnt = meta->task_cnt[a];
      // token of a task row: routed row r belongs to token r / K, shared row R + t to token t
      const bool tok_ok = tok_g < cnt;
      int trow = 0;
      if (tok_ok) {
        const int r = meta->task_rows[a][tok_g];
        trow = is_sh ? tok0 + r - R : r / K;
      }
      int srow_c[2];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int sl = (2 * tig + cc) % TT;
        srow_c[cc] = -1;
        if (sl < cnt) {
          const int r = meta->task_rows[a][sl];
          srow_c[cc] = is_sh ? tok0 + r - R : r / K;
        }
      }
      float acc[2][4];
      ld_item<TT, false>(c, acc, d >> 3, smem_base + lay.xs + trow * xs_stride + tig * 32, smem_base + lay.zero, tok_ok, slot_g, xsum, T,
                         srow_c);
      if (c.alive && c.wk == 0) {
        const int epi = is_sh ? p.sepi : p.epi;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int col = 2 * tig + (j & 1);
          const bool writer = (TT == 8) || (col < TT);
          if (writer && col < cnt) {
            const int dst = meta->task_rows[a][col];
            const float inv = isig[is_sh ? tok0 + dst - R : dst / K];
            const float gv = acc[0][j] * inv, uv = acc[1][j] * inv;
            const float v = (epi == 2) ? swiglu_per_op(gv, uv) : swiglu_cpu_contract(gv, uv);
            st_relaxed_u32(p.h + (size_t)dst * f + n0 + g + ((j >> 1) ? 8 : 0), tag | float_to_bf16_bits(v));
          }
        }
      }
    }
  }
  LD_STAMP(6);

  // ---- down projection: items (task, 32 columns) in task-major order, cut into equal contiguous ranges per
  // CTA; the CTA stages the h rows of the tasks its range touches (this is where it waits for the gate/up
  // tiles of the other CTAs)
  const long long items_dn = (long long)n_tasks * ntd;
  const int dn_lo = (int)(items_dn * blockIdx.x / nblocks), dn_hi = (int)(items_dn * (blockIdx.x + 1) / nblocks);
  ld_csync();  // every team is done with the token rows
  if (tid == 0) {
    int n = 0;
    if (c.alive && dn_hi > dn_lo) {
      for (int a = dn_lo / ntd; a <= (dn_hi - 1) / ntd; ++a)
        for (int r = 0; r < meta->task_cnt[a] && r < kLdMaxT; ++r) {
          const int row = meta->task_rows[a][r];
          if (n < p.hrows) {
            meta->hlist[n] = (unsigned char)row;
            meta->hloc[row] = (unsigned char)n;
          }
          ++n;
        }
      if (n > p.hrows) {  // cannot happen with the host's sizing; never overrun shared memory
        flags[0] = 1;
        atomicExch(p.sync + 3, 1);
        n = 0;
      }
    }
    meta->n_h = n;
  }
  ld_csync();
  const int n_h = meta->n_h;
  ld_stage_rows<true>(xs, qmm_xs_stride(f), xsum, p.hrows, isig, rowmax, p.h, f, meta->hlist, n_h, f >> 3, tag, flags,
                      p.sync + 3);
  LD_STAMP(7);
  if (flags[0]) c.alive = false;
  {
    const int nq = c.alive ? dn_hi - dn_lo : 0;
    const int xs_stride = qmm_xs_stride(f);
#pragma unroll 1
    for (int q = c.team; q < nq; q += kLdTeams) {
      const int i = dn_lo + q;
      const int a = i / ntd, tile = i - a * ntd;
      const int n0 = tile << 5;
      const int cnt = meta->task_cnt[a];
      const bool tok_ok = tok_g < cnt;
      const int srow = tok_ok ? (int)meta->hloc[meta->task_rows[a][tok_g]] : 0;
      int srow_c[2];
#pragma unroll
      for (int cc = 0; cc < 2; ++cc) {
        const int sl = (2 * tig + cc) % TT;
        srow_c[cc] = (sl < cnt) ? (int)meta->hloc[meta->task_rows[a][sl]] : -1;
      }
      float acc[2][4];
      ld_item<TT, true>(c, acc, f >> 3, smem_base + lay.xs + srow * xs_stride + tig * 32, smem_base + lay.zero, tok_ok, slot_g, xsum, p.hrows,
                        srow_c);
      if (c.alive && c.wk == 0) {
#pragma unroll
        for (int m = 0; m < 2; ++m)
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int col = 2 * tig + (j & 1);
            const bool writer = (TT == 8) || (col < TT);
            if (writer && col < cnt) {
              const int dst = meta->task_rows[a][col];
              const float v = acc[m][j] * isig[meta->hloc[dst]];
              // the row goes to its token's home rank: routed row of token tg, slot i -> row tl * K + i there
              // (tl = the token's number on that rank); a shared row stays here, after the routed rows
              uint32_t* yrow;
              if (!EP || dst >= R) {
                yrow = yown + (size_t)dst * d;  // (a shared row: To * K + dst - R, and R = To * K without peers)
                if (EP && dst >= R) yrow = yown + (size_t)(To * K + dst - R) * d;
              } else {
                const int tg = dst / K, home = tg / To;
                yrow = (p.ep_world > 1 ? p.inbox[home] + y_off : yown) + (size_t)((tg - home * To) * K + dst - tg * K) * d;
              }
              uint32_t* yw = yrow + n0 + m * 16 + g + ((j >> 1) ? 8 : 0);
              if (EP)
                st_relaxed_sys_u32(yw, tag | float_to_bf16_bits(v));
              else
                st_relaxed_u32(yw, tag | float_to_bf16_bits(v));
            }
          }
      }
    }
  }
  LD_STAMP(8);

  // ---- ordered combine: 64 output elements per unit, units dealt over the grid; a thread waits for the K
  // (+ shared) projected values of its element (rounded to T, as the separate-kernel path stores them)
  if (flags[0] == 0) {
    const int units = (To * d) >> 6;
    const int mode = p.combine_mode;
    const bool sys_words = EP;  // peers store into this rank's inbox: system-scope polls
    for (int u = (int)blockIdx.x + nblocks * (tid >> 6); u < units; u += nblocks * (kLdConsumers >> 6)) {
      const int o = (u << 6) + (tid & 63);
      const int t = o / d, n = o - t * d;
      uint32_t yw[kLdMaxK + 1];
      int spins = 0;
      bool okc;
      do {
        okc = true;
#pragma unroll
        for (int i = 0; i < kLdMaxK + 1; ++i) {
          yw[i] = tag;
          const uint32_t* src = nullptr;
          if (i < K) src = yown + (size_t)(t * K + i) * d + n;
          if (i == kLdMaxK && p.n_shared) src = yown + (size_t)(To * K + t) * d + n;
          if (src != nullptr) yw[i] = sys_words ? ld_relaxed_sys_u32(src) : ld_relaxed_u32(src);
          okc = okc && ((yw[i] & 0xffff0000u) == tag);
        }
        ++spins;
      } while (!okc && spins < kLdSpinLimit && !((spins & 1023) == 1023 && flags[0]));
      if (!okc) {
        flags[0] = 1;
        atomicExch(p.sync + 3, 1);
        break;
      }
      float a0 = 0.0f;
#pragma unroll
      for (int i = 0; i < kLdMaxK; ++i) {
        if (i < K) {
          float wi = meta->w[(tok0 + t) * K + i];
          if (p.out_flags & 2) wi = round_bf16(wi);
          const float v0 = bf16_bits_to_float(yw[i] & 0xffffu);
          if (mode == ZMOE_COMBINE_FP32 || mode == ZMOE_COMBINE_T) {
            a0 = fmaf(wi, v0, a0);
          } else if (mode == ZMOE_COMBINE_FP32_NO_FMA || mode == ZMOE_COMBINE_NO_FMA) {
            a0 = __fadd_rn(a0, __fmul_rn(wi, v0));
          } else if (mode == ZMOE_COMBINE_EXACT) {
            wi = round_bf16(wi);
            a0 = round_bf16(__fadd_rn(a0, round_bf16(__fmul_rn(wi, v0))));
          } else {
            a0 = round_bf16(__fadd_rn(a0, __fmul_rn(wi, v0)));
          }
        }
      }
      const bool fp32_mode = (mode == ZMOE_COMBINE_FP32 || mode == ZMOE_COMBINE_FP32_NO_FMA);
      if (fp32_mode && !(p.out_flags & 1)) {
        reinterpret_cast<float*>(p.out)[o] = a0;
      } else {
        a0 = round_bf16(a0);
        if (p.n_shared) a0 = __fadd_rn(a0, bf16_bits_to_float(yw[kLdMaxK] & 0xffffu));
        reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(a0);
      }
    }
  }
  LD_STAMP(9);
  LD_STAMP_NS(12);
}

// ------------------------------------------------------------------ host side
constexpr int kLdMaxDevices = 64;
static std::mutex g_ld_mutex;
static int g_ld_sms[kLdMaxDevices] = {};

static int ld_sm_count(int* out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kLdMaxDevices)
    return fail(ZMOE_ERR_UNSUPPORTED, "zmoe_layer_decode: device ordinal %d beyond %d", dev, kLdMaxDevices);
  std::lock_guard<std::mutex> lock(g_ld_mutex);
  if (g_ld_sms[dev] == 0) {
    int n = 0;
    e = cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
    if (e != cudaSuccess || n <= 0)
      return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode: SM count query failed: %s", cudaGetErrorString(e));
    g_ld_sms[dev] = n;
  }
  *out = g_ld_sms[dev];
  return ZMOE_OK;
}

struct LdPlan {
  int hrows, slots;
  LdSmem lay;
};

// Sizes that depend on the grid: the h rows one CTA's share of the down projection can touch, and how many
// ring stages fit beside everything else.  Returns why the shape cannot take the one-launch path (nullptr: it can).
static int ld_world(const zmoe_layer_desc* L) { return L->ep_world > 1 ? L->ep_world : 1; }

// T = the rank's own tokens; the kernel routes T * ep_world of them.
static const char* ld_plan(const zmoe_layer_desc* L, int T_own, int sms, LdPlan* out) {
  const int world = ld_world(L);
  if (world > kLdMaxRanks || L->ep_rank < 0 || L->ep_rank >= world) return "takes at most 8 ranks";
  if (L->E % world != 0) return "needs the expert count to be a multiple of the rank count";
  const int T = T_own * world;
  if (L->qmode != ZMOE_Q_AFFINE4 || L->group_size != 64) return "needs 4-bit affine weights with group size 64";
  if (T_own < 1 || T > kLdMaxT) return "takes 1..8 tokens (over all ranks)";
  if (L->top_k < 1 || L->top_k > kLdMaxK) return "takes top_k <= 8";
  if (L->E < L->top_k || L->E > 256) return "takes at most 256 experts";
  if (L->d_model % 256 != 0 || L->d_ff % 256 != 0) return "needs d_model and d_ff to be multiples of 256";
  if (L->n_shared < 0 || L->n_shared > 1) return "takes at most one shared expert";
  if (sms * kLdMaxMine < L->E) return "needs a GPU with more SMs for this many experts";
  const int rtot = T * L->top_k + (L->n_shared ? T_own : 0);
  int routed_max = T * L->top_k;
  if (routed_max > L->E / world) routed_max = L->E / world;
  const long long items = (long long)(routed_max + (L->n_shared ? 1 : 0)) * (L->d_model / 32);
  const int per_cta = (int)((items + sms - 1) / sms);
  const int span = per_cta > 0 ? (per_cta - 1) / (L->d_model / 32) + 2 : 1;  // tasks a contiguous range can touch
  int hrows = span * T;
  if (hrows > rtot) hrows = rtot;
  const LdSmem fixed = ld_smem(T, L->top_k, L->E, L->d_model, L->d_ff, hrows, 0);
  int slots = (kLdSmemLimit - fixed.total) / kLdSlotBytes;
  if (slots > kLdTeams * kLdMaxDepth) slots = kLdTeams * kLdMaxDepth;
  if (slots < kLdTeams) return "needs more shared memory than an SM has";
  const int route_bytes = ld_align16(T * (4 * L->E + 64 + kLdMaxK) * 4);
  if ((slots - (slots / kLdTeams + (slots % kLdTeams ? 1 : 0))) * kLdSlotBytes < route_bytes)
    return "needs more shared memory than an SM has";
  out->hrows = hrows;
  out->slots = slots;
  out->lay = ld_smem(T, L->top_k, L->E, L->d_model, L->d_ff, hrows, slots);
  return nullptr;
}

static size_t ld_ws_logits_off() { return 256; }
static size_t ld_ws_h_off(const zmoe_layer_desc* L, int T_own) {
  return (ld_ws_logits_off() + (size_t)T_own * ld_world(L) * L->E * 32 + 255) & ~(size_t)255;
}
static size_t ld_ws_y_off(const zmoe_layer_desc* L, int T_own) {
  const size_t rows = (size_t)T_own * ld_world(L) * L->top_k + (L->n_shared ? T_own : 0);
  return (ld_ws_h_off(L, T_own) + rows * L->d_ff * 4 + 255) & ~(size_t)255;
}

template <int TT, bool EP>
static int ld_launch(const LdParams& p, int grid, size_t smem_bytes, cudaStream_t st) {
  auto kern = layer_decode_kernel<TT, EP>;
  cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_bytes);
  if (e != cudaSuccess)
    return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode: shared memory of %zu bytes refused: %s", smem_bytes,
                cudaGetErrorString(e));
  if (p.pdl) {
    // regular launch, one CTA per SM by its size; the caller vouches that no other work holds SMs for long
    e = launch_pdl(kern, dim3(grid), dim3(kLdThreads), smem_bytes, st, p);
    if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode: launch failed: %s", cudaGetErrorString(e));
    return check_launch("layer_decode_kernel");
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid);
  cfg.blockDim = dim3(kLdThreads);
  cfg.dynamicSmemBytes = smem_bytes;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident at once: the waits between CTAs rely on it
  attr[0].val.cooperative = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  e = cudaLaunchKernelEx(&cfg, kern, p);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode: launch failed: %s", cudaGetErrorString(e));
  return check_launch("layer_decode_kernel");
}

}  // namespace zmoe

using namespace zmoe;

extern "C" {

size_t zmoe_layer_decode_workspace_bytes(const zmoe_layer_desc* L, int T) {
  if (!L) return 0;
  int sms = 0;
  if (ld_sm_count(&sms) != ZMOE_OK) return 0;
  LdPlan plan;
  if (ld_plan(L, T, sms, &plan)) return 0;
  const size_t rows = (size_t)T * L->top_k + (L->n_shared ? T : 0);  // the rank's own projected rows
  return ld_ws_y_off(L, T) + rows * L->d_model * 4;
}

size_t zmoe_layer_decode_inbox_bytes(const zmoe_layer_desc* L, int T) {
  if (!L || T < 1) return 0;
  const size_t world = (size_t)ld_world(L);
  const size_t xwords = (size_t)T * world * L->d_model;
  const size_t ywords = ((size_t)T * L->top_k + T) * L->d_model;
  return 2 * (xwords + ywords) * sizeof(uint32_t);
}

int zmoe_layer_decode_status(const void* workspace, int clear, void* stream) {
  ZMOE_REQUIRE(workspace != nullptr, ZMOE_ERR_SHAPE, "zmoe_layer_decode_status: null workspace");
  cudaStream_t st = (cudaStream_t)stream;
  int word = 0;
  int* dev = (int*)workspace + 3;
  cudaError_t e = cudaMemcpyAsync(&word, dev, sizeof(int), cudaMemcpyDeviceToHost, st);
  if (e == cudaSuccess) e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode_status: %s", cudaGetErrorString(e));
  if (word == 0) return ZMOE_OK;
  if (clear) {
    e = cudaMemsetAsync(dev, 0, sizeof(int), st);
    if (e != cudaSuccess) return fail(ZMOE_ERR_CUDA, "zmoe_layer_decode_status: %s", cudaGetErrorString(e));
  }
  return fail(ZMOE_ERR_TIMEOUT,
              "zmoe_layer_decode: a bounded wait ran out in an earlier launch on this workspace (its output is void)");
}

int zmoe_layer_decode(const zmoe_layer_desc* L, const void* x, int ldx, int T, void* workspace,
                      size_t workspace_bytes, float* weights, uint32_t* indices, void* out, void* stream) {
  ZMOE_REQUIRE(L && x && workspace && out, ZMOE_ERR_SHAPE, "zmoe_layer_decode: null pointer");
  int sms = 0;
  int rc = ld_sm_count(&sms);
  if (rc != ZMOE_OK) return rc;
  LdPlan plan;
  const char* why = ld_plan(L, T, sms, &plan);
  ZMOE_REQUIRE(why == nullptr, ZMOE_ERR_UNSUPPORTED, "zmoe_layer_decode: the one-launch path %s", why);
  ZMOE_REQUIRE(L->router_w && L->routed.gate_w && L->routed.gate_scales && L->routed.gate_biases && L->routed.up_w &&
                   L->routed.up_scales && L->routed.up_biases && L->routed.down_w && L->routed.down_scales &&
                   L->routed.down_biases,
               ZMOE_ERR_SHAPE, "zmoe_layer_decode: null router or expert tensor");
  if (L->n_shared)
    ZMOE_REQUIRE(L->shared.gate_w && L->shared.gate_scales && L->shared.gate_biases && L->shared.up_w &&
                     L->shared.up_scales && L->shared.up_biases && L->shared.down_w && L->shared.down_scales &&
                     L->shared.down_biases,
                 ZMOE_ERR_SHAPE, "zmoe_layer_decode: null shared-expert tensor");
  ZMOE_REQUIRE(L->router_family >= 0 && L->router_family <= 2, ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: router family %d", L->router_family);
  if (L->router_family == 2) {
    ZMOE_REQUIRE(L->router_bias != nullptr, ZMOE_ERR_SHAPE, "zmoe_layer_decode: the sigmoid router needs a bias");
    ZMOE_REQUIRE(L->n_group >= 1 && L->n_group <= 32 && L->topk_group >= 1 && L->topk_group <= L->n_group &&
                     L->E % L->n_group == 0,
                 ZMOE_ERR_SHAPE, "zmoe_layer_decode: invalid n_group=%d / topk_group=%d", L->n_group, L->topk_group);
  }
  ZMOE_REQUIRE(!(L->router_family == 0 && L->router_bias), ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: a bias needs the softmax-then-top-k family");
  ZMOE_REQUIRE(L->swiglu_mode == ZMOE_SWIGLU_CPU || L->swiglu_mode == ZMOE_SWIGLU_PER_OP, ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: swiglu_mode %d", L->swiglu_mode);
  ZMOE_REQUIRE(!L->n_shared || L->shared_swiglu_mode == ZMOE_SWIGLU_CPU || L->shared_swiglu_mode == ZMOE_SWIGLU_PER_OP,
               ZMOE_ERR_UNSUPPORTED, "zmoe_layer_decode: shared_swiglu_mode %d", L->shared_swiglu_mode);
  ZMOE_REQUIRE(L->combine_mode >= ZMOE_COMBINE_FP32 && L->combine_mode <= ZMOE_COMBINE_STREAM_T, ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: combine mode %d", L->combine_mode);
  const bool fp32_out = (L->combine_mode == ZMOE_COMBINE_FP32 || L->combine_mode == ZMOE_COMBINE_FP32_NO_FMA) &&
                        !(L->out_flags & 1);
  ZMOE_REQUIRE(!(L->n_shared && fp32_out), ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: a shared expert needs an output in T");
  ZMOE_REQUIRE(ldx >= L->d_model && ldx % 8 == 0 && ((uintptr_t)x % 16) == 0, ZMOE_ERR_ALIGN,
               "zmoe_layer_decode: x rows must be 16-byte aligned (ldx=%d)", ldx);
  ZMOE_REQUIRE(((uintptr_t)L->router_w % 16) == 0 && ((uintptr_t)workspace % 256) == 0, ZMOE_ERR_ALIGN,
               "zmoe_layer_decode: router_w must be 16-byte and the workspace 256-byte aligned");
  const zmoe_expert_bank* banks[2] = {&L->routed, L->n_shared ? &L->shared : nullptr};
  for (int i = 0; i < 2; ++i) {
    if (!banks[i]) continue;
    const void* wptr[3] = {banks[i]->gate_w, banks[i]->up_w, banks[i]->down_w};
    for (int j = 0; j < 3; ++j)
      ZMOE_REQUIRE(((uintptr_t)wptr[j] % 16) == 0, ZMOE_ERR_ALIGN,
                   "zmoe_layer_decode: packed weights must be 16-byte aligned (they are fetched by bulk copies)");
    const void* sptr[6] = {banks[i]->gate_scales, banks[i]->gate_biases, banks[i]->up_scales,
                           banks[i]->up_biases,   banks[i]->down_scales, banks[i]->down_biases};
    for (int j = 0; j < 6; ++j)
      ZMOE_REQUIRE(((uintptr_t)sptr[j] % 8) == 0, ZMOE_ERR_ALIGN,
                   "zmoe_layer_decode: scales and biases must be 8-byte aligned");
  }
  const size_t need = zmoe_layer_decode_workspace_bytes(L, T);
  ZMOE_REQUIRE(workspace_bytes >= need, ZMOE_ERR_WORKSPACE, "zmoe_layer_decode: workspace of %zu bytes, need %zu",
               workspace_bytes, need);
  ZMOE_REQUIRE(L->launch_mode == 0 || L->launch_mode == 1, ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: launch_mode %d", L->launch_mode);

  LdParams p;
  p.x = (const __nv_bfloat16*)x;
  p.ldx = ldx;
  p.T = T;
  p.wr = (const __nv_bfloat16*)L->router_w;
  p.rbias = L->router_bias;
  p.family = L->router_family;
  p.renorm = L->renorm;
  p.n_group = L->n_group;
  p.topk_group = L->topk_group;
  p.scale = (L->router_family == 2) ? L->routed_scale : 1.0f;
  p.E = L->E;
  p.d = L->d_model;
  p.f = L->d_ff;
  p.K = L->top_k;
  auto fill = [](LdBank& gu, LdBank& dn, const zmoe_expert_bank& b) {
    gu.w[0] = b.gate_w;
    gu.w[1] = b.up_w;
    gu.s[0] = (const __nv_bfloat16*)b.gate_scales;
    gu.s[1] = (const __nv_bfloat16*)b.up_scales;
    gu.b[0] = (const __nv_bfloat16*)b.gate_biases;
    gu.b[1] = (const __nv_bfloat16*)b.up_biases;
    dn.w[0] = dn.w[1] = b.down_w;
    dn.s[0] = dn.s[1] = (const __nv_bfloat16*)b.down_scales;
    dn.b[0] = dn.b[1] = (const __nv_bfloat16*)b.down_biases;
  };
  fill(p.gu, p.dn, L->routed);
  fill(p.sgu, p.sdn, L->n_shared ? L->shared : L->routed);
  p.n_shared = L->n_shared;
  p.epi = L->swiglu_mode == ZMOE_SWIGLU_CPU ? 1 : 2;
  p.sepi = L->shared_swiglu_mode == ZMOE_SWIGLU_CPU ? 1 : 2;
  p.combine_mode = L->combine_mode;
  p.out_flags = L->out_flags;
  p.pdl = L->launch_mode;
  p.withhold = (L->debug_flags & ZMOE_DEBUG_WITHHOLD_LOGIT) ? 1 : 0;
  p.stamps = (long long*)L->debug_stamps;
  p.hrows = plan.hrows;
  p.slots = plan.slots;
  const int world = ld_world(L);
  p.ep_world = world;
  p.ep_rank = world > 1 ? L->ep_rank : 0;
  p.e_cnt = L->E / world;
  p.e_lo = p.ep_rank * p.e_cnt;
  p.use_inbox = (world > 1 || (L->debug_flags & ZMOE_DEBUG_FORCE_INBOX)) ? 1 : 0;
  for (int r = 0; r < kLdMaxRanks; ++r) p.inbox[r] = (r < world) ? (uint32_t*)L->ep_inbox[r] : nullptr;
  if (p.use_inbox)
    for (int r = 0; r < world; ++r)
      ZMOE_REQUIRE(p.inbox[r] != nullptr && ((uintptr_t)p.inbox[r] % 16) == 0, ZMOE_ERR_SHAPE,
                   "zmoe_layer_decode: ep_inbox[%d] must be a 16-byte aligned buffer of "
                   "zmoe_layer_decode_inbox_bytes() bytes (zeroed before its first use)", r);
  unsigned char* ws = (unsigned char*)workspace;
  p.sync = (int*)ws;
  p.logits = (uint32_t*)(ws + ld_ws_logits_off());
  p.h = (uint32_t*)(ws + ld_ws_h_off(L, T));
  p.y = (uint32_t*)(ws + ld_ws_y_off(L, T));
  p.weights = weights;
  p.indices = indices;
  p.out = out;

  cudaStream_t st = (cudaStream_t)stream;
  const size_t smem_bytes = (size_t)plan.lay.total;
  const int Tt = T * world;  // rows of one task at most
  if (p.use_inbox) {
    if (Tt == 1) return ld_launch<1, true>(p, sms, smem_bytes, st);
    if (Tt <= 2) return ld_launch<2, true>(p, sms, smem_bytes, st);
    if (Tt <= 4) return ld_launch<4, true>(p, sms, smem_bytes, st);
    return ld_launch<8, true>(p, sms, smem_bytes, st);
  }
  if (Tt == 1) return ld_launch<1, false>(p, sms, smem_bytes, st);
  if (Tt <= 2) return ld_launch<2, false>(p, sms, smem_bytes, st);
  if (Tt <= 4) return ld_launch<4, false>(p, sms, smem_bytes, st);
  return ld_launch<8, false>(p, sms, smem_bytes, st);
}

}  // extern "C"
