// One MoE block for a handful of decode tokens in ONE launch: router linear, top-k,
// fused gate/up + SwiGLU, down projection, ordered weighted combine, shared expert.
//
// The separate-kernel path pays four dependent launches per block; at one token each of
// them is a few microseconds of launch and pipeline-fill latency around ~1 us of memory
// traffic.  Here a persistent grid of one 512-thread CTA per SM (cooperative launch, so
// every CTA is resident) walks three phases.  There is no grid-wide barrier: what one CTA
// produces for the others travels as tagged 32-bit "hand-over words" that a consumer
// re-reads until they carry the current launch's tag.
//
//   phase 1  every CTA stages the T token rows in shared memory (they feed every gate/up
//            tile); the router linear runs one warp per expert row across the whole grid
//            and publishes each logit as a hand-over word;
//   phase 2  every CTA waits for the logits and repeats the top-k of the T rows (cheap,
//            and it spares a second exchange), derives the task list (distinct experts and
//            their rows) in shared memory; gate/up + SwiGLU tiles (task, 16 rows) are dealt
//            to groups of four warps across the grid; h rows are published as hand-over
//            words.  Each warp then already streams the first packed down-projection
//            weights: they depend on the routing only;
//   phase 3  every CTA waits for and stages all h rows, owns 16 output columns at a time,
//            computes them for every task (warps split tasks and K) and combines the K slots
//            of each token in slot order under the requested rounding contract.
//
// The matmul core is the one of qmm.cu: packed codes go from HBM to registers with 8-byte
// streaming loads (for one token an opt-in variant brings them to shared memory with
// cp.async.bulk instead), become bf16 (128 + q) with a shift and a lop3, and meet the token
// rows on the tensor cores (mma.sync m16n8k16, weights are the A operand); scale, bias and
// the 128 offset are applied per group in fp32; spare mma columns carry other groups
// (column multiplexing).  Every wait on another CTA is bounded: when the limit is hit the
// CTA records it in the status word and leaves.
#include <cstdlib>
#include <mutex>

#include "qmm_common.cuh"
#include "router_rows.cuh"

namespace zmoe {

constexpr int kLdThreads = 512;
constexpr int kLdWarps = kLdThreads / 32;
constexpr int kLdMaxT = 8;
constexpr int kLdMaxK = 8;
constexpr int kLdMaxRouted = kLdMaxT * kLdMaxK;      // (token, slot) rows
constexpr int kLdMaxTasks = kLdMaxRouted + 1;
// DPD (kernel template parameter): quads of packed weights a warp keeps in flight in the down projection: 2 when
// a warp's share of an item is two quads anyway (d_ff < 2048), 4 for long rows, where one warp streams a whole
// item and the bytes in flight per SM decide the bandwidth
constexpr bool kLdBulkByDefault = false;  // the bulk-copy form of the one-token kernel
constexpr int kLdSpinLimit = 1 << 21;  // polls of a hand-over word or mbarrier before a CTA gives up (~1 s)

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
  int withhold;           // test hook: expert 0's logit is never published, so every wait for it runs out
  int pdl;                // regular launch with programmatic dependent launch instead of a cooperative one
  int tiles_per_cta;      // upper bound of the 16-column output tiles one CTA owns (sizes ybuf)
  int bulk_off, g_slots;  // bulk-copy variant: byte offset of its shared-memory region, gate/up slots per CTA
  int* sync;         // {-, -, sign-in count, status, launch count}
  uint32_t* logits;  // (T, E) hand-over words, each repeated eight times (one 32-byte sector per logit)
  uint32_t* h;       // (rows, f) hand-over words
  float* weights;
  uint32_t* indices;
  void* out;
};

struct LdMeta {
  int n_tasks, n_routed;
  int idx[kLdMaxRouted];
  float w[kLdMaxRouted];
  int rank[kLdMaxRouted];
  int task_expert[kLdMaxTasks];
  int task_cnt[kLdMaxTasks];
  unsigned char task_rows[kLdMaxTasks][kLdMaxT];
};

struct LdSmem {
  int xs, xsum, sc, red, ybuf, route, meta, zero, total;
};

__host__ __device__ inline int ld_align16(int a) { return (a + 15) & ~15; }

__host__ __device__ inline LdSmem ld_smem(int T, int K, int E, int d, int f, int n_shared, int tiles_per_cta) {
  LdSmem m;
  const int rtot = T * K + (n_shared ? T : 0);
  const int ngd = d / 64, ngf = f / 64;
  int a = 0;
  m.xs = a;
  const int xs1 = T * qmm_xs_stride(d), xs2 = rtot * qmm_xs_stride(f);
  a += ld_align16(xs1 > xs2 ? xs1 : xs2);
  m.xsum = a;
  const int su1 = ngd * T, su2 = ngf * rtot;
  a += ld_align16((su1 > su2 ? su1 : su2) * 4);
  m.sc = a;
  const int sc1 = 4 * 4 * 16 * qmm_sc_stride(ngd);        // gate/up: 4 groups x {gate,up} x {scale,bias} x 16 rows
  const int sc2 = kLdWarps * 2 * 16 * qmm_sc_stride(ngf);  // down: up to 16 groups x {scale,bias} x 16 rows
  a += ld_align16(sc1 > sc2 ? sc1 : sc2);
  m.red = a;
  a += kLdWarps * 32 * 8 * 4;
  m.ybuf = a;
  a += ld_align16(tiles_per_cta * rtot * 16 * 4);  // projected rows of every output tile the CTA owns
  m.route = a;
  a += ld_align16(T * (4 * E + 64 + kLdMaxK) * 4);  // per row: scores, logits, sort keys, group scratch, winners
  m.meta = a;
  a += ld_align16((int)sizeof(LdMeta));
  m.zero = a;
  a += 32;
  m.total = a;
  return m;
}

// ------------------------------------------------------------------ warp-group barrier
__device__ __forceinline__ void ld_group_sync(int gid, int wk_count) {
  if (wk_count == 1)
    __syncwarp();
  else
    asm volatile("bar.sync %0, %1;" ::"r"(gid + 1), "r"(wk_count * 32) : "memory");
}

// ------------------------------------------------------------------ hand-over words
// Values that one CTA produces and others consume (router logits, h rows) travel as 32-bit words
// {launch tag : 16 | bfloat16 : 16}.  A consumer re-reads a word until its tag is the current launch's, so
// the value and its "ready" flag arrive in one relaxed access and no grid-wide barrier is needed.  The tag
// is 1 + (launch count mod 65535): never zero, so a zeroed workspace holds no valid word.
__device__ __forceinline__ uint32_t ld_relaxed_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_v4(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.gpu.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Order-preserving map float -> uint32 (for finite values and infinities; -0 must be folded into +0 first).
__device__ __forceinline__ uint32_t ld_order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ------------------------------------------------------------------ staging of token rows
// Rows go to shared memory with every 8-element block permuted to (0,4,1,5,2,6,3,7) -- the order in
// which a lane's two 16-byte reads give the B fragments of four k16 steps -- plus per-group sums.
// TAGGED: the source holds hand-over words (see below); a block is re-read until its eight tags are the
// current launch's.  Returns false when such a wait ran out.
template <bool TAGGED>
__device__ __forceinline__ bool ld_stage_rows(unsigned char* xs, int xs_stride, float* xsum, int xsum_stride,
                                              const void* src, int ld, int nrows, int K8, uint32_t tag) {
  const int total = nrows * K8;
  const int lane = threadIdx.x & 31;
  bool good = true;
#pragma unroll 1
  for (int base = (int)(threadIdx.x & ~31u); base < total; base += kLdThreads) {
    const int i = base + lane;
    const bool ok = i < total;
    uint4 v = make_uint4(0, 0, 0, 0);
    int t = 0, blk = 0;
    if (ok) {
      t = i / K8;
      blk = i - t * K8;
      if (TAGGED) {
        const uint32_t* w32 = reinterpret_cast<const uint32_t*>(src) + (size_t)t * ld + blk * 8;
        uint4 a, b;
        int spins = 0;
        for (;;) {
          a = ld_relaxed_v4(w32);
          b = ld_relaxed_v4(w32 + 4);
          const uint32_t bad = ((a.x ^ tag) | (a.y ^ tag) | (a.z ^ tag) | (a.w ^ tag) | (b.x ^ tag) | (b.y ^ tag) |
                                (b.z ^ tag) | (b.w ^ tag)) & 0xffff0000u;
          if (bad == 0u) break;
          if (++spins >= kLdSpinLimit) {
            good = false;
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
    if (ok && (lane & 7) == 0) xsum[(blk >> 3) * xsum_stride + t] = part;
  }
  return good;
}

// ------------------------------------------------------------------ routing of the T token rows
// Same arithmetic as the per-row router functions (softmax_topk_row / sigmoid_topk_row: the order of every
// floating-point sum is kept, so scores, indices and weights are bit-identical).  A single warp is slow at
// long dependent instruction sequences, so only what must be is done by one warp per row (waiting for the
// logits, the softmax / sigmoid scores, the weights of the winners); the selection itself -- ranking every
// score against every other one -- is spread over all threads of the CTA.
//
// Step 1, one warp per row: wait for the row's logits (hand-over words written by the router warps of all
// CTAs), compute the selection scores and leave, per expert, the score, the logit and a 64-bit sort key
// {order-preserving score : 32 | ~expert id : 32} in shared memory.  Returns false when the wait ran out.
__device__ __forceinline__ bool ld_route_scores(const uint32_t* g_logits, uint32_t tag, int E, int family,
                                                const float* bias, int n_group, int topk_group, float* vals,
                                                float* lgs, uint2* keys, float* gsc /* 64 floats */, int lane,
                                                long long* dbg = nullptr) {
  constexpr int NJ = 8;  // values per lane: E <= 256
  const int nj = (E + 31) >> 5;
  {
    uint32_t raw[NJ];
    int spins = 0;
    bool ok;
    do {
      ok = true;
#pragma unroll
      for (int j = 0; j < NJ; ++j) {
        raw[j] = tag;
        if (lane + 32 * j < E) raw[j] = ld_relaxed_u32(g_logits + (size_t)(lane + 32 * j) * 8);
        ok = ok && ((raw[j] & 0xffff0000u) == tag);
      }
      ok = __all_sync(0xffffffffu, ok);
    } while (!ok && ++spins < kLdSpinLimit);
    if (!ok) return false;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      if (lane + 32 * j < E) lgs[lane + 32 * j] = bf16_bits_to_float(raw[j] & 0xffffu);
    if (dbg && lane == 0) {
      dbg[22] = clock64();
      dbg[23] = spins;
    }
  }
  // From here on the loops over a lane's values stay rolled (they run once per launch: code size matters more
  // than overlap); every lane touches only its own entries lane, lane + 32, ... of the shared arrays.
  if (family == 0) {
#pragma unroll 1
    for (int j = 0; j < nj; ++j) {
      const int idx = lane + 32 * j;
      if (idx < E) vals[idx] = lgs[idx];
    }
  } else if (family == 1) {
    float mx = -CUDART_INF_F;
#pragma unroll 1
    for (int j = 0; j < nj; ++j) {
      const int idx = lane + 32 * j;
      if (idx < E) mx = fmaxf(mx, lgs[idx]);
    }
    mx = warp_max(mx);
    float sum = 0.0f;
#pragma unroll 1
    for (int j = 0; j < nj; ++j) {
      const int idx = lane + 32 * j;
      const float e = (idx < E) ? expf(lgs[idx] - mx) : 0.0f;
      if (idx < E) vals[idx] = e;
      sum += e;
    }
    sum = warp_sum(sum);
#pragma unroll 1
    for (int j = 0; j < nj; ++j) {
      const int idx = lane + 32 * j;
      if (idx < E) {
        float q = vals[idx] / sum;
        if (bias) q += bias[idx];
        vals[idx] = q;
      }
    }
  } else {
    return true;  // sigmoid family: the scores are computed by all threads (ld_sigmoid_scores)
  }
#pragma unroll 1
  for (int j = 0; j < nj; ++j) {
    const int idx = lane + 32 * j;
    if (idx < E) keys[idx] = make_uint2(~(uint32_t)idx, ld_order_key(vals[idx] + 0.0f));  // .y is the high half
  }
  return true;
}

// Step 1b, sigmoid family, all threads: scores = sigmoid(logit) + bias, group-limited selection (a group's
// score is the sum of its two largest scores; the best topk_group groups are kept, ties to the lower group;
// the experts of the other groups are scored 0.0), then the sort keys.  Maxima and the sum of two numbers do
// not depend on evaluation order, so the result is bit-identical to the one-warp form of sigmoid_topk_row.
// Contains CTA-wide barriers: every thread must call it.
__device__ __forceinline__ void ld_sigmoid_scores(int T, int E, const float* bias, int n_group, int topk_group,
                                                  float* vals, const float* lgs, uint2* keys, float* gsc) {
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  for (int i = tid; i < T * E; i += kLdThreads) vals[i] = sigmoid_stable(lgs[i]) + bias[i % E];
  if (n_group > 1) {  // uniform over the CTA
    __syncthreads();
    const int per = E / n_group;
    for (int pg = wid; pg < T * n_group; pg += kLdWarps) {  // one warp per (row, group)
      const int t = pg / n_group, grp = pg - t * n_group;
      const float* src = vals + (size_t)t * E + grp * per;
      float t1 = -CUDART_INF_F, t2 = -CUDART_INF_F;
      for (int j = lane; j < per; j += 32) {
        const float x = src[j];
        if (x > t1) {
          t2 = t1;
          t1 = x;
        } else if (x > t2) {
          t2 = x;
        }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {  // merge the lanes' (largest, second largest) pairs
        const float o1 = __shfl_xor_sync(0xffffffffu, t1, o);
        const float o2 = __shfl_xor_sync(0xffffffffu, t2, o);
        const float hi = fmaxf(t1, o1);
        t2 = fmaxf(fminf(t1, o1), fmaxf(t2, o2));
        t1 = hi;
      }
      if (lane == 0) gsc[t * 64 + grp] = t1 + t2;
    }
    __syncthreads();
    if (tid < T * n_group) {
      const int t = tid / n_group, grp = tid - t * n_group;
      const float mine = gsc[t * 64 + grp];
      int rank = 0;
      for (int h = 0; h < n_group; ++h) {
        const float o = gsc[t * 64 + h];
        rank += (o > mine) || (o == mine && h < grp);
      }
      gsc[t * 64 + 32 + grp] = (rank < topk_group) ? 1.0f : 0.0f;
    }
    __syncthreads();
    for (int i = tid; i < T * E; i += kLdThreads) {
      const int t = i / E, e = i - t * E;
      if (gsc[t * 64 + 32 + e / per] == 0.0f) vals[i] = 0.0f;
    }
  }
  // each thread reads back only what it wrote itself
  for (int i = tid; i < T * E; i += kLdThreads) keys[i] = make_uint2(~(uint32_t)(i % E), ld_order_key(vals[i] + 0.0f));
}

// Step 2, all threads: rank of every score under (score descending, expert id ascending) -- one unsigned
// 64-bit comparison of the sort keys.  The ranks of a row are a permutation, so the experts ranked below K
// write themselves into slot order.
__device__ __forceinline__ void ld_rank_select(const uint2* keys, int T, int E, int K, int* sel_idx) {
  const int pairs = T * E;
  int P = 1;  // threads that share one score's scan
  while (P < 32 && P * 2 * pairs <= kLdThreads) P *= 2;
  const int lp = 31 - __clz(P);
  const int per_pass = kLdThreads >> lp;
  const int part = threadIdx.x & (P - 1);
  for (int base = 0; base < pairs; base += per_pass) {
    const int pair = base + (threadIdx.x >> lp);
    const bool ok = pair < pairs;
    const int t = ok ? pair / E : 0;
    const int i = ok ? pair - t * E : 0;
    const unsigned long long* row = reinterpret_cast<const unsigned long long*>(keys + (size_t)t * E);
    const unsigned long long mine = row[i];
    int rank = 0;
#pragma unroll 4
    for (int j = part; j < E; j += P) rank += (row[j] > mine);
    for (int o = 1; o < P; o <<= 1) rank += __shfl_xor_sync(0xffffffffu, rank, o);
    if (ok && part == 0 && rank < K) sel_idx[t * K + rank] = i;
  }
}

// Step 3, one warp per row: the weights of the selected experts.  Lane i < K owns slot i; sums run over the
// slots in order 0..K-1 (every lane repeats them), as in the per-row router functions.
__device__ __forceinline__ void ld_finish_row(const float* vals, const float* lgs, int K, int family, int renorm,
                                              float scale, const int* sel_idx, float* w_out, int* idx_out, int lane) {
  const int si = sel_idx[lane < K ? lane : 0];
  const float sv = vals[si];
  float mine;  // the slot's term of the normalising sum
  if (family == 0)
    mine = expf(sv - vals[sel_idx[0]]);
  else if (family == 1)
    mine = sv;
  else
    mine = sigmoid_stable(lgs[si]);
  float sum = 0.0f;
  for (int i = 0; i < K; ++i) sum += __shfl_sync(0xffffffffu, mine, i);
  float w;
  if (family == 0) {
    w = mine / sum;
  } else if (family == 1) {
    const float denom = (renorm == 1) ? sum + 1e-20f : sum;
    w = renorm ? sv / denom : sv;
  } else {
    const float inv = 1.0f / sum;
    w = mine * inv;
    if (scale != 1.0f) w = w * scale;
  }
  if (lane < K) {
    w_out[lane] = w;
    idx_out[lane] = si;
  }
}

// ------------------------------------------------------------------ matmul core (one warp)
template <int NMAT>
__device__ __forceinline__ void ld_load_quad(uint2 (&buf)[4][NMAT][2], const uint32_t* (&wp)[NMAT][2]) {
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      buf[0][m][h] = ldg_stream_u2<0>(wp[m][h]);
      buf[1][m][h] = ldg_stream_u2<32>(wp[m][h]);
      buf[2][m][h] = ldg_stream_u2<64>(wp[m][h]);
      buf[3][m][h] = ldg_stream_u2<96>(wp[m][h]);
    }
  }
}

// Starts one (expert, 16-row tile) item: the first PD quads of this warp's share of K go to registers ...
template <int NMAT, int PD>
__device__ __forceinline__ void ld_issue_w(uint2 (&wbuf)[PD][4][NMAT][2], const uint32_t* (&wp)[NMAT][2],
                                           const LdBank& bank, int e, int N, int K8, int n0, int g, int tig, int wk,
                                           int wk_count, int nq_w) {
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
    const uint32_t* we = bank.w[m] + ((size_t)e * N + n0) * K8 + tig * 2 + wk * 32;
    wp[m][0] = we + (size_t)g * K8;
    wp[m][1] = we + (size_t)(g + 8) * K8;
  }
#pragma unroll
  for (int bq = 0; bq < PD; ++bq) {
    if (bq < nq_w) {
      ld_load_quad<NMAT>(wbuf[bq], wp);
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
        wp[m][0] += wk_count * 32;
        wp[m][1] += wk_count * 32;
      }
    }
  }
}

// ... and the tile's scales and biases to the group's shared-memory area (asynchronous copies, raw T values).
template <int NMAT>
__device__ __forceinline__ void ld_issue_sc(const LdBank& bank, int e, int N, int ngroups, int n0, unsigned char* sraw,
                                            int sc_stride, int gtid, int gsize) {
  const int cpr = ngroups >> 2;  // 8-byte chunks per row
#pragma unroll
  for (int arr = 0; arr < NMAT * 2; ++arr) {
    const __nv_bfloat16* base = ((arr & 1) ? bank.b[arr >> 1] : bank.s[arr >> 1]) + ((size_t)e * N + n0) * ngroups;
    unsigned char* dst = sraw + arr * 16 * sc_stride;
    for (int i = gtid; i < 16 * cpr; i += gsize) {
      const int r = i / cpr;
      const int c = i - r * cpr;
      cp_async_8(dst + r * sc_stride + c * 8, base + (size_t)r * ngroups + c * 4);
    }
  }
}

// Picks the routed or the shared bank field by field (keeps the kernel parameters out of local memory).
__device__ __forceinline__ LdBank ld_pick(const LdBank& a, const LdBank& b, bool second) {
  LdBank r;
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    r.w[m] = second ? b.w[m] : a.w[m];
    r.s[m] = second ? b.s[m] : a.s[m];
    r.b[m] = second ? b.b[m] : a.b[m];
  }
  return r;
}

// Scale, bias and the 128 offset for a block of 8/TT multiplexed groups whose first item in the warp's stream
// is gi0.  Lane (g, tig) owns columns 2*tig and 2*tig+1; srow_c[c] is the staged row of column c's token (-1: none).
template <int NMAT, int TT>
__device__ __forceinline__ void ld_fixup(float (&acc)[NMAT][4], const float (&dg)[NMAT][4], const float* xsum,
                                         int xsum_stride, const int (&srow_c)[2], const unsigned char* sraw,
                                         int sc_stride, int wk, int wk_count, int g, int tig, int gi0, int nq_w) {
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    const int col = 2 * tig + c;
    const int gi_c = gi0 + ((TT == 8) ? 0 : col / TT);
    const int G_c = (wk + (gi_c >> 2) * wk_count) * 4 + (gi_c & 3);
    if ((gi_c >> 2) < nq_w) {
      const float X = (srow_c[c] >= 0) ? xsum[G_c * xsum_stride + srow_c[c]] : 0.0f;
#pragma unroll
      for (int m = 0; m < NMAT; ++m) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          const int r = g + 8 * h;
          const float sv = __bfloat162float(
              *reinterpret_cast<const __nv_bfloat16*>(sraw + ((m * 2 + 0) * 16 + r) * sc_stride + G_c * 2));
          const float bv = __bfloat162float(
              *reinterpret_cast<const __nv_bfloat16*>(sraw + ((m * 2 + 1) * 16 + r) * sc_stride + G_c * 2));
          const float cv = fmaf(-128.0f, sv, bv);
          acc[m][h * 2 + c] = fmaf(sv, dg[m][h * 2 + c], fmaf(cv, X, acc[m][h * 2 + c]));
        }
      }
    }
  }
}

// This warp's share of K for one item.  xoff is the byte offset (in shared memory) of the lane's token row
// plus tig*32; lanes whose column carries no token of this item read the zero page.  The four k16 steps of a
// group go to NACC independent accumulators (summed in a fixed order at the fix-up): a chain of dependent
// mma.sync on one accumulator costs its full latency per step, and at decode sizes nothing else hides it.
template <int NMAT, int PD, int TT, int NACC>
__device__ __forceinline__ void ld_mainloop(float (&acc)[NMAT][4], uint2 (&wbuf)[PD][4][NMAT][2],
                                            const uint32_t* (&wp)[NMAT][2], const unsigned char* smem, int xoff,
                                            bool tok_ok, int zpage, int slot_g, const float* xsum, int xsum_stride,
                                            const int (&srow_c)[2], const unsigned char* sraw, int sc_stride, int wk,
                                            int wk_count, int nq_w, int g, int tig) {
  static_assert(NACC == 1 || NACC == 2 || NACC == 4, "accumulators per matrix");
  constexpr int GPB = 8 / TT;  // groups multiplexed into one accumulator
  float dg[NMAT][NACC][4];
  float dsum[NMAT][4];
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = 0.0f;
#pragma unroll
    for (int n = 0; n < NACC; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) dg[m][n][j] = 0.0f;
  }
  auto fold = [&]() {
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (NACC == 1) dsum[m][j] = dg[m][0][j];
        if (NACC == 2) dsum[m][j] = dg[m][0][j] + dg[m][NACC - 1][j];
        if (NACC == 4) dsum[m][j] = (dg[m][0][j] + dg[m][1 % NACC][j]) + (dg[m][2 % NACC][j] + dg[m][3 % NACC][j]);
      }
  };
  for (int qi = 0; qi < nq_w; qi += PD) {
#pragma unroll
    for (int bq = 0; bq < PD; ++bq) {
      const int quad = wk + (qi + bq) * wk_count;
      if (qi + bq < nq_w) {  // warp-uniform
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int slot = (bq * 4 + j) % GPB;
          if (slot == 0) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m)
#pragma unroll
              for (int n = 0; n < NACC; ++n)
#pragma unroll
                for (int jj = 0; jj < 4; ++jj) dg[m][n][jj] = 0.0f;
          }
          const bool mine = tok_ok && (TT == 8 || slot_g == slot);
          const int xo = mine ? (xoff + quad * 512 + j * 128) : zpage;
          const uint4 xb0 = *reinterpret_cast<const uint4*>(smem + xo);
          const uint4 xb1 = *reinterpret_cast<const uint4*>(smem + xo + 16);
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            const uint2 wa = wbuf[bq][j][m][0];
            const uint2 wb = wbuf[bq][j][m][1];
            mma_bf16_m16n8k16(dg[m][0], deq_imm<0>(wa.x), deq_imm<0>(wb.x), deq_imm<4>(wa.x), deq_imm<4>(wb.x), xb0.x,
                              xb0.y);
            mma_bf16_m16n8k16(dg[m][1 % NACC], deq_imm<8>(wa.x), deq_imm<8>(wb.x), deq_imm<12>(wa.x),
                              deq_imm<12>(wb.x), xb0.z, xb0.w);
            mma_bf16_m16n8k16(dg[m][2 % NACC], deq_imm<0>(wa.y), deq_imm<0>(wb.y), deq_imm<4>(wa.y), deq_imm<4>(wb.y),
                              xb1.x, xb1.y);
            mma_bf16_m16n8k16(dg[m][3 % NACC], deq_imm<8>(wa.y), deq_imm<8>(wb.y), deq_imm<12>(wa.y),
                              deq_imm<12>(wb.y), xb1.z, xb1.w);
          }
          // rolling refill: the registers of the group just consumed take the same group of the quad PD steps
          // ahead at once (keeps the bytes in flight near their maximum instead of dipping once per quad)
          if (qi + bq + PD < nq_w) {
#pragma unroll
            for (int m = 0; m < NMAT; ++m) {
#pragma unroll
              for (int h = 0; h < 2; ++h) {
                if (j == 0) wbuf[bq][0][m][h] = ldg_stream_u2<0>(wp[m][h]);
                if (j == 1) wbuf[bq][1][m][h] = ldg_stream_u2<32>(wp[m][h]);
                if (j == 2) wbuf[bq][2][m][h] = ldg_stream_u2<64>(wp[m][h]);
                if (j == 3) wbuf[bq][3][m][h] = ldg_stream_u2<96>(wp[m][h]);
              }
            }
          }
          if (slot == GPB - 1) {
            fold();
            ld_fixup<NMAT, TT>(acc, dsum, xsum, xsum_stride, srow_c, sraw, sc_stride, wk, wk_count, g, tig,
                               (qi + bq) * 4 + j - (GPB - 1), nq_w);
          }
        }
        if (qi + bq + PD < nq_w) {  // the refilled quad's pointers move on
#pragma unroll
          for (int m = 0; m < NMAT; ++m) {
            wp[m][0] += wk_count * 32;
            wp[m][1] += wk_count * 32;
          }
        }
      }
    }
  }
  // an odd number of quads leaves half a block of eight multiplexed groups without its fix-up
  if (GPB == 8 && (nq_w & 1)) {
    fold();
    ld_fixup<NMAT, TT>(acc, dsum, xsum, xsum_stride, srow_c, sraw, sc_stride, wk, wk_count, g, tig, (nq_w - 1) * 4,
                       nq_w);
  }
}

// Sums the K-split partial results of a group's warps in warp order (result in the group's first warp), then
// folds the multiplexed columns back onto their tokens: afterwards column c < TT of the first warp holds token c.
template <int NMAT, int TT>
__device__ __forceinline__ void ld_reduce_fold(float (&acc)[NMAT][4], float* red, int gid, int wk, int wk_count,
                                               int lane) {
  const int wid = threadIdx.x >> 5;
  if (wk_count > 1) {
    float* mine = red + (wid * 32 + lane) * 8;
    if (wk != 0) {
#pragma unroll
      for (int m = 0; m < NMAT; ++m)
#pragma unroll
        for (int j = 0; j < 4; ++j) mine[m * 4 + j] = acc[m][j];
    }
    ld_group_sync(gid, wk_count);
    if (wk == 0) {
#pragma unroll 1
      for (int o = 1; o < wk_count; ++o) {
        const float* other = red + ((wid + o) * 32 + lane) * 8;
#pragma unroll
        for (int m = 0; m < NMAT; ++m)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[m][j] += other[m * 4 + j];
      }
    }
  }
  if (wk == 0 && TT < 8) {
#pragma unroll
    for (int m = 0; m < NMAT; ++m) {
#pragma unroll
      for (int h = 0; h < 2; ++h) {
        if (TT == 1) {
          acc[m][h * 2] += acc[m][h * 2 + 1];
          acc[m][h * 2 + 1] = 0.0f;
        }
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float v = acc[m][h * 2 + c];
          if (TT <= 2) v += __shfl_xor_sync(0xffffffffu, v, 1);
          v += __shfl_xor_sync(0xffffffffu, v, 2);
          acc[m][h * 2 + c] = v;
        }
      }
    }
  }
}

// ------------------------------------------------------------------ bulk-copy variant (one token)
// With BULK the packed weights do not go to registers: every row of an item is one cp.async.bulk copy into a
// padded shared-memory row (stride = row bytes + 32 == 32 mod 128: the 8-byte fragment reads of a warp hit 32
// different banks), completion is counted on an mbarrier, and the matmul is a compact loop over shared
// memory.  Issuing a copy never blocks the warp, so the copies of all of a CTA's items are in flight while
// the first ones are already being consumed, and the loop body is fetched once instead of a long unrolled
// register pipeline.  Needs 16-byte aligned tensors and rows that fit (d_model, d_ff <= 2048 or so).
__device__ __forceinline__ uint32_t ld_smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ld_mbar_init(uint32_t bar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}
__device__ __forceinline__ void ld_mbar_expect_tx(uint32_t bar, int bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool ld_mbar_try(uint32_t bar, int parity) {
  uint32_t ok;
  asm volatile("{ .reg .pred p; mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0, 1, 0, p; }"
               : "=r"(ok)
               : "r"(bar), "r"(parity)
               : "memory");
  return ok != 0;
}
// Bounded wait for a phase of an mbarrier; false when it ran out.
__device__ __forceinline__ bool ld_mbar_wait(uint32_t bar, int parity) {
  for (int i = 0; i < kLdSpinLimit; ++i)
    if (ld_mbar_try(bar, parity)) return true;
  return false;
}
__device__ __forceinline__ void ld_bulk_g2s(uint32_t dst, const void* src, int bytes, uint32_t bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
               "l"(src), "r"(bytes), "r"(bar)
               : "memory");
}

// One token (TT = 1: eight groups share an accumulator), weights of the item in shared memory: rows m*16 + r at
// `wslot + row * row_stride`.  The warp walks the quads wk, wk + wk_count, ...; the loop is kept rolled.
template <int NMAT, int NACC>
__device__ __forceinline__ void ld_smem_mainloop(float (&acc)[NMAT][4], const unsigned char* wslot, int row_stride,
                                                 const unsigned char* smem, int xoff, int zpage, const float* xsum,
                                                 int xsum_stride, const int (&srow_c)[2], const unsigned char* sraw,
                                                 int sc_stride, int wk, int wk_count, int nq, int g, int tig) {
  float dg[NMAT][NACC][4];
  float dsum[NMAT][4];
#pragma unroll
  for (int m = 0; m < NMAT; ++m) {
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[m][j] = 0.0f;
#pragma unroll
    for (int n = 0; n < NACC; ++n)
#pragma unroll
      for (int j = 0; j < 4; ++j) dg[m][n][j] = 0.0f;
  }
  auto fold = [&]() {
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        if (NACC == 1) dsum[m][j] = dg[m][0][j];
        if (NACC == 2) dsum[m][j] = dg[m][0][j] + dg[m][NACC - 1][j];
        if (NACC == 4) dsum[m][j] = (dg[m][0][j] + dg[m][1 % NACC][j]) + (dg[m][2 % NACC][j] + dg[m][3 % NACC][j]);
      }
  };
  const int nq_w = (nq > wk) ? (nq - wk + wk_count - 1) / wk_count : 0;
  const unsigned char* wlane = wslot + g * row_stride + tig * 8;
  // blocks of eight groups (two of the warp's quads) share the accumulators; one fix-up per block
#pragma unroll 1
  for (int qb = 0; qb < nq_w; qb += 2) {
#pragma unroll
    for (int m = 0; m < NMAT; ++m)
#pragma unroll
      for (int n = 0; n < NACC; ++n)
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) dg[m][n][jj] = 0.0f;
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      if (qb + half >= nq_w) break;
      const int quad = wk + (qb + half) * wk_count;
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const bool mine = (g == half * 4 + j);
        const int xo = mine ? (xoff + quad * 512 + j * 128) : zpage;
        const uint4 xb0 = *reinterpret_cast<const uint4*>(smem + xo);
        const uint4 xb1 = *reinterpret_cast<const uint4*>(smem + xo + 16);
#pragma unroll
        for (int m = 0; m < NMAT; ++m) {
          const unsigned char* wr = wlane + m * 16 * row_stride + quad * 128 + j * 32;
          const uint2 wa = *reinterpret_cast<const uint2*>(wr);
          const uint2 wb = *reinterpret_cast<const uint2*>(wr + 8 * row_stride);
          mma_bf16_m16n8k16(dg[m][0], deq_imm<0>(wa.x), deq_imm<0>(wb.x), deq_imm<4>(wa.x), deq_imm<4>(wb.x), xb0.x,
                            xb0.y);
          mma_bf16_m16n8k16(dg[m][1 % NACC], deq_imm<8>(wa.x), deq_imm<8>(wb.x), deq_imm<12>(wa.x), deq_imm<12>(wb.x),
                            xb0.z, xb0.w);
          mma_bf16_m16n8k16(dg[m][2 % NACC], deq_imm<0>(wa.y), deq_imm<0>(wb.y), deq_imm<4>(wa.y), deq_imm<4>(wb.y),
                            xb1.x, xb1.y);
          mma_bf16_m16n8k16(dg[m][3 % NACC], deq_imm<8>(wa.y), deq_imm<8>(wb.y), deq_imm<12>(wa.y), deq_imm<12>(wb.y),
                            xb1.z, xb1.w);
        }
      }
    }
    fold();
    ld_fixup<NMAT, 1>(acc, dsum, xsum, xsum_stride, srow_c, sraw, sc_stride, wk, wk_count, g, tig, qb * 4, nq_w);
  }
}

// Debug builds (-DZMOE_LD_TIMING) record CTA 0's cycle counter at the phase boundaries in the workspace
// header (8-byte slots from byte 64).
#ifdef ZMOE_LD_TIMING
#define LD_DBG_PTR \
  ((blockIdx.x == 0 && wid == 0) ? reinterpret_cast<long long*>(reinterpret_cast<unsigned char*>(p.sync) + 64) : nullptr)
#define LD_STAMP(i)                                                                     \
  do {                                                                                  \
    if (blockIdx.x == 0 && threadIdx.x == 0)                                            \
      reinterpret_cast<long long*>(reinterpret_cast<unsigned char*>(p.sync) + 64)[i] = clock64(); \
  } while (0)
#else
#define LD_DBG_PTR nullptr
#define LD_STAMP(i) \
  do {              \
  } while (0)
#endif

// ------------------------------------------------------------------ the kernel
template <int TT, bool BULK, int DPD>
__global__ void __launch_bounds__(kLdThreads, 1) layer_decode_kernel(const LdParams p) {
  static_assert(!BULK || TT == 1, "the bulk-copy variant is the one-token kernel");
  extern __shared__ __align__(16) unsigned char smem[];
  __shared__ int wait_failed;  // a bounded wait on another CTA's words ran out somewhere in this CTA
  const int tid = threadIdx.x;
  const int lane = tid & 31;
  const int wid = tid >> 5;
  const int g = lane >> 2;
  const int tig = lane & 3;
  const int slot_g = g / TT;
  const int tok_g = g % TT;

  const int T = p.T, K = p.K, E = p.E, d = p.d, f = p.f;
  const int R = T * K;
  const int rtot = R + (p.n_shared ? T : 0);
  const int ngd = d >> 6, ngf = f >> 6;
  const LdSmem lay = ld_smem(T, K, E, d, f, p.n_shared, p.tiles_per_cta);
  unsigned char* xs = smem + lay.xs;
  float* xsum = reinterpret_cast<float*>(smem + lay.xsum);
  float* red = reinterpret_cast<float*>(smem + lay.red);
  float* ybuf = reinterpret_cast<float*>(smem + lay.ybuf);
  uint2* keys = reinterpret_cast<uint2*>(smem + lay.route);  // 8-byte aligned: the region starts 16-byte aligned
  float* vals = reinterpret_cast<float*>(keys + T * E);
  float* lgs = vals + T * E;
  float* gsc = lgs + T * E;
  int* sel_idx = reinterpret_cast<int*>(gsc + T * 64);
  LdMeta* meta = reinterpret_cast<LdMeta*>(smem + lay.meta);
  const int zpage = lay.zero;
  const int nblocks = gridDim.x;
  bool alive = true;
  // Router rows are constants: the warp's first one is requested before anything that depends on the previous
  // kernel of the stream, so that with programmatic dependent launch its HBM latency hides behind that kernel.
  const int e_first = blockIdx.x + nblocks * wid;
  uint4 wpre[8];
#pragma unroll
  for (int u = 0; u < 8; ++u)
    wpre[u] = (e_first < E && lane + 32 * u < (d >> 3))
                  ? __ldg(reinterpret_cast<const uint4*>(p.wr + (size_t)e_first * d) + lane + 32 * u)
                  : make_uint4(0u, 0u, 0u, 0u);
  if (p.pdl) {
    pdl_trigger();  // the next kernel of the stream may be set up now; it waits for this one to finish
    pdl_wait();     // nothing below may run before the previous kernel has finished and flushed
  }
  // launch count: every thread reads it here; the last CTA to sign in (below) bumps it for the next launch; tag of
  // this launch's words
  const int epoch = __ldcg(p.sync + 4);
  const uint32_t tag = (uint32_t)((epoch % 65535) + 1) << 16;
  if (tid == 0) wait_failed = 0;
  // bulk-copy variant: 16 mbarriers {gate/up slot 0..3, down task 0..}, then the gate/up slots, then the down slots
  const int rs_g = (d >> 1) + 32, rs_d = (f >> 1) + 32;  // padded row strides of the two kinds of slots
  unsigned char* bulk = smem + p.bulk_off;
  const uint32_t bars = ld_smem_u32(bulk);
  unsigned char* gslots = bulk + 128;
  unsigned char* dslots = gslots + p.g_slots * 32 * rs_g;
  if (BULK && tid == 0) {
    for (int i = 0; i < 4; ++i) ld_mbar_init(bars + i * 8, 32);
    for (int i = 4; i < 16; ++i) ld_mbar_init(bars + i * 8, 16);
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
  }

  LD_STAMP(0);
  // ---- phase 0: token rows -> shared memory (permuted, with group sums)
  ld_stage_rows<false>(xs, qmm_xs_stride(d), xsum, T, p.x, p.ldx, T, d >> 3, 0u);
  if (tid < 8) reinterpret_cast<uint32_t*>(smem + zpage)[tid] = 0u;
  for (int i = tid; i < kLdMaxTasks; i += kLdThreads) meta->task_cnt[i] = 0;

  LD_STAMP(1);
  // ---- phase 1: router linear, one warp per expert row over the whole grid.  A lane's eight 16-byte pieces of
  // the row are requested before anything is consumed (one memory round trip); the sum runs over i ascending
  // per lane and then over the lanes, as in the stand-alone router kernels.
  {
    const int nvec = d >> 3;
    for (int e = blockIdx.x + nblocks * wid; e < E; e += nblocks * kLdWarps) {
      const uint4* wrow = reinterpret_cast<const uint4*>(p.wr + (size_t)e * d);
#pragma unroll 1
      for (int t = 0; t < T; ++t) {
        const uint4* xrow = reinterpret_cast<const uint4*>(p.x + (size_t)t * p.ldx);
        float acc = 0.0f;
#pragma unroll 1
        for (int i0 = lane; i0 < nvec; i0 += 256) {
          uint4 wv[8], xv[8];
          const bool have = (e == e_first) && (i0 == lane);  // warp-uniform: the chunk requested at kernel start
#pragma unroll
          for (int u = 0; u < 8; ++u)
            wv[u] = have ? wpre[u] : ((i0 + 32 * u < nvec) ? __ldg(wrow + i0 + 32 * u) : make_uint4(0u, 0u, 0u, 0u));
#pragma unroll
          for (int u = 0; u < 8; ++u)
            xv[u] = (i0 + 32 * u < nvec) ? __ldg(xrow + i0 + 32 * u) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
          for (int u = 0; u < 8; ++u) {
            const uint32_t ww[4] = {wv[u].x, wv[u].y, wv[u].z, wv[u].w};
            const uint32_t xw[4] = {xv[u].x, xv[u].y, xv[u].z, xv[u].w};
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              acc = fmaf(bf16_bits_to_float(ww[q] & 0xffffu), bf16_bits_to_float(xw[q] & 0xffffu), acc);
              acc = fmaf(bf16_bits_to_float(ww[q] >> 16), bf16_bits_to_float(xw[q] >> 16), acc);
            }
          }
        }
        const float sres = warp_sum(acc);
        // eight copies = one full 32-byte sector: L2 holds it whole and never has to merge it with a stale
        // copy from HBM when the other CTAs read it
        if (lane < 8 && !(p.withhold && e == 0))
          st_relaxed_u32(p.logits + ((size_t)t * E + e) * 8 + lane, tag | float_to_bf16_bits(sres));
      }
    }
  }
  LD_STAMP(2);
  __syncthreads();  // wait_failed, the zero page and the cleared task counts are in place
  // Launch count for the next launch.  Every thread of this CTA has read the count by now, so the CTA can sign
  // in; the last CTA of the grid to do so bumps the count (the tags of THIS launch live in registers already)
  // and clears the sign-in counter.  Doing it here, not at the end, keeps the atomic's round trip off the tail.
  if (tid == 0) {
    if (atomicAdd(p.sync + 2, 1) == nblocks - 1) {
      p.sync[4] = epoch + 1;
      p.sync[2] = 0;
    }
  }

  {
    // ---- phase 2a: routing of every row, repeated by every CTA (one warp per row); the logits arrive as
    // hand-over words, so this is also where the CTA waits for the router warps of the other CTAs
    if (wid < T) {
      bool ok;
      ok = ld_route_scores(p.logits + (size_t)wid * E * 8, tag, E, p.family, p.rbias, p.n_group, p.topk_group,
                           vals + wid * E, lgs + wid * E, keys + wid * E, gsc + wid * 64, lane, LD_DBG_PTR);
      if (!ok && lane == 0) {
        wait_failed = 1;
        atomicExch(p.sync + 3, 1);
      }
    }
    __syncthreads();
    if (p.family == 2) {
      ld_sigmoid_scores(T, E, p.rbias, p.n_group, p.topk_group, vals, lgs, keys, gsc);
      __syncthreads();
    }
    LD_STAMP(20);
    if (wait_failed == 0) ld_rank_select(keys, T, E, K, sel_idx);
    __syncthreads();
    LD_STAMP(21);
    if (wid < T && wait_failed == 0)
      ld_finish_row(vals + wid * E, lgs + wid * E, K, p.family, p.renorm, p.scale, sel_idx + wid * K,
                    meta->w + wid * K, meta->idx + wid * K, lane);
    LD_STAMP(3);
    if (T == 1) {
      // one token: its K experts are distinct, so slot a is task a
      if (tid < K) {  // lanes of warp 0, which has just written meta->idx
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
    __syncthreads();
    LD_STAMP(4);
    alive = (wait_failed == 0);
  }
  if (alive) {
    if (blockIdx.x == 0 && tid < R) {
      if (p.weights) p.weights[tid] = meta->w[tid];
      if (p.indices) p.indices[tid] = (uint32_t)meta->idx[tid];
    }
    if (TT > 1 && T > 1) {
      // ---- phase 2b: tasks = distinct experts in order of first use; a task's rows in row order
      if (tid < R) {
        const int e = meta->idx[tid];
        int rk = 0;
        for (int r = 0; r < tid; ++r) rk += (meta->idx[r] == e);
        meta->rank[tid] = rk;
      }
      __syncthreads();
      if (tid < R) {
        const int e = meta->idx[tid];
        int r0 = 0;
        while (meta->idx[r0] != e) ++r0;  // first row of this expert (r0 <= tid)
        int tk = 0;
        for (int r = 0; r < r0; ++r) tk += (meta->rank[r] == 0);
        const int rk = meta->rank[tid];
        if (rk == 0) meta->task_expert[tk] = e;
        if (rk < kLdMaxT) meta->task_rows[tk][rk] = (unsigned char)tid;
        atomicAdd(&meta->task_cnt[tk], 1);
      }
      if (tid == 0) {
        int n = 0;
        for (int r = 0; r < R; ++r) n += (meta->rank[r] == 0);
        meta->n_routed = n;
        meta->n_tasks = n + (p.n_shared ? 1 : 0);
        if (p.n_shared) {
          meta->task_expert[n] = 0;
          meta->task_cnt[n] = T;
          for (int t = 0; t < T; ++t) meta->task_rows[n][t] = (unsigned char)(R + t);
        }
      }
      __syncthreads();
    }
    const int n_tasks = meta->n_tasks;
    const int n_routed = meta->n_routed;
    LD_STAMP(5);

    // ---- phase 2c: gate/up + SwiGLU; items (task, 16-row tile) dealt to groups of four warps over the grid
    {
      constexpr int WK = 4;
      const int gid = wid >> 2, wk = wid & 3;
      const int nq = ngd >> 2;
      const int nq_w = (nq > wk) ? (nq - wk + WK - 1) / WK : 0;
      const int ntiles = f >> 4;
      const int nitems = n_tasks * ntiles;
      const int sc_stride = qmm_sc_stride(ngd);
      unsigned char* sraw = smem + lay.sc + gid * (4 * 16 * sc_stride);
      const int xs_stride = qmm_xs_stride(d);
      int gu_uses = 0;  // how often this team's slot has been filled (parity of its barrier)
      for (int it = gid * nblocks + blockIdx.x; it < nitems; it += nblocks * 4) {
        const int a = it / ntiles;
        const int n0 = (it - a * ntiles) << 4;
        const bool is_sh = a >= n_routed;
        const LdBank bank = ld_pick(p.gu, p.sgu, is_sh);
        const int e = meta->task_expert[a];
        const int cnt = meta->task_cnt[a];
        uint2 wbuf[BULK ? 1 : 2][4][2][2];
        const uint32_t* wp[2][2];
        if (!BULK) ld_issue_w<2, BULK ? 1 : 2>(wbuf, wp, bank, e, f, d >> 3, n0, g, tig, wk, WK, nq_w);
        ld_group_sync(gid, WK);  // the previous item is done with the group's scale area (and weight slot)
        if (BULK) {
          // rows 0..15 gate, 16..31 up: eight lanes of each of the team's warps copy one row each
          if (gu_uses > 0) asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          if (lane < 8) {
            const int r = wk * 8 + lane;
            const uint32_t* src = bank.w[r >> 4] + ((size_t)e * f + n0 + (r & 15)) * (d >> 3);
            ld_mbar_expect_tx(bars + gid * 8, d >> 1);
            ld_bulk_g2s(ld_smem_u32(gslots + (gid * 32 + r) * rs_g), src, d >> 1, bars + gid * 8);
          }
        }
        ld_issue_sc<2>(bank, e, f, ngd, n0, sraw, sc_stride, tid & 127, 128);
        // token of a task row: routed row r belongs to token r / K, shared row R + t to token t
        const bool tok_ok = tok_g < cnt;
        int trow = 0;
        if (tok_ok) {
          const int r = meta->task_rows[a][tok_g];
          trow = is_sh ? r - R : r / K;
        }
        int srow_c[2];
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          const int sl = (2 * tig + c) % TT;
          srow_c[c] = -1;
          if (sl < cnt) {
            const int r = meta->task_rows[a][sl];
            srow_c[c] = is_sh ? r - R : r / K;
          }
        }
        LD_STAMP(11);
        cp_async_wait_all();
        if (BULK && !ld_mbar_wait(bars + gid * 8, gu_uses & 1)) {
          wait_failed = 1;
          atomicExch(p.sync + 3, 1);
        }
        ++gu_uses;
        ld_group_sync(gid, WK);
        LD_STAMP(12);
        float acc[2][4];
        if (BULK)
          ld_smem_mainloop<2, 2>(acc, gslots + gid * 32 * rs_g, rs_g, smem, lay.xs + trow * xs_stride + tig * 32,
                                 zpage, xsum, T, srow_c, sraw, sc_stride, wk, WK, nq, g, tig);
        else
          ld_mainloop<2, BULK ? 1 : 2, TT, 2>(acc, wbuf, wp, smem, lay.xs + trow * xs_stride + tig * 32, tok_ok, zpage,
                                              slot_g, xsum, T, srow_c, sraw, sc_stride, wk, WK, nq_w, g, tig);
        LD_STAMP(13);
        ld_reduce_fold<2, TT>(acc, red, gid, wk, WK, lane);
        LD_STAMP(14);
        if (wk == 0) {
          const int epi = is_sh ? p.sepi : p.epi;
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int col = 2 * tig + (j & 1);
            const bool writer = (TT == 8) || (col < TT);
            if (writer && col < cnt) {
              const float v = (epi == 2) ? swiglu_per_op(acc[0][j], acc[1][j]) : swiglu_cpu_contract(acc[0][j], acc[1][j]);
              const int dst = meta->task_rows[a][col];
              st_relaxed_u32(p.h + (size_t)dst * f + n0 + g + ((j >> 1) ? 8 : 0), tag | float_to_bf16_bits(v));
            }
          }
        }
      }
    }

    LD_STAMP(6);
    // ---- phase 3 set-up.  The CTA owns the 16-column output tiles blockIdx.x, blockIdx.x + grid, ...; an item
    // is (tile, task).  The register-pipelined form takes all of its tiles as one batch, so that the warps have
    // many independent items and few idle rounds; the bulk-copy form has shared-memory slots for one tile.
    const int nqf = ngf >> 2;
    const int ntiles_d = d >> 4;
    const int ntile_mine = ((int)blockIdx.x < ntiles_d) ? (ntiles_d - 1 - (int)blockIdx.x) / nblocks + 1 : 0;
    const int tb = BULK ? 1 : ntile_mine;  // tiles per batch
    int wkc = 1;  // warps that split K for one item
    {
      const int items = (tb < ntile_mine ? tb : ntile_mine) * n_tasks;
      int best = 1 << 30;
      for (int c = 4; c >= 1; c >>= 1) {  // ties go to the smaller split (fewer partial sums)
        if (c > nqf) continue;
        const int groups = kLdWarps / c;
        // a round of items costs its quads plus a fixed latency of about four quads
        const int cost = ((items + groups - 1) / groups) * ((nqf + c - 1) / c + 4);
        if (cost <= best) {
          best = cost;
          wkc = c;
        }
      }
    }
    const int ngrp = kLdWarps / wkc;
    const int gid = wid / wkc, wk = wid % wkc;
    const int nq_w = (nqf > wk) ? (nqf - wk + wkc - 1) / wkc : 0;
    const int sc_stride = qmm_sc_stride(ngf);
    unsigned char* sraw = smem + lay.sc + gid * (2 * 16 * sc_stride);
    const int gtid = tid - gid * wkc * 32;
    const int nb0 = tb < ntile_mine ? tb : ntile_mine;  // tiles of the first batch
    const int pre_tl = gid / n_tasks, pre_a = gid - pre_tl * n_tasks;  // the group's first item
    const int pre_n0 = ((int)blockIdx.x + pre_tl * nblocks) << 4;

    uint2 wbuf[BULK ? 1 : DPD][4][1][2];
    const uint32_t* wp[1][2];
    // the first item's packed weights and scales depend on the routing only: stream them before waiting for h
    const bool pre = gid < nb0 * n_tasks;
    if (BULK) {
      // all tasks of the CTA's first tile: warp a copies the 16 rows of task a into down slot a
      if ((int)blockIdx.x < ntiles_d && wid < n_tasks && lane < 16) {
        const LdBank bank = ld_pick(p.dn, p.sdn, wid >= n_routed);
        const uint32_t* src = bank.w[0] + ((size_t)meta->task_expert[wid] * d + (blockIdx.x << 4) + lane) * (f >> 3);
        ld_mbar_expect_tx(bars + (4 + wid) * 8, f >> 1);
        ld_bulk_g2s(ld_smem_u32(dslots + (wid * 16 + lane) * rs_d), src, f >> 1, bars + (4 + wid) * 8);
      }
    } else if (pre) {
      ld_issue_w<1, BULK ? 1 : DPD>(wbuf, wp, ld_pick(p.dn, p.sdn, pre_a >= n_routed), meta->task_expert[pre_a],
                                          d, f >> 3, pre_n0, g, tig, wk, wkc, nq_w);
    }
    __syncthreads();  // every group of this CTA is done with the gate/up scale areas, which the next copies reuse
    if (pre)
      ld_issue_sc<1>(ld_pick(p.dn, p.sdn, pre_a >= n_routed), meta->task_expert[pre_a], d, ngf, pre_n0, sraw,
                     sc_stride, gtid, wkc * 32);
    LD_STAMP(7);
    {
      // ---- phase 3: stage every h row (hand-over words: this is where the CTA waits for the gate/up tiles of
      // the other CTAs), then 16 output columns at a time: all tasks, then the combine
      const int xs_stride = qmm_xs_stride(f);
      const bool good = ld_stage_rows<true>(xs, xs_stride, xsum, rtot, p.h, f, rtot, f >> 3, tag);
      if (!good) {
        wait_failed = 1;
        atomicExch(p.sync + 3, 1);
      }
      __syncthreads();
      LD_STAMP(9);
      alive = (wait_failed == 0);
    }
    if (alive) {
      const int xs_stride = qmm_xs_stride(f);
      int d_uses = 0;  // how often the down slots have been filled (parity of their barriers)
      for (int b0 = 0; b0 < ntile_mine; b0 += tb, ++d_uses) {
        const int nb = (tb < ntile_mine - b0) ? tb : ntile_mine - b0;  // tiles of this batch
        if (BULK && d_uses > 0) {
          // the previous tile ended with a CTA-wide barrier: every slot is free again
          asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
          if (wid < n_tasks && lane < 16) {
            const LdBank bank = ld_pick(p.dn, p.sdn, wid >= n_routed);
            const int n0b = ((int)blockIdx.x + b0 * nblocks) << 4;
            const uint32_t* src = bank.w[0] + ((size_t)meta->task_expert[wid] * d + n0b + lane) * (f >> 3);
            ld_mbar_expect_tx(bars + (4 + wid) * 8, f >> 1);
            ld_bulk_g2s(ld_smem_u32(dslots + (wid * 16 + lane) * rs_d), src, f >> 1, bars + (4 + wid) * 8);
          }
        }
        for (int item = gid; item < nb * n_tasks; item += ngrp) {
          const int tl = item / n_tasks;
          const int a = item - tl * n_tasks;
          const int n0 = ((int)blockIdx.x + (b0 + tl) * nblocks) << 4;
          const bool is_sh = a >= n_routed;
          const int cnt = meta->task_cnt[a];
          if (!(pre && b0 == 0 && item == gid)) {
            const LdBank bank = ld_pick(p.dn, p.sdn, is_sh);
            if (!BULK)
              ld_issue_w<1, BULK ? 1 : DPD>(wbuf, wp, bank, meta->task_expert[a], d, f >> 3, n0, g, tig, wk, wkc,
                                                  nq_w);
            ld_group_sync(gid, wkc);  // the previous item is done with the group's scale area
            ld_issue_sc<1>(bank, meta->task_expert[a], d, ngf, n0, sraw, sc_stride, gtid, wkc * 32);
          }
          const bool tok_ok = tok_g < cnt;
          const int srow = tok_ok ? meta->task_rows[a][tok_g] : 0;
          int srow_c[2];
#pragma unroll
          for (int c = 0; c < 2; ++c) {
            const int sl = (2 * tig + c) % TT;
            srow_c[c] = (sl < cnt) ? (int)meta->task_rows[a][sl] : -1;
          }
          LD_STAMP(15);
          cp_async_wait_all();
          if (BULK && !ld_mbar_wait(bars + (4 + a) * 8, d_uses & 1)) {
            wait_failed = 1;  // the results of this launch are void; the status word says so
            atomicExch(p.sync + 3, 1);
          }
          ld_group_sync(gid, wkc);
          LD_STAMP(16);
          float acc[1][4];
          if (BULK)
            ld_smem_mainloop<1, 4>(acc, dslots + a * 16 * rs_d, rs_d, smem, lay.xs + srow * xs_stride + tig * 32, zpage,
                                   xsum, rtot, srow_c, sraw, sc_stride, wk, wkc, nqf, g, tig);
          else
            ld_mainloop<1, BULK ? 1 : DPD, TT, 4>(acc, wbuf, wp, smem, lay.xs + srow * xs_stride + tig * 32, tok_ok,
                                                        zpage, slot_g, xsum, rtot, srow_c, sraw, sc_stride, wk, wkc,
                                                        nq_w, g, tig);
          LD_STAMP(17);
          ld_reduce_fold<1, TT>(acc, red, gid, wk, wkc, lane);
          LD_STAMP(18);
          if (wk == 0) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              const int col = 2 * tig + (j & 1);
              const bool writer = (TT == 8) || (col < TT);
              if (writer && col < cnt)
                ybuf[(tl * rtot + (int)meta->task_rows[a][col]) * 16 + g + ((j >> 1) ? 8 : 0)] = acc[0][j];
            }
          }
        }
        __syncthreads();
        LD_STAMP(19);
        // ordered combine: thread (tile, token, column) walks the K slots; projected values are rounded to T
        // first, as the separate-kernel path stores them
        for (int idx = tid; idx < nb * T * 16; idx += kLdThreads) {
          const int tl = idx / (T * 16);
          const int t = (idx - tl * T * 16) >> 4, n = idx & 15;
          const float* yb = ybuf + tl * rtot * 16;
          const int mode = p.combine_mode;
          float a0 = 0.0f;
#pragma unroll 1
          for (int i = 0; i < K; ++i) {
            float wi = meta->w[t * K + i];
            if (p.out_flags & 2) wi = round_bf16(wi);
            const float v0 = round_bf16(yb[(t * K + i) * 16 + n]);
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
          const size_t oo = (size_t)t * d + (((int)blockIdx.x + (b0 + tl) * nblocks) << 4) + n;
          const bool fp32_mode = (mode == ZMOE_COMBINE_FP32 || mode == ZMOE_COMBINE_FP32_NO_FMA);
          if (fp32_mode && !(p.out_flags & 1)) {
            reinterpret_cast<float*>(p.out)[oo] = a0;
          } else {
            a0 = round_bf16(a0);
            if (p.n_shared) a0 = __fadd_rn(a0, round_bf16(yb[(R + t) * 16 + n]));
            reinterpret_cast<__nv_bfloat16*>(p.out)[oo] = __float2bfloat16_rn(a0);
          }
        }
        __syncthreads();
      }
    }
  }

  LD_STAMP(10);
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

// Output tiles per CTA that the shared-memory layout provides for: right for grids of 128 CTAs or more.
static int ld_tiles_assumed(int d_model) { return (d_model / 16 + 127) / 128; }

// Why a block shape cannot take the one-launch path (nullptr: it can).
static const char* ld_unsupported(const zmoe_layer_desc* L, int T) {
  if (L->qmode != ZMOE_Q_AFFINE4 || L->group_size != 64) return "needs 4-bit affine weights with group size 64";
  if (T < 1 || T > kLdMaxT) return "takes 1..8 tokens";
  if (L->top_k < 1 || L->top_k > kLdMaxK) return "takes top_k <= 8";
  if (L->E < L->top_k || L->E > 256) return "takes at most 256 experts";
  if (L->d_model % 256 != 0 || L->d_ff % 256 != 0) return "needs d_model and d_ff to be multiples of 256";
  if (L->n_shared < 0 || L->n_shared > 1) return "takes at most one shared expert";
  const LdSmem lay = ld_smem(T, L->top_k, L->E, L->d_model, L->d_ff, L->n_shared, ld_tiles_assumed(L->d_model));
  if (lay.total > 220 * 1024) return "needs more shared memory than an SM has";
  return nullptr;
}

static size_t ld_ws_logits_off() { return 256; }
static size_t ld_ws_h_off(const zmoe_layer_desc* L, int T) {
  return (ld_ws_logits_off() + (size_t)T * L->E * 32 + 255) & ~(size_t)255;
}

template <int TT, bool BULK, int DPD>
static int ld_launch(const LdParams& p, int grid, size_t smem_bytes, cudaStream_t st) {
  auto kern = layer_decode_kernel<TT, BULK, DPD>;
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
  if (!L || ld_unsupported(L, T)) return 0;
  const size_t rows = (size_t)T * L->top_k + (L->n_shared ? T : 0);
  return ld_ws_h_off(L, T) + rows * L->d_ff * 4;
}

int zmoe_layer_decode(const zmoe_layer_desc* L, const void* x, int ldx, int T, void* workspace,
                      size_t workspace_bytes, float* weights, uint32_t* indices, void* out, void* stream) {
  ZMOE_REQUIRE(L && x && workspace && out, ZMOE_ERR_SHAPE, "zmoe_layer_decode: null pointer");
  const char* why = ld_unsupported(L, T);
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
    const void* ptrs[9] = {banks[i]->gate_w,    banks[i]->gate_scales, banks[i]->gate_biases,
                           banks[i]->up_w,      banks[i]->up_scales,   banks[i]->up_biases,
                           banks[i]->down_w,    banks[i]->down_scales, banks[i]->down_biases};
    for (int j = 0; j < 9; ++j)
      ZMOE_REQUIRE(((uintptr_t)ptrs[j] % 8) == 0, ZMOE_ERR_ALIGN,
                   "zmoe_layer_decode: packed weights, scales and biases must be 8-byte aligned");
  }
  const size_t need = zmoe_layer_decode_workspace_bytes(L, T);
  ZMOE_REQUIRE(workspace_bytes >= need, ZMOE_ERR_WORKSPACE, "zmoe_layer_decode: workspace of %zu bytes, need %zu",
               workspace_bytes, need);

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
  ZMOE_REQUIRE(L->launch_mode == 0 || L->launch_mode == 1, ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: launch_mode %d", L->launch_mode);
  p.pdl = L->launch_mode;
  // ZMOE_LD_TEST_WITHHOLD=1 (read once per process) makes the bounded waits run out on purpose: the kernel must
  // end by itself with the status word set and leave the context usable
  static const bool withhold = getenv("ZMOE_LD_TEST_WITHHOLD") != nullptr && atoi(getenv("ZMOE_LD_TEST_WITHHOLD")) != 0;
  p.withhold = withhold ? 1 : 0;
  unsigned char* ws = (unsigned char*)workspace;
  p.sync = (int*)ws;
  p.logits = (uint32_t*)(ws + ld_ws_logits_off());
  p.h = (uint32_t*)(ws + ld_ws_h_off(L, T));
  p.weights = weights;
  p.indices = indices;
  p.out = out;

  int sms = 0;
  int rc = ld_sm_count(&sms);
  if (rc != ZMOE_OK) return rc;
  p.tiles_per_cta = ld_tiles_assumed(L->d_model);
  ZMOE_REQUIRE((L->d_model / 16 + sms - 1) / sms <= p.tiles_per_cta, ZMOE_ERR_UNSUPPORTED,
               "zmoe_layer_decode: this GPU has %d SMs, the one-launch path is laid out for 128 or more", sms);
  const LdSmem lay = ld_smem(T, L->top_k, L->E, L->d_model, L->d_ff, L->n_shared, p.tiles_per_cta);
  cudaStream_t st = (cudaStream_t)stream;
  p.bulk_off = 0;
  p.g_slots = 0;
  if (T == 1) {
    // bulk-copy variant: every tensor 16-byte aligned and its shared-memory slots fit beside the rest
    // ZMOE_LD_BULK=1 / ZMOE_LD_NO_BULK=1 force the choice (read once per process)
    static const bool force_on = getenv("ZMOE_LD_BULK") != nullptr && atoi(getenv("ZMOE_LD_BULK")) != 0;
    static const bool force_off = getenv("ZMOE_LD_NO_BULK") != nullptr && atoi(getenv("ZMOE_LD_NO_BULK")) != 0;
    const bool no_bulk = force_off || !(force_on || kLdBulkByDefault);
    bool aligned = true;
    for (int i = 0; i < 2; ++i) {
      if (!banks[i]) continue;
      const void* wptr[3] = {banks[i]->gate_w, banks[i]->up_w, banks[i]->down_w};
      for (int j = 0; j < 3; ++j) aligned = aligned && (((uintptr_t)wptr[j] % 16) == 0);
    }
    const int n_tasks = L->top_k + (L->n_shared ? 1 : 0);
    const int items = n_tasks * (L->d_ff / 16);
    int g_slots = (items + sms - 1) / sms;
    if (g_slots > 4) g_slots = 4;
    const int rs_g = L->d_model / 2 + 32, rs_d = L->d_ff / 2 + 32;
    const int bulk_off = (lay.total + 127) & ~127;
    const size_t total = (size_t)bulk_off + 128 + (size_t)g_slots * 32 * rs_g + (size_t)n_tasks * 16 * rs_d;
    if (!no_bulk && aligned && n_tasks <= 12 && total <= 220 * 1024) {
      p.bulk_off = bulk_off;
      p.g_slots = g_slots;
      return ld_launch<1, true, 2>(p, sms, total, st);
    }
    if (L->d_ff >= 2048) return ld_launch<1, false, 4>(p, sms, lay.total, st);
    return ld_launch<1, false, 2>(p, sms, lay.total, st);
  }
  if (L->d_ff >= 2048) {
    if (T <= 2) return ld_launch<2, false, 4>(p, sms, lay.total, st);
    if (T <= 4) return ld_launch<4, false, 4>(p, sms, lay.total, st);
    return ld_launch<8, false, 4>(p, sms, lay.total, st);
  }
  if (T <= 2) return ld_launch<2, false, 2>(p, sms, lay.total, st);
  if (T <= 4) return ld_launch<4, false, 2>(p, sms, lay.total, st);
  return ld_launch<8, false, 2>(p, sms, lay.total, st);
}

}  // extern "C"
