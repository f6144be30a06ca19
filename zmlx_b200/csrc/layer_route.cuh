// Pieces of the one-launch decode block that do not touch the expert matmuls: hand-over words, the router
// linear's summation order (shared with the stand-alone router kernels so that both give the same bits) and
// the routing of the T token rows inside a CTA.
#pragma once

#include <math_constants.h>

#include "common.cuh"

namespace zmoe {

constexpr int kLdConsumers = 512;              // threads that compute (16 warps)
constexpr int kLdWarps = kLdConsumers / 32;    // consumer warps
constexpr int kLdThreads = kLdConsumers + 128;  // plus four producer warps (one per team) that only issue copies
constexpr int kLdMaxT = 8;
constexpr int kLdMaxK = 8;
constexpr int kLdMaxRouted = kLdMaxT * kLdMaxK;  // (token, slot) rows
constexpr int kLdMaxTasks = kLdMaxRouted + 1;
constexpr int kLdSpinLimit = 1 << 21;  // polls of a hand-over word, flag or mbarrier before a warp gives up (~1 s)

// Barrier of the consumer threads only (the producer warp never joins it).
__device__ __forceinline__ void ld_csync() { asm volatile("bar.sync 1, %0;" ::"n"(kLdConsumers) : "memory"); }

// ------------------------------------------------------------------ hand-over words
// Values that one CTA produces and others consume (router logits, activated rows, projected rows) travel as
// 32-bit words {launch tag:16 | bfloat16:16}.  A consumer re-reads a word until its tag is the current
// launch's, so the value and its "ready" flag arrive in one relaxed access and no grid-wide barrier is needed.
// The tag is 1 + (launch count mod 65535): never zero, so a zeroed workspace holds no valid word.
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
__device__ __forceinline__ void st_relaxed_v4(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.gpu.global.v4.u32 [%0], {%1,%1,%1,%1};" ::"l"(p), "r"(v) : "memory");
}

// System-scope forms for words that another GPU writes or reads (expert parallel: token rows and projected rows
// cross NVLink as the same tagged words, stored straight into the owner's buffer).
__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_relaxed_sys_v4(const uint32_t* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p)
               : "memory");
  return v;
}
__device__ __forceinline__ void st_relaxed_sys_u32(uint32_t* p, uint32_t v) {
  asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void st_relaxed_sys_v4(uint32_t* p, const uint4& v) {
  asm volatile("st.relaxed.sys.global.v4.u32 [%0], {%1,%2,%3,%4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
               : "memory");
}

// Order-preserving map float -> uint32 (-0 must be folded into +0 first).  NaN maps to 0, below every number
// (the order a stable descending argsort gives: NaN scores come last, among themselves by ascending id), so
// the keys of a row are totally ordered whatever it holds.
__device__ __forceinline__ uint32_t ld_order_key(float v) {
  const uint32_t u = __float_as_uint(v);
  if (v != v) return 0u;
  return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

// ------------------------------------------------------------------ router linear: the summation order
// A logit is sum_k x[k] * Wr[e][k] in float.  The row is cut into kRouterSegs interleaved segments of 16-byte
// pieces: piece i belongs to segment (i / 32) % kRouterSegs, lane i % 32.  A lane chains fused multiply-adds
// over its pieces of one segment in ascending order, the 32 lanes of a segment are summed by the xor butterfly,
// and the segment sums are added in ascending order.  The one-launch block gives one segment to each of its 16
// warps (one memory round trip for a 14 KB row); the stand-alone kernels walk the segments with one warp.
// Both call this function, so their logits agree bit for bit.
constexpr int kRouterSegs = 16;

__device__ __forceinline__ float router_fma8(const uint4& wv, const uint4& xv, float acc) {
  const uint32_t ww[4] = {wv.x, wv.y, wv.z, wv.w};
  const uint32_t xw[4] = {xv.x, xv.y, xv.z, xv.w};
#pragma unroll
  for (int q = 0; q < 4; ++q) {
    acc = fmaf(bf16_bits_to_float(ww[q] & 0xffffu), bf16_bits_to_float(xw[q] & 0xffffu), acc);
    acc = fmaf(bf16_bits_to_float(ww[q] >> 16), bf16_bits_to_float(xw[q] >> 16), acc);
  }
  return acc;
}

// Lane partial of segment `seg`: pieces seg*32 + lane + 32*kRouterSegs*r, r = 0, 1, ...
__device__ __forceinline__ float router_segment_partial(const uint4* wrow, const uint4* xrow, int nvec, int seg,
                                                        int lane) {
  float acc = 0.0f;
  for (int i = seg * 32 + lane; i < nvec; i += 32 * kRouterSegs) acc = router_fma8(__ldg(wrow + i), __ldg(xrow + i), acc);
  return acc;
}

// The whole logit by one warp (all lanes return it).
__device__ __forceinline__ float router_logit_warp(const uint4* wrow, const uint4* xrow, int nvec, int lane) {
  float total = 0.0f;
  const int nseg = min(kRouterSegs, (nvec + 31) >> 5);
  for (int s = 0; s < nseg; ++s) total += warp_sum(router_segment_partial(wrow, xrow, nvec, s, lane));
  return total;
}

// The logits of one weight row against TB token rows at once: the same arithmetic per token as
// router_logit_warp (segment partials, then one warp sum per segment, added in segment order), with the TB
// independent chains interleaved so that their loads and shuffles overlap.
template <int TB>
__device__ __forceinline__ void router_logit_warp_multi(const uint4* wrow, const uint4* const (&xrow)[TB], int nvec,
                                                        int lane, float (&total)[TB]) {
#pragma unroll
  for (int t = 0; t < TB; ++t) total[t] = 0.0f;
  const int nseg = min(kRouterSegs, (nvec + 31) >> 5);
  for (int s = 0; s < nseg; ++s) {
    float acc[TB];
#pragma unroll
    for (int t = 0; t < TB; ++t) acc[t] = 0.0f;
    for (int i = s * 32 + lane; i < nvec; i += 32 * kRouterSegs) {
      const uint4 wv = __ldg(wrow + i);
#pragma unroll
      for (int t = 0; t < TB; ++t) acc[t] = router_fma8(wv, __ldg(xrow[t] + i), acc[t]);
    }
#pragma unroll
    for (int t = 0; t < TB; ++t) total[t] += warp_sum(acc[t]);
  }
}

// ------------------------------------------------------------------ routing of the T token rows
// Same arithmetic as the per-row router functions (softmax_topk_row / sigmoid_topk_row: the order of every
// floating-point sum is kept, so scores, indices and weights are bit-identical).  A single warp is slow at
// long dependent instruction sequences, so only what must be is done by one warp per row (waiting for the
// logits, the softmax scores, the weights of the winners); the selection itself -- ranking every score
// against every other one -- is spread over all consumer threads of the CTA.
//
// Step 1, one warp per row: wait for the row's logits (hand-over words written by the router threads of all
// CTAs), compute the selection scores and leave, per expert, the score, the logit and a 64-bit sort key
// {order-preserving score : 32 | ~expert id : 32} in shared memory.  Returns false when the wait ran out.
__device__ __forceinline__ bool ld_route_scores(const uint32_t* g_logits, uint32_t tag, int E, int family,
                                                const float* bias, float* vals, float* lgs, uint2* keys, int lane) {
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

// Step 1b, sigmoid family, all consumer threads: scores = sigmoid(logit) + bias, group-limited selection (a
// group's score is the sum of its two largest scores; the best topk_group groups are kept, ties to the lower
// group; the experts of the other groups are scored 0.0), then the sort keys.  Maxima and the sum of two
// numbers do not depend on evaluation order, so the result is bit-identical to the one-warp form of
// sigmoid_topk_row.  Contains consumer-wide barriers: every consumer thread must call it.
__device__ __forceinline__ void ld_sigmoid_scores(int T, int E, const float* bias, int n_group, int topk_group,
                                                  float* vals, const float* lgs, uint2* keys, float* gsc) {
  const int tid = threadIdx.x, lane = tid & 31, wid = tid >> 5;
  for (int i = tid; i < T * E; i += kLdConsumers) vals[i] = sigmoid_stable(lgs[i]) + bias[i % E];
  if (n_group > 1) {  // uniform over the CTA
    ld_csync();
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
    ld_csync();
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
    ld_csync();
    for (int i = tid; i < T * E; i += kLdConsumers) {
      const int t = i / E, e = i - t * E;
      if (gsc[t * 64 + 32 + e / per] == 0.0f) vals[i] = 0.0f;
    }
  }
  // each thread reads back only what it wrote itself
  for (int i = tid; i < T * E; i += kLdConsumers)
    keys[i] = make_uint2(~(uint32_t)(i % E), ld_order_key(vals[i] + 0.0f));
}

// Steps 1b and 2 of the sigmoid family by ONE warp per row, in registers: no consumer-wide barrier and no pass
// through shared memory between the score, the group-limited selection and the top-k.  For E <= 256 with either no
// groups or groups of exactly 32 experts (E == 32 * n_group: expert lane + 32 j belongs to group j, so a group's
// members are one register across the warp).  The arithmetic is that of ld_sigmoid_scores + ld_topk_select:
// maxima, the sum of a group's two largest scores, ranks under (value descending, index ascending) and order keys
// do not depend on evaluation order, so indices are bit-identical.
__device__ __forceinline__ void ld_sigmoid_route_warp(int E, int K, const float* bias, int n_group, int topk_group,
                                                      const float* lgs, int* sel_idx, int lane) {
  constexpr int NJ = 8;
  float v[NJ];
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    const int idx = lane + 32 * j;
    v[j] = idx < E ? sigmoid_stable(lgs[idx]) + bias[idx] : -CUDART_INF_F;
  }
  if (n_group > 1) {
    float gs[NJ];
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      float t1 = v[j], t2 = -CUDART_INF_F;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {  // merge the lanes' (largest, second largest) pairs
        const float o1 = __shfl_xor_sync(0xffffffffu, t1, o);
        const float o2 = __shfl_xor_sync(0xffffffffu, t2, o);
        const float hi = fmaxf(t1, o1);
        t2 = fmaxf(fminf(t1, o1), fmaxf(t2, o2));
        t1 = hi;
      }
      gs[j] = t1 + t2;
    }
#pragma unroll
    for (int j = 0; j < NJ; ++j) {
      int rank = 0;
#pragma unroll
      for (int h = 0; h < NJ; ++h)
        if (h < n_group) rank += (gs[h] > gs[j]) || (gs[h] == gs[j] && h < j);
      if (j < n_group && rank >= topk_group) v[j] = 0.0f;
    }
  }
  uint32_t kv[NJ];
  unsigned live = 0u;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    kv[j] = ld_order_key(v[j] + 0.0f);
    if (lane + 32 * j < E) live |= 1u << j;
  }
#pragma unroll 1
  for (int r = 0; r < K; ++r) {
    uint32_t bk = 0u;
    int bj = -1;
#pragma unroll
    for (int j = 0; j < NJ; ++j)
      if (((live >> j) & 1u) && (bj < 0 || kv[j] > bk)) {
        bk = kv[j];
        bj = j;
      }
    const uint32_t mx = __reduce_max_sync(0xffffffffu, bj >= 0 ? bk : 0u);
    const unsigned none = 0x7fffffffu;
    const unsigned win = __reduce_min_sync(0xffffffffu, (bj >= 0 && bk == mx) ? (unsigned)(lane + 32 * bj) : none);
    if (lane == 0) sel_idx[r] = win == none ? 0 : (int)win;
    if (win != none && (int)(win & 31u) == lane) live &= ~(1u << (win >> 5));
  }
  __syncwarp();
}

// Step 2, small expert counts: rank of every score under (score descending, expert id ascending) by all
// consumer threads -- one unsigned 64-bit comparison of the sort keys per pair.  The ranks of a row are a
// permutation, so the experts ranked below K write themselves into slot order.
__device__ __forceinline__ void ld_rank_select(const uint2* keys, int T, int E, int K, int* sel_idx) {
  const int pairs = T * E;
  int P = 1;  // threads that share one score's scan
  while (P < 32 && P * 2 * pairs <= kLdConsumers) P *= 2;
  const int lp = 31 - __clz(P);
  const int per_pass = kLdConsumers >> lp;
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

// Step 2, large expert counts (where all-pairs ranking costs too many comparisons): the same selection in two
// rounds of warp arg-max:
//   (a) one warp per 32 consecutive experts of a row picks its own K best, best first.  A round = one
//       redux.sync.max over the lanes' order keys, a ballot of the lanes that hold the maximum, and the lowest
//       such lane (= the lowest expert id among equals) leaves the race;
//   (b) one warp per row picks the K best of the (E / 32) * 8 candidates the same way.  Candidate c = 8 * w + r is
//       warp w's r-th pick: among equal scores a smaller c is a smaller expert id (ids grow with w, and a warp
//       emits equal scores in ascending id order), so "lowest candidate among equals" is the canonical tie rule.
// The result equals ranking every score against every other one.  cand_key / cand_idx hold 64 entries per row.
// Contains a consumer-wide barrier: every consumer thread must call it.
__device__ __forceinline__ void ld_topk_select(const uint2* keys, int T, int E, int K, uint32_t* cand_key,
                                               int* cand_idx, int* sel_idx) {
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  const int nw = (E + 31) >> 5;  // <= 8
  for (int task = wid; task < T * nw; task += kLdWarps) {
    const int t = task / nw, w = task - t * nw;
    const int i = w * 32 + lane;
    bool live = i < E;
    const uint32_t key = live ? keys[(size_t)t * E + i].y : 0u;
#pragma unroll 1
    for (int r = 0; r < kLdMaxK; ++r) {
      const uint32_t mx = __reduce_max_sync(0xffffffffu, live ? key : 0u);
      const uint32_t ball = __ballot_sync(0xffffffffu, live && key == mx);
      const int src = __ffs(ball) - 1;  // -1: the warp has run out of experts
      if (lane == 0) {
        cand_key[t * 64 + w * 8 + r] = mx;
        cand_idx[t * 64 + w * 8 + r] = (r < K && src >= 0) ? w * 32 + src : -1;
      }
      if (lane == src) live = false;
    }
  }
  ld_csync();
  if (wid < T) {
    const int t = wid;
    const int nc = nw * 8;
    const int i0 = cand_idx[t * 64 + lane];
    const int i1 = (lane + 32 < nc) ? cand_idx[t * 64 + lane + 32] : -1;
    bool v0 = lane < nc && i0 >= 0, v1 = i1 >= 0;
    const uint32_t k0 = cand_key[t * 64 + lane], k1 = (lane + 32 < nc) ? cand_key[t * 64 + lane + 32] : 0u;
#pragma unroll 1
    for (int r = 0; r < K; ++r) {
      const uint32_t m0 = v0 ? k0 : 0u, m1 = v1 ? k1 : 0u;
      const uint32_t mx = __reduce_max_sync(0xffffffffu, max(m0, m1));
      const uint32_t b0 = __ballot_sync(0xffffffffu, v0 && k0 == mx);
      const uint32_t b1 = __ballot_sync(0xffffffffu, v1 && k1 == mx);
      const int src = b0 ? __ffs(b0) - 1 : __ffs(b1) - 1;
      const int won = __shfl_sync(0xffffffffu, b0 ? i0 : i1, src < 0 ? 0 : src);
      if (lane == 0) sel_idx[t * K + r] = (src >= 0 && won >= 0) ? won : 0;
      if (lane == src) {
        if (b0)
          v0 = false;
        else
          v1 = false;
      }
    }
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

}  // namespace zmoe
