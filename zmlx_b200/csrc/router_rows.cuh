// Per-token-row router device functions shared by the router kernels and the fused decode-layer kernel.
// One warp owns one token row; the row's E scores live in registers (E <= 1024); top-k order is
// (score descending, expert id ascending).
#pragma once

#include <math_constants.h>

#include "common.cuh"
#include "layer_route.cuh"

namespace zmoe {

constexpr int kMaxVPL = 32;  // values per lane: E <= 1024
constexpr int kMaxK = 16;

__device__ __forceinline__ float load_logit(const void* p, int dtype, size_t i) {
  if (dtype == ZMOE_F32) return reinterpret_cast<const float*>(p)[i];
  return __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i]);
}

// Top-k of the lane-strided values v[j] (expert id = lane + 32*j) by ranking: every value
// counts how many others beat it under the canonical order (value descending, id ascending);
// the ranks are a permutation, so the entries ranked below K write themselves straight into
// slot order.  `scratch` is E + 2 * kMaxK floats owned by the warp.  All lanes end with the
// winners in sel_val/sel_idx.
template <int VPL>
__device__ __forceinline__ void warp_topk_masked(float (&v)[VPL], int E, int K, int lane, float* sel_val,
                                                 int* sel_idx, float* scratch) {
  // ranking runs on order-preserving integer keys (ld_order_key): a total order even when a row holds NaN
  // (NaN ranks below every number), so the ranks are always a permutation and every slot gets written
  uint32_t* keys = reinterpret_cast<uint32_t*>(scratch);
  float* out_v = scratch + E;
  int* out_i = reinterpret_cast<int*>(scratch + E + kMaxK);
  __syncwarp();
  uint32_t kv[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int idx = lane + 32 * j;
    kv[j] = ld_order_key(v[j] + 0.0f);
    if (idx < E) keys[idx] = kv[j];
  }
  if (lane < K) out_i[lane] = 0;
  __syncwarp();
  int rank[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) rank[j] = 0;
  for (int o = 0; o < E; ++o) {
    const uint32_t ok = keys[o];  // broadcast read
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      const int idx = lane + 32 * j;
      rank[j] += (ok > kv[j]) || (ok == kv[j] && o < idx);
    }
  }
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    const int idx = lane + 32 * j;
    if (idx < E && rank[j] < K) {
      out_v[rank[j]] = v[j];
      out_i[rank[j]] = idx;
    }
  }
  __syncwarp();
  for (int r = 0; r < K; ++r) {
    sel_val[r] = out_v[r];
    sel_idx[r] = min(max(out_i[r], 0), E - 1);
  }
}

// One warp routes one token row (softmax family); see zmoe_router_softmax_topk.
template <int VPL>
__device__ __forceinline__ void softmax_topk_row(const void* __restrict__ logits, int dtype, int row, int E, int K,
                                                 int flavour, const float* __restrict__ bias, int renorm,
                                                 float* __restrict__ weights, uint32_t* __restrict__ indices,
                                                 int lane, float* scratch) {
  float v[VPL];
  float mx = -CUDART_INF_F;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int idx = lane + 32 * j;
    v[j] = (idx < E) ? load_logit(logits, dtype, (size_t)row * E + idx) : -CUDART_INF_F;
    mx = fmaxf(mx, v[j]);
  }
  float sel_val[kMaxK];
  int sel_idx[kMaxK];
  if (flavour == ZMOE_ROUTER_TOPK_THEN_SOFTMAX) {
    warp_topk_masked<VPL>(v, E, K, lane, sel_val, sel_idx, scratch);
    if (lane == 0) {
      float m = sel_val[0];
      float s = 0.0f;
      for (int i = 0; i < K; ++i) s += expf(sel_val[i] - m);
      for (int i = 0; i < K; ++i) {
        weights[(size_t)row * K + i] = expf(sel_val[i] - m) / s;
        indices[(size_t)row * K + i] = (uint32_t)sel_idx[i];
      }
    }
    return;
  }
  // full softmax [+ bias] -> top-k -> optional renormalisation
  mx = warp_max(mx);
  float sum = 0.0f;
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int idx = lane + 32 * j;
    v[j] = (idx < E) ? expf(v[j] - mx) : 0.0f;
    sum += v[j];
  }
  sum = warp_sum(sum);
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int idx = lane + 32 * j;
    if (idx < E) {
      v[j] = v[j] / sum;
      if (bias) v[j] += bias[idx];
    }
  }
  warp_topk_masked<VPL>(v, E, K, lane, sel_val, sel_idx, scratch);
  if (lane == 0) {
    float denom = 1.0f;
    if (renorm) {
      float sk = 0.0f;
      for (int i = 0; i < K; ++i) sk += sel_val[i];
      denom = (renorm == 1) ? sk + 1e-20f : sk;
    }
    for (int i = 0; i < K; ++i) {
      weights[(size_t)row * K + i] = renorm ? sel_val[i] / denom : sel_val[i];
      indices[(size_t)row * K + i] = (uint32_t)sel_idx[i];
    }
  }
}

// sigmoid + selection bias, optional group-limited selection.  One warp routes one token row;
// `sc` is 2 * E + 64 + 2 * kMaxK floats of scratch owned by the warp (scores, group scores and
// keep flags, then the top-k scratch).
template <int VPL>
__device__ __forceinline__ void sigmoid_topk_row(const void* __restrict__ logits, int dtype, int row, int E, int K,
                                                 const float* __restrict__ bias, int n_group, int topk_group,
                                                 float scale, float* __restrict__ weights,
                                                 uint32_t* __restrict__ indices, int lane, float* sc) {
  float* gsc = sc + E;
  float* gkeep = gsc + 32;
  float v[VPL];
#pragma unroll
  for (int j = 0; j < VPL; ++j) {
    int idx = lane + 32 * j;
    if (idx < E) {
      float aff = sigmoid_stable(load_logit(logits, dtype, (size_t)row * E + idx));
      v[j] = aff + bias[idx];
      sc[idx] = v[j];
    } else {
      v[j] = -CUDART_INF_F;
    }
  }
  if (n_group > 1) {
    __syncwarp();
    const int per = E / n_group;
    for (int g0 = 0; g0 < n_group; g0 += 32) {
      // this build keeps n_group <= 32 (validated on the host); loop kept for clarity
      int g = g0 + lane;
      if (g < n_group) {
        float t1 = -CUDART_INF_F, t2 = -CUDART_INF_F;
        for (int j = 0; j < per; ++j) {
          float x = sc[g * per + j];
          if (x > t1) {
            t2 = t1;
            t1 = x;
          } else if (x > t2) {
            t2 = x;
          }
        }
        gsc[g] = t1 + t2;
      }
    }
    __syncwarp();
    if (lane < n_group) {
      float mine = gsc[lane];
      int rank = 0;
      for (int h = 0; h < n_group; ++h) {
        float o = gsc[h];
        rank += (o > mine) || (o == mine && h < lane);
      }
      gkeep[lane] = (rank < topk_group) ? 1.0f : 0.0f;
    }
    __syncwarp();
#pragma unroll
    for (int j = 0; j < VPL; ++j) {
      int idx = lane + 32 * j;
      if (idx < E && gkeep[idx / per] == 0.0f) v[j] = 0.0f;
    }
  }
  float sel_val[kMaxK];
  int sel_idx[kMaxK];
  warp_topk_masked<VPL>(v, E, K, lane, sel_val, sel_idx, sc + E + 64);
  if (lane == 0) {
    float aff[kMaxK];
    float sum = 0.0f;
    for (int i = 0; i < K; ++i) {
      aff[i] = sigmoid_stable(load_logit(logits, dtype, (size_t)row * E + sel_idx[i]));
      sum += aff[i];
    }
    float inv = 1.0f / sum;
    for (int i = 0; i < K; ++i) {
      float w = aff[i] * inv;
      if (scale != 1.0f) w = w * scale;
      weights[(size_t)row * K + i] = w;
      indices[(size_t)row * K + i] = (uint32_t)sel_idx[i];
    }
  }
}

}  // namespace zmoe
