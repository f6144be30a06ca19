// Builds the token-sorted expert plan inside one CTA (shared by the stand-alone plan
// kernel and the fused router kernel).
#pragma once

#include "common.cuh"

namespace zmoe {

// One CTA of NTHREADS threads groups `rows` (pair, m) rows by expert: histogram, exclusive
// scan, scatter.  `sm` needs 2 * E + 2 * NTHREADS + 2 ints (8-byte aligned).  The order of rows inside an expert's
// segment is arbitrary; every output row is computed from its own input row only, so
// results do not depend on it.  All threads of the CTA must call this.
template <int NTHREADS>
__device__ __forceinline__ void build_plan_block(const int* lhs, int lhs_div, const int* rhs, int P, int M, int E,
                                                 int* plan_base, int* sm) {
  int* count = sm;               // E
  int* cursor = sm + E;          // E
  // NTHREADS 64-bit cells: rows in the low half, number of experts that own rows in the high half
  unsigned long long* scan_tmp = reinterpret_cast<unsigned long long*>(sm + 2 * E + (((size_t)sm >> 2) & 1));
  const int rows = P * M;
  PlanView pv = plan_view(plan_base, rows, E);
  const int tid = threadIdx.x;
  __shared__ int bad;
  if (tid == 0) bad = 0;
  for (int e = tid; e < E; e += NTHREADS) count[e] = 0;
  __syncthreads();
  for (int p = tid; p < P; p += NTHREADS) {
    int e = rhs[p];
    if (e >= 0 && e < E)
      atomicAdd(&count[e], M);
    else
      bad = 1;
  }
  __syncthreads();
  // exclusive scan over E (chunked by NTHREADS), plus compaction of the experts that own rows
  int base = 0, abase = 0;
  for (int e0 = 0; e0 < E; e0 += NTHREADS) {
    int e = e0 + tid;
    int c = (e < E) ? count[e] : 0;
    int flag = c > 0;
    scan_tmp[tid] = (unsigned long long)(unsigned)c | ((unsigned long long)flag << 32);  // both scans in one pass
    __syncthreads();
    for (int o = 1; o < NTHREADS; o <<= 1) {
      unsigned long long v = (tid >= o) ? scan_tmp[tid - o] : 0ull;
      __syncthreads();
      scan_tmp[tid] += v;
      __syncthreads();
    }
    const unsigned long long packed = scan_tmp[tid];
    const unsigned long long ptotal = scan_tmp[NTHREADS - 1];
    __syncthreads();
    const int incl = (int)(packed & 0xFFFFFFFFull), aincl = (int)(packed >> 32);
    if (e < E) {
      int off = base + incl - c;
      pv.offset[e] = off;
      cursor[e] = off;
      if (flag) {
        const int a = abase + aincl - 1;
        pv.active[a] = e;
        reinterpret_cast<int4*>(pv.tasks)[a] = make_int4(e, off, c, 0);
      }
    }
    base += (int)(ptotal & 0xFFFFFFFFull);
    abase += (int)(ptotal >> 32);
  }
  for (int a = abase + tid; a < E; a += NTHREADS) reinterpret_cast<int4*>(pv.tasks)[a] = make_int4(0, 0, 0, 0);
  if (tid == 0) {
    pv.offset[E] = base;
    pv.hdr[0] = abase;
    pv.hdr[1] = rows;
    pv.hdr[3] = E;
  }
  __syncthreads();
  for (int p = tid; p < P; p += NTHREADS) {
    int e = rhs[p];
    if (e < 0 || e >= E) continue;
    int pos = atomicAdd(&cursor[e], M);
    int src = (lhs ? lhs[p] : p / lhs_div) * M;
    for (int m = 0; m < M; ++m) {
      pv.row_src[pos + m] = src + m;
      pv.row_dst[pos + m] = p * M + m;
    }
  }
  __syncthreads();
  if (tid == 0) pv.hdr[2] = bad;
}

}  // namespace zmoe
