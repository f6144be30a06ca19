/*
 * libzmoe -- C ABI of the B200 (sm_100a) MoE decode hot path.
 *
 * Every entry point replaces one piece of the reference (ZMLX v0.8.5 on MLX);
 * the reference interface each one stands in for is cited as file:line
 * relative to the ZMLX tree ("patch:" = integrations/mlx_local_integration/
 * gather_qmm_swiglu.patch, "moe.py" = src/zmlx/kernels/moe.py).
 *
 * Conventions (modelled on the reference's only C ABI, zig/shim/shim.h:48-127):
 *   - plain pointers and sizes; all data pointers are DEVICE pointers owned by
 *     the caller; the library allocates no user-visible memory;
 *   - every call takes a cudaStream_t (passed as void*), only enqueues work and
 *     returns; nothing synchronises the device;
 *   - return value: 0 on success, a negative ZMOE_ERR_* otherwise; no call
 *     throws, exits or traps the device; zmoe_last_error() gives the message
 *     of the calling thread's last failure;
 *   - dtype T is bfloat16 (16-bit pattern); packed 4-bit tensors are uint32
 *     with code i of a row in word i/8 at bit 4*(i%8)
 *     (src/zmlx/kernels/quant.py:109-120); affine scales/biases are T, shaped
 *     (E, N, K/group_size); mxfp4 scales are e8m0 bytes shaped (E, N, K/32).
 */
#ifndef ZMOE_H_
#define ZMOE_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ZMOE_ABI_VERSION 2

enum zmoe_status {
  ZMOE_OK = 0,
  ZMOE_ERR_SHAPE = -1,
  ZMOE_ERR_DTYPE = -2,
  ZMOE_ERR_ALIGN = -3,
  ZMOE_ERR_UNSUPPORTED = -4,
  ZMOE_ERR_CUDA = -5,
  ZMOE_ERR_TIMEOUT = -6,
  ZMOE_ERR_WORKSPACE = -7
};

enum zmoe_dtype { ZMOE_F32 = 0, ZMOE_BF16 = 1 };

/* Quantisation modes of the expert weights. */
enum zmoe_qmode {
  ZMOE_Q_AFFINE4 = 0, /* MLX affine 4-bit, w = q*scale + bias per group */
  ZMOE_Q_MXFP4 = 1    /* e2m1 codes, one e8m0 scale per 32 along K      */
};

/* Rounding contract of the SwiGLU epilogue. */
enum zmoe_swiglu_mode {
  ZMOE_SWIGLU_CPU = 0,   /* gate, up rounded to T; g*1/(1+exp(-g))*u in float; one rounding (patch:47-55) */
  ZMOE_SWIGLU_PER_OP = 1, /* every elementwise op rounded to T, sigmoid as 1/(1+exp|g|) (src/zmlx/msl.py:20-24,
                             src/zmlx/kernels/transformer.py:882-897) */
  ZMOE_SWIGLU_FP32 = 2    /* gate and up stay in float through g*sigmoid(g)*u, sigmoid as 1/(1+exp|g|); one
                             rounding at the store (the dense fused GEMV, src/zmlx/kernels/quant.py:103-124).
                             zmoe_gather_qmm_swiglu with affine weights only. */
};

/* Rounding contract of the weighted combine (slots summed in order 0..K-1). */
enum zmoe_combine_mode {
  ZMOE_COMBINE_FP32 = 0,        /* moe_combine_fp32          moe.py:1020-1026 : float acc (fma), float out   */
  ZMOE_COMBINE_FP32_NO_FMA = 1, /* moe_combine_fp32_no_fma   moe.py:1075-1095 : product rounded, float out   */
  ZMOE_COMBINE_T = 2,           /* moe_combine               moe.py:840-846   : float acc (fma), T out       */
  ZMOE_COMBINE_NO_FMA = 3,      /* moe_combine_no_fma        moe.py:899-912   : product rounded, T out       */
  ZMOE_COMBINE_EXACT = 4,       /* moe_combine_exact         moe.py:963-970   : product and sum rounded to T */
  ZMOE_COMBINE_STREAM_T = 5     /* _weighted_accumulate_kernel moe.py:1821-1841: acc = T(float(acc) + w*v)   */
};

/* Router flavours of zmoe_router_softmax_topk. */
enum zmoe_softmax_router {
  ZMOE_ROUTER_TOPK_THEN_SOFTMAX = 0, /* top-k of logits, softmax over the k   moe.py:1287-1315, 1380-1386 */
  ZMOE_ROUTER_SOFTMAX_THEN_TOPK = 1  /* full softmax [+bias], top-k, optional renorm   moe.py:1326-1396;
                                        Qwen3: src/zmlx/patch/patterns/moe_mlp.py:260-266 */
};

int zmoe_abi_version(void);

/* Message of this thread's last failing call ("" if none). Never NULL. */
const char* zmoe_last_error(void);

/* ------------------------------------------------------------------ routers */

/*
 * topk_gating_softmax / Qwen3 gating / GPT-OSS gating.
 * Replaces: moe.py:1239-1396 (topk_gating_softmax), moe.py:1448-1490
 * (router_argpartition_logits_topk), moe_mlp.py:226-274.
 * logits (T, E) of logits_dtype; bias (E) float or NULL; renorm: 0 none, 1 divide
 * by (sum + 1e-20) (moe.py:196), 2 divide by sum (moe_mlp.py:265).
 * Outputs: weights (T, K) float, indices (T, K) uint32, slot order = score
 * descending, ties to the lower expert id.  E <= 1024, K <= 16.
 */
int zmoe_router_softmax_topk(const void* logits, int logits_dtype, int T, int E, int K, int flavour,
                             const float* bias, int renorm, float* weights, uint32_t* indices, void* stream);

/*
 * deepseek_router_topk_sigmoid (+ the routed_scaling_factor multiply of the gate).
 * Replaces: moe.py:1745-1817 (kernel moe.py:1502-1679) and
 * src/zmlx/patch/patterns/deepseek_router.py:108-120.
 * score = sigmoid(l) + bias; with n_group > 1 a group's score is the sum of its two
 * largest scores, the best topk_group groups are kept (ties to the lower group) and
 * the others are scored 0.0; weights = sigmoid(l)[sel] / sum, then * scale.
 */
int zmoe_router_sigmoid_bias_topk(const void* logits, int logits_dtype, int T, int E, int K, const float* bias,
                                  int n_group, int topk_group, float scale, float* weights, uint32_t* indices,
                                  void* stream);

/*
 * Router linear: logits[t, e] = T( sum_k x[t,k] * Wr[e,k] ), x (T, d) T, Wr (E, d) T.
 * Replaces the model's gate matmul (deepseek_router.py:107, `x @ weight.T`) on the
 * fused-layer path.  out_dtype selects T or float logits.
 */
int zmoe_router_logits(const void* x, const void* wr, int T, int E, int d, void* logits, int out_dtype,
                       void* stream);

/*
 * Fused router for one MoE block: router linear (T logits, as above), the family's top-k and
 * the token-sorted expert plan over the T*K (token, slot) pairs, in ONE launch.
 * family 0: top-k of logits then softmax (moe.py:1287-1315); 1: softmax then top-k with
 * `renorm` as in zmoe_router_softmax_topk (moe_mlp.py:260-266); 2: sigmoid + bias with
 * n_group / topk_group / scale as in zmoe_router_sigmoid_bias_topk.  Replaces the gate call and
 * `_gating` of the patched block (moe_mlp.py:202-289) on the fused-layer path.
 * logits (T, E) T is written as a by-product; plan may be NULL; counter is one int of device
 * memory that must be zero before the first call (the kernel leaves it zero).
 */
int zmoe_route(const void* x, const void* wr, int T, int E, int d, int K, int family, const float* bias, int renorm,
               int n_group, int topk_group, float scale, void* logits, float* weights, uint32_t* indices, void* plan,
               size_t plan_bytes, int* counter, void* stream);

/* --------------------------------------------------- token-sorted expert plan */

/*
 * The gather ops take (lhs, rhs) index pairs (patch:754-781).  A "plan" groups the
 * pairs by expert so that each expert's weights are streamed once for all of its
 * rows.  Pair p, row m reads x row lhs[p]*M + m, uses expert rhs[p] and writes
 * output row p*M + m.  lhs == NULL means lhs[p] = p / lhs_div (lhs_div >= 1).
 * plan must hold zmoe_plan_bytes(P*M, E) bytes.  No reference counterpart: MLX
 * re-reads an expert per row (patch:576).
 */
size_t zmoe_plan_bytes(int rows, int E);
int zmoe_build_plan(const int32_t* lhs, int lhs_div, const int32_t* rhs, int P, int M, int E, void* plan,
                    size_t plan_bytes, void* stream);

/* ------------------------------------------------------------ expert matmuls */

/*
 * mx.gather_qmm_swiglu: out[r, :] = swiglu(x_r @ Wg[e_r].T, x_r @ Wu[e_r].T).
 * Replaces: python binding patch:995-1013, op patch:695-800, Metal kernel
 * patch:329-510, CPU eval patch:64-192; wrapper src/zmlx/kernels/fused_moe.py:39-106.
 * x (x_rows, K) T with row stride ldx; weights (E, N, K/8) uint32; out (rows, N) T.
 * biases are ignored for ZMOE_Q_MXFP4.  rows_hint is an upper bound on the rows of
 * any one expert (e.g. the token count for top-k routing); it sizes shared memory.
 * K % 64 == 0 (affine: K % group_size == 0, group_size == 64).
 */
int zmoe_gather_qmm_swiglu(const void* x, int x_rows, int ldx, const uint32_t* gate_w, const void* gate_scales,
                           const void* gate_biases, const uint32_t* up_w, const void* up_scales,
                           const void* up_biases, int E, int N, int K, int group_size, int qmode,
                           const void* plan, int rows, int rows_hint, void* out, int swiglu_mode, void* stream);

/*
 * mx.gather_qmm(transpose=True): out[r, :] = T(x_r @ W[e_r].T).
 * Replaces the third-party op at its call sites moe.py:1219-1229, 2147-2157 and
 * moe_mlp.py:571-574 (switch_mlp.down_proj).  With x_by_output_row != 0 output row r
 * reads x row r (the down projection after gather_qmm_swiglu, whose output rows are
 * already one per pair) instead of the plan's lhs row (bit 0).  Bit 1 of x_by_output_row
 * declares that the plan was written before the kernel that produced x started; the call
 * may then stream its first weights while that kernel is still running.
 */
int zmoe_gather_qmm(const void* x, int x_rows, int ldx, const uint32_t* w, const void* scales, const void* biases,
                    int E, int N, int K, int group_size, int qmode, const void* plan, int rows, int rows_hint,
                    int x_by_output_row, void* out, void* stream);

/* ------------------------------------------------------------------- combine */

/*
 * out[t, d] = sum_i w[t, i] * y[t, i, d] under one of the reference's five rounding
 * contracts (+ the streaming one).  Replaces moe.py:859-1127 and the accumulate
 * kernels moe.py:1821-1921; `post_scale` != 1 is unused by the reference (pass 1).
 * y (T, K, D) of y_dtype; w (T, K) of w_dtype; out (T, D): float for the FP32
 * modes, T otherwise.  residual (T, D) T or NULL is added after the combine and the
 * sum rounded to T (the `y + shared_experts(x)` of moe_mlp.py:1059-1061); it needs a
 * T-output mode, or an FP32 mode with out_t bit 0 set (cast to T first, moe_mlp.py:1002).
 * out_t bit 1: round the weights to T before use (`weights.astype(x.dtype)`,
 * moe_mlp.py:288).
 */
int zmoe_moe_combine(const void* y, int y_dtype, const void* w, int w_dtype, int T, int K, int D, int mode,
                     void* out, int out_t, const void* residual, void* stream);

/*
 * Elementwise SwiGLU on T tensors: out[i] = silu(gate[i]) * up[i] under `swiglu_mode`.
 * Replaces transformer.swiglu2 (src/zmlx/kernels/transformer.py:925-1005) and its GLM specialisation
 * glm_fused_swiglu (src/zmlx/kernels/discovered/glm_fused_swiglu.py:65-90), which the patched block uses on its
 * unfused path (src/zmlx/patch/patterns/moe_mlp.py:712-716); ZMOE_SWIGLU_PER_OP is their in-T arithmetic.
 */
int zmoe_swiglu(const void* gate, const void* up, long long n, int swiglu_mode, void* out, void* stream);

/*
 * gather_qmm_combine_quantized: out[t] = sum_k gate[t,k] * T(act[t,k] @ W[idx[t,k]].T).
 * Replaces moe.py:2043-2174 (and the K-vectorised form moe.py:1198-1236).
 * act (T*K, Kin) T; plan built over rhs = idx (T*K pairs, lhs = identity);
 * scratch must hold T*K*N T values; the call clears it first, so a pair whose expert id lies
 * outside 0..E-1 (dropped by the plan) contributes zero.
 */
int zmoe_gather_qmm_combine(const void* act, int ldx, const uint32_t* w, const void* scales, const void* biases,
                            int E, int N, int Kin, int group_size, int qmode, const void* plan, int T, int K,
                            const void* gate, int gate_dtype, int mode, void* scratch, void* out, int out_t,
                            void* stream);

/*
 * The same operation as zmoe_gather_qmm_combine for callers that have no scratch buffer to give and
 * must not allocate one: code running inside a CUDA-graph capture or a real-time serving loop where
 * cudaMalloc (a device-wide synchronising call) is off limits, and hosts that bind this library from a
 * runtime whose allocator they cannot reach.  It has no counterpart in the reference.
 *
 * The T*K*N projected rows live in a 4 MiB array inside the library image (every GPU that loads the
 * library holds it until the process exits), so T*K*N must not exceed 2,097,152; larger calls fail
 * with ZMOE_ERR_WORKSPACE and a message.  The call allocates nothing.  The first call on each device
 * looks up the array's device address (a one-time, non-stream runtime query): make that first call
 * outside any stream capture.  All calls on a device share the array: two calls that may overlap on the
 * GPU (different streams) race with each other; calls on one stream are safe.  The used part of the
 * array is zeroed at the start of every call.
 */
int zmoe_gather_qmm_combine_noalloc(const void* act, int ldx, const uint32_t* w, const void* scales,
                                    const void* biases, int E, int N, int Kin, int group_size, int qmode,
                                    const void* plan, int T, int K, const void* gate, int gate_dtype, int mode,
                                    void* out, int out_t, void* stream);

/* --------------------------------------------------------- one-launch decode block */

/* Packed tensors of one expert bank: (E, N, K/8) uint32 weights, (E, N, K/64) T scales and biases. */
typedef struct zmoe_expert_bank {
  const uint32_t* gate_w;
  const void* gate_scales;
  const void* gate_biases;
  const uint32_t* up_w;
  const void* up_scales;
  const void* up_biases;
  const uint32_t* down_w;
  const void* down_scales;
  const void* down_biases;
} zmoe_expert_bank;

/*
 * One MoE block as the patched module sees it (attribute contract of
 * src/zmlx/patch/patterns/moe_mlp.py:392-409,778-809 and deepseek_router.py:58-69).
 * router_family / router_bias / renorm / n_group / topk_group / routed_scale as in zmoe_route;
 * combine_mode and out_flags as `mode` and `out_t` of zmoe_moe_combine; n_shared is 0 or 1 and
 * the shared expert has the routed experts' d_ff.
 */
typedef struct zmoe_layer_desc {
  int32_t E, d_model, d_ff, top_k;
  int32_t group_size, qmode;
  int32_t router_family, renorm, n_group, topk_group;
  float routed_scale;
  int32_t n_shared;
  int32_t swiglu_mode, shared_swiglu_mode;
  int32_t combine_mode, out_flags;
  int32_t launch_mode; /* 0: cooperative launch (every CTA guaranteed resident).  1: regular launch with
                          programmatic dependent launch -- the kernel is set up while the previous kernel of the
                          stream still runs, which saves ~3 us per block in a chain of blocks; the caller vouches
                          that nothing else (another stream, another process) keeps SMs busy for long: CTAs that
                          cannot become resident make the bounded waits run out (status word, no hang) */
  const void* router_w;     /* (E, d_model) T */
  const float* router_bias; /* (E) or NULL */
  zmoe_expert_bank routed;
  zmoe_expert_bank shared;  /* ignored when n_shared == 0 */
  int32_t debug_flags;      /* 0 in production; ZMOE_DEBUG_* bits are test hooks */
  int32_t reserved;
  void* debug_stamps;       /* NULL in production; else 32 int64 of device memory: CTA 0 records its cycle
                               counter at the phase boundaries (router linear, token staging, logits received,
                               top-k, task list, gate/up done, h staged, down done, combine done) */
  /* Expert parallel (zero / NULL when the block lives on one GPU).  E stays the router's expert count; the
     `routed` bank holds this rank's E / ep_world experts (experts ep_rank * E / ep_world ...); router and
     shared expert are replicated.  ep_inbox[r] is rank r's inbox as seen from THIS rank: its own buffer for
     r == ep_rank, a peer mapping (zmoe_ep_import) otherwise. */
  int32_t ep_world, ep_rank;
  void* ep_inbox[8];
} zmoe_layer_desc;

/* debug_flags bit: expert 0's router logit is never published, so that every CTA's bounded wait for it runs
   out -- the launch must end by itself with the status word set (failure detection without a GPU fault). */
#define ZMOE_DEBUG_WITHHOLD_LOGIT 1
/* debug_flags bit: with ep_world <= 1, still send the token rows and the projected rows through ep_inbox[0]
   (the expert-parallel data path on one GPU, for tests). */
#define ZMOE_DEBUG_FORCE_INBOX 2

/*
 * The whole patched block forward for a few decode tokens (src/zmlx/patch/patterns/moe_mlp.py:883-1063:
 * gate -> experts -> combine -> + shared_experts(x)) in ONE launch: router linear, the family's
 * top-k, gather_qmm_swiglu, the down projection, the ordered combine and the shared expert.  Same
 * arithmetic contracts as the separate entry points above.  Covers 4-bit affine weights with group
 * size 64, 1..8 tokens, top_k <= 8, E <= 256, d_model and d_ff multiples of 256, packed weights 16-byte
 * aligned, as long as the token rows fit in shared memory beside the weight stages; other shapes fail with
 * ZMOE_ERR_UNSUPPORTED (zmoe_layer_decode_workspace_bytes returns 0 for them) and take the separate calls.
 * Both functions need the CUDA device of the call to be current (sizes depend on its SM count).
 *
 * workspace: zmoe_layer_decode_workspace_bytes(L, T) bytes, 256-byte aligned, ALL ZERO before the first
 * call, then left to the library and used with the same T (zero it again before changing T).  It starts
 * with five ints {-, -, sign-in count, status, launch count}.  CTAs hand the router logits, the activated
 * rows and the projected rows to each other through the workspace as tagged 32-bit words and re-read a word
 * until it carries the current launch's tag; every such wait is bounded, and one that runs out sets status
 * to 1 and ends the launch with `out` undefined (read it with zmoe_layer_decode_status).  One workspace
 * serves one stream at a time.
 * x (T, d_model) T with row stride ldx; out (T, d_model) T (float for the FP32 combine modes without
 * out_flags bit 0); weights (T, top_k) float and indices (T, top_k) uint32 receive the routing when not
 * NULL.
 */
size_t zmoe_layer_decode_workspace_bytes(const zmoe_layer_desc* L, int T);
int zmoe_layer_decode(const zmoe_layer_desc* L, const void* x, int ldx, int T, void* workspace,
                      size_t workspace_bytes, float* weights, uint32_t* indices, void* out, void* stream);

/*
 * Expert parallel form of zmoe_layer_decode (no reference counterpart: the reference runs on one device and
 * only disables its MoE pattern under tensor parallelism, src/zmlx/exo.py:141-151; the exchange sits where its
 * dispatch and combine kernels are, moe.py:776-827 and :831-1127).  Every rank calls zmoe_layer_decode with
 * its own T tokens, the same launch count on every rank.  In ONE launch per rank: the rank stores its token
 * rows into every rank's inbox (plain peer stores of tagged words), routes all T * ep_world tokens, runs the
 * (token, slot) rows whose expert it holds, and the down projection stores each projected row straight into
 * the inbox of the token's home rank, which combines its own tokens' rows in slot order after a bounded wait
 * -- bit-identical to the one-GPU order.  No collective call, nothing to synchronise on the host.  T * ep_world
 * must not exceed 8.  Each rank owns an inbox of zmoe_layer_decode_inbox_bytes(L, T) bytes, zeroed before its
 * first use, in memory the peers can map (zmoe_ep_alloc / zmoe_ep_export / zmoe_ep_import below, or any other
 * peer-accessible allocation).
 */
size_t zmoe_layer_decode_inbox_bytes(const zmoe_layer_desc* L, int T);

/* Peer-mappable device memory for the inboxes: allocate (zeroed), export a 64-byte handle, map a peer's
   handle, and undo both.  These are set-up calls: they allocate and synchronise. */
int zmoe_ep_alloc(size_t bytes, void** ptr);
int zmoe_ep_free(void* ptr);
int zmoe_ep_export(const void* ptr, void* handle64);
int zmoe_ep_import(const void* handle64, void** ptr);
int zmoe_ep_unmap(void* ptr);

/*
 * Status of the launches that have used `workspace`: copies the status word to the host on `stream` and WAITS
 * for the stream (the one call of this library that synchronises; make it where the caller synchronises
 * anyway, e.g. when it reads the block's output).  Returns ZMOE_OK, or ZMOE_ERR_TIMEOUT when a bounded wait
 * ran out in some launch since the word was last cleared; with clear != 0 the word is zeroed again on
 * `stream`.  No reference counterpart (the reference has no cross-CTA waits).
 */
int zmoe_layer_decode_status(const void* workspace, int clear, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ZMOE_H_ */
