/*
 * deltanet_b200.h -- C ABI of the B200 (sm_100a) delta-rule recurrence library.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream (passed as
 * void* so that this header needs no CUDA include), only ENQUEUES work on that stream,
 * allocates nothing, keeps no pointer after it returns, and reports problems through an
 * int status (0 = ok; see dn_status_string).  The caller owns every buffer.
 *
 * The functions replace, one for one, the device work behind the reference package's
 * differentiable operator (paths are those inside the reference project):
 *
 *   reference interface                                              replaced by
 *   -----------------------------------------------------------------------------------------
 *   custom-VJP op fwd     src/deltanet_tpu/gdn2.py:1479-1494,1176-1389   dn_chunk_fwd
 *   custom-VJP op bwd     src/deltanet_tpu/gdn2.py:1496-1766             dn_chunk_bwd
 *   pallas_prepass_fwd    src/deltanet_tpu/gdn2.py:1262-1276 (body 115-240)   dn_prepass_fwd
 *   pallas_split_fwd      src/deltanet_tpu/gdn2.py:1331-1376 (body 585-652)   dn_state_fwd
 *   pallas_recompute_states src/deltanet_tpu/gdn2.py:1614-1630 (body 655-695) dn_recompute_states
 *   pallas_split_bwd      src/deltanet_tpu/gdn2.py:1674-1690 (body 698-769)   dn_state_bwd
 *   pallas_prepass_bwd    src/deltanet_tpu/gdn2.py:1737-1752 (body 243-582)   dn_prepass_bwd
 *   segment canonicalisation src/deltanet_tpu/gdn2.py:2081-2094               dn_canonical_segments
 *   gdn2_decode_step core src/deltanet_tpu/gdn2.py:2393-2489                  dn_decode_step
 *
 * Tensor layouts are the reference's own, un-broadcast and un-padded:
 *   q,k   (B, L, Hk, K)      v, out, d_out   (B, L, Hv, V)      state  (B, Hv, K, V)
 *   g,b   (B, L, gh[, gc])   gh in {1,Hk,Hv}, gc in {1,K}        w  (B, L, wh[, wc]), wc in {1,V}
 *   segment ids (B, L) int32, canonical (they step by one at every document change).
 * L need not be a multiple of the chunk: rows past L behave as the reference's padding.
 *
 * "Exec heads": as in the reference (gdn2.py:1992-2007) the recurrence runs on H = Hk heads of
 * value width Vw = (Hv/Hk)*V when neither g nor b is given per value head, and on H = Hv heads
 * of width Vw = V otherwise.  Residual and scratch buffers use the exec-head layout (B,H,NC,...).
 */
#ifndef DELTANET_B200_H_
#define DELTANET_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* element types */
enum { DN_F32 = 0, DN_BF16 = 1 };
/* matmul precision, the reference's precision="fp32" | "bf16" (gdn2.py:28-35) */
enum { DN_PREC_FP32 = 0, DN_PREC_BF16 = 1 };

/* flags */
enum {
  DN_QK_L2NORM      = 1u << 0, /* normalise q,k in the kernel prologue (gdn2.py:2113-2122 / 133-138) */
  DN_FUSE_PROLOGUE  = 1u << 1, /* g,b,w are pre-activations (gdn2.py:133-142, adjoints 558-575)   */
  DN_HAS_INIT       = 1u << 2, /* an initial state is given (gdn2.py:613-617)                      */
  DN_STABILITY_GUARD= 1u << 3, /* stability_guard: decay clamped to <= -1e-6 (activated, with DN_FUSE_PROLOGUE;
                                  else the given g) and, without the fused prologue, b to >= 0 (gdn2.py:1972-1974) */
  DN_STATE_FP32_MM  = 1u << 4, /* state_fp32_matmul (gdn2.py:625)                                   */
  DN_INFERENCE      = 1u << 5, /* forward only: no T / chunk-state residuals (gdn2.py:1257,1322)    */
  DN_TRUNC_DT_BF16  = 1u << 6, /* truncate_bwd_dT_bf16 (gdn2.py:327-330)                            */
  DN_RESET_PER_HEAD = 1u << 7, /* decode: reset is (B,Hv), one flag per sequence and value head      */
  DN_SP_SKIP_PROVISIONAL = 1u << 8 /* dn_sp_summary: leave the outputs of the chunks that depend on the
                                      incoming state to dn_sp_correct_fwd, which rewrites exactly those  */
};

/* status codes */
enum {
  DN_OK = 0,
  DN_ERR_BAD_SHAPE = 1,      /* a dimension outside what the kernels support          */
  DN_ERR_BAD_DTYPE = 2,
  DN_ERR_NULL_POINTER = 3,   /* a required buffer is NULL                              */
  DN_ERR_SCRATCH_TOO_SMALL = 4,
  DN_ERR_CUDA_LAUNCH = 5,    /* cudaGetLastError() after a launch was not cudaSuccess  */
  DN_ERR_UNSUPPORTED = 6,
  DN_ERR_STATIC_SCRATCH_EXCEEDED = 7, /* dn_prepass_fwd_static: the shape needs more scratch than the built-in array */
  DN_ERR_DEVICE_WAIT = 8     /* an EARLIER kernel gave up a bounded wait: results since then are not to be
                                trusted; nothing was enqueued by this call (see dn_device_error_reset)  */
};

typedef struct dn_shape {
  int32_t B, L, Hk, Hv, K, V;
  int32_t chunk;               /* 64 or 128 (see dn_exec.chunk)                */
  int32_t g_heads, g_cols;     /* layout of g (see above)                      */
  int32_t b_heads, b_cols;
  int32_t w_heads, w_cols;
  int32_t qkv_dtype;           /* dtype of q,k,v,out,d_out,dq,dk,dv            */
  int32_t gate_dtype;          /* dtype of g,b,w,dg,db,dw                      */
  int32_t precision;           /* DN_PREC_*                                    */
  uint32_t flags;
  float scale;                 /* query scale (already resolved, gdn2.py:1978) */
} dn_shape;

/* Exec-head view of a shape (what the residual layouts are expressed in). */
typedef struct dn_exec {
  int32_t H, Vw, G, NC;        /* exec heads, value width, value heads per exec head, chunks */
  int32_t pre_dtype;           /* dtype of W,U,M,qe,ke: bf16 in bf16 precision else f32 (gdn2.py:1247) */
  int32_t chunk;               /* rows per tile the kernels use, the C of every layout below.  Equal to
                                  dn_shape.chunk except on the tensor-core path (bf16 precision, K = 128,
                                  Vw in {128,256}): there tiles are 128 rows, the M of a tcgen05.mma, and a
                                  request for 64 runs with pairs of requested chunks merged into one tile
                                  (the chunked form regroups the token recurrence exactly; only the points
                                  where the state is rounded to bf16 move).  NC = ceil(L / chunk).          */
} dn_exec;
int dn_exec_view(const dn_shape* s, dn_exec* out);

/*
 * Residuals written by the forward and read by the backward: the reference's residual tuple
 * (gdn2.py:1384-1388).  All in exec-head layout; C = dn_exec.chunk, NC = ceil(L / C).
 *
 * The five pre_dtype tiles are opaque to the caller: only the library's own entry points read
 * them.  Each (batch, head, chunk) tile holds rows x cols elements, row-major in general; for shapes
 * that take the tensor-core path (precision bf16 without DN_STATE_FP32_MM, K = 128, Vw in {128,256},
 * DN_FORCE_SIMT unset) a tile is stored as the tensor cores' operand image, [col / 8][row][8 elements], so that
 * every kernel copies it into shared memory as it lies.  The sizes are the same in both layouts.
 * On that path T holds a bf16 image in the first half of its slot, and the chunk-entry states are kept
 * as a bf16 operand image only (half the bytes; dn_residual_bytes accounts for it).  The dV / dH
 * buffers that dn_state_bwd hands to dn_prepass_bwd are opaque in the same way (bf16 images plus the
 * partial sums of the decay cotangent); a caller only sizes them (fp32 element counts) and passes
 * them on.
 */
typedef struct dn_residuals {
  void*  W;        /* (B,H,NC) tiles of C x K    pre_dtype */
  void*  U;        /* (B,H,NC) tiles of C x Vw   pre_dtype */
  void*  M;        /* (B,H,NC) tiles of C x C    pre_dtype */
  void*  qe;       /* (B,H,NC) tiles of C x K    pre_dtype */
  void*  ke;       /* (B,H,NC) tiles of C x K    pre_dtype */
  float* lam_end;  /* (B,H,NC,K)     */
  float* T;        /* (B,H,NC,C,C)   or NULL (inference); opaque */
  float* states;   /* (B,H,NC,K,Vw)  chunk-entry states (fp32; a bf16 image on the tensor-core path), or NULL (inference) */
} dn_residuals;

/* Bytes of one packed residual block, and a helper that carves the block into the struct. */
size_t dn_residual_bytes(const dn_shape* s);
int dn_residual_carve(const dn_shape* s, void* block, dn_residuals* out);

/* Scratch bytes needed by dn_chunk_fwd / dn_chunk_bwd (upper bound over their phases). */
size_t dn_scratch_bytes(const dn_shape* s, int for_backward, int recompute);

/* (B,L) raw ids -> canonical ids; first_is_new (B) may be NULL (gdn2.py:2081-2094). */
int dn_canonical_segments(const int32_t* raw, const int32_t* first_is_new, int32_t* out,
                          int32_t B, int32_t L, void* stream);

/* The same ids from cumulative sequence lengths cu_seqlens (n_cu int32 values on the device, the
 * first 0 and the last L, strictly increasing; applied to every batch row, gdn2.py:2037-2052). */
int dn_cu_seqlens_segments(const int32_t* cu_seqlens, int32_t n_cu, const int32_t* first_is_new, int32_t* out,
                           int32_t B, int32_t L, void* stream);

/*
 * Forward of the chunked recurrence.  seg may be NULL (one document).  init_state
 * (B,Hv,K,V) f32 is read when DN_HAS_INIT.  final_state (B,Hv,K,V) f32 may be NULL.
 * res == NULL means "keep nothing" (inference, or recompute_states): the prepass
 * outputs then live in scratch only.
 *
 * Streams: all work is ordered on `stream`.  For shapes whose B*H*NC work items leave the last
 * round of the one-CTA-per-SM kernels mostly empty, dn_chunk_fwd and dn_chunk_bwd cut the chunk
 * axis in two and run part of the inter-chunk chain on a library-owned side stream next to the
 * chunk-parallel kernel of the other part; the side stream forks from `stream` and joins back into
 * it through events before the call's last kernel, so the caller still sees one stream-ordered
 * operation (and may capture it in a graph).  The side stream and its two events are created on the
 * first such call per device; make that call outside stream capture.  DN_NO_OVERLAP=1 in the
 * environment turns the split off.
 */
int dn_chunk_fwd(const dn_shape* s,
                 const void* q, const void* k, const void* v,
                 const void* g, const void* b, const void* w,
                 const int32_t* seg, const float* init_state,
                 void* out, float* final_state,
                 const dn_residuals* res, void* scratch, size_t scratch_bytes, void* stream);

/*
 * Backward.  res == NULL means recompute_states=True: the prepass and the chunk states are
 * rebuilt in scratch first (gdn2.py:1545-1630).  d_final_state and d_init may be NULL.
 * dq,dk have q's shape; dv has v's; dg,db,dw have the shapes g,b,w were given in.
 */
int dn_chunk_bwd(const dn_shape* s,
                 const void* q, const void* k, const void* v,
                 const void* g, const void* b, const void* w,
                 const int32_t* seg, const float* init_state,
                 const dn_residuals* res,
                 const void* d_out, const float* d_final_state,
                 void* dq, void* dk, void* dv, void* dg, void* db, void* dw, float* d_init,
                 void* scratch, size_t scratch_bytes, void* stream);

/* ---- the single phases (same buffers as above) ------------------------------------------ */
int dn_prepass_fwd(const dn_shape* s, const void* q, const void* k, const void* v,
                   const void* g, const void* b, const void* w, const int32_t* seg,
                   const dn_residuals* res, void* scratch, size_t scratch_bytes, void* stream);

int dn_state_fwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                 const float* init_state, void* out, float* final_state, void* stream);

int dn_recompute_states(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                        const float* init_state, void* stream);

/*
 * Reverse chain.  Writes, in exec-head layout, dV (B,H,NC,C,Vw) f32 -- the cotangent of
 * U, the reference's dU -- and dH (B,H,NC,K,Vw) f32, the state cotangent each chunk
 * receives from its successor.  The remaining per-chunk cotangents of the reference's
 * state-backward kernel (dW, dM, dqe, dke, d lambda_end) are contractions over the value
 * width that do not depend on the chain; dn_prepass_bwd forms them chunk-parallel.
 */
int dn_state_bwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                 const void* d_out, const float* d_final_state,
                 float* dV, float* dH, float* d_init, void* stream);

int dn_prepass_bwd(const dn_shape* s, const void* q, const void* k, const void* v,
                   const void* g, const void* b, const void* w, const int32_t* seg,
                   const dn_residuals* res, const void* d_out, const float* dV, const float* dH,
                   void* dq, void* dk, void* dv, void* dg, void* db, void* dw,
                   void* scratch, size_t scratch_bytes, void* stream);

/* ---- sequence sharding --------------------------------------------------------------------
 * The reference has no sequence-parallel implementation, only the hooks for one (initial_state,
 * output_final_state and initial_state_segment_id, src/deltanet_tpu/gdn2.py:2081-2085; README
 * "when a packed sequence is split across calls or chips").  These two entry points are what a
 * sharded caller adds on top of the phases above.  The state pass of a shard is affine in the
 * incoming state, S_out = P S_in + Q per (batch, exec head), with Q the final state from S_in = 0.
 *
 * dn_sp_transition: P (B,H,K,K) f32 of a shard whose prepass residuals are `res` (W, ke, lam_end are
 *   read).  identity is a (B,H,K,K) f32 buffer holding the identity per head.
 * dn_sp_apply: S_out[b,hv] = P[b,hv/G] S_in[b,hv] + Q[b,hv] (Q may be NULL), or with P transposed
 *   (the adjoint, for the state cotangent).  States are (B, H*G, K, V) f32.  keep (B bytes, may be NULL):
 *   batch rows whose byte is 0 get S_out = 0 (the next shard starts a new document there).
 */
int dn_sp_transition(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                     const float* identity, float* P, void* stream);
/*
 * The cheaper schedule built on the same fact (what a shard computes after its first document boundary
 * does not depend on the incoming state at all):
 *
 * dn_sp_summary: ONE launch that runs the state pass from a zero state over the whole shard -- writing
 *   outputs (out may be NULL) and chunk-entry states (res->states may be NULL) as dn_state_fwd does, and
 *   Q (B,Hv,K,V) -- while K extra columns per (batch, exec head) start from the identity with U = 0 and
 *   end as P (B,H,K,K).  Everything it writes for chunks after the first boundary is final.  With
 *   DN_SP_SKIP_PROVISIONAL in the shape's flags (tensor-core path) it does not write the outputs of the
 *   chunks before that point, which the caller must then obtain from dn_sp_correct_fwd.
 * dn_sp_correct_fwd: the forward chain again from the true incoming state S_in (B,Hv,K,V), stopping at
 *   the first chunk whose results no longer depend on it; rewrites out and the chunk-entry states of the
 *   chunks it walks.  The shard's final state is P S_in + Q (dn_sp_apply); this call does not produce it.
 *   The shape must carry DN_HAS_INIT.
 * dn_sp_correct_bwd: the mirror image for the reverse chain: after dn_state_bwd with a NULL
 *   d_final_state (cotangent 0, which also gives d_init0), this walks back from the true d_final_state
 *   and stops where dH no longer depends on it, rewriting dV and dH of the chunks it walks.  The shard's
 *   d_init is P^T d_final_state + d_init0.
 */
int dn_sp_summary(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                  void* out, float* Q, float* P, void* stream);
int dn_sp_correct_fwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                      const float* S_in, void* out, void* stream);
int dn_sp_correct_bwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                      const void* d_out, const float* d_final_state, float* dV, float* dH, void* stream);
int dn_sp_apply(const float* P, const float* S_in, const float* Q, float* S_out, const uint8_t* keep, int32_t B,
                int32_t H, int32_t G, int32_t K, int32_t V, int32_t transpose, void* stream);

/*
 * Allocation-free forward prepass.  No counterpart in the reference.
 *
 * Same results as dn_prepass_fwd, for callers that cannot give the library a scratch buffer
 * because they cannot allocate device memory where they call it: a runtime whose call handlers
 * may not allocate and that was not asked for scratch when the call was built, a serving loop
 * with a frozen memory plan, a sandboxed plugin without access to the CUDA allocator.  The
 * scratch is a fixed array of dn_static_scratch_bytes() (32 MiB) inside the library image; every
 * GPU that loads the library holds it until the process exits.  The function calls no cudaMalloc,
 * cudaFree or other allocating routine.
 *
 *  - Shapes whose prepass needs more scratch than the array return DN_ERR_STATIC_SCRATCH_EXCEEDED
 *    (the tensor-core path, bf16 precision with chunk = K = 128, needs 9.3 MiB and always fits;
 *    the fp32 path fits for chunk = K = V = 64).
 *  - The first call on each device looks up the array's device address (with that device
 *    current).  Make that first call outside any stream capture.
 *  - All calls share the one array and it keeps the previous call's contents.  Nothing in it has
 *    to start at zero (every word is written before it is read within a call), but two calls that
 *    overlap on the GPU -- different streams, or different host threads -- race on it: serialise them.
 */
size_t dn_static_scratch_bytes(void);
int dn_prepass_fwd_static(const dn_shape* s, const void* q, const void* k, const void* v,
                          const void* g, const void* b, const void* w, const int32_t* seg,
                          const dn_residuals* res, void* stream);

/* ---- the steps either side of the recurrence in a Gated DeltaNet layer -------------------------------
 * The reference shows them in its layer example (examples/qwen3_5_layer_parity.py:144-159): the projected
 * activations go through a short depthwise causal convolution and SiLU and are split into q, k, v; the
 * gate pre-activations become g = -exp(A_log) * softplus(a + dt_bias) and beta = sigmoid(b); the
 * recurrence's output is normalised per value head and gated, y = weight * rmsnorm(o) * silu(z).  All are
 * bound by HBM bytes: each kernel reads its inputs once and writes its outputs once.
 *
 * producer: mixed (B,L,D), D = 2*Hk*K + Hv*V, channel order q | k | v; conv_w (D,W) fp32 with tap W-1 on the
 *   current token, W in {2,3,4}; conv_b (D) fp32 or NULL; seg (B,L) canonical ids (>= 0) or NULL -- taps that
 *   would reach into another document (or before token 0) read zero.  q,k (B,L,Hk,K), v (B,L,Hv,V), in `dtype`.
 *   backward: dq,dk,dv -> d_mixed (B,L,D), d_conv_w (D,W), d_conv_b (D, may be NULL); scratch of
 *   dn_gdn_producer_scratch_bytes holds per-tile partial sums (added in a fixed order).
 * gates: a, b (B,L,Hv) in `dtype`; A_log, dt_bias (Hv) fp32; g, beta (B,L,Hv) fp32 -- the per-head scalar
 *   gates chunk_gdn takes.  backward: dg, dbeta fp32 -> da, db in `dtype`, dA_log, d_dt_bias (Hv) fp32.
 * gated rmsnorm: o, z, y (rows, V) in `dtype`, rows = B*L*Hv, V in {64,128}; weight (V) fp32; the normalised
 *   value is rounded to `dtype` before the weight is applied.  backward: dy -> d_o, d_z, d_weight (V) fp32.
 */
size_t dn_gdn_producer_scratch_bytes(int32_t B, int32_t L, int32_t D, int32_t W);
int dn_gdn_producer_fwd(const void* mixed, const float* conv_w, const float* conv_b, const int32_t* seg,
                        int32_t B, int32_t L, int32_t Hk, int32_t Hv, int32_t K, int32_t V, int32_t W, int32_t dtype,
                        void* q, void* k, void* v, void* stream);
int dn_gdn_producer_bwd(const void* mixed, const float* conv_w, const float* conv_b, const int32_t* seg,
                        int32_t B, int32_t L, int32_t Hk, int32_t Hv, int32_t K, int32_t V, int32_t W, int32_t dtype,
                        const void* dq, const void* dk, const void* dv, void* d_mixed, float* d_conv_w, float* d_conv_b,
                        void* scratch, size_t scratch_bytes, void* stream);
int dn_gdn_gates_fwd(const void* a, const void* b, const float* A_log, const float* dt_bias, int32_t B, int32_t L,
                     int32_t Hv, int32_t dtype, float* g, float* beta, void* stream);
int dn_gdn_gates_bwd(const void* a, const void* b, const float* A_log, const float* dt_bias, const float* dg,
                     const float* dbeta, int32_t B, int32_t L, int32_t Hv, int32_t dtype, void* da, void* db,
                     float* dA_log, float* d_dt_bias, void* stream);
size_t dn_gated_rmsnorm_scratch_bytes(int64_t rows, int32_t V);
int dn_gated_rmsnorm_fwd(const void* o, const void* z, const float* weight, int64_t rows, int32_t V, int32_t dtype,
                         float eps, void* y, void* stream);
int dn_gated_rmsnorm_bwd(const void* o, const void* z, const float* weight, int64_t rows, int32_t V, int32_t dtype,
                         float eps, const void* dy, void* d_o, void* d_z, float* d_weight, void* scratch,
                         size_t scratch_bytes, void* stream);

/* ---- decode ------------------------------------------------------------------------------ */
typedef struct dn_decode_shape {
  int32_t B, Hk, Hv, K, V;
  int32_t g_heads, g_cols, b_heads, b_cols, w_heads, w_cols;
  int32_t qkv_dtype, gate_dtype;
  int32_t state_in_dtype, state_out_dtype;
  uint32_t flags;              /* DN_QK_L2NORM, DN_STABILITY_GUARD, DN_RESET_PER_HEAD */
  float scale, stability_tau;
} dn_decode_shape;

/*
 * One token for B sequences.  state_in and state_out may be the same buffer when their
 * dtypes match (in-place update).  reset, (B) uint8 or (B,Hv) with DN_RESET_PER_HEAD, may be NULL
 * (the reference broadcasts reset over (B,Hv,K,V), gdn2.py:2404-2410).  out is (B,Hv,V) in qkv_dtype.
 */
int dn_decode_step(const dn_decode_shape* s,
                   const void* q, const void* k, const void* v,
                   const void* g, const void* b, const void* w,
                   const void* state_in, const uint8_t* reset,
                   void* out, void* state_out, void* stream);

/*
 * Diagnostic (no reference counterpart): D[128 x N] = A B^T in bf16 with fp32 accumulation through
 * the library's tcgen05 building blocks, one CTA.  a_mn / b_mn = 0: the operand is given as
 * (rows, Kc) with the contraction index contiguous; = 1: as (Kc, rows) with the row index
 * contiguous.  N in {32,64,128,256}, Kc a multiple of 16 up to 256.  *err is set to 1 if a bounded
 * wait inside the kernel gave up.
 */
int dn_selftest_umma(int32_t a_mn, int32_t b_mn, int32_t N, int32_t Kc, const void* A, const void* B,
                     float* D, int32_t* err, void* stream);

/*
 * The library's error word (no reference counterpart).  Every wait inside a kernel (on a tensor-core
 * or copy barrier) is bounded; a kernel whose wait gives up finishes without the affected work and
 * stores 1 into the word.  The word sits in pinned host memory the device writes directly, so the
 * host sees it without synchronising: once it is set, every enqueueing entry point returns
 * DN_ERR_DEVICE_WAIT instead of enqueueing (results produced since the failed wait are not to be
 * trusted) until dn_device_error_reset() clears it.  dn_device_error() synchronises with the current
 * device first and then returns the word (0 or 1): the check for "did everything I enqueued so far
 * run to completion normally".
 */
int dn_device_error(void);
void dn_device_error_reset(void);

/*
 * stability_guard's cap of a recurrent state (gdn2.py:2180-2188, 2224-2238): each of the n_states
 * consecutive fp32 (K,V) matrices is scaled in place by min(1, tau / sqrt(sum S^2 + 1e-6)).
 */
int dn_cap_state(float* state, int64_t n_states, int32_t K, int32_t V, float tau, void* stream);

/*
 * Diagnostic (no reference counterpart): the number of kernels dn_chunk_fwd (backward = 0) or
 * dn_chunk_bwd (backward = 1; recompute = 1 adds the rebuilt prepass and states) enqueues for this
 * shape on the current device.  0 for an invalid shape.  A pure query: creates no stream or event.
 */
int dn_launch_count(const dn_shape* s, int backward, int recompute);
/* Diagnostic (no reference counterpart): kernels this library has launched in this process so far
 * (every successful launch of one of its own kernels counts one), for callers that report launch counts. */
int64_t dn_launches_total(void);

const char* dn_status_string(int status);
int dn_version(void);

#ifdef __cplusplus
}
#endif
#endif /* DELTANET_B200_H_ */
