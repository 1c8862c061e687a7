// Argument blocks and host launchers of the kernels behind the C ABI.
#pragma once
#include "dn_common.cuh"

namespace dn {

struct PrepassFwdArgs {
  Geo g;
  const void *q, *k, *v, *gg, *b, *w;
  const int32_t* seg;
  dn_residuals res;
  float* scratch;
  size_t scratch_per_cta;
  int items;
  int smem_tile_off;
  int c_begin, c_end;          // chunk range [c_begin, c_end) of every (batch, head); tensor-core path only
};

struct StateArgs {
  Geo g;
  dn_residuals res;
  const int32_t* seg;
  const float* init_state;   // (B,Hv,K,V) or null
  void* out;                 // (B,L,Hv,V) qkv dtype, or null (states only)
  float* final_state;        // (B,Hv,K,V) or null
  float* states;             // (B,H,NC,K,Vw) chunk-entry states or null
  // backward chain
  const void* d_out;
  const float* d_final;
  float* dV;                 // (B,H,NC,C,Vw)
  float* dH;                 // (B,H,NC,K,Vw)
  float* d_init;             // (B,Hv,K,V) or null
  // Chunk range [c_begin, c_end) of the chain (tensor-core path only; 0, NC = the whole chain).  A
  // forward pass that starts at c_begin > 0 reads its state from `carry`, one that stops before NC
  // leaves it there; the backward pass uses it the other way round.  (B,H,K,Vw) fp32.
  int c_begin, c_end;
  float* carry;
  int* err;                  // error word (bounded waits report here); set by the launchers
  // Sequence-sharded use.  P_out (B,H,K,K): the forward launch carries K extra "value" columns per
  // (batch, head) that start from the identity with U = 0 and end as the shard's transition matrix
  // (grid.x grows by K / VS slices; those slices write neither outputs nor chunk states).
  // until_independent: the chain stops at the first chunk whose results no longer depend on the
  // state it was started from (a document boundary cuts the dependence); outputs, chunk states, dV
  // and dH of the chunks before that point are (re)written, nothing else is, and neither the final
  // state nor d_init is produced.
  // skip_provisional (forward, tensor-core path): outputs of the chunks that still depend on the state the
  // launch started from are not computed; the caller runs an until_independent pass over them afterwards.
  float* P_out;
  bool until_independent;
  bool skip_provisional;
};

struct PrepassBwdArgs {
  Geo g;
  const void *q, *k, *v, *gg, *b, *w;
  const int32_t* seg;
  dn_residuals res;
  const void* d_out;
  const float *dV, *dH;
  // gradient sinks at exec-head granularity: either the user's buffer (typed) or f32 staging
  void *dq, *dk, *dv, *dg, *db, *dw;
  int dq_dt, dg_dt, db_dt, dw_dt;   // dtype actually written (f32 when staged)
  float* scratch;
  size_t scratch_per_cta;
  int items;
  int* err;                        // device error word (bounded waits report here)
  int c_begin, c_end;              // chunk range [c_begin, c_end) of every (batch, head); tensor-core path only
  bool bulk_v;                     // v, w, dv, dw move by bulk copies (set by the launcher)
};

// Called right after every kernel launch of the library: DN_OK or DN_ERR_CUDA_LAUNCH from
// cudaGetLastError(), and one more in the library's count of kernels it has launched.
int launch_status();
long long launches_total();

size_t prepass_fwd_scratch_per_cta(const Geo& g);
size_t prepass_bwd_scratch_per_cta(const Geo& g);

int launch_prepass_fwd(const Geo& g, const void* q, const void* k, const void* v, const void* gg,
                       const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                       float* scratch, size_t scratch_floats, cudaStream_t st);
bool prepass_fwd_tc_eligible(const Geo& g);
size_t prepass_fwd_tc_scratch_per_cta();
int launch_prepass_fwd_tc(const Geo& g, const void* q, const void* k, const void* v, const void* gg,
                          const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                          float* scratch, size_t scratch_floats, cudaStream_t st, int c_begin = 0, int c_end = -1);
int launch_state_fwd(const StateArgs& a, cudaStream_t st);
// tensor-core (tcgen05) variants of the chain kernels, used when state_tc_eligible()
bool state_tc_eligible(const Geo& g);
int launch_state_fwd_tc(const StateArgs& a, cudaStream_t st);
int launch_state_bwd_tc(const StateArgs& a, cudaStream_t st);
// The library's error word (dn_misc.cu): device address for the kernels; read without / with a
// device synchronisation; clear.
int* device_error_ptr();
int peek_device_error();
int read_device_error();
void reset_device_error();
int launch_state_bwd(const StateArgs& a, cudaStream_t st);
int launch_prepass_bwd(PrepassBwdArgs& a, size_t scratch_floats, cudaStream_t st);
int launch_prepass_bwd_tc(PrepassBwdArgs& a, size_t scratch_floats, cudaStream_t st);
bool prepass_bwd_tc_eligible(const Geo& g);
size_t prepass_bwd_tc_scratch_per_cta(const Geo& g);
int launch_canonical_segments(const int32_t* raw, const int32_t* first_is_new, int32_t* out,
                              int B, int L, cudaStream_t st);
int launch_cu_seqlens_segments(const int32_t* cu, int n_cu, const int32_t* first_is_new, int32_t* out,
                               int B, int L, cudaStream_t st);
// sums `groups` consecutive heads: in (rows, heads_out*groups, cols) f32 -> out (rows, heads_out, cols)
int launch_group_sum(const float* in, void* out, int out_dt, size_t rows, int heads_out, int groups,
                     int cols, cudaStream_t st);
// S_out[b, h*G+g] = op(P[b,h]) S_in[b, h*G+g] (+ Q); op = transpose when asked.  P (B,H,K,K), states (B,H*G,K,V).
int launch_sp_apply(const float* P, const float* S_in, const float* Q, float* S_out, const uint8_t* keep, int B, int H,
                    int G, int K, int V, int transpose, cudaStream_t st);
// Frobenius cap of n_states fp32 (K,V) states in place: S <- S * min(1, tau / sqrt(|S|^2 + 1e-6))
int launch_cap_state(float* state, int64_t n_states, int KV, float tau, cudaStream_t st);
int launch_decode(const dn_decode_shape& s, const void* q, const void* k, const void* v,
                  const void* g, const void* b, const void* w, const void* state_in,
                  const uint8_t* reset, void* out, void* state_out, cudaStream_t st);

}  // namespace dn
