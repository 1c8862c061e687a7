// extern "C" surface declared in include/deltanet_b200.h: argument checks, buffer carving,
// and the order in which the kernels are enqueued.  Nothing here allocates device memory or
// synchronises.
#include <cstdlib>
#include <mutex>

#include "dn_kernels.cuh"

using namespace dn;

static inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// ---- overlap of the chunk-parallel kernels with the chains ------------------------------------
// The chunk-parallel kernels run one CTA per SM over B*H*NC work items; when that count leaves the
// last round of CTAs mostly empty (192 items on 148 SMs), dn_chunk_fwd / dn_chunk_bwd cut the chunk
// axis in two and run the chain of one part on a side stream next to the chunk-parallel kernel of
// the other part.  The side stream forks from and joins back into the caller's stream through
// events, so the caller still sees one stream-ordered operation.  The stream and its events are
// created on the first such call per device (host objects; do that call outside stream capture).
// DN_NO_OVERLAP=1 turns the split off.
namespace {
struct Overlap {
  cudaStream_t side = nullptr;
  cudaEvent_t ev[2] = {nullptr, nullptr};
  bool tried = false, ok = false;
  // Held while one call enqueues its fork/join: a record and the wait that refers to it must not be
  // separated by another host thread's record of the same event.
  std::mutex enqueue;
};
bool overlap_disabled() {
  static const bool off = [] { const char* e = std::getenv("DN_NO_OVERLAP"); return e && e[0] == '1'; }();
  return off;
}
Overlap* overlap_for_device() {
  static Overlap table[64];
  static std::mutex mu;
  if (overlap_disabled()) return nullptr;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  Overlap& o = table[dev];
  if (!o.tried) {
    o.tried = true;
    o.ok = cudaStreamCreateWithFlags(&o.side, cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&o.ev[0], cudaEventDisableTiming) == cudaSuccess &&
           cudaEventCreateWithFlags(&o.ev[1], cudaEventDisableTiming) == cudaSuccess;
    if (!o.ok) cudaGetLastError();
  }
  return o.ok ? &o : nullptr;
}
// First chunk of the second part, or 0 for "do not split": the first part [0, cut) holds the whole
// rounds of CTAs, the second part [cut, NC) the last, partly filled round.
int overlap_cut(const Geo& g) {
  if (!g.img || !state_tc_eligible(g) || (g.flags & DN_STATE_FP32_MM)) return 0;
  const int per_chunk = g.B * g.H, n = per_chunk * g.NC, sms = sm_count();
  if (g.NC < 4 || n <= sms || n > 4 * sms) return 0;
  const int rounds = (n + sms - 1) / sms, tail = n - (rounds - 1) * sms;
  if (tail * 4 > sms * 3) return 0;                       // the last round is well filled already
  const int cut = ((rounds - 1) * sms) / per_chunk;
  return (cut >= 1 && cut < g.NC) ? cut : 0;
}
size_t carry_bytes(const Geo& g) { return align_up((size_t)g.B * g.H * g.K * g.Vw * sizeof(float)); }
}  // namespace

extern "C" {

int dn_version(void) { return 1; }

int dn_device_error(void) { return read_device_error(); }
void dn_device_error_reset(void) { reset_device_error(); }
int64_t dn_launches_total(void) { return launches_total(); }

const char* dn_status_string(int st) {
  switch (st) {
    case DN_OK: return "ok";
    case DN_ERR_BAD_SHAPE: return "unsupported shape (K,V in {64,128}; chunk in {64,128}; gate heads in {1,Hk,Hv})";
    case DN_ERR_BAD_DTYPE: return "unsupported dtype or precision";
    case DN_ERR_NULL_POINTER: return "a required buffer is NULL";
    case DN_ERR_SCRATCH_TOO_SMALL: return "scratch buffer too small (see dn_scratch_bytes)";
    case DN_ERR_CUDA_LAUNCH: return "a CUDA kernel launch failed";
    case DN_ERR_UNSUPPORTED: return "unsupported combination of options";
    case DN_ERR_DEVICE_WAIT: return "an earlier kernel gave up a bounded wait (see dn_device_error / dn_device_error_reset)";
    case DN_ERR_STATIC_SCRATCH_EXCEEDED: return "this shape needs more scratch than the built-in static array (see dn_static_scratch_bytes)";
    default: return "unknown status";
  }
}

int dn_exec_view(const dn_shape* s, dn_exec* out) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (!out) return DN_ERR_NULL_POINTER;
  out->H = g.H; out->Vw = g.Vw; out->G = g.G; out->NC = g.NC; out->pre_dtype = g.pre_dt; out->chunk = g.C;
  return DN_OK;
}

// Residual block layout: W | U | M | qe | ke | lam_end | T | states, each 256-byte aligned.
static void residual_sizes(const Geo& g, size_t sz[8]) {
  const size_t n = (size_t)g.B * g.H * g.NC, ps = dt_size(g.pre_dt);
  const bool keep = !(g.flags & DN_INFERENCE);
  sz[0] = n * g.C * g.K * ps;
  sz[1] = n * g.C * g.Vw * ps;
  sz[2] = n * g.C * g.C * ps;
  sz[3] = sz[0];
  sz[4] = sz[0];
  sz[5] = n * g.K * sizeof(float);
  sz[6] = keep ? n * g.C * g.C * sizeof(float) : 0;
  sz[7] = keep ? n * g.K * g.Vw * (g.img ? 2 : sizeof(float)) : 0;            // image path: a bf16 operand image (states_img)
}

size_t dn_residual_bytes(const dn_shape* s) {
  Geo g;
  if (make_geo(s, &g)) return 0;
  size_t sz[8], tot = 0;
  residual_sizes(g, sz);
  for (int i = 0; i < 8; ++i) tot += align_up(sz[i]);
  return tot;
}

int dn_residual_carve(const dn_shape* s, void* block, dn_residuals* out) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (!block || !out) return DN_ERR_NULL_POINTER;
  size_t sz[8];
  residual_sizes(g, sz);
  char* p = reinterpret_cast<char*>(block);
  void* ptr[8];
  for (int i = 0; i < 8; ++i) { ptr[i] = sz[i] ? p : nullptr; p += align_up(sz[i]); }
  out->W = ptr[0]; out->U = ptr[1]; out->M = ptr[2]; out->qe = ptr[3]; out->ke = ptr[4];
  out->lam_end = reinterpret_cast<float*>(ptr[5]);
  out->T = reinterpret_cast<float*>(ptr[6]);
  out->states = reinterpret_cast<float*>(ptr[7]);
  return DN_OK;
}

// ---- scratch accounting -------------------------------------------------------------------
static size_t fwd_kernel_scratch(const Geo& g) {
  size_t items = (size_t)g.B * g.H * g.NC;
  size_t ctas = items < (size_t)sm_count() ? items : (size_t)sm_count();
  return align_up(ctas * prepass_fwd_scratch_per_cta(g) * sizeof(float));
}
static size_t bwd_kernel_scratch(const Geo& g) {
  size_t items = (size_t)g.B * g.H * g.NC;
  size_t ctas = items < (size_t)2 * sm_count() ? items : (size_t)2 * sm_count();
  return align_up(ctas * prepass_bwd_scratch_per_cta(g) * sizeof(float));
}
static size_t staging_bytes(const Geo& g) {
  // f32 staging of gradients that must be summed over heads afterwards
  size_t rows = (size_t)g.B * g.L, tot = 0;
  if (g.qk_div > 1) tot += 2 * align_up(rows * g.H * g.K * sizeof(float));
  if (g.gH != g.H) tot += align_up(rows * g.H * g.gC * sizeof(float));
  if (g.bH != g.H) tot += align_up(rows * g.H * g.bC * sizeof(float));
  if (g.wH != g.Hv) tot += align_up(rows * g.Hv * g.wC * sizeof(float));
  return tot;
}
static size_t full_residual_bytes(const dn_shape* s) {
  dn_shape t = *s;
  t.flags &= ~DN_INFERENCE;
  return dn_residual_bytes(&t);
}

size_t dn_scratch_bytes(const dn_shape* s, int for_backward, int recompute) {
  Geo g;
  if (make_geo(s, &g)) return 0;
  const size_t n = (size_t)g.B * g.H * g.NC;
  if (!for_backward) {
    // forward without residuals keeps the prepass outputs in scratch
    return fwd_kernel_scratch(g) + align_up(dn_residual_bytes(s)) + carry_bytes(g);
  }
  size_t tot = bwd_kernel_scratch(g) > fwd_kernel_scratch(g) ? bwd_kernel_scratch(g) : fwd_kernel_scratch(g);
  tot += align_up(n * g.C * g.Vw * sizeof(float));   // dV
  tot += align_up(n * g.K * g.Vw * sizeof(float));   // dH
  tot += staging_bytes(g);
  tot += carry_bytes(g);
  if (recompute) tot += align_up(full_residual_bytes(s));
  return tot;
}

int dn_canonical_segments(const int32_t* raw, const int32_t* first_is_new, int32_t* out,
                          int32_t B, int32_t L, void* stream) {
  if (!raw || !out) return DN_ERR_NULL_POINTER;
  if (B < 1 || L < 1) return DN_ERR_BAD_SHAPE;
  return launch_canonical_segments(raw, first_is_new, out, B, L, (cudaStream_t)stream);
}

int dn_cu_seqlens_segments(const int32_t* cu_seqlens, int32_t n_cu, const int32_t* first_is_new, int32_t* out,
                           int32_t B, int32_t L, void* stream) {
  if (!cu_seqlens || !out) return DN_ERR_NULL_POINTER;
  if (B < 1 || L < 1 || n_cu < 2) return DN_ERR_BAD_SHAPE;
  return launch_cu_seqlens_segments(cu_seqlens, n_cu, first_is_new, out, B, L, (cudaStream_t)stream);
}

// ---- phases -------------------------------------------------------------------------------
int dn_prepass_fwd(const dn_shape* s, const void* q, const void* k, const void* v,
                   const void* g_, const void* b, const void* w, const int32_t* seg,
                   const dn_residuals* res, void* scratch, size_t scratch_bytes, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!q || !k || !v || !g_ || !b || !w || !res || !scratch) return DN_ERR_NULL_POINTER;
  if (!res->W || !res->U || !res->M || !res->qe || !res->ke || !res->lam_end) return DN_ERR_NULL_POINTER;
  return launch_prepass_fwd(g, q, k, v, g_, b, w, seg, *res, reinterpret_cast<float*>(scratch),
                            scratch_bytes / sizeof(float), (cudaStream_t)stream);
}

int dn_state_fwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                 const float* init_state, void* out, float* final_state, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || (!out && !final_state && !res->states)) return DN_ERR_NULL_POINTER;
  if ((g.flags & DN_HAS_INIT) && !init_state) return DN_ERR_NULL_POINTER;
  StateArgs a{};
  a.g = g; a.res = *res; a.seg = seg; a.init_state = (g.flags & DN_HAS_INIT) ? init_state : nullptr;
  a.out = out; a.final_state = final_state; a.states = res->states;
  return launch_state_fwd(a, (cudaStream_t)stream);
}

int dn_recompute_states(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                        const float* init_state, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || !res->states) return DN_ERR_NULL_POINTER;
  if ((g.flags & DN_HAS_INIT) && !init_state) return DN_ERR_NULL_POINTER;
  StateArgs a{};
  a.g = g; a.res = *res; a.seg = seg; a.init_state = (g.flags & DN_HAS_INIT) ? init_state : nullptr;
  a.states = res->states;
  return launch_state_fwd(a, (cudaStream_t)stream);
}

int dn_state_bwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                 const void* d_out, const float* d_final_state,
                 float* dV, float* dH, float* d_init, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || !d_out || !dV || !dH) return DN_ERR_NULL_POINTER;
  if (g.img && !res->states) return DN_ERR_NULL_POINTER;      // dLambda_end is reduced in the reverse chain on this path
  StateArgs a{};
  a.g = g; a.res = *res; a.seg = seg; a.d_out = d_out; a.d_final = d_final_state;
  a.dV = dV; a.dH = dH; a.d_init = (g.flags & DN_HAS_INIT) ? d_init : nullptr;
  return launch_state_bwd(a, (cudaStream_t)stream);
}

// The chunk-parallel backward in three steps: carve the gradient staging out of `p` and fill the
// argument block; launch (a chunk range, on a stream); the head sums.
namespace {
struct BwdPlan {
  PrepassBwdArgs a{};
  float *sq = nullptr, *sk = nullptr, *sg = nullptr, *sb = nullptr, *sw = nullptr;
  size_t scratch_floats = 0;
  void *dq, *dk, *dg, *db, *dw;
};
int plan_prepass_bwd(const Geo& g, const void* q, const void* k, const void* v, const void* g_,
                     const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                     const void* d_out, const float* dV, const float* dH,
                     void* dq, void* dk, void* dv, void* dg, void* db, void* dw,
                     char* p, size_t bytes, BwdPlan& pl) {
  const size_t rows = (size_t)g.B * g.L;
  char* end = p + bytes;
  PrepassBwdArgs& a = pl.a;
  a.g = g; a.q = q; a.k = k; a.v = v; a.gg = g_; a.b = b; a.w = w; a.seg = seg; a.res = res;
  a.d_out = d_out; a.dV = dV; a.dH = dH;
  a.dq = dq; a.dk = dk; a.dv = dv; a.dg = dg; a.db = db; a.dw = dw;
  pl.dq = dq; pl.dk = dk; pl.dg = dg; pl.db = db; pl.dw = dw;
  a.dq_dt = g.qkv_dt; a.dg_dt = a.db_dt = a.dw_dt = g.gate_dt;
  auto take = [&](size_t nfl) { float* r = reinterpret_cast<float*>(p); p += align_up(nfl * sizeof(float)); return r; };
  if (g.qk_div > 1) { pl.sq = take(rows * g.H * g.K); pl.sk = take(rows * g.H * g.K); a.dq = pl.sq; a.dk = pl.sk; a.dq_dt = DN_F32; }
  if (g.gH != g.H) { pl.sg = take(rows * g.H * g.gC); a.dg = pl.sg; a.dg_dt = DN_F32; }
  if (g.bH != g.H) { pl.sb = take(rows * g.H * g.bC); a.db = pl.sb; a.db_dt = DN_F32; }
  if (g.wH != g.Hv) { pl.sw = take(rows * g.Hv * g.wC); a.dw = pl.sw; a.dw_dt = DN_F32; }
  if (p > end) return DN_ERR_SCRATCH_TOO_SMALL;
  a.scratch = reinterpret_cast<float*>(p);
  pl.scratch_floats = (size_t)(end - p) / sizeof(float);
  return DN_OK;
}
int launch_plan(BwdPlan& pl, int c_begin, int c_end, cudaStream_t st) {
  pl.a.c_begin = c_begin; pl.a.c_end = c_end;
  return launch_prepass_bwd(pl.a, pl.scratch_floats, st);
}
int finish_plan(const Geo& g, const BwdPlan& pl, cudaStream_t st) {
  const size_t rows = (size_t)g.B * g.L;
  int rc;
  if (pl.sq) {
    if ((rc = launch_group_sum(pl.sq, pl.dq, g.qkv_dt, rows, g.Hk, g.qk_div, g.K, st))) return rc;
    if ((rc = launch_group_sum(pl.sk, pl.dk, g.qkv_dt, rows, g.Hk, g.qk_div, g.K, st))) return rc;
  }
  if (pl.sg && (rc = launch_group_sum(pl.sg, pl.dg, g.gate_dt, rows, g.gH, g.H / g.gH, g.gC, st))) return rc;
  if (pl.sb && (rc = launch_group_sum(pl.sb, pl.db, g.gate_dt, rows, g.bH, g.H / g.bH, g.bC, st))) return rc;
  if (pl.sw && (rc = launch_group_sum(pl.sw, pl.dw, g.gate_dt, rows, g.wH, g.Hv / g.wH, g.wC, st))) return rc;
  return DN_OK;
}
}  // namespace

static int run_prepass_bwd(const Geo& g, const void* q, const void* k, const void* v, const void* g_,
                           const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                           const void* d_out, const float* dV, const float* dH,
                           void* dq, void* dk, void* dv, void* dg, void* db, void* dw,
                           char* p, size_t bytes, cudaStream_t st) {
  BwdPlan pl;
  int rc = plan_prepass_bwd(g, q, k, v, g_, b, w, seg, res, d_out, dV, dH, dq, dk, dv, dg, db, dw, p, bytes, pl);
  if (rc) return rc;
  if ((rc = launch_plan(pl, 0, 0, st))) return rc;
  return finish_plan(g, pl, st);
}

int dn_prepass_bwd(const dn_shape* s, const void* q, const void* k, const void* v,
                   const void* g_, const void* b, const void* w, const int32_t* seg,
                   const dn_residuals* res, const void* d_out, const float* dV, const float* dH,
                   void* dq, void* dk, void* dv, void* dg, void* db, void* dw,
                   void* scratch, size_t scratch_bytes, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!q || !k || !v || !g_ || !b || !w || !res || !d_out || !dV || !dH || !scratch) return DN_ERR_NULL_POINTER;
  if (!dq || !dk || !dv || !dg || !db || !dw) return DN_ERR_NULL_POINTER;
  if (!res->W || !res->U || !res->T || !res->states || !res->lam_end) return DN_ERR_NULL_POINTER;
  return run_prepass_bwd(g, q, k, v, g_, b, w, seg, *res, d_out, dV, dH, dq, dk, dv, dg, db, dw,
                         reinterpret_cast<char*>(scratch), scratch_bytes, (cudaStream_t)stream);
}

// ---- the operator boundary ------------------------------------------------------------------
int dn_chunk_fwd(const dn_shape* s, const void* q, const void* k, const void* v,
                 const void* g_, const void* b, const void* w, const int32_t* seg,
                 const float* init_state, void* out, float* final_state,
                 const dn_residuals* res, void* scratch, size_t scratch_bytes, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!q || !k || !v || !g_ || !b || !w || !out || !scratch) return DN_ERR_NULL_POINTER;
  if ((g.flags & DN_HAS_INIT) && !init_state) return DN_ERR_NULL_POINTER;
  char* p = reinterpret_cast<char*>(scratch);
  char* end = p + scratch_bytes;
  dn_residuals local;
  if (!res) {
    dn_shape t = *s;
    t.flags |= DN_INFERENCE;                      // nothing is kept: no T, no chunk states
    size_t need = align_up(dn_residual_bytes(&t));
    if (p + need > end) return DN_ERR_SCRATCH_TOO_SMALL;
    if ((rc = dn_residual_carve(&t, p, &local))) return rc;
    p += need;
    res = &local;
  }
  const int cut = overlap_cut(g);
  Overlap* ov = cut ? overlap_for_device() : nullptr;
  if (ov && p + carry_bytes(g) <= end) {
    // prepass of chunks [0, cut); then the chain over those chunks (side stream) next to the
    // prepass of chunks [cut, NC); then the rest of the chain
    if (!res->W || !res->U || !res->M || !res->qe || !res->ke || !res->lam_end) return DN_ERR_NULL_POINTER;
    std::lock_guard<std::mutex> lock(ov->enqueue);
    cudaStream_t st = (cudaStream_t)stream;
    float* carry = reinterpret_cast<float*>(p);
    p += carry_bytes(g);
    float* sc = reinterpret_cast<float*>(p);
    const size_t scf = (size_t)(end - p) / sizeof(float);
    StateArgs a{};
    a.g = g; a.res = *res; a.seg = seg; a.init_state = (g.flags & DN_HAS_INIT) ? init_state : nullptr;
    a.out = out; a.final_state = final_state; a.states = res->states; a.carry = carry;
    if ((rc = launch_prepass_fwd_tc(g, q, k, v, g_, b, w, seg, *res, sc, scf, st, 0, cut))) return rc;
    if (cudaEventRecord(ov->ev[0], st) != cudaSuccess || cudaStreamWaitEvent(ov->side, ov->ev[0], 0) != cudaSuccess)
      return DN_ERR_CUDA_LAUNCH;
    // forked: whatever fails from here on, the side stream is joined back before returning
    a.c_begin = 0; a.c_end = cut;
    const int rc_side = launch_state_fwd_tc(a, ov->side);
    const cudaError_t e1 = cudaEventRecord(ov->ev[1], ov->side);
    const int rc_main = launch_prepass_fwd_tc(g, q, k, v, g_, b, w, seg, *res, sc, scf, st, cut, g.NC);
    const cudaError_t e2 = cudaStreamWaitEvent(st, ov->ev[1], 0);
    if (rc_side) return rc_side;
    if (rc_main) return rc_main;
    if (e1 != cudaSuccess || e2 != cudaSuccess) return DN_ERR_CUDA_LAUNCH;
    a.c_begin = cut; a.c_end = g.NC;
    return launch_state_fwd_tc(a, st);
  }
  if ((rc = dn_prepass_fwd(s, q, k, v, g_, b, w, seg, res, p, (size_t)(end - p), stream))) return rc;
  return dn_state_fwd(s, res, seg, init_state, out, final_state, stream);
}

int dn_chunk_bwd(const dn_shape* s, const void* q, const void* k, const void* v,
                 const void* g_, const void* b, const void* w, const int32_t* seg,
                 const float* init_state, const dn_residuals* res,
                 const void* d_out, const float* d_final_state,
                 void* dq, void* dk, void* dv, void* dg, void* db, void* dw, float* d_init,
                 void* scratch, size_t scratch_bytes, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!q || !k || !v || !g_ || !b || !w || !d_out || !scratch) return DN_ERR_NULL_POINTER;
  if (!dq || !dk || !dv || !dg || !db || !dw) return DN_ERR_NULL_POINTER;
  if (g.flags & DN_INFERENCE) return DN_ERR_UNSUPPORTED;
  cudaStream_t st = (cudaStream_t)stream;
  char* p = reinterpret_cast<char*>(scratch);
  char* end = p + scratch_bytes;
  const size_t n = (size_t)g.B * g.H * g.NC;
  auto take = [&](size_t bytes) { char* r = p; p += align_up(bytes); return r; };
  float* dV = reinterpret_cast<float*>(take(n * g.C * g.Vw * sizeof(float)));
  float* dH = reinterpret_cast<float*>(take(n * g.K * g.Vw * sizeof(float)));
  if (p > end) return DN_ERR_SCRATCH_TOO_SMALL;
  dn_residuals local;
  if (!res) {
    // recompute_states: rebuild the prepass outputs (with T) and the chunk-entry states
    size_t need = align_up(full_residual_bytes(s));
    if (p + need > end) return DN_ERR_SCRATCH_TOO_SMALL;
    if ((rc = dn_residual_carve(s, p, &local))) return rc;
    p += need;
    if ((rc = dn_prepass_fwd(s, q, k, v, g_, b, w, seg, &local, p, (size_t)(end - p), stream))) return rc;
    if ((rc = dn_recompute_states(s, &local, seg, init_state, stream))) return rc;
    res = &local;
  }
  if (!res->T || !res->states) return DN_ERR_NULL_POINTER;
  const int cut = prepass_bwd_tc_eligible(g) ? overlap_cut(g) : 0;
  Overlap* ov = cut ? overlap_for_device() : nullptr;
  if (ov && p + carry_bytes(g) <= end) {
    // reverse chain over chunks [cut, NC); then the chunk-parallel backward of those chunks (side
    // stream, the partly filled round of CTAs) next to the rest of the chain; then the
    // chunk-parallel backward of chunks [0, cut) and the head sums
    if (!res->W || !res->U || !res->lam_end) return DN_ERR_NULL_POINTER;
    std::lock_guard<std::mutex> lock(ov->enqueue);
    float* carry = reinterpret_cast<float*>(p);
    p += carry_bytes(g);
    BwdPlan pl;
    if ((rc = plan_prepass_bwd(g, q, k, v, g_, b, w, seg, *res, d_out, dV, dH, dq, dk, dv, dg, db, dw,
                               p, (size_t)(end - p), pl))) return rc;
    StateArgs a{};
    a.g = g; a.res = *res; a.seg = seg; a.d_out = d_out; a.d_final = d_final_state;
    a.dV = dV; a.dH = dH; a.d_init = (g.flags & DN_HAS_INIT) ? d_init : nullptr; a.carry = carry;
    a.c_begin = cut; a.c_end = g.NC;
    if ((rc = launch_state_bwd_tc(a, st))) return rc;
    if (cudaEventRecord(ov->ev[0], st) != cudaSuccess || cudaStreamWaitEvent(ov->side, ov->ev[0], 0) != cudaSuccess)
      return DN_ERR_CUDA_LAUNCH;
    // forked: whatever fails from here on, the side stream is joined back before returning
    const int rc_side = launch_plan(pl, cut, g.NC, ov->side);
    const cudaError_t e1 = cudaEventRecord(ov->ev[1], ov->side);
    a.c_begin = 0; a.c_end = cut;
    const int rc_main = launch_state_bwd_tc(a, st);
    const cudaError_t e2 = cudaStreamWaitEvent(st, ov->ev[1], 0);
    if (rc_side) return rc_side;
    if (rc_main) return rc_main;
    if (e1 != cudaSuccess || e2 != cudaSuccess) return DN_ERR_CUDA_LAUNCH;
    if ((rc = launch_plan(pl, 0, cut, st))) return rc;
    return finish_plan(g, pl, st);
  }
  if ((rc = dn_state_bwd(s, res, seg, d_out, d_final_state, dV, dH, d_init, stream))) return rc;
  return run_prepass_bwd(g, q, k, v, g_, b, w, seg, *res, d_out, dV, dH, dq, dk, dv, dg, db, dw,
                         p, (size_t)(end - p), st);
}

// ---- sequence-parallel helpers ------------------------------------------------------------------
// Transition matrix of a shard: the map S_in -> S_out of the state pass is affine, S_out = P S_in + Q
// with P (K x K) per (batch, exec head).  P is the state pass run on K "value" columns with U = 0
// and S_in = I, because the recurrence acts on every value column independently.
int dn_sp_transition(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                     const float* identity, float* P, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || !identity || !P) return DN_ERR_NULL_POINTER;
  Geo t = g;                       // same chunks and heads, value width K, one "value head" per exec head
  t.Hv = g.H; t.G = 1; t.V = g.K; t.Vw = g.K; t.qk_div = 1;
  t.flags |= DN_HAS_INIT;
  StateArgs a{};
  a.g = t; a.res = *res; a.res.U = nullptr; a.res.states = nullptr; a.seg = seg;
  a.init_state = identity; a.final_state = P;
  return launch_state_fwd(a, (cudaStream_t)stream);
}

// One launch for a shard's affine summary: the state pass from a zero state WITH outputs and chunk
// states (complete for every chunk after the shard's first document boundary, provisional before it),
// carrying K extra columns that start from the identity and end as P.
int dn_sp_summary(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                  void* out, float* Q, float* P, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || !Q || !P) return DN_ERR_NULL_POINTER;
  if (!res->W || !res->U || !res->ke || !res->lam_end || (out && (!res->M || !res->qe))) return DN_ERR_NULL_POINTER;
  StateArgs a{};
  a.g = g; a.res = *res; a.seg = seg; a.init_state = nullptr;
  a.out = out; a.final_state = Q; a.states = res->states; a.P_out = P;
  a.skip_provisional = (g.flags & DN_SP_SKIP_PROVISIONAL) != 0;
  return launch_state_fwd(a, (cudaStream_t)stream);
}

// The forward chain again from the shard's true incoming state, over the chunks that depend on it.
int dn_sp_correct_fwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                      const float* S_in, void* out, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || !S_in || (!out && !res->states)) return DN_ERR_NULL_POINTER;
  if (!(g.flags & DN_HAS_INIT)) return DN_ERR_UNSUPPORTED;
  StateArgs a{};
  a.g = g; a.res = *res; a.seg = seg; a.init_state = S_in;
  a.out = out; a.states = res->states; a.until_independent = true;
  return launch_state_fwd(a, (cudaStream_t)stream);
}

// The reverse chain again from the shard's true incoming state cotangent, over the chunks that depend on it.
int dn_sp_correct_bwd(const dn_shape* s, const dn_residuals* res, const int32_t* seg,
                      const void* d_out, const float* d_final_state, float* dV, float* dH, void* stream) {
  Geo g;
  int rc = make_geo(s, &g);
  if (rc) return rc;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!res || !d_out || !d_final_state || !dV || !dH) return DN_ERR_NULL_POINTER;
  if (g.img && !res->states) return DN_ERR_NULL_POINTER;
  StateArgs a{};
  a.g = g; a.res = *res; a.seg = seg; a.d_out = d_out; a.d_final = d_final_state;
  a.dV = dV; a.dH = dH; a.until_independent = true;
  return launch_state_bwd(a, (cudaStream_t)stream);
}

int dn_launch_count(const dn_shape* s, int backward, int recompute) {
  Geo g;
  if (make_geo(s, &g)) return 0;
  const bool split_f = overlap_cut(g) && !overlap_disabled();      // (a pure query: creates no stream)
  const bool split_b = split_f && prepass_bwd_tc_eligible(g);
  if (!backward) return split_f ? 4 : 2;
  int n = split_b ? 4 : 2;
  if (recompute) n += 2;
  n += (g.qk_div > 1 ? 2 : 0) + (g.gH != g.H) + (g.bH != g.H) + (g.wH != g.Hv);   // head sums
  return n;
}

int dn_sp_apply(const float* P, const float* S_in, const float* Q, float* S_out, const uint8_t* keep, int32_t B,
                int32_t H, int32_t G, int32_t K, int32_t V, int32_t transpose, void* stream) {
  if (!P || !S_in || !S_out) return DN_ERR_NULL_POINTER;
  if (B < 1 || H < 1 || G < 1 || K < 1 || V < 1) return DN_ERR_BAD_SHAPE;
  return launch_sp_apply(P, S_in, Q, S_out, keep, B, H, G, K, V, transpose, (cudaStream_t)stream);
}

int dn_decode_step(const dn_decode_shape* s, const void* q, const void* k, const void* v,
                   const void* g_, const void* b, const void* w, const void* state_in,
                   const uint8_t* reset, void* out, void* state_out, void* stream) {
  if (!s || !q || !k || !v || !g_ || !b || !w || !state_in || !out || !state_out) return DN_ERR_NULL_POINTER;
  if (s->B < 1 || s->Hk < 1 || s->Hv % s->Hk) return DN_ERR_BAD_SHAPE;
  if ((s->K != 64 && s->K != 128) || (s->V != 64 && s->V != 128)) return DN_ERR_BAD_SHAPE;
  auto okh = [&](int h) { return h == 1 || h == s->Hk || h == s->Hv; };
  if (!okh(s->g_heads) || !okh(s->b_heads) || !okh(s->w_heads)) return DN_ERR_BAD_SHAPE;
  if ((s->g_cols != 1 && s->g_cols != s->K) || (s->b_cols != 1 && s->b_cols != s->K) ||
      (s->w_cols != 1 && s->w_cols != s->V)) return DN_ERR_BAD_SHAPE;
  if (state_in == state_out && s->state_in_dtype != s->state_out_dtype) return DN_ERR_UNSUPPORTED;
  if (peek_device_error()) return DN_ERR_DEVICE_WAIT;
  return launch_decode(*s, q, k, v, g_, b, w, state_in, reset, out, state_out, (cudaStream_t)stream);
}

int dn_cap_state(float* state, int64_t n_states, int32_t K, int32_t V, float tau, void* stream) {
  if (!state) return DN_ERR_NULL_POINTER;
  if (n_states < 1 || K < 1 || V < 1 || !(tau > 0.f)) return DN_ERR_BAD_SHAPE;
  return launch_cap_state(state, n_states, K * V, tau, (cudaStream_t)stream);
}

}  // extern "C"
