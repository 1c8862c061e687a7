// Per-chunk preparation shared by the tensor-core prepass kernels (chunk = K = 128):
// activated and normalised rows of q, k, b, g read straight from the user's tensors in
// 8-element pieces, the cumulative log-decay in shared memory, and the bf16 operand images of
// one level of the hierarchical A/M factorisation.
#pragma once
#include "dn_common.cuh"
#include "dn_umma.cuh"

namespace dn {
namespace prep {

constexpr int C = 128, K = 128;
constexpr int IMG = 128 * 16;          // uint4 per 128x128 bf16 image
constexpr int LP = 132;                // row pitch (floats) of the shared-memory Lambda array: 16-byte
                                       // shifts between rows keep row-strided float4 reads conflict-free

// What a kernel instantiation knows about its inputs at compile time.  MODE 0: q/k/v in bf16, gates
// in fp32 and already activated (no fused prologue), every gate with one value per channel; MODE 1:
// the same with q/k/v in fp32; MODE 2: nothing (dtypes, gate widths and the prologue are run-time
// properties, every load sits behind a branch and both activation paths are compiled in); MODE 3:
// bf16 q/k/v, fp32 activated gates with ONE value per head (Gated DeltaNet's scalar decay and beta);
// MODE 4: bf16 q/k/v, fp32 activated gates, the decay per channel and ONE erase / write gate value per head
// (the KDA layout).
template <int MODE>
struct InCfg {
  static constexpr bool fixed = MODE != 2;
  static constexpr bool scalar_gates = MODE == 3;                 // the decay is one scalar per (token, head)
  static constexpr bool scalar_bw = MODE == 3 || MODE == 4;       // b and w are
  static constexpr int qkv_dt = MODE == 1 ? DN_F32 : DN_BF16;
};
inline int input_mode(const Geo& g) {
  if (g.gate_dt != DN_F32 || (g.flags & (DN_FUSE_PROLOGUE | DN_STABILITY_GUARD))) return 2;
  if (g.gC == g.K && g.bC == g.K && g.wC == g.V) return g.qkv_dt == DN_BF16 ? 0 : 1;
  if (g.gC == 1 && g.bC == 1 && g.wC == 1 && g.qkv_dt == DN_BF16) return 3;
  if (g.gC == g.K && g.bC == 1 && g.wC == 1 && g.qkv_dt == DN_BF16) return 4;
  return 2;
}

// Where one (batch, exec head, chunk) reads its rows from.
struct Rows {
  const void *q, *k, *gg, *b;
  int qkv_dt, gate_dt;
  size_t qk_row0;        // element offset of (token t0, head hq, channel 0) in q / k
  size_t qk_pitch;       // elements between tokens
  size_t g_row0, g_pitch;   // same for g (channel 0 of its head)
  size_t b_row0, b_pitch;
  int gC, bC;            // channels per row of g / b: 1 or K
  int rows_valid;        // tokens of the chunk that exist
  bool l2, fuse, guard, round_in;
  float scale;
  const float *rq, *rk;  // per-row normalisers (shared memory), 1 when l2 is off
};

// Eight consecutive elements of one of the operator's INPUT tensors (read-only path: never for
// memory the running kernel writes).
__device__ __forceinline__ void load8(const void* base, size_t off, int dt, float (&x)[8]) {
  if (dt == DN_BF16) umma::unpack8(__ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + off)), x);
  else {
    const float4 a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off));
    const float4 b = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off + 4));
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
}
__device__ __forceinline__ void zero8(float (&x)[8]) {
#pragma unroll
  for (int i = 0; i < 8; ++i) x[i] = 0.f;
}

// raw q / k piece (channels 8p..8p+7 of chunk row x), zero on rows past the end.  The load itself
// is unconditional (a row past the end reads row 0 and is zeroed afterwards), so that a caller's
// loads can all be in flight together.
__device__ __forceinline__ void raw_q8(const Rows& r, int x, int p, float (&o)[8]) {
  const bool live = x < r.rows_valid;
  load8(r.q, r.qk_row0 + (size_t)(live ? x : 0) * r.qk_pitch + 8 * p, r.qkv_dt, o);
  if (!live) zero8(o);
}
__device__ __forceinline__ void raw_k8(const Rows& r, int x, int p, float (&o)[8]) {
  const bool live = x < r.rows_valid;
  load8(r.k, r.qk_row0 + (size_t)(live ? x : 0) * r.qk_pitch + 8 * p, r.qkv_dt, o);
  if (!live) zero8(o);
}
// q_hat = l2norm(q) * scale, k_hat = l2norm(k), each rounded to the input dtype when the
// prologue is not fused (the reference stores them in the input dtype, gdn2.py:2113-2122)
__device__ __forceinline__ void qhat8(const Rows& r, int x, int p, float (&o)[8]) {
  raw_q8(r, x, p, o);
  const float f = r.rq[x];
#pragma unroll
  for (int i = 0; i < 8; ++i) { o[i] = (o[i] * f) * r.scale; if (r.round_in) o[i] = bf16r(o[i]); }
}
__device__ __forceinline__ void khat8(const Rows& r, int x, int p, float (&o)[8]) {
  raw_k8(r, x, p, o);
  if (!r.l2) return;
  const float f = r.rk[x];
#pragma unroll
  for (int i = 0; i < 8; ++i) { o[i] *= f; if (r.round_in) o[i] = bf16r(o[i]); }
}
// raw gate pieces (a per-head scalar is broadcast over the channels)
__device__ __forceinline__ void raw_gate8(const void* base, size_t row0, size_t pitch, int cols, int dt, int x, int p,
                                          float (&o)[8]) {
  if (cols == 1) {
    const float v = ldf_ro(base, row0 + (size_t)x * pitch, dt);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = v;
  } else {
    load8(base, row0 + (size_t)x * pitch + 8 * p, dt, o);
  }
}
// activated erase gate b
__device__ __forceinline__ void bact8(const Rows& r, int x, int p, float (&o)[8]) {
  const bool live = x < r.rows_valid;
  raw_gate8(r.b, r.b_row0, r.b_pitch, r.bC, r.gate_dt, live ? x : 0, p, o);
  if (r.fuse) {
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = 1.f / (1.f + expf(-o[i]));
  } else if (r.guard) {                       // stability_guard on a given gate: b >= 0 (gdn2.py:1973)
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = fmaxf(o[i], 0.f);
  }
  if (!live) zero8(o);
}
// activated log-decay g (<= 0)
__device__ __forceinline__ void gact8(const Rows& r, int x, int p, float (&o)[8]) {
  const bool live = x < r.rows_valid;
  raw_gate8(r.gg, r.g_row0, r.g_pitch, r.gC, r.gate_dt, live ? x : 0, p, o);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    if (r.fuse) { o[i] = -expf(fminf(o[i], 5.f)); if (r.guard) o[i] = fminf(o[i], -1e-6f); }
    else { o[i] = o[i] <= 0.f ? o[i] : 0.f; if (r.guard) o[i] = fminf(o[i], -1e-6f); }
  }
  if (!live) zero8(o);
}
// beta = b_act * k_hat
__device__ __forceinline__ void beta8(const Rows& r, int x, int p, float (&o)[8]) {
  float kk[8];
  bact8(r, x, p, o);
  khat8(r, x, p, kk);
#pragma unroll
  for (int i = 0; i < 8; ++i) o[i] *= kk[i];
}

// Row normalisers, 512 threads, a warp covering 8 rows x 4 pieces: thread (myrow = 8*warp + (lane&7),
// lgrp = lane>>3) sums its 4 pieces of q and k, the four threads of a row sit 8 lanes apart.
__device__ __forceinline__ void row_norms_8x4(const Rows& r, int myrow, int lgrp, float* rq, float* rk) {
  float sq = 0.f, sk = 0.f;
  if (r.l2) {                       // rows past the end read as zero
#pragma unroll
    for (int it = 0; it < 4; ++it) {
      float qv[8], kv[8];
      raw_q8(r, myrow, it * 4 + lgrp, qv);
      raw_k8(r, myrow, it * 4 + lgrp, kv);
#pragma unroll
      for (int i = 0; i < 8; ++i) { sq = fmaf(qv[i], qv[i], sq); sk = fmaf(kv[i], kv[i], sk); }
    }
  }
  sq += __shfl_xor_sync(0xffffffffu, sq, 8);  sk += __shfl_xor_sync(0xffffffffu, sk, 8);
  sq += __shfl_xor_sync(0xffffffffu, sq, 16); sk += __shfl_xor_sync(0xffffffffu, sk, 16);
  if (lgrp == 0) {
    rq[myrow] = r.l2 ? rsqrtf(sq + 1e-6f) : 1.f;
    rk[myrow] = r.l2 ? rsqrtf(sk + 1e-6f) : 1.f;
  }
}

// Cumulative log-decay of the chunk into shared memory (C rows of pitch LP, fp32), restarting at
// document changes.  512 threads: thread (channel c, quarter qd) loads and scans 32 rows in
// registers; the quarters are chained through `tot` (4 x 128 floats of shared memory) and `reset`
// (4 ints: a document starts inside the quarter).  seg_s must be visible before; a __syncthreads()
// is needed after.
__device__ __forceinline__ void lambda_scan_512(const Rows& r, const int* seg_s, float* LAM, float* tot, int* reset) {
  const int c = threadIdx.x & 127, qd = threadIdx.x >> 7, x0 = qd * 32;
  const size_t gcol = r.gC == 1 ? 0 : c;
  float v[32];
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int x = x0 + i;
    const bool live = x < r.rows_valid;
    float gv = ldf_ro(r.gg, r.g_row0 + (size_t)(live ? x : 0) * r.g_pitch + gcol, r.gate_dt);
    if (r.fuse) { gv = -expf(fminf(gv, 5.f)); if (r.guard) gv = fminf(gv, -1e-6f); }
    else { gv = gv <= 0.f ? gv : 0.f; if (r.guard) gv = fminf(gv, -1e-6f); }
    v[i] = live ? gv : 0.f;
  }
  float run = 0.f;
  int nr = 32;                                   // first row of the quarter that starts a document
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int x = x0 + i;
    if (x > 0 && seg_s[x] != seg_s[x - 1]) { run = 0.f; if (nr == 32) nr = i; }
    run += v[i];
    v[i] = run;
  }
  tot[qd * 128 + c] = run;
  if (c == 0) reset[qd] = nr < 32;
  __syncthreads();
  float carry = 0.f;
  for (int q2 = qd - 1; q2 >= 0; --q2) {
    carry += tot[q2 * 128 + c];
    if (reset[q2]) break;
  }
#pragma unroll
  for (int i = 0; i < 32; ++i) LAM[(x0 + i) * LP + c] = v[i] + (i < nr ? carry : 0.f);
}

__device__ __forceinline__ int level_ref(int x, int s) { return (x / (2 * s)) * 2 * s + s; }

// exp(min(a - b, 0)) for eight channels of two LAM rows
__device__ __forceinline__ void decay8(const float* la, const float* lb, float (&f)[8]) {
  const float4 a0 = *reinterpret_cast<const float4*>(la), a1 = *reinterpret_cast<const float4*>(la + 4);
  const float4 b0 = *reinterpret_cast<const float4*>(lb), b1 = *reinterpret_cast<const float4*>(lb + 4);
  const float d[8] = {a0.x - b0.x, a0.y - b0.y, a0.z - b0.z, a0.w - b0.w, a1.x - b1.x, a1.y - b1.y, a1.z - b1.z, a1.w - b1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = umma::ex2_fast(fminf(d[i], 0.f) * DN_LOG2E);
}

// Operand images of level s (pairs of adjacent s-row blocks; reference row = first row of the
// lower block).  Every row has one role per level: rows of the upper blocks (x < ref) carry
// k_hat * exp(Lam_ref - Lam_x) in BOTH images; rows of the lower blocks carry
// beta * exp(Lam_x - Lam_ref) in KR and q_hat * exp(Lam_x - Lam_ref) in QK.  All scale factors are
// <= 1.  One piece (row x, channel group p) per call, stored at image[p*128 + x].
__device__ __forceinline__ void build_level_from(const float (&kh)[8], const float (&ba)[8], const float (&qh)[8],
                                                 const float* LAM, int s, int x, int p, uint4* KR, uint4* QK) {
  const int ref = level_ref(x, s);
  const bool lower = x >= ref;
  float f[8], o1[8], o2[8];
  decay8(LAM + (lower ? x : ref) * LP + 8 * p, LAM + (lower ? ref : x) * LP + 8 * p, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float kf = kh[i] * f[i];
    o1[i] = lower ? (ba[i] * kh[i]) * f[i] : kf;
    o2[i] = lower ? qh[i] * f[i] : kf;
  }
  KR[p * 128 + x] = umma::pack8(o1);
  QK[p * 128 + x] = umma::pack8(o2);
}
// The same from beta = b_act * k_hat already formed (operands cached on chip).
__device__ __forceinline__ void build_level_from_beta(const float (&kh)[8], const float (&be)[8], const float (&qh)[8],
                                                      const float* LAM, int s, int x, int p, uint4* KR, uint4* QK) {
  const int ref = level_ref(x, s);
  const bool lower = x >= ref;
  float f[8], o1[8], o2[8];
  decay8(LAM + (lower ? x : ref) * LP + 8 * p, LAM + (lower ? ref : x) * LP + 8 * p, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float kf = kh[i] * f[i];
    o1[i] = lower ? be[i] * f[i] : kf;
    o2[i] = lower ? qh[i] * f[i] : kf;
  }
  KR[p * 128 + x] = umma::pack8(o1);
  QK[p * 128 + x] = umma::pack8(o2);
}
__device__ __forceinline__ void build_level_piece(const Rows& r, const float* LAM, int s, int x, int p, uint4* KR, uint4* QK) {
  float kh[8], ba[8], qh[8];
  khat8(r, x, p, kh);              // all three loads are issued before the role is looked at
  bact8(r, x, p, ba);
  qhat8(r, x, p, qh);
  build_level_from(kh, ba, qh, LAM, s, x, p, KR, QK);
}

// Which level owns entry (row block bi, column block bj) of the strictly lower block triangle:
// 0 -> s = 16, 1 -> s = 32, 2 -> s = 64 (the highest bit in which the 16-row block indices differ).
__device__ __forceinline__ int owner_level(int bi, int bj) {
  const int x = bi ^ bj;
  return x >= 4 ? 2 : (x >= 2 ? 1 : 0);
}

template <class CF = InCfg<2>>
__device__ __forceinline__ Rows make_rows(const Geo& g, const void* q, const void* k, const void* gg, const void* b,
                                          int bidx, int h, int t0, const float* rq, const float* rk) {
  Rows r;
  r.q = q; r.k = k; r.gg = gg; r.b = b;
  r.qkv_dt = CF::fixed ? CF::qkv_dt : g.qkv_dt;
  r.gate_dt = CF::fixed ? DN_F32 : g.gate_dt;
  const size_t tok0 = (size_t)bidx * g.L + t0;
  r.qk_pitch = (size_t)g.Hk * K;
  r.qk_row0 = tok0 * r.qk_pitch + (size_t)(h / g.qk_div) * K;
  r.gC = CF::fixed ? (CF::scalar_gates ? 1 : K) : g.gC;
  r.bC = CF::fixed ? (CF::scalar_bw ? 1 : K) : g.bC;
  r.g_pitch = (size_t)g.gH * g.gC;
  r.g_row0 = tok0 * r.g_pitch + (size_t)g.gate_head(h, g.gH) * g.gC;
  r.b_pitch = (size_t)g.bH * g.bC;
  r.b_row0 = tok0 * r.b_pitch + (size_t)g.gate_head(h, g.bH) * g.bC;
  r.rows_valid = g.L - t0 < C ? g.L - t0 : C;
  r.l2 = g.flags & DN_QK_L2NORM;
  r.fuse = CF::fixed ? false : (g.flags & DN_FUSE_PROLOGUE) != 0;
  r.guard = CF::fixed ? false : (g.flags & DN_STABILITY_GUARD) != 0;
  r.round_in = !r.fuse && g.qkv_dt == DN_BF16;
  r.scale = g.scale;
  r.rq = rq; r.rk = rk;
  return r;
}

}  // namespace prep
}  // namespace dn
