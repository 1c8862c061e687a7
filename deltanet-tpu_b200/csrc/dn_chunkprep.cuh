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
// in fp32, every gate with one value per channel; MODE 1: the same with q/k/v in fp32; MODE 2:
// nothing (dtypes and gate widths are run-time properties, every load sits behind a branch).
template <int MODE>
struct InCfg {
  static constexpr bool fixed = MODE != 2;
  static constexpr int qkv_dt = MODE == 0 ? DN_BF16 : DN_F32;
};
inline int input_mode(const Geo& g) {
  const bool full = g.gC == g.K && g.bC == g.K && g.wC == g.V && g.gate_dt == DN_F32;
  if (!full) return 2;
  return g.qkv_dt == DN_BF16 ? 0 : 1;
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
    else o[i] = o[i] <= 0.f ? o[i] : 0.f;
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

// Row normalisers: one warp per row.
template <int NT>
__device__ __forceinline__ void row_norms(const Rows& r, float* rq, float* rk) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int x = warp; x < C; x += NT / 32) {
    float sq = 0.f, sk = 0.f;
    if (r.l2 && x < r.rows_valid) {
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const float a = ldf_ro(r.q, r.qk_row0 + (size_t)x * r.qk_pitch + lane + 32 * u, r.qkv_dt);
        const float b = ldf_ro(r.k, r.qk_row0 + (size_t)x * r.qk_pitch + lane + 32 * u, r.qkv_dt);
        sq += a * a;
        sk += b * b;
      }
    }
    sq = warp_sum(sq);
    sk = warp_sum(sk);
    if (lane == 0) {
      rq[x] = r.l2 ? rsqrtf(sq + 1e-6f) : 1.f;
      rk[x] = r.l2 ? rsqrtf(sk + 1e-6f) : 1.f;
    }
  }
}

// Cumulative log-decay of the chunk into shared memory (C rows of pitch LP, fp32), restarting at
// document changes.  Needs a __syncthreads() before and leaves one after.
template <int NT>
__device__ __forceinline__ void build_lambda(const Rows& r, const int* seg_s, float* LAM) {
  for (int e = threadIdx.x; e < IMG; e += NT) {
    const int x = e >> 4, p = e & 15;
    float gv[8];
    gact8(r, x, p, gv);
    float4* d = reinterpret_cast<float4*>(LAM + x * LP + 8 * p);
    d[0] = make_float4(gv[0], gv[1], gv[2], gv[3]);
    d[1] = make_float4(gv[4], gv[5], gv[6], gv[7]);
  }
  __syncthreads();
  if (threadIdx.x < K) {
    float run = 0.f;
    int prev = seg_s[0];
#pragma unroll 4
    for (int i = 0; i < C; ++i) {
      const int s = seg_s[i];
      if (s != prev) run = 0.f;
      prev = s;
      run += LAM[i * LP + threadIdx.x];
      LAM[i * LP + threadIdx.x] = run;
    }
  }
  __syncthreads();
}

__device__ __forceinline__ int level_ref(int x, int s) { return (x / (2 * s)) * 2 * s + s; }

// exp(min(a - b, 0)) for eight channels of two LAM rows
__device__ __forceinline__ void decay8(const float* la, const float* lb, float (&f)[8]) {
  const float4 a0 = *reinterpret_cast<const float4*>(la), a1 = *reinterpret_cast<const float4*>(la + 4);
  const float4 b0 = *reinterpret_cast<const float4*>(lb), b1 = *reinterpret_cast<const float4*>(lb + 4);
  const float d[8] = {a0.x - b0.x, a0.y - b0.y, a0.z - b0.z, a0.w - b0.w, a1.x - b1.x, a1.y - b1.y, a1.z - b1.z, a1.w - b1.w};
#pragma unroll
  for (int i = 0; i < 8; ++i) f[i] = exp2f(fminf(d[i], 0.f) * DN_LOG2E);
}

// Operand images of level s (pairs of adjacent s-row blocks; reference row = first row of the
// lower block): rows of the lower blocks carry beta and q_hat scaled by exp(Lam_x - Lam_ref),
// rows of the upper blocks carry k_hat scaled by exp(Lam_ref - Lam_x); the other rows are 0.
// Piece e = (p = channel group, x = row) sits at image[p*128 + x].
template <int NT>
__device__ __forceinline__ void build_level(const Rows& r, const float* LAM, int s, uint4* RB, uint4* RQ, uint4* KC) {
  const uint4 zero = make_uint4(0, 0, 0, 0);
  for (int e = threadIdx.x; e < IMG; e += NT) {
    const int p = e >> 7, x = e & 127;
    const int ref = level_ref(x, s);
    float f[8], a[8];
    if (x >= ref) {
      decay8(LAM + x * LP + 8 * p, LAM + ref * LP + 8 * p, f);
      if (RB) {
        beta8(r, x, p, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] *= f[i];
        RB[e] = umma::pack8(a);
      }
      if (RQ) {
        qhat8(r, x, p, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] *= f[i];
        RQ[e] = umma::pack8(a);
      }
      if (KC) KC[e] = zero;
    } else {
      if (KC) {
        decay8(LAM + ref * LP + 8 * p, LAM + x * LP + 8 * p, f);
        khat8(r, x, p, a);
#pragma unroll
        for (int i = 0; i < 8; ++i) a[i] *= f[i];
        KC[e] = umma::pack8(a);
      }
      if (RB) RB[e] = zero;
      if (RQ) RQ[e] = zero;
    }
  }
}

// The same images for the backward, where every row has one role per level: rows of the upper
// blocks (x < ref) carry k_hat * exp(Lam_ref - Lam_x) in BOTH images; rows of the lower blocks carry
// beta * exp(Lam_x - Lam_ref) in KR and q_hat * exp(Lam_x - Lam_ref) in QK.  One piece (row x,
// channel group p) per call.
__device__ __forceinline__ void build_level_piece(const Rows& r, const float* LAM, int s, int x, int p, uint4* KR, uint4* QK) {
  const int ref = level_ref(x, s);
  const bool lower = x >= ref;
  float f[8], kh[8], ba[8], qh[8];
  khat8(r, x, p, kh);              // all three loads are issued before the role is looked at
  bact8(r, x, p, ba);
  qhat8(r, x, p, qh);
  decay8(LAM + (lower ? x : ref) * LP + 8 * p, LAM + (lower ? ref : x) * LP + 8 * p, f);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const float kf = kh[i] * f[i];
    ba[i] = lower ? (ba[i] * kh[i]) * f[i] : kf;
    qh[i] = lower ? qh[i] * f[i] : kf;
  }
  KR[p * 128 + x] = umma::pack8(ba);
  QK[p * 128 + x] = umma::pack8(qh);
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
  r.gC = CF::fixed ? K : g.gC;
  r.bC = CF::fixed ? K : g.bC;
  r.g_pitch = (size_t)g.gH * g.gC;
  r.g_row0 = tok0 * r.g_pitch + (size_t)g.gate_head(h, g.gH) * g.gC;
  r.b_pitch = (size_t)g.bH * g.bC;
  r.b_row0 = tok0 * r.b_pitch + (size_t)g.gate_head(h, g.bH) * g.bC;
  r.rows_valid = g.L - t0 < C ? g.L - t0 : C;
  r.l2 = g.flags & DN_QK_L2NORM; r.fuse = g.flags & DN_FUSE_PROLOGUE; r.guard = g.flags & DN_STABILITY_GUARD;
  r.round_in = !r.fuse && g.qkv_dt == DN_BF16;
  r.scale = g.scale;
  r.rq = rq; r.rk = rk;
  return r;
}

}  // namespace prep
}  // namespace dn
