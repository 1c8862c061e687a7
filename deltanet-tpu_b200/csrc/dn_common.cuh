// Shared device helpers: dtype-agnostic loads/stores, the exec-head view of a shape,
// segment flags, and a CTA-wide fp32 GEMM on operands given as index functors.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/deltanet_b200.h"

#define DN_THREADS 256
#define DN_LOG2E 1.4426950408889634f

namespace dn {

// true when the environment asks for the fp32 SIMT kernels everywhere (DN_FORCE_SIMT=1)
bool force_simt();
// streaming multiprocessors of the current device (queried once per device)
int sm_count();

// --------------------------------------------------------------------------- geometry
// Everything a kernel needs to know about where a (batch, exec head, chunk) lives.
struct Geo {
  int B, L, Hk, Hv, K, V, C, NC;
  int H, Vw, G;          // exec heads, value width, value heads per exec head
  int qk_div;            // q/k head of exec head h is h / qk_div
  int gH, gC, bH, bC, wH, wC;
  int qkv_dt, gate_dt, pre_dt, prec;
  uint32_t flags;
  float scale;
  // Layout of the bf16 residual tiles W, U, M, qe, ke.  false: row-major (rows x cols).  true: the
  // operand image of the tensor-core kernels, [col / 8][row][8] -- a tile is then copied into shared
  // memory as it lies, and a thread that owns one row writes 16 bytes next to its neighbours'.
  // Chosen once per shape (prepass on the tensor cores <=> image layout); every kernel reading or
  // writing these tiles goes through rix().
  bool img;
  __host__ __device__ bool bf16_mode() const { return prec == DN_PREC_BF16; }
  __host__ __device__ bool state_bf16() const { return prec == DN_PREC_BF16 && !(flags & DN_STATE_FP32_MM); }
  // head of a gate tensor that exec head h (and, for w, value head hv) reads
  __host__ __device__ int gate_head(int h, int nheads) const {
    if (nheads == 1) return 0;
    if (nheads == H) return h;
    return h / (H / nheads);             // H == Hv and the gate sits at Hk heads
  }
  __host__ __device__ int w_head(int hv) const {
    if (wH == 1) return 0;
    if (wH == Hv) return hv;
    return hv / (Hv / wH);               // w given per key head
  }
};

inline int make_geo(const dn_shape* s, Geo* g) {
  if (!s) return DN_ERR_NULL_POINTER;
  if (s->B < 1 || s->L < 1 || s->Hk < 1 || s->Hv < 1 || s->Hv % s->Hk) return DN_ERR_BAD_SHAPE;
  if ((s->K != 64 && s->K != 128) || (s->V != 64 && s->V != 128)) return DN_ERR_BAD_SHAPE;
  if (s->chunk != 64 && s->chunk != 128) return DN_ERR_BAD_SHAPE;
  auto okh = [&](int h) { return h == 1 || h == s->Hk || h == s->Hv; };
  if (!okh(s->g_heads) || !okh(s->b_heads) || !okh(s->w_heads)) return DN_ERR_BAD_SHAPE;
  if ((s->g_cols != 1 && s->g_cols != s->K) || (s->b_cols != 1 && s->b_cols != s->K) ||
      (s->w_cols != 1 && s->w_cols != s->V)) return DN_ERR_BAD_SHAPE;
  if ((s->qkv_dtype != DN_F32 && s->qkv_dtype != DN_BF16) ||
      (s->gate_dtype != DN_F32 && s->gate_dtype != DN_BF16)) return DN_ERR_BAD_DTYPE;
  if (s->precision != DN_PREC_FP32 && s->precision != DN_PREC_BF16) return DN_ERR_BAD_DTYPE;
  g->B = s->B; g->L = s->L; g->Hk = s->Hk; g->Hv = s->Hv; g->K = s->K; g->V = s->V;
  bool at_hv = (s->Hk < s->Hv) && (s->g_heads == s->Hv || s->b_heads == s->Hv);
  // More than two value heads per key head would make a tile wider than the tensor-core kernels take
  // (G V > 256): such calls use the per-value-head view too (the key-side work is repeated per value head,
  // the key-side gradients are summed over the group as for gates given per value head).
  if (s->Hk < s->Hv && s->precision == DN_PREC_BF16 && !(s->flags & DN_STATE_FP32_MM) && s->K == 128 && s->V == 128 &&
      (s->Hv / s->Hk) * s->V > 256 && !force_simt())
    at_hv = true;
  if (at_hv) { g->H = s->Hv; g->Vw = s->V; g->G = 1; g->qk_div = s->Hv / s->Hk; }
  else       { g->H = s->Hk; g->G = s->Hv / s->Hk; g->Vw = g->G * s->V; g->qk_div = 1; }
  if (g->Vw > 1024) return DN_ERR_BAD_SHAPE;
  // Rows per tile.  The tensor-core kernels work on 128-row tiles (the M of a tcgen05.mma), so in
  // bf16 precision a request for chunk 64 is run with two requested chunks merged into one tile:
  // the chunked form is an exact regrouping of the token recurrence, results differ only in where
  // the state is rounded to bf16 (every 128 tokens instead of every 64).  dn_exec_view reports the
  // tile height actually used; every buffer size follows from it.
  const bool tc_shape = s->precision == DN_PREC_BF16 && !(s->flags & DN_STATE_FP32_MM) && s->K == 128 &&
                        (g->Vw == 128 || g->Vw == 256) && !force_simt();
  g->C = (tc_shape && s->chunk == 64) ? 128 : s->chunk;
  g->NC = (s->L + g->C - 1) / g->C;
  g->gH = s->g_heads; g->gC = s->g_cols; g->bH = s->b_heads; g->bC = s->b_cols;
  g->wH = s->w_heads; g->wC = s->w_cols;
  g->qkv_dt = s->qkv_dtype; g->gate_dt = s->gate_dtype; g->prec = s->precision;
  g->pre_dt = s->precision == DN_PREC_BF16 ? DN_BF16 : DN_F32;
  g->flags = s->flags; g->scale = s->scale;
  g->img = tc_shape;
  return DN_OK;
}

// On the image path three more arrays are kept as bf16 operand images, [col / 8][128 rows][8]:
//   * the chunk-entry states (the only copy on this path: the `states` slot holds the image): states_img();
//   * T, in the first half of its fp32-sized slot;
//   * dV and dH, in the first half of their fp32-sized buffers; the second half of the dH buffer
//     carries the partial sums of dLambda_end, (item, column slice of 32, K) fp32: dlend_part().
__host__ __device__ __forceinline__ const __nv_bfloat16* states_img(const Geo& g, const float* states) {
  (void)g;
  return reinterpret_cast<const __nv_bfloat16*>(states);
}
__host__ __device__ __forceinline__ float* dlend_part(const Geo& g, float* dH) {
  return dH + (size_t)g.B * g.H * g.NC * g.K * g.Vw / 2;
}

// element index of (row, col) in a residual tile of 128 rows (image layout) or `ncols` columns (row-major)
__host__ __device__ __forceinline__ size_t rix(bool img, int row, int col, int ncols) {
  return img ? ((size_t)((col >> 3) * 128 + row) << 3) + (col & 7) : (size_t)row * ncols + col;
}

// Optional phase clock (compile with -DDN_PHASE_TIMING): CTA 0 records clock64 at marked points of
// its first item and prints the differences.  Compiled out otherwise.
#ifdef DN_PHASE_TIMING
static __device__ long long g_phase_marks[48];
#define DN_MARK(i) do { if (blockIdx.x == 0 && threadIdx.x == 0) g_phase_marks[i] = clock64(); } while (0)
#else
#define DN_MARK(i) do { } while (0)
#endif

// --------------------------------------------------------------------------- dtype helpers
// A bounded wait gave up: raise the library's error word (a plain store; the word may live in
// host memory that the device reaches over the bus).
__device__ __forceinline__ void report_timeout(int* err) {
  if (err) { *reinterpret_cast<volatile int*>(err) = 1; __threadfence_system(); }
}

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

__device__ __forceinline__ float ldf(const void* p, size_t i, int dt) {
  return dt == DN_BF16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p)[i])
                       : reinterpret_cast<const float*>(p)[i];
}
// the same load through the read-only path: only for data no thread of the running kernel writes
__device__ __forceinline__ float ldf_ro(const void* p, size_t i, int dt) {
  return dt == DN_BF16 ? __bfloat162float(__ldg(reinterpret_cast<const __nv_bfloat16*>(p) + i))
                       : __ldg(reinterpret_cast<const float*>(p) + i);
}
__device__ __forceinline__ void stf(void* p, size_t i, float v, int dt) {
  if (dt == DN_BF16) reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
  else reinterpret_cast<float*>(p)[i] = v;
}
__host__ __device__ __forceinline__ size_t dt_size(int dt) { return dt == DN_BF16 ? 2 : 4; }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// Segment id of token t of row b; rows past L repeat the last id (edge padding).
__device__ __forceinline__ int seg_at(const int32_t* seg, int b, int t, int L) {
  if (!seg) return 0;
  return seg[(size_t)b * L + (t < L ? t : L - 1)];
}
// Flags of chunk c (reference: gdn2.py:1291-1302).
__device__ __forceinline__ void chunk_flags(const int32_t* seg, const Geo& g, int b, int c,
                                            bool& is_new_doc, bool& all_same_doc) {
  int first = seg_at(seg, b, c * g.C, g.L);
  int last = seg_at(seg, b, c * g.C + g.C - 1, g.L);
  int prev = c == 0 ? ((g.flags & DN_HAS_INIT) ? 0 : -1) : seg_at(seg, b, c * g.C - 1, g.L);
  is_new_doc = first != prev;
  all_same_doc = first == last;
}

// --------------------------------------------------------------------------- CTA GEMM
// C[M x N] = A[M x Kc] * B[Kc x N] with fa(i,k), fb(k,j) giving operand elements and
// epi(i,j,acc) consuming results.  256 threads, 64x64 output tiles, fp32 FMA.  M, N, Kc
// need not be multiples of the tile (out-of-range operand elements are read as 0 and
// out-of-range results are not passed to epi).  A_KFAST / B_NFAST say which index of the
// operand is contiguous in memory, which only steers the (coalesced) tile-load mapping.
// `tile` is 2*16*68 floats of shared memory.  Ends with a __syncthreads().
constexpr int GT = 64, GK = 16, GS = 68;
constexpr int GEMM_SMEM_FLOATS = 2 * GK * GS;

template <bool A_KFAST, bool B_NFAST, class FA, class FB, class EPI>
__device__ __forceinline__ void cta_gemm(int M, int N, int Kc, FA fa, FB fb, EPI epi, float* tile) {
  float* As = tile;
  float* Bs = tile + GK * GS;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  for (int m0 = 0; m0 < M; m0 += GT) {
    for (int n0 = 0; n0 < N; n0 += GT) {
      float acc[4][4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) acc[r][c] = 0.f;
      for (int k0 = 0; k0 < Kc; k0 += GK) {
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          int idx = tid + r * DN_THREADS;
          int i, kk;
          if (A_KFAST) { kk = idx & 15; i = idx >> 4; } else { i = idx & 63; kk = idx >> 6; }
          float v = 0.f;
          if (m0 + i < M && k0 + kk < Kc) v = fa(m0 + i, k0 + kk);
          As[kk * GS + i] = v;
          int j, k2;
          if (B_NFAST) { j = idx & 63; k2 = idx >> 6; } else { k2 = idx & 15; j = idx >> 4; }
          float u = 0.f;
          if (n0 + j < N && k0 + k2 < Kc) u = fb(k0 + k2, n0 + j);
          Bs[k2 * GS + j] = u;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GK; ++kk) {
          float4 a = *reinterpret_cast<const float4*>(&As[kk * GS + ty * 4]);
          float4 b = *reinterpret_cast<const float4*>(&Bs[kk * GS + tx * 4]);
          float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
          for (int r = 0; r < 4; ++r)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[r][c] = fmaf(av[r], bv[c], acc[r][c]);
        }
        __syncthreads();
      }
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          int i = m0 + ty * 4 + r, j = n0 + tx * 4 + c;
          if (i < M && j < N) epi(i, j, acc[r][c]);
        }
    }
  }
  __syncthreads();
}

}  // namespace dn
