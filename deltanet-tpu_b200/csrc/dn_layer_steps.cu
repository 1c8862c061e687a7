// The steps either side of the recurrence in a Gated DeltaNet layer, as the reference's layer example
// wires them (examples/qwen3_5_layer_parity.py:144-159 of the reference project):
//
//   producer   mixed (B,L,D), D = 2*Hk*K + Hv*V  --depthwise causal conv (width W <= 4) + SiLU-->  q | k | v
//              a, b (B,L,Hv)  -->  g = -exp(A_log) * softplus(a + dt_bias),  beta = sigmoid(b)
//   consumer   y = weight * rmsnorm(o) * silu(z) per (token, value head), o and z of shape (rows, V)
//
// All of it is element-wise or a short stencil over tokens, i.e. bound by HBM bytes: every kernel
// below reads each input once with 16-byte accesses (a thread owns 8 channels and walks a run of
// tokens with the stencil window in registers, so the halo is 3 rows per run) and writes each output
// once.  Parameter gradients (conv weight, bias, A_log, dt_bias, norm weight) are reduced in a fixed
// order through per-tile partial sums, so results are bit-reproducible.
#include "dn_kernels.cuh"
#include "dn_umma.cuh"

namespace dn {
namespace {

constexpr int CG = 8;            // channels per thread (one 16-byte bf16 vector)
constexpr int PT = 128;          // threads per CTA of the producer kernels (= 1024 channels)
constexpr int TT_FWD = 64;       // tokens per thread run, forward
constexpr int TT_BWD = 256;      // tokens per thread run, backward (also the tile of the weight-gradient partials)
constexpr int MAXW = 4;

__device__ __forceinline__ float silu(float x) { return x * __frcp_rn(1.f + __expf(-x)); }
// d silu(x) / dx = s + x s (1 - s), s = sigmoid(x)
__device__ __forceinline__ float dsilu(float x) {
  const float s = __frcp_rn(1.f + __expf(-x));
  return s * (1.f + x * (1.f - s));
}

__device__ __forceinline__ void st8(void* base, size_t off, int dt, const float (&v)[8]) {
  if (dt == DN_BF16) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + off) = umma::pack8(v);
  else {
    float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off);
    d[0] = make_float4(v[0], v[1], v[2], v[3]);
    d[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

struct ProducerArgs {
  const void* mixed;             // (B,L,D)
  const float* w;                // (D,W) depthwise taps; tap W-1 multiplies the current token
  const float* bias;             // (D) or null
  const int32_t* seg;            // (B,L) or null: taps from another document read as zero
  int B, L, D, W, dt;
  int qk_dim, Hk_K;              // Hk*K: channels [0,HkK) -> q, [HkK, 2HkK) -> k, rest -> v
  void *q, *k, *v;               // forward outputs / backward: their cotangents
  void* d_mixed;                 // backward
  float* part;                   // backward: (tiles, D, W+1) partial sums of d w | d bias
};

// sigmoid by one MUFU op (tanh.approx, relative error ~2^-11): used where the result is rounded to bf16 anyway
__device__ __forceinline__ float sigmoid_fast(float x) {
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.5f * x));
  return fmaf(0.5f, t, 0.5f);
}
template <bool FAST> __device__ __forceinline__ float silu_t(float x) {
  if (FAST) return x * sigmoid_fast(x);
  return silu(x);
}
template <bool FAST> __device__ __forceinline__ float dsilu_t(float x) {
  if (FAST) { const float sg = sigmoid_fast(x); return sg * (1.f + x * (1.f - sg)); }
  return dsilu(x);
}

// One row of CG (4 or 8) channels as it was loaded (conversion to fp32 happens when the row is used, so a
// batch of loads can be issued back to back without holding CG floats per row).
template <bool BF16, int CG_> struct Raw;
template <> struct Raw<true, 8> {
  uint4 r;
  __device__ __forceinline__ void load(const void* base, size_t off) {
    r = __ldg(reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(base) + off));
  }
  __device__ __forceinline__ void get(float (&x)[8]) const { umma::unpack8(r, x); }
};
template <> struct Raw<false, 8> {
  float4 a, b;
  __device__ __forceinline__ void load(const void* base, size_t off) {
    const float4* p = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    a = __ldg(p); b = __ldg(p + 1);
  }
  __device__ __forceinline__ void get(float (&x)[8]) const {
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
  }
};
template <> struct Raw<true, 4> {
  uint2 r;
  __device__ __forceinline__ void load(const void* base, size_t off) {
    r = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + off));
  }
  __device__ __forceinline__ void get(float (&x)[4]) const {
    x[0] = __uint_as_float(r.x << 16); x[1] = __uint_as_float(r.x & 0xffff0000u);
    x[2] = __uint_as_float(r.y << 16); x[3] = __uint_as_float(r.y & 0xffff0000u);
  }
};
template <> struct Raw<false, 4> {
  float4 a;
  __device__ __forceinline__ void load(const void* base, size_t off) {
    a = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off));
  }
  __device__ __forceinline__ void get(float (&x)[4]) const { x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; }
};
template <> struct Raw<true, 2> {
  uint32_t r;
  __device__ __forceinline__ void load(const void* base, size_t off) {
    r = __ldg(reinterpret_cast<const uint32_t*>(reinterpret_cast<const __nv_bfloat16*>(base) + off));
  }
  __device__ __forceinline__ void get(float (&x)[2]) const { x[0] = __uint_as_float(r << 16); x[1] = __uint_as_float(r & 0xffff0000u); }
};
template <> struct Raw<false, 2> {
  float2 a;
  __device__ __forceinline__ void load(const void* base, size_t off) {
    a = __ldg(reinterpret_cast<const float2*>(reinterpret_cast<const float*>(base) + off));
  }
  __device__ __forceinline__ void get(float (&x)[2]) const { x[0] = a.x; x[1] = a.y; }
};
template <bool BF16> __device__ __forceinline__ void st4(void* base, size_t off, const float (&v)[4]) {
  if (BF16) *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(base) + off) = make_uint2(umma::pack2(v[0], v[1]), umma::pack2(v[2], v[3]));
  else *reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off) = make_float4(v[0], v[1], v[2], v[3]);
}

// The token loops below keep a ring of NS batches of NB rows in shared memory, filled by asynchronous
// copies (cp.async) that cost no registers: while batch i is walked with the stencil window in registers,
// the rows of batches i+1 .. i+NS-1 are on their way (12 rows of 16 or 32 bytes per thread).  A thread
// reads back only the slots it filled itself, so the ring needs no block-wide synchronisation.
template <int BYTES> __device__ __forceinline__ void cp_async_row(void* dst, const void* src);
template <> __device__ __forceinline__ void cp_async_row<16>(void* dst, const void* src) { umma::cp_async16(dst, src); }
template <> __device__ __forceinline__ void cp_async_row<8>(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(umma::smem_u32(dst)), "l"(src) : "memory");
}
// CGN channels of one row from the ring: PIECE bytes per copy, pieces of one row PT * PIECE bytes apart
template <bool BF16, int CGN> __device__ __forceinline__ void ring_get(const uint8_t* slot, float (&x)[CGN]);
template <> __device__ __forceinline__ void ring_get<true, 8>(const uint8_t* slot, float (&x)[8]) {
  umma::unpack8(*reinterpret_cast<const uint4*>(slot), x);
}
template <> __device__ __forceinline__ void ring_get<false, 8>(const uint8_t* slot, float (&x)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(slot), b = *reinterpret_cast<const float4*>(slot + PT * 16);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w; x[4] = b.x; x[5] = b.y; x[6] = b.z; x[7] = b.w;
}
template <> __device__ __forceinline__ void ring_get<true, 4>(const uint8_t* slot, float (&x)[4]) {
  const uint2 r = *reinterpret_cast<const uint2*>(slot);
  x[0] = __uint_as_float(r.x << 16); x[1] = __uint_as_float(r.x & 0xffff0000u);
  x[2] = __uint_as_float(r.y << 16); x[3] = __uint_as_float(r.y & 0xffff0000u);
}
template <> __device__ __forceinline__ void ring_get<false, 4>(const uint8_t* slot, float (&x)[4]) {
  const float4 a = *reinterpret_cast<const float4*>(slot);
  x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
}

template <int W, bool BF16>
__global__ void __launch_bounds__(PT, 4) producer_fwd_kernel(ProducerArgs a) {
  constexpr int NB = 4, NS = BF16 ? 4 : 2;           // rows per batch, batches in the ring (32 KB either way)
  constexpr int ES = BF16 ? 2 : 4, NP = CG * ES / 16;  // element size; 16-byte copies per row and thread
  __shared__ __align__(16) uint8_t ring[NS * NB * NP * PT * 16];
  __shared__ int seg_sm[TT_FWD + MAXW];              // document ids of rows t0-(W-1) .. t_end-1 (-1 before the sequence)
  const int tid = threadIdx.x;
  const bool active = (blockIdx.y * PT + tid) * CG < a.D;
  const int c0 = active ? (blockIdx.y * PT + tid) * CG : 0;
  const int tiles_per_row = (a.L + TT_FWD - 1) / TT_FWD;
  const int b = blockIdx.x / tiles_per_row, t0 = (blockIdx.x % tiles_per_row) * TT_FWD;
  const size_t row0 = (size_t)b * a.L;
  const int t_end = min(t0 + TT_FWD, a.L);
  const int nbatch = (t_end - t0 + NB - 1) / NB;
  const char* src = reinterpret_cast<const char*>(a.mixed);
  auto fetch = [&](int bi) {                           // rows past the end read the last row and are not stored
    if (bi < nbatch) {
#pragma unroll
      for (int n = 0; n < NB; ++n) {
        const int t = min(t0 + bi * NB + n, a.L - 1);
        const char* g = src + ((row0 + t) * a.D + c0) * ES;
        uint8_t* d = ring + ((size_t)(((bi % NS) * NB + n) * NP) * PT + tid) * 16;
#pragma unroll
        for (int h = 0; h < NP; ++h) umma::cp_async16(d + h * PT * 16, g + h * 16);
      }
    }
    umma::cp_async_commit();
  };
#pragma unroll
  for (int bi = 0; bi < NS - 1; ++bi) fetch(bi);
  for (int i = tid; i < TT_FWD + W - 1; i += PT) {
    const int t = t0 - (W - 1) + i;
    seg_sm[i] = t < 0 ? -1 : (a.seg ? __ldg(a.seg + row0 + min(t, a.L - 1)) : 0);
  }
  float wt[MAXW][CG], bs[CG];
#pragma unroll
  for (int j = 0; j < MAXW; ++j)
#pragma unroll
    for (int i = 0; i < CG; ++i) wt[j][i] = j < W ? __ldg(a.w + (size_t)(c0 + i) * W + j) : 0.f;
#pragma unroll
  for (int i = 0; i < CG; ++i) bs[i] = a.bias ? __ldg(a.bias + c0 + i) : 0.f;
  // window: xw[j] = x[t - (W-1) + j], j = 0..W-1 (tap j)
  float xw[MAXW][CG];
  int sw[MAXW];
#pragma unroll
  for (int j = 0; j < MAXW; ++j) {
    sw[j] = -1;
#pragma unroll
    for (int i = 0; i < CG; ++i) xw[j][i] = 0.f;
  }
  __syncthreads();
#pragma unroll
  for (int h = W - 1; h >= 1; --h) {                 // halo rows t0-h
    const int t = t0 - h, j = W - 1 - h;
    if (t >= 0) {
      Raw<BF16, CG> r;
      r.load(a.mixed, (row0 + t) * a.D + c0);
      r.get(xw[j]);
      sw[j] = seg_sm[j];
    }
  }
  const int HkK = a.Hk_K, Dv = a.D - 2 * HkK;
  // where this thread's channels go: q, k or v, each token-major
  char* obase; size_t ostride, ooff;
  if (c0 < HkK) { obase = (char*)a.q; ostride = HkK; ooff = c0; }
  else if (c0 < 2 * HkK) { obase = (char*)a.k; ostride = HkK; ooff = c0 - HkK; }
  else { obase = (char*)a.v; ostride = Dv; ooff = c0 - 2 * HkK; }
#pragma unroll 1
  for (int bi = 0; bi < nbatch; ++bi) {
    fetch(bi + NS - 1);
    umma::cp_async_wait<NS - 1>();
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      const int t = t0 + bi * NB + n;
      ring_get<BF16, CG>(ring + ((size_t)(((bi % NS) * NB + n) * NP) * PT + tid) * 16, xw[W - 1]);
      const int s = seg_sm[bi * NB + n + W - 1];
      sw[W - 1] = s;
      float y[CG];
#pragma unroll
      for (int i = 0; i < CG; ++i) y[i] = bs[i];
#pragma unroll
      for (int j = 0; j < MAXW; ++j) {
        if (j < W && sw[j] == s) {
#pragma unroll
          for (int i = 0; i < CG; ++i) y[i] = fmaf(wt[j][i], xw[j][i], y[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < CG; ++i) y[i] = silu_t<BF16>(y[i]);
      if (active && t < t_end) st8(obase, (row0 + t) * ostride + ooff, BF16 ? DN_BF16 : DN_F32, y);
#pragma unroll
      for (int j = 0; j + 1 < MAXW; ++j) {
        if (j + 1 < W) {
          sw[j] = sw[j + 1];
#pragma unroll
          for (int i = 0; i < CG; ++i) xw[j][i] = xw[j + 1][i];
        }
      }
    }
  }
  umma::cp_async_wait<0>();
}

// Backward of the producer over one run of TT_BWD tokens: with pre[u] the conv output of token u and
// dpre[u] = dy[u] * silu'(pre[u]),
//   d x[s]    = sum_j w[j] * dpre[s + (W-1-j)]      (taps inside the same document)
//   d w[j]   += dpre[u] * x[u - (W-1) + j],   d bias += dpre[u]    (u inside this run)
// The loop walks u over the run plus W-1 rows of look-ahead and emits d x with a lag of W-1.  A thread
// owns CB = 4 channels here (the windows of x and dpre and the parameter-gradient accumulators are
// 10 CB + registers), so that twice as many threads are resident as with 8.
constexpr int CB = 4;
template <int W, bool BF16>
__global__ void __launch_bounds__(PT, 4) producer_bwd_kernel(ProducerArgs a) {
  constexpr int NB = 4, NS = BF16 ? 4 : 2;
  constexpr int ES = BF16 ? 2 : 4, RB = CB * ES;     // bytes per row, thread and tensor: 8 or 16
  __shared__ __align__(16) uint8_t ring[NS * NB * 2 * PT * RB];       // x rows | cotangent rows
  __shared__ int seg_sm[TT_BWD + 2 * MAXW];          // document ids of rows t0-(W-1) .. u_end-1 (-1 / -2 outside the sequence)
  const int tid = threadIdx.x;
  const bool active = (blockIdx.y * PT + tid) * CB < a.D;
  const int c0 = active ? (blockIdx.y * PT + tid) * CB : 0;
  const int tiles_per_row = (a.L + TT_BWD - 1) / TT_BWD;
  const int b = blockIdx.x / tiles_per_row, t0 = (blockIdx.x % tiles_per_row) * TT_BWD;
  const size_t row0 = (size_t)b * a.L;
  const int t_end = min(t0 + TT_BWD, a.L);
  const int u_end = t_end + W - 1;                   // look-ahead rows; rows >= L contribute nothing
  const int nbatch = (u_end - t0 + NB - 1) / NB;
  const int HkK = a.Hk_K, Dv = a.D - 2 * HkK;
  const char* gbase; size_t gstride, goff;           // this thread's channels of the cotangent of q, k or v
  if (c0 < HkK) { gbase = (const char*)a.q; gstride = HkK; goff = c0; }
  else if (c0 < 2 * HkK) { gbase = (const char*)a.k; gstride = HkK; goff = c0 - HkK; }
  else { gbase = (const char*)a.v; gstride = Dv; goff = c0 - 2 * HkK; }
  const char* xsrc = reinterpret_cast<const char*>(a.mixed);
  auto fetch = [&](int bi) {                         // rows past the end read the last row and count as not live
    if (bi < nbatch) {
#pragma unroll
      for (int n = 0; n < NB; ++n) {
        const int u = min(t0 + bi * NB + n, a.L - 1);
        uint8_t* d = ring + ((size_t)(((bi % NS) * NB + n) * 2) * PT + tid) * RB;
        cp_async_row<RB>(d, xsrc + ((row0 + u) * a.D + c0) * ES);
        cp_async_row<RB>(d + PT * RB, gbase + ((row0 + u) * gstride + goff) * ES);
      }
    }
    umma::cp_async_commit();
  };
#pragma unroll
  for (int bi = 0; bi < NS - 1; ++bi) fetch(bi);
  for (int i = tid; i < TT_BWD + 2 * MAXW; i += PT) {
    const int t = t0 - (W - 1) + i;
    seg_sm[i] = t < 0 ? -1 : (t >= a.L ? -2 : (a.seg ? __ldg(a.seg + row0 + t) : 0));
  }
  float wt[MAXW][CB], bs[CB], dwt[MAXW][CB], dbs[CB];
#pragma unroll
  for (int j = 0; j < MAXW; ++j)
#pragma unroll
    for (int i = 0; i < CB; ++i) { wt[j][i] = j < W ? __ldg(a.w + (size_t)(c0 + i) * W + j) : 0.f; dwt[j][i] = 0.f; }
#pragma unroll
  for (int i = 0; i < CB; ++i) { bs[i] = a.bias ? __ldg(a.bias + c0 + i) : 0.f; dbs[i] = 0.f; }
  float xw[MAXW][CB], dp[MAXW][CB];      // xw[j] = x[u-(W-1)+j]; dp[j] = dpre[u-(W-1)+j]
  int sw[MAXW];
#pragma unroll
  for (int j = 0; j < MAXW; ++j) {
    sw[j] = -1;
#pragma unroll
    for (int i = 0; i < CB; ++i) { xw[j][i] = 0.f; dp[j][i] = 0.f; }
  }
  __syncthreads();
#pragma unroll
  for (int h = W - 1; h >= 1; --h) {
    const int t = t0 - h, j = W - 1 - h;
    if (t >= 0) {
      Raw<BF16, CB> r;
      r.load(a.mixed, (row0 + t) * a.D + c0);
      r.get(xw[j]);
      sw[j] = seg_sm[j];
    }
  }
#pragma unroll 1
  for (int bi = 0; bi < nbatch; ++bi) {
    fetch(bi + NS - 1);
    umma::cp_async_wait<NS - 1>();
#pragma unroll
    for (int n = 0; n < NB; ++n) {
      const int u = t0 + bi * NB + n;
      const bool live = u < a.L;
      float dy[CB];
      const uint8_t* slot = ring + ((size_t)(((bi % NS) * NB + n) * 2) * PT + tid) * RB;
      ring_get<BF16, CB>(slot, xw[W - 1]);
      ring_get<BF16, CB>(slot + PT * RB, dy);
      const int s = seg_sm[bi * NB + n + W - 1];     // -2 past the end of the sequence: matches no tap
      sw[W - 1] = s;
      float pre[CB];
#pragma unroll
      for (int i = 0; i < CB; ++i) pre[i] = bs[i];
#pragma unroll
      for (int j = 0; j < MAXW; ++j) {
        if (j < W && sw[j] == s) {
#pragma unroll
          for (int i = 0; i < CB; ++i) pre[i] = fmaf(wt[j][i], xw[j][i], pre[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < CB; ++i) dp[W - 1][i] = live ? dy[i] * dsilu_t<BF16>(pre[i]) : 0.f;
      if (u < t_end) {                               // parameter gradients of the rows this run owns
#pragma unroll
        for (int j = 0; j < MAXW; ++j) {
          if (j < W && sw[j] == s) {
#pragma unroll
            for (int i = 0; i < CB; ++i) dwt[j][i] = fmaf(dp[W - 1][i], xw[j][i], dwt[j][i]);
          }
        }
#pragma unroll
        for (int i = 0; i < CB; ++i) dbs[i] += dp[W - 1][i];
      }
      // d x of token sx = u - (W-1): output token sx + (W-1-j) used it through tap j; that token sits at window slot W-1-j
      const int sx = u - (W - 1);
      if (sx >= t0 && sx < t_end) {
        float dx[CB];
#pragma unroll
        for (int i = 0; i < CB; ++i) dx[i] = 0.f;
        const int s0 = sw[0];                        // document of token sx (slot 0 of the window)
#pragma unroll
        for (int j = 0; j < MAXW; ++j) {
          if (j < W && sw[W - 1 - j] == s0) {
#pragma unroll
            for (int i = 0; i < CB; ++i) dx[i] = fmaf(wt[j][i], dp[W - 1 - j][i], dx[i]);
          }
        }
        if (active) st4<BF16>(a.d_mixed, (row0 + sx) * a.D + c0, dx);
      }
#pragma unroll
      for (int j = 0; j + 1 < MAXW; ++j) {
        if (j + 1 < W) {
          sw[j] = sw[j + 1];
#pragma unroll
          for (int i = 0; i < CB; ++i) { xw[j][i] = xw[j + 1][i]; dp[j][i] = dp[j + 1][i]; }
        }
      }
    }
  }
  umma::cp_async_wait<0>();
  if (!active) return;
  float* p = a.part + ((size_t)blockIdx.x * a.D + c0) * (W + 1);
#pragma unroll
  for (int i = 0; i < CB; ++i) {
#pragma unroll
    for (int j = 0; j < MAXW; ++j)
      if (j < W) p[i * (W + 1) + j] = dwt[j][i];
    p[i * (W + 1) + W] = dbs[i];
  }
}

// out[e] = sum over tiles of part[tile][e] in a fixed order: a CTA takes 32 elements; each of its 8 warps
// adds one eighth of the tiles in ascending order (independent loads, several in flight), and the eight
// partial sums are added in ascending order.
__global__ void __launch_bounds__(256) tile_sum_kernel(const float* part, int tiles, size_t n, float* out_a, float* out_b,
                                                       int W) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, grp = threadIdx.x >> 5;
  const size_t e = (size_t)blockIdx.x * 32 + lane;
  const int per = (tiles + 7) / 8, tb = grp * per, te = min(tb + per, tiles);
  float s = 0.f;
  if (e < n) {
    int t = tb;
    for (; t + 8 <= te; t += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = __ldg(part + (size_t)(t + u) * n + e);
#pragma unroll
      for (int u = 0; u < 8; ++u) s += v[u];
    }
    for (; t < te; ++t) s += __ldg(part + (size_t)t * n + e);
  }
  red[grp][lane] = s;
  __syncthreads();
  if (grp != 0 || e >= n) return;
  s = red[0][lane];
#pragma unroll
  for (int k = 1; k < 8; ++k) s += red[k][lane];
  if (W < 0) { out_a[e] = s; return; }
  const size_t c = e / (W + 1);
  const int j = (int)(e - c * (W + 1));
  if (j < W) out_a[c * W + j] = s;
  else if (out_b) out_b[c] = s;
}

// ---- gates ------------------------------------------------------------------------------------------
__device__ __forceinline__ float softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

__global__ void __launch_bounds__(256) gates_fwd_kernel(const void* a_, const void* b_, int dt, const float* A_log,
                                                        const float* dt_bias, size_t n, int Hv, float* g, float* beta) {
  const size_t e = (size_t)blockIdx.x * 256 + threadIdx.x;
  if (e >= n) return;
  const int h = (int)(e % Hv);
  g[e] = -expf(A_log[h]) * softplus(ldf_ro(a_, e, dt) + dt_bias[h]);
  beta[e] = 1.f / (1.f + expf(-ldf_ro(b_, e, dt)));
}

// da, db element-wise; dA_log[h] = sum dg * g, d dt_bias[h] = sum dg * dg/d(a): one CTA per head, fixed order
__global__ void __launch_bounds__(256) gates_bwd_kernel(const void* a_, const void* b_, int dt, const float* A_log,
                                                        const float* dt_bias, const float* dg, const float* dbeta,
                                                        size_t tokens, int Hv, void* da, void* db, float* dA_log,
                                                        float* d_dt_bias) {
  const int h = blockIdx.x;
  const float Ae = -expf(A_log[h]), bias = dt_bias[h];
  float sA = 0.f, sB = 0.f;
  for (size_t t = threadIdx.x; t < tokens; t += 256) {
    const size_t e = t * Hv + h;
    const float x = ldf_ro(a_, e, dt) + bias;
    const float sp = softplus(x), sg = 1.f / (1.f + expf(-x));
    const float d = dg[e];
    const float dx = d * Ae * sg;
    stf(da, e, dx, dt);
    const float be = 1.f / (1.f + expf(-ldf_ro(b_, e, dt)));
    stf(db, e, dbeta[e] * be * (1.f - be), dt);
    sA += d * Ae * sp;
    sB += dx;
  }
  __shared__ float red[2][256];
  red[0][threadIdx.x] = sA; red[1][threadIdx.x] = sB;
  __syncthreads();
  for (int o = 128; o > 0; o >>= 1) {
    if (threadIdx.x < o) { red[0][threadIdx.x] += red[0][threadIdx.x + o]; red[1][threadIdx.x] += red[1][threadIdx.x + o]; }
    __syncthreads();
  }
  if (threadIdx.x == 0) { dA_log[h] = red[0][0]; d_dt_bias[h] = red[1][0]; }
}

// ---- gated RMSNorm -----------------------------------------------------------------------------------
// One warp per row of V (64 or 128) elements, EPL = V / 32 per lane.  The normalised value is rounded to
// the input dtype before the weight is applied, as the layer this mirrors does.
template <int EPL>
__device__ __forceinline__ void ld_row(const void* base, size_t off, int dt, float (&x)[EPL]) {
  if (dt == DN_BF16) {
    const __nv_bfloat16* p = reinterpret_cast<const __nv_bfloat16*>(base) + off;
    if (EPL == 4) {
      const uint2 u = __ldg(reinterpret_cast<const uint2*>(p));
      x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xffff0000u);
      x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xffff0000u);
    } else {
      const uint32_t u = __ldg(reinterpret_cast<const uint32_t*>(p));
      x[0] = __uint_as_float(u << 16); x[1] = __uint_as_float(u & 0xffff0000u);
    }
  } else {
    const float* p = reinterpret_cast<const float*>(base) + off;
    if (EPL == 4) { const float4 u = __ldg(reinterpret_cast<const float4*>(p)); x[0] = u.x; x[1] = u.y; x[2] = u.z; x[3] = u.w; }
    else { const float2 u = __ldg(reinterpret_cast<const float2*>(p)); x[0] = u.x; x[1] = u.y; }
  }
}
template <int EPL>
__device__ __forceinline__ void st_row(void* base, size_t off, int dt, const float (&x)[EPL]) {
  if (dt == DN_BF16) {
    __nv_bfloat16* p = reinterpret_cast<__nv_bfloat16*>(base) + off;
    if (EPL == 4) *reinterpret_cast<uint2*>(p) = make_uint2(umma::pack2(x[0], x[1]), umma::pack2(x[2], x[3]));
    else *reinterpret_cast<uint32_t*>(p) = umma::pack2(x[0], x[1]);
  } else {
    float* p = reinterpret_cast<float*>(base) + off;
    if (EPL == 4) *reinterpret_cast<float4*>(p) = make_float4(x[0], x[1], x[2], x[3]);
    else *reinterpret_cast<float2*>(p) = make_float2(x[0], x[1]);
  }
}

// A warp takes NR rows per batch with two sets of registers: the rows of batch i + 1 are requested
// before batch i is worked on (rows past the end read the last row and are not stored), so 2 NR
// (forward) or 3 NR (backward) loads per lane are always in flight.
template <int EPL, bool BF16>
__global__ void __launch_bounds__(256) gated_rmsnorm_fwd_kernel(const void* o, const void* z, const float* weight,
                                                                size_t rows, float eps, void* y, float* rstd) {
  constexpr int V = EPL * 32, NR = 4, dt = BF16 ? DN_BF16 : DN_F32;
  const int lane = threadIdx.x & 31;
  float w[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) w[i] = __ldg(weight + lane * EPL + i);
  const size_t stride = (size_t)gridDim.x * 8;
  const size_t rbeg = (size_t)blockIdx.x * 8 + (threadIdx.x >> 5);
  Raw<BF16, EPL> rx[2][NR], rz[2][NR];
  auto fetch = [&](size_t r0, int slot) {
#pragma unroll
    for (int u = 0; u < NR; ++u) {
      const size_t r = min(r0 + u * stride, rows - 1);
      rx[slot][u].load(o, r * V + lane * EPL);
      rz[slot][u].load(z, r * V + lane * EPL);
    }
  };
  if (rbeg < rows) fetch(rbeg, 0);
  int slot = 0;
#pragma unroll 2
  for (size_t r0 = rbeg; r0 < rows; r0 += stride * NR, slot ^= 1) {
    if (r0 + stride * NR < rows) fetch(r0 + stride * NR, slot ^ 1);
#pragma unroll
    for (int u = 0; u < NR; ++u) {
      const size_t r = r0 + u * stride;
      float x[EPL], zz[EPL], out[EPL];
      rx[slot][u].get(x);
      rz[slot][u].get(zz);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) ss = fmaf(x[i], x[i], ss);
      ss = warp_sum(ss);
      const float rs = rsqrtf(ss * (1.f / V) + eps);
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        float n = x[i] * rs;
        if (BF16) n = bf16r(n);
        out[i] = w[i] * n * silu_t<BF16>(zz[i]);
      }
      if (r < rows) {
        st_row<EPL>(y, r * V + lane * EPL, dt, out);
        if (rstd && lane == 0) rstd[r] = rs;
      }
    }
  }
}

template <int EPL, bool BF16>
__global__ void __launch_bounds__(256) gated_rmsnorm_bwd_kernel(const void* o, const void* z, const float* weight,
                                                                size_t rows, float eps, const void* dy, void* d_o, void* d_z,
                                                                float* part) {
  constexpr int V = EPL * 32, NR = 2, dt = BF16 ? DN_BF16 : DN_F32;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  float w[EPL], dwp[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) { w[i] = __ldg(weight + lane * EPL + i); dwp[i] = 0.f; }
  const size_t stride = (size_t)gridDim.x * 8;
  const size_t rbeg = (size_t)blockIdx.x * 8 + warp;
  Raw<BF16, EPL> rx[2][NR], rz[2][NR], rg[2][NR];
  auto fetch = [&](size_t r0, int slot) {
#pragma unroll
    for (int u = 0; u < NR; ++u) {
      const size_t r = min(r0 + u * stride, rows - 1);
      rx[slot][u].load(o, r * V + lane * EPL);
      rz[slot][u].load(z, r * V + lane * EPL);
      rg[slot][u].load(dy, r * V + lane * EPL);
    }
  };
  if (rbeg < rows) fetch(rbeg, 0);
  int slot = 0;
#pragma unroll 2
  for (size_t r0 = rbeg; r0 < rows; r0 += stride * NR, slot ^= 1) {
    if (r0 + stride * NR < rows) fetch(r0 + stride * NR, slot ^ 1);
#pragma unroll
    for (int u = 0; u < NR; ++u) {                   // rows in ascending order: the weight gradient's order of addition is fixed
      const size_t r = r0 + u * stride;
      if (r >= rows) break;
      float x[EPL], zz[EPL], g[EPL], dn_[EPL], n[EPL], dzo[EPL], dxo[EPL];
      rx[slot][u].get(x);
      rz[slot][u].get(zz);
      rg[slot][u].get(g);
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) ss = fmaf(x[i], x[i], ss);
      ss = warp_sum(ss);
      const float rs = rsqrtf(ss * (1.f / V) + eps);
      float dot = 0.f;
#pragma unroll
      for (int i = 0; i < EPL; ++i) {
        n[i] = x[i] * rs;
        const float nr = BF16 ? bf16r(n[i]) : n[i];
        const float sg = BF16 ? sigmoid_fast(zz[i]) : __frcp_rn(1.f + __expf(-zz[i]));
        const float sl = zz[i] * sg;
        dzo[i] = g[i] * w[i] * nr * (sg * (1.f + zz[i] * (1.f - sg)));
        dn_[i] = g[i] * w[i] * sl;
        dwp[i] = fmaf(g[i] * nr, sl, dwp[i]);
        dot = fmaf(dn_[i], n[i], dot);
      }
      dot = warp_sum(dot) * (1.f / V);
#pragma unroll
      for (int i = 0; i < EPL; ++i) dxo[i] = rs * (dn_[i] - n[i] * dot);
      st_row<EPL>(d_o, r * V + lane * EPL, dt, dxo);
      st_row<EPL>(d_z, r * V + lane * EPL, dt, dzo);
    }
  }
  __shared__ float red[8][V];
#pragma unroll
  for (int i = 0; i < EPL; ++i) red[warp][lane * EPL + i] = dwp[i];
  __syncthreads();
  for (int c = threadIdx.x; c < V; c += 256) {
    float sacc = 0.f;
#pragma unroll
    for (int k = 0; k < 8; ++k) sacc += red[k][c];
    part[(size_t)blockIdx.x * V + c] = sacc;
  }
}

// CTAs of 8 warps that walk the rows with a grid stride: as many as are resident at once (per_sm per SM,
// from the occupancy of the kernel instance; 8 is the upper bound the scratch is sized for)
int norm_grid(size_t rows, int per_sm = 8) {
  const size_t want = (rows + 7) / 8, cap = (size_t)sm_count() * (per_sm < 1 ? 1 : (per_sm > 8 ? 8 : per_sm));
  return (int)(want < cap ? (want ? want : 1) : cap);
}
template <typename KernelT> int resident_ctas(KernelT kernel) {
  int n = 0;
  if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, 256, 0) != cudaSuccess) { cudaGetLastError(); n = 4; }
  return n;
}

}  // namespace
}  // namespace dn

using namespace dn;

extern "C" {

size_t dn_gdn_producer_scratch_bytes(int32_t B, int32_t L, int32_t D, int32_t W) {
  if (B < 1 || L < 1 || D < 1 || W < 2 || W > 4) return 0;
  const size_t tiles = (size_t)B * ((L + TT_BWD - 1) / TT_BWD);
  return tiles * D * (W + 1) * sizeof(float);
}

static int producer_args(ProducerArgs& a, const void* mixed, const float* conv_w, const float* conv_b, const int32_t* seg,
                         int32_t B, int32_t L, int32_t Hk, int32_t Hv, int32_t K, int32_t V, int32_t W, int32_t dtype) {
  if (!mixed || !conv_w) return DN_ERR_NULL_POINTER;
  if (B < 1 || L < 1 || Hk < 1 || Hv < 1 || (K != 64 && K != 128) || (V != 64 && V != 128) || W < 2 || W > MAXW) return DN_ERR_BAD_SHAPE;
  if (dtype != DN_F32 && dtype != DN_BF16) return DN_ERR_BAD_DTYPE;
  a.mixed = mixed; a.w = conv_w; a.bias = conv_b; a.seg = seg;
  a.B = B; a.L = L; a.D = 2 * Hk * K + Hv * V; a.W = W; a.dt = dtype; a.Hk_K = Hk * K; a.qk_dim = K;
  return DN_OK;
}

int dn_gdn_producer_fwd(const void* mixed, const float* conv_w, const float* conv_b, const int32_t* seg,
                        int32_t B, int32_t L, int32_t Hk, int32_t Hv, int32_t K, int32_t V, int32_t W, int32_t dtype,
                        void* q, void* k, void* v, void* stream) {
  ProducerArgs a{};
  int rc = producer_args(a, mixed, conv_w, conv_b, seg, B, L, Hk, Hv, K, V, W, dtype);
  if (rc) return rc;
  if (!q || !k || !v) return DN_ERR_NULL_POINTER;
  a.q = q; a.k = k; a.v = v;
  dim3 grid(B * ((L + TT_FWD - 1) / TT_FWD), (a.D / CG + PT - 1) / PT);
  cudaStream_t st = (cudaStream_t)stream;
  const bool bf = dtype == DN_BF16;
#define DN_GO(WW) (bf ? producer_fwd_kernel<WW, true><<<grid, PT, 0, st>>>(a) : producer_fwd_kernel<WW, false><<<grid, PT, 0, st>>>(a))
  if (W == 4) DN_GO(4); else if (W == 3) DN_GO(3); else DN_GO(2);
#undef DN_GO
  return launch_status();
}

int dn_gdn_producer_bwd(const void* mixed, const float* conv_w, const float* conv_b, const int32_t* seg,
                        int32_t B, int32_t L, int32_t Hk, int32_t Hv, int32_t K, int32_t V, int32_t W, int32_t dtype,
                        const void* dq, const void* dk, const void* dv, void* d_mixed, float* d_conv_w, float* d_conv_b,
                        void* scratch, size_t scratch_bytes, void* stream) {
  ProducerArgs a{};
  int rc = producer_args(a, mixed, conv_w, conv_b, seg, B, L, Hk, Hv, K, V, W, dtype);
  if (rc) return rc;
  if (!dq || !dk || !dv || !d_mixed || !d_conv_w || !scratch) return DN_ERR_NULL_POINTER;
  if (scratch_bytes < dn_gdn_producer_scratch_bytes(B, L, a.D, W)) return DN_ERR_SCRATCH_TOO_SMALL;
  a.q = const_cast<void*>(dq); a.k = const_cast<void*>(dk); a.v = const_cast<void*>(dv);
  a.d_mixed = d_mixed; a.part = reinterpret_cast<float*>(scratch);
  const int tiles = B * ((L + TT_BWD - 1) / TT_BWD);
  dim3 grid(tiles, (a.D / CB + PT - 1) / PT);
  cudaStream_t st = (cudaStream_t)stream;
  const bool bf = dtype == DN_BF16;
#define DN_GO(WW) (bf ? producer_bwd_kernel<WW, true><<<grid, PT, 0, st>>>(a) : producer_bwd_kernel<WW, false><<<grid, PT, 0, st>>>(a))
  if (W == 4) DN_GO(4); else if (W == 3) DN_GO(3); else DN_GO(2);
#undef DN_GO
  if ((rc = launch_status())) return rc;
  const size_t n = (size_t)a.D * (W + 1);
  tile_sum_kernel<<<(unsigned)((n + 31) / 32), 256, 0, st>>>(a.part, tiles, n, d_conv_w, d_conv_b, W);
  return launch_status();
}

int dn_gdn_gates_fwd(const void* a, const void* b, const float* A_log, const float* dt_bias, int32_t B, int32_t L,
                     int32_t Hv, int32_t dtype, float* g, float* beta, void* stream) {
  if (!a || !b || !A_log || !dt_bias || !g || !beta) return DN_ERR_NULL_POINTER;
  if (B < 1 || L < 1 || Hv < 1) return DN_ERR_BAD_SHAPE;
  if (dtype != DN_F32 && dtype != DN_BF16) return DN_ERR_BAD_DTYPE;
  const size_t n = (size_t)B * L * Hv;
  gates_fwd_kernel<<<(unsigned)((n + 255) / 256), 256, 0, (cudaStream_t)stream>>>(a, b, dtype, A_log, dt_bias, n, Hv, g, beta);
  return launch_status();
}

int dn_gdn_gates_bwd(const void* a, const void* b, const float* A_log, const float* dt_bias, const float* dg,
                     const float* dbeta, int32_t B, int32_t L, int32_t Hv, int32_t dtype, void* da, void* db,
                     float* dA_log, float* d_dt_bias, void* stream) {
  if (!a || !b || !A_log || !dt_bias || !dg || !dbeta || !da || !db || !dA_log || !d_dt_bias) return DN_ERR_NULL_POINTER;
  if (B < 1 || L < 1 || Hv < 1) return DN_ERR_BAD_SHAPE;
  if (dtype != DN_F32 && dtype != DN_BF16) return DN_ERR_BAD_DTYPE;
  gates_bwd_kernel<<<Hv, 256, 0, (cudaStream_t)stream>>>(a, b, dtype, A_log, dt_bias, dg, dbeta, (size_t)B * L, Hv, da, db,
                                                         dA_log, d_dt_bias);
  return launch_status();
}

size_t dn_gated_rmsnorm_scratch_bytes(int64_t rows, int32_t V) {
  if (rows < 1 || V < 1) return 0;
  return (size_t)norm_grid((size_t)rows) * V * sizeof(float);
}

int dn_gated_rmsnorm_fwd(const void* o, const void* z, const float* weight, int64_t rows, int32_t V, int32_t dtype,
                         float eps, void* y, void* stream) {
  if (!o || !z || !weight || !y) return DN_ERR_NULL_POINTER;
  if (rows < 1 || (V != 64 && V != 128)) return DN_ERR_BAD_SHAPE;
  if (dtype != DN_F32 && dtype != DN_BF16) return DN_ERR_BAD_DTYPE;
  cudaStream_t st = (cudaStream_t)stream;
  auto go = [&](auto kernel) {
    const int grid = norm_grid((size_t)rows, resident_ctas(kernel));
    kernel<<<grid, 256, 0, st>>>(o, z, weight, (size_t)rows, eps, y, nullptr);
  };
  if (dtype == DN_BF16) { if (V == 128) go(gated_rmsnorm_fwd_kernel<4, true>); else go(gated_rmsnorm_fwd_kernel<2, true>); }
  else { if (V == 128) go(gated_rmsnorm_fwd_kernel<4, false>); else go(gated_rmsnorm_fwd_kernel<2, false>); }
  return launch_status();
}

int dn_gated_rmsnorm_bwd(const void* o, const void* z, const float* weight, int64_t rows, int32_t V, int32_t dtype,
                         float eps, const void* dy, void* d_o, void* d_z, float* d_weight, void* scratch,
                         size_t scratch_bytes, void* stream) {
  if (!o || !z || !weight || !dy || !d_o || !d_z || !d_weight || !scratch) return DN_ERR_NULL_POINTER;
  if (rows < 1 || (V != 64 && V != 128)) return DN_ERR_BAD_SHAPE;
  if (dtype != DN_F32 && dtype != DN_BF16) return DN_ERR_BAD_DTYPE;
  if (scratch_bytes < dn_gated_rmsnorm_scratch_bytes(rows, V)) return DN_ERR_SCRATCH_TOO_SMALL;
  cudaStream_t st = (cudaStream_t)stream;
  float* part = reinterpret_cast<float*>(scratch);
  int grid = 0;
  auto go = [&](auto kernel) {
    grid = norm_grid((size_t)rows, resident_ctas(kernel));
    kernel<<<grid, 256, 0, st>>>(o, z, weight, (size_t)rows, eps, dy, d_o, d_z, part);
  };
  if (dtype == DN_BF16) { if (V == 128) go(gated_rmsnorm_bwd_kernel<4, true>); else go(gated_rmsnorm_bwd_kernel<2, true>); }
  else { if (V == 128) go(gated_rmsnorm_bwd_kernel<4, false>); else go(gated_rmsnorm_bwd_kernel<2, false>); }
  int rc = launch_status();
  if (rc) return rc;
  tile_sum_kernel<<<(unsigned)((V + 31) / 32), 256, 0, st>>>(part, grid, (size_t)V, d_weight, nullptr, -1);
  return launch_status();
}

}  // extern "C"
