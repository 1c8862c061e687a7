// Single-token decode step: streams the (B,Hv,K,V) state through registers exactly once.
//
// Math (src/deltanet_tpu/gdn2.py:2471-2478 of the reference), per sequence and value head:
//     Sd = diag(exp g) S ;  e = Sd^T (b*k) ;  v_new = w*v - e ;  S' = Sd + k v_new^T ;  o = S'^T q
// o uses the un-rounded S'; S' is then cast to the output state dtype (gdn2.py:2478-2489).
//
// The update is independent per value column, so one CTA owns a K x 64 column slab of one
// (sequence, value head): every thread loads its share with 16-byte vector loads issued
// back to back, the two reductions over K go through shared memory, and the slab is written
// back with 16-byte stores.  Bytes moved = state read once + state written once.
#include "dn_kernels.cuh"

namespace dn {

constexpr int DV = 64;                 // value columns per CTA
constexpr int DEC_THREADS = 256;

template <typename T> struct Vec16;    // 16-byte vector of state elements
template <> struct Vec16<float> { static constexpr int N = 4; };
template <> struct Vec16<__nv_bfloat16> { static constexpr int N = 8; };

template <typename T>
__device__ __forceinline__ void load16(const T* p, float (&x)[Vec16<T>::N]);
template <>
__device__ __forceinline__ void load16<float>(const float* p, float (&x)[4]) {
  float4 v = __ldcs(reinterpret_cast<const float4*>(p));
  x[0] = v.x; x[1] = v.y; x[2] = v.z; x[3] = v.w;
}
template <>
__device__ __forceinline__ void load16<__nv_bfloat16>(const __nv_bfloat16* p, float (&x)[8]) {
  uint4 v = __ldcs(reinterpret_cast<const uint4*>(p));
  const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    x[2 * i] = __uint_as_float(u[i] << 16);
    x[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
  }
}
template <int N>
__device__ __forceinline__ void store_row(float* p, const float (&x)[N]) {
#pragma unroll
  for (int i = 0; i < N; i += 4) __stcs(reinterpret_cast<float4*>(p + i), make_float4(x[i], x[i + 1], x[i + 2], x[i + 3]));
}
template <int N>
__device__ __forceinline__ void store_row(__nv_bfloat16* p, const float (&x)[N]) {
  static_assert(N % 8 == 0 || N == 4, "row width");
  if (N == 4) {
    __nv_bfloat162 a = __floats2bfloat162_rn(x[0], x[1]), b = __floats2bfloat162_rn(x[2], x[3]);
    uint2 v = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
    __stcs(reinterpret_cast<uint2*>(p), v);
  } else {
#pragma unroll
    for (int i = 0; i < N; i += 8) {
      uint32_t u[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        __nv_bfloat162 h = __floats2bfloat162_rn(x[i + 2 * j], x[i + 2 * j + 1]);
        u[j] = *reinterpret_cast<uint32_t*>(&h);
      }
      __stcs(reinterpret_cast<uint4*>(p + i), make_uint4(u[0], u[1], u[2], u[3]));
    }
  }
}

struct DecodeArgs {
  dn_decode_shape s;
  const void *q, *k, *v, *g, *b, *w;
  const void* state_in;
  const uint8_t* reset;
  void* out;
  void* state_out;
};

__device__ __forceinline__ int dec_gate_head(int hv, int nheads, int Hk, int Hv) {
  if (nheads == 1) return 0;
  if (nheads == Hv) return hv;
  return hv / (Hv / Hk);
}

template <typename SI, typename SO, int KD, int DVT = DV, int NTH = DEC_THREADS>
__global__ void __launch_bounds__(NTH) decode_kernel(DecodeArgs a) {
  constexpr int CPT = Vec16<SI>::N;        // columns per thread
  constexpr int VC = DVT / CPT;             // vector columns per row slab
  constexpr int RG = NTH / VC;     // row groups
  constexpr int R = KD / RG;               // rows per thread
  const dn_decode_shape& s = a.s;
  const int V = s.V;
  const int nslab = V / DVT;
  const int slab = blockIdx.x % nslab, hv = (blockIdx.x / nslab) % s.Hv, b = blockIdx.x / (nslab * s.Hv);
  const int tid = threadIdx.x, vc = tid % VC, rg = tid / VC;
  const int col0 = slab * DVT + vc * CPT;

  __shared__ float qs[KD], ks[KD], dec[KD], beta[KD];
  __shared__ float red[RG][DVT + 4];
  __shared__ float vnew[DVT], wvs[DVT], nrm[2];

  // ---- state loads first: they are the long-latency part
  const size_t sbase = ((size_t)b * s.Hv + hv) * KD * V;
  const SI* Sin = reinterpret_cast<const SI*>(a.state_in) + sbase;
  const bool zero = a.reset && a.reset[(s.flags & DN_RESET_PER_HEAD) ? b * s.Hv + hv : b];
  float S[R][CPT];
#pragma unroll
  for (int r = 0; r < R; ++r) {
    if (zero) {
#pragma unroll
      for (int c = 0; c < CPT; ++c) S[r][c] = 0.f;
    } else {
      load16<SI>(Sin + (size_t)(rg + r * RG) * V + col0, S[r]);
    }
  }

  // ---- token vectors
  const int G = s.Hv / s.Hk, hk = hv / G;
  const bool guard = s.flags & DN_STABILITY_GUARD;
  if (tid < 64) {
    // two warps: warp 0 normalises q, warp 1 normalises k
    const int wq = tid >> 5, lane = tid & 31;
    const void* src = wq == 0 ? a.q : a.k;
    float x[KD / 32], ss = 0.f;
#pragma unroll
    for (int u = 0; u < KD / 32; ++u) {
      x[u] = ldf(src, ((size_t)b * s.Hk + hk) * KD + lane + 32 * u, s.qkv_dtype);
      ss += x[u] * x[u];
    }
    ss = warp_sum(ss);
    float r = 1.f;
    if (s.flags & DN_QK_L2NORM) r = 1.f / sqrtf(ss + 1e-6f);
#pragma unroll
    for (int u = 0; u < KD / 32; ++u) {
      if (wq == 0) qs[lane + 32 * u] = x[u] * r * s.scale;
      else ks[lane + 32 * u] = x[u] * r;
    }
  } else if (tid < 64 + DVT) {
    const int j = tid - 64, cv = slab * DVT + j;
    const float vv = ldf(a.v, ((size_t)b * s.Hv + hv) * V + cv, s.qkv_dtype);
    const int hw = dec_gate_head(hv, s.w_heads, s.Hk, s.Hv);
    const float ww = ldf(a.w, ((size_t)b * s.w_heads + hw) * s.w_cols + (s.w_cols == 1 ? 0 : cv), s.gate_dtype);
    wvs[j] = ww * vv;
  }
  __syncthreads();
  if (tid < KD) {
    const int hg = dec_gate_head(hv, s.g_heads, s.Hk, s.Hv), hb = dec_gate_head(hv, s.b_heads, s.Hk, s.Hv);
    float gg = ldf(a.g, ((size_t)b * s.g_heads + hg) * s.g_cols + (s.g_cols == 1 ? 0 : tid), s.gate_dtype);
    float bb = ldf(a.b, ((size_t)b * s.b_heads + hb) * s.b_cols + (s.b_cols == 1 ? 0 : tid), s.gate_dtype);
    gg = fminf(gg, 0.f);
    if (guard) { bb = fmaxf(bb, 0.f); gg = fminf(gg, -1e-6f); }
    dec[tid] = expf(gg);
    beta[tid] = bb * ks[tid];
  }
  __syncthreads();

  // ---- decay, erase projection e = Sd^T beta
  float part[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) part[c] = 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int kk = rg + r * RG;
    const float d = dec[kk], be = beta[kk];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      S[r][c] *= d;
      part[c] = fmaf(be, S[r][c], part[c]);
    }
  }
#pragma unroll
  for (int c = 0; c < CPT; ++c) red[rg][vc * CPT + c] = part[c];
  __syncthreads();
  if (tid < DVT) {
    float e = 0.f;
#pragma unroll
    for (int r = 0; r < RG; ++r) e += red[r][tid];
    vnew[tid] = wvs[tid] - e;
  }
  __syncthreads();
  // ---- rank-one write, output projection o = S'^T q
  float vn[CPT];
#pragma unroll
  for (int c = 0; c < CPT; ++c) { vn[c] = vnew[vc * CPT + c]; part[c] = 0.f; }
  float sq = 0.f;
#pragma unroll
  for (int r = 0; r < R; ++r) {
    const int kk = rg + r * RG;
    const float kx = ks[kk], qx = qs[kk];
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
      S[r][c] = fmaf(kx, vn[c], S[r][c]);
      part[c] = fmaf(qx, S[r][c], part[c]);
      sq = fmaf(S[r][c], S[r][c], sq);
    }
  }
  __syncthreads();                     // red is reused
#pragma unroll
  for (int c = 0; c < CPT; ++c) red[rg][vc * CPT + c] = part[c];
  __syncthreads();
  if (tid < DVT) {
    float o = 0.f;
#pragma unroll
    for (int r = 0; r < RG; ++r) o += red[r][tid];
    stf(a.out, ((size_t)b * s.Hv + hv) * V + slab * DVT + tid, o, s.qkv_dtype);
  }
  (void)sq; (void)nrm;
  // ---- state out
  SO* Sout = reinterpret_cast<SO*>(a.state_out) + sbase;
#pragma unroll
  for (int r = 0; r < R; ++r) store_row<CPT>(Sout + (size_t)(rg + r * RG) * V + col0, S[r]);
}

// ---------------------------------------------------------------------------------------------
// Bulk-copy pipeline for the common serving case: K = V = 128, state in and out in one dtype, bf16 q/k/v,
// fp32 gates, each either per channel or one scalar per head.  The (128,128) state of one (sequence, value head) is 32 KB (bf16) or 64 KB (fp32)
// of contiguous global memory, so it moves with ONE bulk asynchronous copy each way
// (cp.async.bulk, completion on an mbarrier / a bulk group); the token vectors ride on the same
// barrier.  A persistent CTA keeps a ring of STAGES tiles: while tile i is updated in place in
// shared memory, tiles i+1 .. i+STAGES-1 are in flight and tile i-1 drains to global memory.  No
// register ever holds a byte that is waiting for memory, which is what limited the slab kernel.
// Every barrier wait is bounded; a wait that gives up sets the library's error word and the CTA
// stops taking tiles.
namespace bulk {

constexpr int NT = 256, STAGES = 3, KD = 128, VD = 128;
// one stage of the ring: the state tile (SB bytes per element), then q, k, v (bf16) and g, b, w (fp32)
template <int SB>
struct Stage {
  static constexpr int TILE = KD * VD * SB;
  static constexpr int OFF_Q = TILE, OFF_K = OFF_Q + 256, OFF_V = OFF_K + 256, OFF_G = OFF_V + 256,
                       OFF_B = OFF_G + 512, OFF_W = OFF_B + 512, BYTES = OFF_W + 512;   // 35072 / 67840, multiples of 128
};
constexpr uint32_t SPIN = 1u << 22;

__device__ __forceinline__ uint32_t s32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void bar_init(uint64_t* b, uint32_t n) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(s32(b)), "r"(n) : "memory");
}
__device__ __forceinline__ void bar_expect(uint64_t* b, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(b)), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool bar_wait(uint64_t* b, uint32_t parity) {
  for (uint32_t it = 0; it < SPIN; ++it) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(s32(b)), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* b) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(s32(dst)), "l"(src), "r"(bytes), "r"(s32(b)) : "memory");
}
__device__ __forceinline__ void bulk_store(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(s32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void fence_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// SB: bytes per state element, 2 (bf16, two CTAs per SM) or 4 (fp32, one).  SC: some gate is one scalar per
// head (the all-per-channel instance carries none of that code).
template <int SB, bool SC>
__global__ void __launch_bounds__(NT, SB == 2 ? 2 : 1) decode_bulk_kernel(DecodeArgs a, int tiles, int* err) {
  using LY = Stage<SB>;
  constexpr int TILE = LY::TILE, OFF_Q = LY::OFF_Q, OFF_K = LY::OFF_K, OFF_V = LY::OFF_V, OFF_G = LY::OFF_G,
                OFF_B = LY::OFF_B, OFF_W = LY::OFF_W, STAGE_BYTES = LY::BYTES;
  extern __shared__ __align__(128) uint8_t ring[];
  __shared__ __align__(8) uint64_t full[STAGES];
  __shared__ float qs[KD], ks[KD], dec[KD], beta[KD], wv[VD], vnew[VD];
  __shared__ float red[NT / 32][VD];
  __shared__ int dead_s;
  const dn_decode_shape& s = a.s;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int G = s.Hv / s.Hk;
  const bool l2 = s.flags & DN_QK_L2NORM, guard = s.flags & DN_STABILITY_GUARD;

  // a gate that is one scalar per head cannot travel as a bulk copy (16 bytes at least): it comes by a
  // 4-byte cp.async of the issuing thread, one committed group per issued tile
  const bool gs = SC && s.g_cols == 1, bs = SC && s.b_cols == 1, ws = SC && s.w_cols == 1;
  constexpr bool any_scalar = SC;
  const uint32_t tx_bytes = TILE + 3 * 256 + (gs ? 0 : 512) + (bs ? 0 : 512) + (ws ? 0 : 512);
  auto gate = [&](uint8_t* dst, const void* base, int b, int heads, int hv, bool scalar, uint64_t* bar) {
    const float* src = reinterpret_cast<const float*>(base) + ((size_t)b * heads + dec_gate_head(hv, heads, s.Hk, s.Hv)) * (scalar ? 1 : KD);
    if (scalar) asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s32(dst)), "l"(src) : "memory");
    else bulk_load(dst, src, 512, bar);
  };
  auto issue = [&](int tile, int st) {               // one thread: the tile's state and token vectors
    const int hv = tile % s.Hv, b = tile / s.Hv, hk = hv / G;
    uint8_t* dst = ring + (size_t)st * STAGE_BYTES;
    bar_expect(&full[st], tx_bytes);
    bulk_load(dst, reinterpret_cast<const uint8_t*>(a.state_in) + (size_t)tile * TILE, TILE, &full[st]);
    bulk_load(dst + OFF_Q, reinterpret_cast<const __nv_bfloat16*>(a.q) + ((size_t)b * s.Hk + hk) * KD, 256, &full[st]);
    bulk_load(dst + OFF_K, reinterpret_cast<const __nv_bfloat16*>(a.k) + ((size_t)b * s.Hk + hk) * KD, 256, &full[st]);
    bulk_load(dst + OFF_V, reinterpret_cast<const __nv_bfloat16*>(a.v) + ((size_t)b * s.Hv + hv) * VD, 256, &full[st]);
    gate(dst + OFF_G, a.g, b, s.g_heads, hv, gs, &full[st]);
    gate(dst + OFF_B, a.b, b, s.b_heads, hv, bs, &full[st]);
    gate(dst + OFF_W, a.w, b, s.w_heads, hv, ws, &full[st]);
  };
  // (a group is committed whether or not a tile was issued, so that the count below stays in step)
  auto commit_scalars = [&]() { if (any_scalar) asm volatile("cp.async.commit_group;" ::: "memory"); };

  if (tid == 0) {
    for (int i = 0; i < STAGES; ++i) bar_init(&full[i], 1);
    dead_s = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  // everything above touched shared memory only; what follows reads what earlier kernels of the stream wrote
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // the next launch of the stream may take the places of this grid's CTAs as they leave (all of them are resident)
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
  const int first = blockIdx.x, stride = gridDim.x;
  if (tid == NT - 1)
    for (int i = 0; i < STAGES - 1; ++i) {
      if (first + i * stride < tiles) issue(first + i * stride, i);
      commit_scalars();
    }

  const int vc = tid & 15, rg = tid >> 4;              // 8 columns, rows rg + 16 r
  int it = 0;
  for (int tile = first; tile < tiles; tile += stride, ++it) {
    const int st = it % STAGES;
    const uint32_t parity = (uint32_t)(it / STAGES) & 1u;
    if (!bar_wait(&full[st], parity)) { dead_s = 1; report_timeout(err); }
    // STAGES - 1 + it groups are committed by now and this tile's is number it: all but the newest STAGES - 2
    if (any_scalar && tid == NT - 1) asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
    __syncthreads();
    if (dead_s) break;
    uint8_t* buf = ring + (size_t)st * STAGE_BYTES;
    const int hv = tile % s.Hv, b = tile / s.Hv;
    const bool zero = a.reset && a.reset[(s.flags & DN_RESET_PER_HEAD) ? b * s.Hv + hv : b];

    // ---- token vectors in one phase: warps 0..3 take k (every warp computes the norm for itself),
    //      the decay and beta = b * k_hat; warps 4..7 take q and w * v
    {
      const bool kside = tid < 128;
      const int j = tid & 127;
      const __nv_bfloat16* src = reinterpret_cast<const __nv_bfloat16*>(buf + (kside ? OFF_K : OFF_Q));
      float ss = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) { const float x = __bfloat162float(src[lane + 32 * u]); ss += x * x; }
      ss = warp_sum(ss);
      const float r = l2 ? 1.f / sqrtf(ss + 1e-6f) : 1.f;
      const float mine = __bfloat162float(src[j]) * r;
      if (kside) {
        float gg = fminf(reinterpret_cast<const float*>(buf + OFF_G)[gs ? 0 : j], 0.f), bb = reinterpret_cast<const float*>(buf + OFF_B)[bs ? 0 : j];
        if (guard) { bb = fmaxf(bb, 0.f); gg = fminf(gg, -1e-6f); }
        ks[j] = mine;
        dec[j] = expf(gg);
        beta[j] = bb * mine;
      } else {
        qs[j] = mine * s.scale;
        wv[j] = reinterpret_cast<const float*>(buf + OFF_W)[ws ? 0 : j] * __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(buf + OFF_V)[j]);
      }
    }
    // refill the stage that tile it-1 used: its store (issued a while ago) must have finished reading
    // shared memory
    if (tid == NT - 1) {
      bulk_wait_read<0>();
      const int nxt = tile + (STAGES - 1) * stride;
      if (nxt < tiles) issue(nxt, (it + STAGES - 1) % STAGES);
      commit_scalars();
    }
    __syncthreads();

    // ---- decay, erase projection e = Sd^T beta
    uint4* tile4 = reinterpret_cast<uint4*>(buf);          // row kk: 16 (bf16) or 32 (fp32) vectors; a thread owns 8 columns
    float S[8][8], part[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) part[c] = 0.f;
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int kk = rg + 16 * r;
      const float d = dec[kk], be = beta[kk];
      if (SB == 2) {
        const uint4 v = tile4[kk * 16 + vc];
        const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {                        // a reset sequence starts from zeros whatever the buffer holds
          S[r][2 * j] = zero ? 0.f : __uint_as_float(u[j] << 16) * d;
          S[r][2 * j + 1] = zero ? 0.f : __uint_as_float(u[j] & 0xffff0000u) * d;
        }
      } else {
        const uint4 v0 = tile4[kk * 32 + 2 * vc], v1 = tile4[kk * 32 + 2 * vc + 1];
        const uint32_t u[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
#pragma unroll
        for (int j = 0; j < 8; ++j) S[r][j] = zero ? 0.f : __uint_as_float(u[j]) * d;
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) part[c] = fmaf(be, S[r][c], part[c]);
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], 16);    // the warp's two row groups
    if (lane < 16) {
#pragma unroll
      for (int c = 0; c < 8; ++c) red[warp][8 * vc + c] = part[c];
    }
    __syncthreads();
    if (tid < VD) {
      float e = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < NT / 32; ++w8) e += red[w8][tid];
      vnew[tid] = wv[tid] - e;
    }
    __syncthreads();
    // ---- rank-one write, output projection o = S'^T q, new state back into the tile
    float vn[8];
#pragma unroll
    for (int c = 0; c < 8; ++c) { vn[c] = vnew[8 * vc + c]; part[c] = 0.f; }
#pragma unroll
    for (int r = 0; r < 8; ++r) {
      const int kk = rg + 16 * r;
      const float kx = ks[kk], qx = qs[kk];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        S[r][c] = fmaf(kx, vn[c], S[r][c]);
        part[c] = fmaf(qx, S[r][c], part[c]);
      }
      if (SB == 2) {
        uint32_t u[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          __nv_bfloat162 h2 = __floats2bfloat162_rn(S[r][2 * j], S[r][2 * j + 1]);
          u[j] = *reinterpret_cast<uint32_t*>(&h2);
        }
        tile4[kk * 16 + vc] = make_uint4(u[0], u[1], u[2], u[3]);
      } else {
        tile4[kk * 32 + 2 * vc] = make_uint4(__float_as_uint(S[r][0]), __float_as_uint(S[r][1]), __float_as_uint(S[r][2]), __float_as_uint(S[r][3]));
        tile4[kk * 32 + 2 * vc + 1] = make_uint4(__float_as_uint(S[r][4]), __float_as_uint(S[r][5]), __float_as_uint(S[r][6]), __float_as_uint(S[r][7]));
      }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) part[c] += __shfl_xor_sync(0xffffffffu, part[c], 16);
    if (lane < 16) {
#pragma unroll
      for (int c = 0; c < 8; ++c) red[warp][8 * vc + c] = part[c];
    }
    fence_async();                                           // the tile was written through the generic proxy
    __syncthreads();
    if (tid == NT - 1) {                                     // the thread that also waits on the bulk groups
      bulk_store(reinterpret_cast<uint8_t*>(a.state_out) + (size_t)tile * TILE, buf, TILE);
      bulk_commit();
    }
    if (tid < VD) {
      float o = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < NT / 32; ++w8) o += red[w8][tid];
      reinterpret_cast<__nv_bfloat16*>(a.out)[((size_t)b * s.Hv + hv) * VD + tid] = __float2bfloat16_rn(o);
    }
    // the next tile's first barrier orders these reads of red / vnew before they are rewritten
  }
  if (tid == NT - 1) {
    asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
    if (any_scalar) asm volatile("cp.async.wait_all;" ::: "memory");
  }
}

inline bool eligible(const DecodeArgs& a) {
  const dn_decode_shape& s = a.s;
  if (s.K != KD || s.V != VD) return false;
  if (s.state_in_dtype != s.state_out_dtype || s.qkv_dtype != DN_BF16 || s.gate_dtype != DN_F32) return false;
  if ((s.g_cols != KD && s.g_cols != 1) || (s.b_cols != KD && s.b_cols != 1) || (s.w_cols != VD && s.w_cols != 1)) return false;
  const void* ptrs[] = {a.q, a.k, a.v, a.g, a.b, a.w, a.state_in, a.state_out};
  for (const void* p : ptrs)
    if (reinterpret_cast<uintptr_t>(p) & 15) return false;
  return true;
}

}  // namespace bulk

// Frobenius cap of the returned state (gdn2.py:2484-2487): one CTA per (sequence, value head).
template <typename SO>
__global__ void __launch_bounds__(256) decode_cap_kernel(SO* state, int KV, float tau) {
  SO* p = state + (size_t)blockIdx.x * KV;
  __shared__ float wsum[8];
  float s = 0.f;
  for (int e = threadIdx.x; e < KV; e += 256) { float x = (float)p[e]; s += x * x; }
  s = warp_sum(s);
  if ((threadIdx.x & 31) == 0) wsum[threadIdx.x >> 5] = s;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) tot += wsum[i];
  const float f = fminf(1.f, tau / sqrtf(tot + 1e-6f));
  if (f < 1.f)
    for (int e = threadIdx.x; e < KV; e += 256) p[e] = (SO)((float)p[e] * f);
}

template <typename SI, typename SO>
static int launch_decode_t(const DecodeArgs& a, cudaStream_t st) {
  const dn_decode_shape& s = a.s;
  const int grid = s.B * s.Hv * (s.V / DV);
  if (s.K == 128) decode_kernel<SI, SO, 128><<<grid, DEC_THREADS, 0, st>>>(a);
  else decode_kernel<SI, SO, 64><<<grid, DEC_THREADS, 0, st>>>(a);
  if (launch_status()) return DN_ERR_CUDA_LAUNCH;
  if (s.flags & DN_STABILITY_GUARD) {
    decode_cap_kernel<SO><<<s.B * s.Hv, 256, 0, st>>>(reinterpret_cast<SO*>(a.state_out), s.K * s.V, s.stability_tau);
    if (launch_status()) return DN_ERR_CUDA_LAUNCH;
  }
  return DN_OK;
}

int launch_cap_state(float* state, int64_t n_states, int KV, float tau, cudaStream_t st) {
  decode_cap_kernel<float><<<(unsigned)n_states, 256, 0, st>>>(state, KV, tau);
  return launch_status();
}

int launch_decode(const dn_decode_shape& s, const void* q, const void* k, const void* v,
                  const void* g, const void* b, const void* w, const void* state_in,
                  const uint8_t* reset, void* out, void* state_out, cudaStream_t st) {
  DecodeArgs a{s, q, k, v, g, b, w, state_in, reset, out, state_out};
  if (bulk::eligible(a) && !force_simt()) {
    const int tiles = s.B * s.Hv;
    const bool sb16 = s.state_in_dtype == DN_BF16;
    const bool sc = s.g_cols == 1 || s.b_cols == 1 || s.w_cols == 1;
    const int slots = (sb16 ? 2 : 1) * sm_count();
    const int grid = tiles < slots ? tiles : slots;
    const size_t smem = (size_t)bulk::STAGES * (sb16 ? bulk::Stage<2>::BYTES : bulk::Stage<4>::BYTES);
    // Programmatic dependent launch: the CTAs of this launch may become resident while the kernel before it
    // in the stream is still finishing (a decode loop is a chain of short launches of this kernel); they set
    // up their barriers and then wait, inside the kernel, for that kernel to have completed before they touch
    // global memory.
    auto go = [&](auto kern) {
      cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaLaunchConfig_t cfg{};
      cfg.gridDim = dim3((unsigned)grid); cfg.blockDim = dim3(bulk::NT); cfg.dynamicSmemBytes = smem; cfg.stream = st;
      cudaLaunchAttribute attr[1];
      attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
      attr[0].val.programmaticStreamSerializationAllowed = 1;
      cfg.attrs = attr; cfg.numAttrs = 1;
      cudaLaunchKernelEx(&cfg, kern, a, tiles, device_error_ptr());
    };
    if (sb16) { if (sc) go(bulk::decode_bulk_kernel<2, true>); else go(bulk::decode_bulk_kernel<2, false>); }
    else      { if (sc) go(bulk::decode_bulk_kernel<4, true>); else go(bulk::decode_bulk_kernel<4, false>); }
    if (launch_status()) return DN_ERR_CUDA_LAUNCH;
    if (s.flags & DN_STABILITY_GUARD) {
      if (sb16) decode_cap_kernel<__nv_bfloat16><<<s.B * s.Hv, 256, 0, st>>>(reinterpret_cast<__nv_bfloat16*>(a.state_out), s.K * s.V, s.stability_tau);
      else decode_cap_kernel<float><<<s.B * s.Hv, 256, 0, st>>>(reinterpret_cast<float*>(a.state_out), s.K * s.V, s.stability_tau);
      if (launch_status()) return DN_ERR_CUDA_LAUNCH;
    }
    return DN_OK;
  }
  const bool ib = s.state_in_dtype == DN_BF16, ob = s.state_out_dtype == DN_BF16;
  if (ib && ob) return launch_decode_t<__nv_bfloat16, __nv_bfloat16>(a, st);
  if (ib && !ob) return launch_decode_t<__nv_bfloat16, float>(a, st);
  if (!ib && ob) return launch_decode_t<float, __nv_bfloat16>(a, st);
  return launch_decode_t<float, float>(a, st);
}

}  // namespace dn
