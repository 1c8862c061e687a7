// Prepass forward on the tcgen05 tensor cores (bf16 precision, chunk = K = 128, value width
// 128 or 256).  Produces the same outputs as the fp32 formulation in dn_prepass_fwd.cu
// (reference body: src/deltanet_tpu/gdn2.py:115-240), with the bf16 tiles W, U, M, qe, ke written
// as tensor-core operand images ([col / 8][row][8], see Geo::img).
//
// A and M.  A_ij = sum_c beta_ic exp(Lam_ic - Lam_jc) k_jc cannot in general be one matrix product
// because the decay couples i, j and the channel c.  Two cases reduce to plain products and are taken
// when they apply: one scalar decay per (token, head), where exp(lam_i - lam_j) is applied entry-wise
// to the Gram products beta k k^T and q k^T while they drain; and channel-wise decay that stays
// within e^{+-32} of each document's midpoint over the chunk (tested per chunk on the device),
// where with f = exp(Lam - midpoint) the images k / f, q f, beta k f give A and M by one product
// each.  Otherwise it is built hierarchically: at level s in {16,32,64}
// the chunk is cut into pairs of adjacent s-row blocks, and for a pair with rows I (lower block),
// columns J (upper block) and reference row r = first row of I
//     A[I,J] = (beta_I * exp(Lam_I - Lam_r)) (k_J * exp(Lam_r - Lam_J))^T ,
// with both scale factors <= 1 (the cumulative decay is monotone inside a document), so nothing
// can overflow however strong the decay.  In one level every row is either a row of its pair
// (lower block) or a column (upper block), so two images suffice: KR holds the beta-images on lower
// rows and the k-images on upper rows, QK the q-images and the k-images, and
//     level part of A = KR KR^T,   level part of M = QK KR^T       (one 128^3 MMA each);
// entries outside the level's blocks are finite garbage that the drain ignores (entry (i,j) belongs
// to the level of the highest bit in which i>>4 and j>>4 differ).  A level's drain shares a barrier
// interval with the next level's image build (the images are free once the level's products have
// completed).  The 16x16 diagonal blocks are evaluated exactly, pair by pair, on the CUDA cores;
// when k_hat and q_hat are exactly bf16 this pass runs first and parks k_hat | q_hat (two bf16 per
// column) and beta in tensor memory, from where the qe / ke / X pass and all level images are built
// without touching global memory again.  The reference does the same with 32-row blocks and one
// reference per block row (gdn2.py:162-197).
//
// T = (I+A)^-1 is obtained as in the fp32 formulation (substitution on 16x16 blocks + block
// merges, fp32 in shared memory); W = T X and U = T Y are tcgen05 MMAs on bf16 operands, which
// is also where the reference rounds to bf16 (gdn2.py:226-230).
//
// 512 threads per CTA, one CTA per SM, looping over (batch, exec head, chunk) items.  Phases that
// read the operator's row-major tensors let a warp cover 8 rows x 4 pieces of 8 channels (row =
// 8 * warp + (lane & 7) fixed per thread) with every load issued unconditionally; phases that drain
// tensor memory own one row per thread, which the image layout of the outputs (and the panel
// layout [col / 4][row][4] of the fp32 scratch that carries A to the inverse) turns into stores of
// 512 contiguous bytes per warp.
#ifdef DN_PHASE_TIMING
#include <cstdio>
#endif
#include "dn_chunkprep.cuh"
#include "dn_kernels.cuh"

namespace dn {
namespace {

using namespace prep;
constexpr int NT = 512;
constexpr int AP = 132;                              // row pitch (floats) of A, T in shared memory
constexpr int OFF_IMG = C * LP * 4;                  // level images / k cache / A start after Lambda
constexpr int OFF_TM = OFF_IMG + C * AP * 4;         // merge scratch (16 KB)
constexpr int OFF_XI = 160 * 1024;                   // X image: survives the inverse
constexpr int OFF_TI = 192 * 1024;                   // T image
constexpr int SMEM_BYTES = 224 * 1024;
static_assert(OFF_TM + 16384 <= OFF_XI, "merge scratch below the X image");
static_assert(OFF_IMG + 2 * 32768 <= OFF_XI, "level images below the X image");

__device__ __forceinline__ int p4v(int row, int col) { return ((col >> 2) << 7) + row; }
__device__ __forceinline__ int p4f(int row, int col) { return ((((col >> 2) << 7) + row) << 2) + (col & 3); }

// One merge level of the inverse: for every pair of adjacent S-row blocks (lower rows I, upper rows J)
//   T[I,J] = -T[I,I] (A[I,J] T[J,J]).
// 512 threads = (row pair of I) x (16 column groups of S/16 columns) x pairs; a thread owns a
// 2 x (S/16) tile of outputs, so one step of the contraction costs two scalar loads and one
// vector load from shared memory for 2 * S/16 multiply-adds.
template <int S>
__device__ __forceinline__ void merge_level(const float* As, float* Ts, float* Tm) {
  constexpr int NJ = S / 16;
  const int cg = threadIdx.x & 15, rest = threadIdx.x >> 4;     // rest = pair * (S/2) + row pair in I
  const int p = rest / (S / 2), il = 2 * (rest - p * (S / 2));
  const int i = 2 * p * S + S + il, j0 = 2 * p * S + cg * NJ, m0 = 2 * p * S;
  float acc0[NJ], acc1[NJ];
#pragma unroll
  for (int u = 0; u < NJ; ++u) acc0[u] = acc1[u] = 0.f;
#pragma unroll 4
  for (int m = 0; m < S; ++m) {
    const float a0 = As[i * AP + m0 + m], a1 = As[(i + 1) * AP + m0 + m];
    const float* t = Ts + (m0 + m) * AP + j0;
#pragma unroll
    for (int u = 0; u < NJ; ++u) { acc0[u] = fmaf(a0, t[u], acc0[u]); acc1[u] = fmaf(a1, t[u], acc1[u]); }
  }
#pragma unroll
  for (int u = 0; u < NJ; ++u) {
    Tm[(p * S + il) * S + cg * NJ + u] = acc0[u];
    Tm[(p * S + il + 1) * S + cg * NJ + u] = acc1[u];
  }
  __syncthreads();
#pragma unroll
  for (int u = 0; u < NJ; ++u) acc0[u] = acc1[u] = 0.f;
#pragma unroll 4
  for (int m = 0; m < S; ++m) {
    const float t0 = Ts[i * AP + m0 + S + m], t1 = Ts[(i + 1) * AP + m0 + S + m];
    const float* t = Tm + (p * S + m) * S + cg * NJ;
#pragma unroll
    for (int u = 0; u < NJ; ++u) { acc0[u] = fmaf(t0, t[u], acc0[u]); acc1[u] = fmaf(t1, t[u], acc1[u]); }
  }
#pragma unroll
  for (int u = 0; u < NJ; ++u) { Ts[i * AP + j0 + u] = -acc0[u]; Ts[(i + 1) * AP + j0 + u] = -acc1[u]; }
  __syncthreads();
}

template <int VW, int MODE>
__global__ void __launch_bounds__(NT, 1) prepass_fwd_tc_kernel(PrepassFwdArgs a, int* err) {
  using CF = InCfg<MODE>;
  extern __shared__ __align__(128) uint8_t smraw[];
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_base;
  __shared__ int seg_s[C];
  __shared__ int reset_s[4];
  __shared__ float rq_s[C], rk_s[C], bsc_s[C];
  __shared__ uint8_t ds_s[C], de_s[C];                  // first / last row of each row's document inside the chunk
  const Geo& g = a.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int myrow = warp * 8 + (lane & 7), lgrp = lane >> 3;
  float* LAM = reinterpret_cast<float*>(smraw);
  uint4* KR = reinterpret_cast<uint4*>(smraw + OFF_IMG);
  uint4* QK = KR + IMG;
  float* KHs = reinterpret_cast<float*>(smraw + OFF_IMG);          // k_hat cache (pitch AP), diagonal pass
  float* TOTL = reinterpret_cast<float*>(smraw + OFF_IMG);         // partial sums of the decay scan
  uint4* XI = reinterpret_cast<uint4*>(smraw + OFF_XI);
  float* Ts = reinterpret_cast<float*>(smraw);                     // inverse: T over Lambda,
  float* As = reinterpret_cast<float*>(smraw + OFF_IMG);           //          A over the images / cache
  float* Tm = reinterpret_cast<float*>(smraw + OFF_TM);
  uint4* TI = reinterpret_cast<uint4*>(smraw + OFF_TI);
  uint4* YI = reinterpret_cast<uint4*>(smraw + OFF_IMG);           // Y image over A, after the inverse

  float* Ag = a.scratch + (size_t)blockIdx.x * a.scratch_per_cta;     // A (fp32, masked), panel layout
  float4* Ag4 = reinterpret_cast<float4*>(Ag);

  if (tid == 0) { umma::mbar_init(&mma_bar, 1); umma::fence_mbar_init(); }
  if (warp == 0) umma::tmem_alloc(&tmem_base, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &mma_bar, 0u, err, false};

  const bool fuse = CF::fixed ? false : (g.flags & DN_FUSE_PROLOGUE) != 0;     // the fixed modes have no fused prologue
  // tensor-memory columns: level products at [0, 256); operand cache at [256, 384) (k_hat | q_hat, two
  // bf16 per column) and [384, 512) (beta, fp32)
  constexpr uint32_t COL_KQ = 256, COL_BE = 384;

  // work items in chunk-major order inside the chunk range: all heads of chunk c_begin first
  for (int e_item = blockIdx.x; e_item < a.items; e_item += gridDim.x) {
    const int bh = e_item % (g.B * g.H), c_idx = a.c_begin + e_item / (g.B * g.H);
    const int h = bh % g.H, b = bh / g.H;
    const int item = bh * g.NC + c_idx;
    const int t0 = c_idx * C;
    const size_t ibase = (size_t)item;
    uint4* Wimg = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.res.W) + ibase * C * K);
    uint4* Uimg = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.res.U) + ibase * C * VW);
    uint4* Mimg = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.res.M) + ibase * C * C);
    __nv_bfloat16* Mel = reinterpret_cast<__nv_bfloat16*>(a.res.M) + ibase * C * C;
    uint4* QEimg = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.res.qe) + ibase * C * K);
    uint4* KEimg = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.res.ke) + ibase * C * K);

    DN_MARK(0);
    for (int i = tid; i < C; i += NT) seg_s[i] = seg_at(a.seg, b, t0 + i, g.L);
    const Rows r = make_rows<CF>(g, a.q, a.k, a.gg, a.b, b, h, t0, rq_s, rk_s);
    const int qdt = r.qkv_dt, gdt = r.gate_dt;           // compile-time constants in the fixed modes
    const int wC = CF::fixed ? (CF::scalar_bw ? 1 : g.V) : g.wC;
    const bool tm_cache = r.round_in;                    // k_hat, q_hat exactly bf16: they can be packed two per column
    __syncthreads();
    const int seg0 = seg_s[0], segL = seg_s[C - 1];
    row_norms_8x4(r, myrow, lgrp, rq_s, rk_s);             // no barrier in between: the loads of q, k and g
    lambda_scan_512(r, seg_s, LAM, TOTL, reset_s);         // are all in flight together
    __syncthreads();

    // ---- 16x16 diagonal blocks, exact.  k_hat, q_hat and beta of 64 rows at a time are cached in
    //      shared memory (fp32; one global round trip per half); four warps per block take every
    //      fourth row i, lanes own 4 channels, and every pair (i, j <= i) is one warp reduction.
    const uint32_t tm_lane = cx.tmem + ((uint32_t)((warp & 3) * 32) << 16);
    auto diag_pass = [&]() {
#pragma unroll 1
    for (int half = 0; half < 2; ++half) {
      float* QHs = KHs + 64 * AP;                                       // q_hat (pitch AP)
      float* BEs = reinterpret_cast<float*>(smraw + OFF_TI);            // beta (pitch 128)
#pragma unroll
      for (int it = 0; it < 2; ++it) {
        const int w = it * 16 + warp, xr = (w & 7) * 8 + (lane & 7), p = (w >> 3) * 4 + lgrp, x = half * 64 + xr;
        float kh[8], qh[8], ba[8];
        khat8(r, x, p, kh);
        qhat8(r, x, p, qh);
        bact8(r, x, p, ba);
#pragma unroll
        for (int i = 0; i < 8; ++i) ba[i] *= kh[i];
        *reinterpret_cast<float4*>(KHs + xr * AP + 8 * p) = make_float4(kh[0], kh[1], kh[2], kh[3]);
        *reinterpret_cast<float4*>(KHs + xr * AP + 8 * p + 4) = make_float4(kh[4], kh[5], kh[6], kh[7]);
        *reinterpret_cast<float4*>(QHs + xr * AP + 8 * p) = make_float4(qh[0], qh[1], qh[2], qh[3]);
        *reinterpret_cast<float4*>(QHs + xr * AP + 8 * p + 4) = make_float4(qh[4], qh[5], qh[6], qh[7]);
        *reinterpret_cast<float4*>(BEs + xr * 128 + 8 * p) = make_float4(ba[0], ba[1], ba[2], ba[3]);
        *reinterpret_cast<float4*>(BEs + xr * 128 + 8 * p + 4) = make_float4(ba[4], ba[5], ba[6], ba[7]);
      }
      __syncthreads();
      DN_MARK(20 + 3 * half);
      if (tm_cache && ((warp & 3) >> 1) == half) {
        // every later pass (qe / ke / X, the three levels) reads k_hat, q_hat and beta from tensor
        // memory: thread = row (its own lane), the four warps of a lane quarter take 32 channels each
        const int xr = (warp & 3) * 32 + lane - 64 * half, cg0 = (warp >> 2) * 32;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int c0 = cg0 + 8 * j;
          float kq[8], be8[8];
          const float4 k0 = *reinterpret_cast<const float4*>(KHs + xr * AP + c0), k1 = *reinterpret_cast<const float4*>(KHs + xr * AP + c0 + 4);
          const float4 q0 = *reinterpret_cast<const float4*>(QHs + xr * AP + c0), q1 = *reinterpret_cast<const float4*>(QHs + xr * AP + c0 + 4);
          const float4 b0 = *reinterpret_cast<const float4*>(BEs + xr * 128 + c0), b1 = *reinterpret_cast<const float4*>(BEs + xr * 128 + c0 + 4);
          const float kk[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w}, qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i)                   // both are exactly representable in bf16 here
            kq[i] = __uint_as_float((__float_as_uint(kk[i]) >> 16) | (__float_as_uint(qq[i]) & 0xffff0000u));
          be8[0] = b0.x; be8[1] = b0.y; be8[2] = b0.z; be8[3] = b0.w; be8[4] = b1.x; be8[5] = b1.y; be8[6] = b1.z; be8[7] = b1.w;
          umma::tmem_st8(tm_lane + COL_KQ + c0, kq);
          umma::tmem_st8(tm_lane + COL_BE + c0, be8);
        }
        umma::tmem_wait_st();
      }
      const int lb = warp >> 2, r0 = (half * 4 + lb) * 16, c0 = lb * 16;   // block rows in the chunk / in the caches
#pragma unroll 1
      for (int i = warp & 3; i < 16; i += 4) {
        const int ri = r0 + i;
        const float4 q4 = *reinterpret_cast<const float4*>(QHs + (c0 + i) * AP + 4 * lane);
        const float4 b4 = *reinterpret_cast<const float4*>(BEs + (c0 + i) * 128 + 4 * lane);
        const float4 li = *reinterpret_cast<const float4*>(LAM + ri * LP + 4 * lane);
        const float qi[4] = {q4.x, q4.y, q4.z, q4.w}, bi4[4] = {b4.x, b4.y, b4.z, b4.w};
        float arow = 0.f, mrow = 0.f;                  // lane j (< 16) keeps entry (ri, r0 + j)
        const bool hi16 = lane & 16, hi8 = lane & 8, hi4 = lane & 4;
#pragma unroll 1
        for (int j = 0; j <= i; j += 4) {              // four columns per step, reduced together (see below)
          float v[8];
#pragma unroll
          for (int u = 0; u < 4; ++u) {
            const int cj = j + u < 16 ? j + u : 15;    // (a column past the block is computed and dropped)
            const float4 kk = *reinterpret_cast<const float4*>(KHs + (c0 + cj) * AP + 4 * lane);
            const float4 ll = *reinterpret_cast<const float4*>(LAM + (r0 + cj) * LP + 4 * lane);
            const float e0 = kk.x * umma::ex2_fast(fminf(li.x - ll.x, 0.f) * DN_LOG2E), e1 = kk.y * umma::ex2_fast(fminf(li.y - ll.y, 0.f) * DN_LOG2E);
            const float e2 = kk.z * umma::ex2_fast(fminf(li.z - ll.z, 0.f) * DN_LOG2E), e3 = kk.w * umma::ex2_fast(fminf(li.w - ll.w, 0.f) * DN_LOG2E);
            v[2 * u] = bi4[0] * e0 + bi4[1] * e1 + bi4[2] * e2 + bi4[3] * e3;
            v[2 * u + 1] = qi[0] * e0 + qi[1] * e1 + qi[2] * e2 + qi[3] * e3;
          }
          // eight sums over the 32 lanes in 9 shuffles: at each of the first three steps a lane hands
          // over the half it drops and adds what it receives to the half it keeps
          float w4[4], u2[2], z;
#pragma unroll
          for (int t = 0; t < 4; ++t) {
            const float got = __shfl_xor_sync(0xffffffffu, hi16 ? v[t] : v[4 + t], 16);
            w4[t] = (hi16 ? v[4 + t] : v[t]) + got;
          }
#pragma unroll
          for (int t = 0; t < 2; ++t) {
            const float got = __shfl_xor_sync(0xffffffffu, hi8 ? w4[t] : w4[2 + t], 8);
            u2[t] = (hi8 ? w4[2 + t] : w4[t]) + got;
          }
          {
            const float got = __shfl_xor_sync(0xffffffffu, hi4 ? u2[0] : u2[1], 4);
            z = (hi4 ? u2[1] : u2[0]) + got;
          }
          z += __shfl_xor_sync(0xffffffffu, z, 2);
          z += __shfl_xor_sync(0xffffffffu, z, 1);
          // lane 16*(u>>1) + 8*(u&1) + 4*t now holds column j+u's sum of kind t (0: A, 1: M)
          const int u = lane - j;                      // the column this lane keeps, if 0 <= u < 4
          const int src = (u >= 0 && u < 4) ? 16 * (u >> 1) + 8 * (u & 1) : 0;
          const float pa = __shfl_sync(0xffffffffu, z, src), pm = __shfl_sync(0xffffffffu, z, src + 4);
          if (u >= 0 && u < 4 && lane <= i) {
            const bool same = seg_s[ri] == seg_s[r0 + lane];
            arow = (lane < i && same) ? pa : 0.f;
            mrow = same ? pm : 0.f;
          }
        }
        if (lane < 16) {
          umma::st_keep1(Ag + p4f(ri, r0 + lane), arow);
          Mel[rix(true, ri, r0 + lane, C)] = __float2bfloat16_rn(mrow);
        }
      }
      DN_MARK(21 + 3 * half);
      __syncthreads();
      DN_MARK(22 + 3 * half);
    }
    };

    // ---- qe, ke, the X = [first doc] beta e^Lam operand image and the images of the first level for
    //      one piece (row x, channels 8p..8p+7), from k_hat, q_hat and beta = b_act * k_hat
    auto xi_piece = [&](int x, int p, const float (&kh)[8], const float (&qh)[8], const float (&be)[8]) {
      const bool first = seg_s[x] == seg0, last = seg_s[x] == segL;
      float lam[8], lend[8], o[8], el[8];
      *reinterpret_cast<float4*>(lam) = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p);
      *reinterpret_cast<float4*>(lam + 4) = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p + 4);
      *reinterpret_cast<float4*>(lend) = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p);
      *reinterpret_cast<float4*>(lend + 4) = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p + 4);
#pragma unroll
      for (int i = 0; i < 8; ++i) el[i] = umma::exp_neg(fminf(lam[i], 0.f));
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = first ? qh[i] * el[i] : 0.f;
      QEimg[p * 128 + x] = umma::pack8(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = last ? kh[i] * umma::exp_neg(fminf(lend[i] - lam[i], 0.f)) : 0.f;
      KEimg[p * 128 + x] = umma::pack8(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = first ? be[i] * el[i] : 0.f;
      XI[p * 128 + x] = umma::pack8(o);
      build_level_from_beta(kh, be, qh, LAM, 16, x, p, KR, QK);
    };
    // the cached operands of row x = this thread's tensor-memory lane, piece p
    auto cached_piece = [&](int p, float (&kh)[8], float (&qh)[8], float (&be)[8]) {
      float kq[8];
      umma::tmem_ld8(tm_lane + COL_KQ + 8 * p, kq);
      umma::tmem_ld8(tm_lane + COL_BE + 8 * p, be);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        kh[i] = __uint_as_float(__float_as_uint(kq[i]) << 16);
        qh[i] = __uint_as_float(__float_as_uint(kq[i]) & 0xffff0000u);
      }
    };
    auto xi_pass = [&]() {
      if (tm_cache) {
        const int x = (warp & 3) * 32 + lane;
#pragma unroll 2
        for (int j = 0; j < 4; ++j) {
          const int p = (warp >> 2) * 4 + j;
          float kh[8], qh[8], be[8];
          cached_piece(p, kh, qh, be);
          xi_piece(x, p, kh, qh, be);
        }
      } else {
#pragma unroll 2
        for (int it = 0; it < 4; ++it) {
          const int p = it * 4 + lgrp;
          float qh[8], kh[8], be[8];
          qhat8(r, myrow, p, qh);
          khat8(r, myrow, p, kh);
          bact8(r, myrow, p, be);
#pragma unroll
          for (int i = 0; i < 8; ++i) be[i] *= kh[i];
          xi_piece(myrow, p, kh, qh, be);
        }
      }
      if (tid < K) a.res.lam_end[ibase * K + tid] = LAM[(C - 1) * LP + tid];
    };

    if constexpr (CF::scalar_gates) {
      // ---- one scalar decay and one scalar beta per (token, head): the decay leaves the channel sum,
      //      A_ij = beta_i e^{lam_i - lam_j} (k_i . k_j),  M_ij = e^{lam_i - lam_j} (q_i . k_j),
      //      so A and M are two Gram products on the plain bf16 images of k_hat and q_hat, and the decay
      //      (exact, <= 1) is applied per entry by the drain.  No levels, no diagonal pass.
      DN_MARK(1);
      {
        const int x = myrow;
        const bool first = seg_s[x] == seg0, last = seg_s[x] == segL;
        const bool live = x < r.rows_valid;
        const float lam = LAM[x * LP], lend = LAM[(C - 1) * LP];
        const float el = umma::exp_neg(fminf(lam, 0.f)), eke = umma::exp_neg(fminf(lend - lam, 0.f));
        const float bx = live ? ldf_ro(r.b, r.b_row0 + (size_t)x * r.b_pitch, DN_F32) : 0.f;
#pragma unroll 2
        for (int it = 0; it < 4; ++it) {
          const int p = it * 4 + lgrp;
          float qh[8], kh[8], o[8];
          qhat8(r, x, p, qh);
          khat8(r, x, p, kh);
          KR[p * 128 + x] = umma::pack8(kh);
          QK[p * 128 + x] = umma::pack8(qh);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = first ? qh[i] * el : 0.f;
          QEimg[p * 128 + x] = umma::pack8(o);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = last ? kh[i] * eke : 0.f;
          KEimg[p * 128 + x] = umma::pack8(o);
#pragma unroll
          for (int i = 0; i < 8; ++i) o[i] = first ? (bx * kh[i]) * el : 0.f;
          XI[p * 128 + x] = umma::pack8(o);
        }
        if (lgrp == 0) bsc_s[x] = bx;
        if (tid < K) a.res.lam_end[ibase * K + tid] = lend;
      }
      DN_MARK(2);
      umma::pre_issue_sync();
      umma::issue<128, false, false>(cx, KR, KR, K, 0, false);             // k_hat k_hat^T
      umma::issue<128, false, false>(cx, QK, KR, K, 128, false);           // q_hat k_hat^T
      umma::commit_wait(cx);
      DN_MARK(3);
      {
        const int quarter = warp & 3, group = warp >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t tbase = cx.tmem + ((uint32_t)(quarter * 32) << 16);
        const float lrow = LAM[row * LP] * DN_LOG2E, brow = bsc_s[row];
        const int srow = seg_s[row];
#pragma unroll 1
        for (int cc = 0; cc < 32; cc += 16) {
          const int col = group * 32 + cc;
          float va[16], vm[16];
          if (!cx.dead && col <= quarter * 32 + 31) {    // warp-uniform: a piece wholly above the warp's rows is zeros
            umma::tmem_ld16(tbase + col, va);
            umma::tmem_ld16(tbase + 128 + col, vm);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) va[i] = vm[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = col + i;
            const bool same = srow == seg_s[j];
            const float f = umma::ex2_fast(fminf(lrow - LAM[j * LP] * DN_LOG2E, 0.f));
            va[i] = (same && j < row) ? brow * f * va[i] : 0.f;
            vm[i] = (same && j <= row) ? f * vm[i] : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) umma::st_keep4(Ag4 + p4v(row, col + 4 * i), make_float4(va[4 * i], va[4 * i + 1], va[4 * i + 2], va[4 * i + 3]));
          Mimg[(col / 8) * 128 + row] = umma::pack8p(vm);
          Mimg[(col / 8 + 1) * 128 + row] = umma::pack8p(vm + 8);
        }
        umma::tc_fence_before();
      }
      __syncthreads();
      DN_MARK(6);
    } else {
    // ---- Channel-wise decay.  When the decay of every document inside the chunk is moderate in every
    //      channel, A and M are single Gram products as well: with m_c the midpoint of a document's
    //      cumulative decay in channel c and f_ic = e^{Lam_ic - m_c},
    //        A_ij = sum_c (beta_ic f_ic) (k_jc / f_jc),   M_ij = sum_c (q_ic f_ic) (k_jc / f_jc)
    //      for i, j in one document, and every factor stays within e^{+-FAST_HALF_RANGE}: nothing can
    //      overflow, and bf16 keeps its relative precision at any magnitude.  Chunks with a stronger decay
    //      (half range above the bound in some channel of some document) take the hierarchical
    //      factorisation below, whose factors never exceed 1 whatever the decay.
    constexpr float FAST_HALF_RANGE = 32.f;
    if (tid < C) {                              // first and last row of each row's document inside the chunk
      const int sx = seg_s[tid];
      int lo = 0, hi = tid;                     // seg_s is non-decreasing: binary searches
      while (lo < hi) { const int mid = (lo + hi) >> 1; if (seg_s[mid] < sx) lo = mid + 1; else hi = mid; }
      ds_s[tid] = (uint8_t)lo;
      lo = tid; hi = C - 1;
      while (lo < hi) { const int mid = (lo + hi + 1) >> 1; if (seg_s[mid] > sx) hi = mid - 1; else lo = mid; }
      de_s[tid] = (uint8_t)lo;
    }
    __syncthreads();
    // one test per document and channel, at the document's last row: threads (row x, channel quarter)
    bool strong = false;
    {
      const int x = tid & 127;
      if (de_s[x] == x) {
        const float* ls = LAM + ds_s[x] * LP + (tid >> 7) * 32;
        const float* le = LAM + x * LP + (tid >> 7) * 32;
#pragma unroll 8
        for (int c = 0; c < 32; ++c) strong |= 0.5f * (ls[c] - le[c]) > FAST_HALF_RANGE;
      }
    }
    const bool fast = !__syncthreads_or(strong);
    if (fast) {
      DN_MARK(1);
      uint4* BT = reinterpret_cast<uint4*>(smraw + OFF_TI);      // third image (beta f); the T image is built later
      {
        const int x = myrow;
        const bool first = seg_s[x] == seg0, last = seg_s[x] == segL;
        const float* lam_s = LAM + ds_s[x] * LP;
        const float* lam_e = LAM + de_s[x] * LP;
#pragma unroll 2
        for (int it = 0; it < 4; ++it) {
          const int p = it * 4 + lgrp;
          float qh[8], kh[8], be[8], lam[8], ls[8], le[8], lend[8], o1[8], o2[8], o3[8];
          qhat8(r, x, p, qh);
          khat8(r, x, p, kh);
          bact8(r, x, p, be);
          *reinterpret_cast<float4*>(lam) = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p);
          *reinterpret_cast<float4*>(lam + 4) = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p + 4);
          *reinterpret_cast<float4*>(ls) = *reinterpret_cast<const float4*>(lam_s + 8 * p);
          *reinterpret_cast<float4*>(ls + 4) = *reinterpret_cast<const float4*>(lam_s + 8 * p + 4);
          *reinterpret_cast<float4*>(le) = *reinterpret_cast<const float4*>(lam_e + 8 * p);
          *reinterpret_cast<float4*>(le + 4) = *reinterpret_cast<const float4*>(lam_e + 8 * p + 4);
          *reinterpret_cast<float4*>(lend) = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p);
          *reinterpret_cast<float4*>(lend + 4) = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p + 4);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            be[i] *= kh[i];                                             // beta = b_act * k_hat
            const float d = (lam[i] - 0.5f * (ls[i] + le[i])) * DN_LOG2E;      // log2 f, |d| <= FAST_HALF_RANGE * log2 e
            const float f = umma::ex2_fast(d), fi = umma::ex2_fast(-d);
            o1[i] = kh[i] * fi;
            o2[i] = qh[i] * f;
            o3[i] = be[i] * f;
          }
          KR[p * 128 + x] = umma::pack8(o1);
          QK[p * 128 + x] = umma::pack8(o2);
          BT[p * 128 + x] = umma::pack8(o3);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float el = umma::exp_neg(fminf(lam[i], 0.f));
            o1[i] = first ? qh[i] * el : 0.f;
            o2[i] = last ? kh[i] * umma::exp_neg(fminf(lend[i] - lam[i], 0.f)) : 0.f;
            o3[i] = first ? be[i] * el : 0.f;
          }
          QEimg[p * 128 + x] = umma::pack8(o1);
          KEimg[p * 128 + x] = umma::pack8(o2);
          XI[p * 128 + x] = umma::pack8(o3);
        }
        if (tid < K) a.res.lam_end[ibase * K + tid] = LAM[(C - 1) * LP + tid];
      }
      DN_MARK(2);
      umma::pre_issue_sync();
      umma::issue<128, false, false>(cx, BT, KR, K, 0, false);             // A = (beta f) (k / f)^T
      umma::issue<128, false, false>(cx, QK, KR, K, 128, false);           // M = (q f) (k / f)^T
      umma::commit_wait(cx);
      DN_MARK(3);
      {
        const int quarter = warp & 3, group = warp >> 2;
        const int row = quarter * 32 + lane;
        const uint32_t tbase = cx.tmem + ((uint32_t)(quarter * 32) << 16);
        const int srow = seg_s[row];
#pragma unroll 1
        for (int cc = 0; cc < 32; cc += 16) {
          const int col = group * 32 + cc;
          float va[16], vm[16];
          if (!cx.dead && col <= quarter * 32 + 31) {    // warp-uniform: a piece wholly above the warp's rows is zeros
            umma::tmem_ld16(tbase + col, va);
            umma::tmem_ld16(tbase + 128 + col, vm);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) va[i] = vm[i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int j = col + i;
            const bool same = srow == seg_s[j];
            va[i] = (same && j < row) ? va[i] : 0.f;
            vm[i] = (same && j <= row) ? vm[i] : 0.f;
          }
#pragma unroll
          for (int i = 0; i < 4; ++i) umma::st_keep4(Ag4 + p4v(row, col + 4 * i), make_float4(va[4 * i], va[4 * i + 1], va[4 * i + 2], va[4 * i + 3]));
          Mimg[(col / 8) * 128 + row] = umma::pack8p(vm);
          Mimg[(col / 8 + 1) * 128 + row] = umma::pack8p(vm + 8);
        }
        umma::tc_fence_before();
      }
      __syncthreads();
      DN_MARK(6);
    } else {
    DN_MARK(1);
    if (tm_cache) diag_pass();                 // first: it also fills the tensor-memory operand cache
    xi_pass();

    DN_MARK(2);
    // ---- A and M, level by level: two images, two MMAs, one predicated drain per level
    auto build = [&](int lv) {
      if (tm_cache) {
        const int x = (warp & 3) * 32 + lane;
#pragma unroll 2
        for (int j = 0; j < 4; ++j) {
          const int p = (warp >> 2) * 4 + j;
          float kh[8], qh[8], be[8];
          cached_piece(p, kh, qh, be);
          build_level_from_beta(kh, be, qh, LAM, 16 << lv, x, p, KR, QK);
        }
      } else {
#pragma unroll 2
        for (int it = 0; it < 4; ++it) build_level_piece(r, LAM, 16 << lv, myrow, it * 4 + lgrp, KR, QK);
      }
    };
    auto drain_level = [&](int lv) {
      const int quarter = warp & 3, group = warp >> 2;
      const int row = quarter * 32 + lane, bi = row >> 4, bi0 = quarter * 2;
      const uint32_t tbase = cx.tmem + ((uint32_t)(quarter * 32) << 16);
#pragma unroll 1
      for (int cc = 0; cc < 32; cc += 16) {
        const int col = group * 32 + cc, bj = col >> 4;
        // warp-uniform skip: neither of the warp's two row blocks has this piece at this level
        const bool own0 = bj < bi0 && owner_level(bi0, bj) == lv, own1 = bj < bi0 + 1 && owner_level(bi0 + 1, bj) == lv;
        const bool upper = lv == 0 && bj > bi0;                  // zero fill, once
        if (!own0 && !own1 && !upper) continue;
        float va[16], vm[16];
        if (!cx.dead && (own0 || own1)) {
          umma::tmem_ld16(tbase + col, va);
          umma::tmem_ld16(tbase + 128 + col, vm);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) va[i] = vm[i] = 0.f;
        }
        const bool mine = bj < bi && owner_level(bi, bj) == lv;
        const bool zero_fill = lv == 0 && bj > bi;
        if (!mine && !zero_fill) continue;
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          const bool keep = mine && seg_s[row] == seg_s[col + i];
          va[i] = keep ? va[i] : 0.f;
          vm[i] = keep ? vm[i] : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) umma::st_keep4(Ag4 + p4v(row, col + 4 * i), make_float4(va[4 * i], va[4 * i + 1], va[4 * i + 2], va[4 * i + 3]));
        Mimg[(col / 8) * 128 + row] = umma::pack8p(vm);
        Mimg[(col / 8 + 1) * 128 + row] = umma::pack8p(vm + 8);
      }
      umma::tc_fence_before();
    };
#pragma unroll 1
    for (int lv = 0; lv < 3; ++lv) {                       // (the images of level 0 were built above)
      const uint32_t tcol = 0;                             // the drain of level lv is over before level lv + 1 is issued
      umma::pre_issue_sync();
      umma::issue<128, false, false>(cx, KR, KR, K, tcol, false);          // A: KR KR^T
      umma::issue<128, false, false>(cx, QK, KR, K, tcol + 128, false);    // M: QK KR^T
      umma::commit_wait(cx);
      DN_MARK(3 + lv);
      if (lv < 2) build(lv + 1);
      drain_level(lv);
    }
    __syncthreads();

    DN_MARK(6);
    if (!tm_cache) diag_pass();
    }
    }

    DN_MARK(7);
    // The inverse below works out of shared memory for a while: ask for this item's rows of v and w (read
    // right after it, for the first time) to be brought into L2 meanwhile.
    if (tid < r.rows_valid) {
      const size_t tok = (size_t)b * g.L + t0 + tid;
      const uint32_t qe = (uint32_t)dt_size(qdt), ge = (uint32_t)dt_size(gdt);
      umma::prefetch_l2(reinterpret_cast<const uint8_t*>(a.v) + (tok * g.Hv * g.V + (size_t)h * VW) * qe, VW * qe);
      if (wC == g.V && g.wH == g.Hv)
        umma::prefetch_l2(reinterpret_cast<const uint8_t*>(a.w) + (tok * g.Hv * g.V + (size_t)h * VW) * ge, VW * ge);
    }
    // ---- T = (I + A)^-1 in fp32: substitution on the diagonal blocks, then block merges
    {
      float4* As4 = reinterpret_cast<float4*>(As);
      float4* Ts4 = reinterpret_cast<float4*>(Ts);
#pragma unroll 4
      for (int e = tid; e < 32 * C; e += NT) {
        const int q = e >> 7, i = e & 127;
        As4[i * (AP / 4) + q] = umma::ld_keep4(Ag4 + e);
      }
      for (int e = tid; e < C * AP / 4; e += NT) Ts4[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    if (tid < C) {
      const int j = tid, blk0 = j & ~15, jl = j & 15;
      float col[16];
#pragma unroll
      for (int m = 0; m < 16; ++m) col[m] = m == jl ? 1.f : 0.f;
#pragma unroll
      for (int i = 1; i < 16; ++i) {
        float av[16];
#pragma unroll
        for (int u = 0; u < (i + 3) / 4; ++u)
          *reinterpret_cast<float4*>(av + 4 * u) = *reinterpret_cast<const float4*>(As + (blk0 + i) * AP + blk0 + 4 * u);
        float s = 0.f;
#pragma unroll
        for (int m = 0; m < i; ++m) s = fmaf(av[m], col[m], s);
        if (i > jl) col[i] = -s;
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) Ts[(blk0 + i) * AP + j] = col[i];
    }
    __syncthreads();
    DN_MARK(8);
    merge_level<16>(As, Ts, Tm);
    merge_level<32>(As, Ts, Tm);
    merge_level<64>(As, Ts, Tm);
    DN_MARK(9);
    // ---- W = T X, U = T Y on the tensor cores
    {
      // T as K-major A: piece (p = j/8, x = i).  The same image is the residual the backward reads
      // (bf16, in the first half of T's fp32-sized slot): it rounds T to bf16 there anyway.
      uint4* Tg = a.res.T ? reinterpret_cast<uint4*>(a.res.T + ibase * C * C) : nullptr;
      for (int e = tid; e < IMG; e += NT) {
        const int p = e >> 7, x = e & 127;
        const uint4 v = umma::ld8_f32(Ts + x * AP + 8 * p);
        TI[e] = v;
        if (Tg) Tg[e] = v;
      }
    }
    {                                                           // Y = w*v as MN-major B
      const int x = myrow, t = t0 + x;
      const bool live = t < g.L;
      const size_t tokr = (size_t)b * g.L + (live ? t : t0);
#pragma unroll 4
      for (int it = 0; it < VW / 32; ++it) {
        const int p = it * 4 + lgrp;
        const int col0 = h * VW + 8 * p, hv = col0 / g.V, cv = col0 - hv * g.V;
        float vv[8], ww[8], f[8];
        load8(a.v, tokr * g.Hv * g.V + col0, qdt, vv);
        if (wC == 1) {
          const float w1 = ldf_ro(a.w, tokr * g.wH + g.w_head(hv), gdt);
#pragma unroll
          for (int i = 0; i < 8; ++i) ww[i] = w1;
        } else {
          load8(a.w, (tokr * g.wH + g.w_head(hv)) * wC + cv, gdt, ww);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float wa = fuse ? 1.f / (1.f + expf(-ww[i])) : ww[i];
          f[i] = live ? wa * vv[i] : 0.f;
        }
        YI[p * 128 + x] = umma::pack8(f);
      }
    }
    umma::pre_issue_sync();
    umma::issue<128, false, true>(cx, TI, XI, C, 0, false);
    umma::issue<VW, false, true>(cx, TI, YI, C, 128, false);
    umma::commit_wait(cx);
    DN_MARK(10);
    umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
      Wimg[(col / 8) * 128 + row] = umma::pack8p(v);
      Wimg[(col / 8 + 1) * 128 + row] = umma::pack8p(v + 8);
    });
    umma::drain<NT, VW>(cx, 128, [&](int row, int col, const float (&v)[16]) {
      Uimg[(col / 8) * 128 + row] = umma::pack8p(v);
      Uimg[(col / 8 + 1) * 128 + row] = umma::pack8p(v + 8);
    });
    __syncthreads();
#ifdef DN_PHASE_TIMING
    DN_MARK(11);
    if (blockIdx.x == 0 && tid == 0 && e_item == 0) {
      for (int i = 1; i < 12; ++i) printf("fwd mark %d -> %d: %lld\n", i - 1, i, g_phase_marks[i] - g_phase_marks[i - 1]);
      printf("fwd item total %lld\n", g_phase_marks[11] - g_phase_marks[0]);
      printf("fwd D: stage0 %lld compute0(warp0) %lld wait0 %lld stage1 %lld compute1 %lld wait1 %lld\n", g_phase_marks[20] - g_phase_marks[6],
             g_phase_marks[21] - g_phase_marks[20], g_phase_marks[22] - g_phase_marks[21], g_phase_marks[23] - g_phase_marks[22],
             g_phase_marks[24] - g_phase_marks[23], g_phase_marks[25] - g_phase_marks[24]);
    }
#endif
  }
  umma::tc_fence_before();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, 512);
}

}  // namespace

bool prepass_fwd_tc_eligible(const Geo& g) { return g.img; }

size_t prepass_fwd_tc_scratch_per_cta() { return (size_t)C * C; }

int launch_prepass_fwd_tc(const Geo& g, const void* q, const void* k, const void* v, const void* gg,
                          const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                          float* scratch, size_t scratch_floats, cudaStream_t st, int c_begin, int c_end) {
  PrepassFwdArgs a;
  a.g = g; a.q = q; a.k = k; a.v = v; a.gg = gg; a.b = b; a.w = w; a.seg = seg; a.res = res;
  a.c_begin = c_begin; a.c_end = c_end < 0 ? g.NC : c_end;
  a.items = g.B * g.H * (a.c_end - a.c_begin);
  if (a.items <= 0) return DN_OK;
  a.scratch_per_cta = prepass_fwd_tc_scratch_per_cta();
  a.smem_tile_off = 0;
  const int grid = a.items < sm_count() ? a.items : sm_count();
  if (scratch_floats < (size_t)grid * a.scratch_per_cta) return DN_ERR_SCRATCH_TOO_SMALL;
  a.scratch = scratch;
  int* err = device_error_ptr();
  auto go = [&](auto kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    kernel<<<grid, NT, SMEM_BYTES, st>>>(a, err);
  };
  const int mode = input_mode(g);
  if (g.Vw == 256) {
    if (mode == 0) go(prepass_fwd_tc_kernel<256, 0>); else if (mode == 1) go(prepass_fwd_tc_kernel<256, 1>); else if (mode == 3) go(prepass_fwd_tc_kernel<256, 3>); else if (mode == 4) go(prepass_fwd_tc_kernel<256, 4>); else go(prepass_fwd_tc_kernel<256, 2>);
  } else {
    if (mode == 0) go(prepass_fwd_tc_kernel<128, 0>); else if (mode == 1) go(prepass_fwd_tc_kernel<128, 1>); else if (mode == 3) go(prepass_fwd_tc_kernel<128, 3>); else if (mode == 4) go(prepass_fwd_tc_kernel<128, 4>); else go(prepass_fwd_tc_kernel<128, 2>);
  }
  return launch_status();
}

}  // namespace dn
