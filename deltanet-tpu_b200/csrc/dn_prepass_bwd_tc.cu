// Chunk-parallel backward on the tcgen05 tensor cores (bf16 precision, chunk = K = 128, value
// width 128 or 256): the adjoint of the state step's value-width contractions, of the prepass
// (reference: src/deltanet_tpu/gdn2.py:243-493, 750-762) and of the fused prologue (558-575).
//
// Per (batch, exec head, chunk), 512 threads, one CTA per SM, in this order:
//   G. nine matrix products (bwd_gemms_tc): V_new, dqe, dM, dW, dke, dX, dY, dA.  Every operand is a
//      bf16 image fetched by one bulk copy; dLambda_end comes from the reverse chain's partial sums.
//   V. dv and dw from the bf16 image of dY that G leaves in shared memory; in the headline mode the
//      rows of v, w, dv, dw move by bulk copies through padded staging rows.
//   L. row normalisers and the cumulative log-decay of the chunk in shared memory.
//   D/H. adjoints of A and M, i.e. dbeta', dq', dk', by one of three routes:
//      (a) one scalar decay per (token, head): with f_ij = e^{lam_i - lam_j} applied entry-wise to dA and dM,
//          two rounds of two products on the plain images of k_hat and q_hat;
//      (b) channel-wise decay that stays within e^{+-32} of each document's midpoint over the chunk (tested
//          per chunk on the device): the same two rounds on images of k_hat / f, q_hat f, beta k_hat f with
//          f = e^{Lam - midpoint}; the results are scaled by f, f, 1 / f when phase E reads them;
//          on (a) and (b) the three accumulators stay in tensor memory for phase E;
//      (c) otherwise: D. the 16x16 diagonal blocks of dA and dM, exact, one thread per (block, channel), from
//          shared-memory caches of k_hat, q_hat, beta (64 rows at a time), which initialises dbeta', dq', dk'
//          in the scratch and parks k_hat | q_hat (two bf16 per column) and beta in tensor memory; then
//          H. the three-level factorisation of the forward: in one level every row is either a ROW of the
//          level's entries (lower block of its pair) or a COLUMN (upper block), so with dA_s / dM_s the
//          entries the level owns, KR the image holding beta-images on lower rows and k-images on upper
//          rows, and QK holding q-images / k-images,
//            T1 = (dA_s + dA_s^T) KR,   T2 = (dM_s + dM_s^T) QK        (four MMAs, one drain)
//            lower rows:  dbeta' += rowfac * T1,  dq' += rowfac * T2
//            upper rows:  dk'    += colfac * (T1 + T2)
//          with the same exp(Lam - Lam_ref) factors (all <= 1) as the forward; a level's drain overlaps the
//          next level's image build.
//   E. combination into dLambda, d q_hat, d k_hat, d b (written), the l2norm adjoint and dq, dk, in the
//      thread mapping of a tensor-memory drain; the operands of the second half wait in tensor memory.
//   R. dg by a within-document reverse cumulative sum plus the Lambda_end path; written with the
//      gate adjoint.
//
// Thread mappings: phases that touch the operator's row-major tensors let a warp cover 8 rows x 4
// pieces of 8 channels (row = 8 * warp + (lane & 7) is fixed per thread); phases that drain or use
// tensor memory own one row per thread (row = the thread's lane of its warp's lane quarter) and use
// the panel layout of the scratch (see the header).
#ifdef DN_PHASE_TIMING
#include <cstdio>
#endif
#include "dn_chunkprep.cuh"
#include "dn_kernels.cuh"
#include "dn_prepass_bwd_tc.cuh"

namespace dn {
namespace {

using namespace prep;
constexpr int NT = 512;

__device__ __forceinline__ void ld2x4(const float4* p, float (&o)[8]) {      // scratch written by this CTA
  const float4 a = umma::ld_keep4(p), b = umma::ld_keep4(p + 128);
  o[0] = a.x; o[1] = a.y; o[2] = a.z; o[3] = a.w; o[4] = b.x; o[5] = b.y; o[6] = b.z; o[7] = b.w;
}
__device__ __forceinline__ void out8(void* base, size_t off, int dt, const float (&v)[8]) {
  if (dt == DN_BF16) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(base) + off) = umma::pack8(v);
  else {
    float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off);
    d[0] = make_float4(v[0], v[1], v[2], v[3]);
    d[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// One row i of a diagonal block: columns [0, JF) always, columns [JF, JF + JP) while j < i.
template <int JF, int JP>
__device__ __forceinline__ void diag_row(int i, float li, const float (&lam)[16], const float (&kh)[16], float (&sk)[16],
                                         const float4* da4, const float4* dm4, float be, float qv, float& sb, float& sq) {
  constexpr int NJ = JF + JP, NV = (NJ + 3) / 4;
  float da[4 * NV], dm[4 * NV];
#pragma unroll
  for (int u = 0; u < NV; ++u) {
    const float4 va = da4[u], vm = dm4[u];
    da[4 * u] = va.x; da[4 * u + 1] = va.y; da[4 * u + 2] = va.z; da[4 * u + 3] = va.w;
    dm[4 * u] = vm.x; dm[4 * u + 1] = vm.y; dm[4 * u + 2] = vm.z; dm[4 * u + 3] = vm.w;
  }
  sb = 0.f; sq = 0.f;
#pragma unroll
  for (int j = 0; j < NJ; ++j) {
    if (j < JF || j < i) {
      const float e = umma::ex2_fast(fminf(li - lam[j], 0.f));
      const float ek = e * kh[j];
      sb = fmaf(da[j], ek, sb);
      sq = fmaf(dm[j], ek, sq);
      sk[j] = fmaf(fmaf(da[j], be, dm[j] * qv), e, sk[j]);
    }
  }
}

template <int VW, int MODE>
__global__ void __launch_bounds__(NT, 1) prepass_bwd_tc_kernel(PrepassBwdArgs a) {
  using CF = InCfg<MODE>;
  extern __shared__ __align__(128) uint8_t smraw[];
  __shared__ uint64_t mma_bar, v_bar, g_bar;
  __shared__ uint32_t tmem_base;
  __shared__ int seg_s[C];
  __shared__ int reset_s[8];                 // per 32-row quarter: a document starts inside it
  __shared__ uint8_t ds_s[C], de_s[C];       // first / last row of each row's document inside the chunk
  __shared__ float rq_s[C], rk_s[C], dlend_s[K], dlend_b_s[C];     // dlend_b_s: the activated scalar erase gate per row (scalar-gate path)
  const Geo& g = a.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int myrow = warp * 8 + (lane & 7), lgrp = lane >> 3;      // the 8 rows x 4 pieces mapping
  constexpr int OFF_IMG = C * LP * 4;
  float* LAM = reinterpret_cast<float*>(smraw);
  uint4* I_DA = reinterpret_cast<uint4*>(smraw + OFF_IMG);
  uint4* I_DM = I_DA + IMG;
  uint4* I_KR = I_DM + IMG;
  uint4* I_QK = I_KR + IMG;
  float* DLs = reinterpret_cast<float*>(smraw + OFF_IMG);          // dLambda (pitch LP), over the images
  float* DKs = DLs + C * LP;                                        // dke*ke   (pitch LP)
  float* TOT = reinterpret_cast<float*>(smraw + 3 * C * LP * 4);   // 3 x 4 x 128 partial sums of phases E and R
  float* TOTL = reinterpret_cast<float*>(smraw + OFF_IMG);         // 4 x 128 partial sums of phase L

  const size_t CK = (size_t)C * K, CV = (size_t)C * VW, CC = (size_t)C * C;
  float* sc = a.scratch + (size_t)blockIdx.x * a.scratch_per_cta;
  float* DQE = sc;          float* DKE = DQE + CK;   float* DX = DKE + CK;
  float* DBP = DX + CK;     float* DQP = DBP + CK;   float* DKP = DQP + CK;
  float* DM = DKP + CK;     float* DA = DM + CC;
  float4* DA4 = reinterpret_cast<float4*>(DA);
  float4* DM4 = reinterpret_cast<float4*>(DM);
  float4* DBP4 = reinterpret_cast<float4*>(DBP);
  float4* DQP4 = reinterpret_cast<float4*>(DQP);
  float4* DKP4 = reinterpret_cast<float4*>(DKP);
  const float4* DX4 = reinterpret_cast<const float4*>(DX);
  const float4* DQE4 = reinterpret_cast<const float4*>(DQE);
  const float4* DKE4 = reinterpret_cast<const float4*>(DKE);

  if (tid == 0) { umma::mbar_init(&mma_bar, 1); umma::mbar_init(&v_bar, 1); umma::mbar_init(&g_bar, 1); umma::fence_mbar_init(); }
  uint32_t v_phase = 0;
  ImgLoader imgld{&g_bar, 0u, a.err};
  const bool bulk_v = MODE == 0 && a.bulk_v;
  // tensor-memory columns: level products T1 | T2 at [0, 256); operand cache of the level sweep at
  // [256, 384) (k_hat | q_hat, two bf16 per column) and [384, 512) (beta, fp32)
  constexpr uint32_t COL_KQ = 256, COL_BE = 384;
  if (warp == 0) umma::tmem_alloc(&tmem_base, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &mma_bar, 0u, a.err, false};

  const bool l2 = g.flags & DN_QK_L2NORM;
  const bool fuse = CF::fixed ? false : (g.flags & DN_FUSE_PROLOGUE) != 0;     // the fixed modes have no fused prologue
  const bool guard = CF::fixed ? false : (g.flags & DN_STABILITY_GUARD) != 0;
  const bool trunc = g.flags & DN_TRUNC_DT_BF16;

  // work items in chunk-major order inside the chunk range: all heads of chunk c_begin first
  for (int e_item = blockIdx.x; e_item < a.items; e_item += gridDim.x) {
    const int bh = e_item % (g.B * g.H), c_idx = a.c_begin + e_item / (g.B * g.H);
    const int h = bh % g.H, b = bh / g.H;
    const int item = bh * g.NC + c_idx;
    const int t0 = c_idx * C;
    const size_t ibase = (size_t)item;
    DN_MARK(0);
    for (int i = tid; i < C; i += NT) seg_s[i] = seg_at(a.seg, b, t0 + i, g.L);
    bool is_new, all_same;
    chunk_flags(a.seg, g, b, c_idx, is_new, all_same);
    __syncthreads();
    const int seg0 = seg_s[0], segL = seg_s[C - 1];
    const Rows r = make_rows<CF>(g, a.q, a.k, a.gg, a.b, b, h, t0, rq_s, rk_s);
    const int qdt = r.qkv_dt, gdt = r.gate_dt;           // compile-time constants in the fixed modes
    const int wC = CF::fixed ? (CF::scalar_bw ? 1 : g.V) : g.wC;
    const bool tm_cache = r.round_in;                    // k_hat, q_hat exactly bf16: they can be packed two per column

    // staging rows of phase V (headline mode): v as bf16 and w as fp32, one row per token, padded pitches
    constexpr int VP = 256 + 16, WP = 512 + 16;            // row pitches in bytes (padding: no bank conflicts)
    uint8_t* const VB = smraw + 68 * 1024;
    uint8_t* const WB = VB + 128 * VP;
    auto v_rows_request = [&](int pass) {                  // all threads: one bulk copy per row and tensor
      const int rows = g.L - t0 < C ? g.L - t0 : C;
      const int hv = h * (VW / 128) + pass;
      const size_t tok = (size_t)b * g.L + t0 + tid;
      if (tid == 0) umma::mbar_expect_tx(&v_bar, (uint32_t)rows * (256 + 512));
      __syncthreads();
      if (tid < rows) {
        umma::bulk_load(VB + tid * VP, reinterpret_cast<const __nv_bfloat16*>(a.v) + (tok * g.Hv + hv) * 128, 256, &v_bar);
        umma::bulk_load(WB + tid * WP, reinterpret_cast<const float*>(a.w) + (tok * g.wH + g.w_head(hv)) * 128, 512, &v_bar);
      }
    };

    // ---- G. the matrix products (and dLambda_end from the carried state)
    {
      BwdTcIo io;
      io.W = reinterpret_cast<const __nv_bfloat16*>(a.res.W) + ibase * CK;
      io.U = reinterpret_cast<const __nv_bfloat16*>(a.res.U) + ibase * CV;
      io.S = states_img(g, a.res.states) + ibase * K * VW;
      io.dH = reinterpret_cast<const __nv_bfloat16*>(a.dH) + ibase * K * VW;
      io.dV = reinterpret_cast<const __nv_bfloat16*>(a.dV) + ibase * CV;
      io.T = reinterpret_cast<const __nv_bfloat16*>(a.res.T + ibase * CC);
      io.slices = VW / 32;
      io.dlend_part = dlend_part(g, const_cast<float*>(a.dH)) + ibase * (VW / 32) * K;
      io.lam_end = a.res.lam_end + ibase * K;
      io.d_out = a.d_out; io.qkv_dt = CF::fixed ? CF::qkv_dt : g.qkv_dt;
      io.dO_off = ((size_t)b * g.L + t0) * g.Hv * g.V + (size_t)h * VW;
      io.dO_pitch = (size_t)g.Hv * g.V;
      io.rows_valid = g.L - t0 < C ? g.L - t0 : C;
      io.DQE = DQE; io.DKE = DKE; io.DX = DX; io.DM = DM; io.DA = DA;
      io.dlend_s = dlend_s; io.all_same = all_same;
      io.seg_s = seg_s; io.trunc = trunc;
      // the rows of v and w of the first value head are requested as soon as the products are done: they
      // travel while the last accumulator drains (phase V below waits for them)
      bwd_gemms_tc<VW, NT>(cx, smraw, io, imgld, [&]() {
        if (bulk_v) v_rows_request(0);
      });
    }

    // ---- V. dv = dY * w_act, dw = dY * v (+ sigmoid adjoint; summed over a value head's columns
    //         when w is one scalar per head): 8 rows x 4 pieces per warp step.  dY is read from the
    //         bf16 operand image the products left in shared memory (slot X), i.e. rounded to bf16
    //         like every other operand of this precision mode.
    //         In the headline mode (bf16 v, fp32 per-channel w, V = 128) the rows of v and w come in
    //         and the rows of dv and dw go out by bulk asynchronous copies, one per row and tensor,
    //         through padded staging rows in shared memory: a 128-column pass (one value head) moves
    //         384 KB without a single load or store instruction of the CUDA cores touching global memory.
    if (bulk_v) {
      const int rows = g.L - t0 < C ? g.L - t0 : C;
      const uint4* Ximg = reinterpret_cast<const uint4*>(smraw);
#pragma unroll 1
      for (int pass = 0; pass < VW / 128; ++pass) {
        const int hv = h * (VW / 128) + pass;                // V == 128: one value head per pass
        const size_t tok = (size_t)b * g.L + t0 + tid;
        if (pass > 0) v_rows_request(pass);                  // (pass 0 was requested before the last drain of phase G)
        if (!umma::mbar_wait(&v_bar, v_phase)) umma::report_timeout(a.err);
        v_phase ^= 1u;
#pragma unroll
        for (int it = 0; it < 4; ++it) {
          const int p = it * 4 + lgrp, x = myrow;
          uint4* pv = reinterpret_cast<uint4*>(VB + x * VP + 16 * p);
          float4* pw = reinterpret_cast<float4*>(WB + x * WP + 32 * p);
          float vv[8], dy[8], dv8[8];
          umma::unpack8(*pv, vv);
          const float4 w0 = pw[0], w1 = pw[1];
          const float ww[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
          umma::unpack8(Ximg[(pass * 16 + p) * 128 + x], dy);
#pragma unroll
          for (int i = 0; i < 8; ++i) { dv8[i] = dy[i] * ww[i]; vv[i] *= dy[i]; }
          *pv = umma::pack8(dv8);
          pw[0] = make_float4(vv[0], vv[1], vv[2], vv[3]);
          pw[1] = make_float4(vv[4], vv[5], vv[6], vv[7]);
        }
        umma::fence_async_smem();
        __syncthreads();
        if (tid < rows) {
          umma::bulk_store(reinterpret_cast<__nv_bfloat16*>(a.dv) + (tok * g.Hv + hv) * 128, VB + tid * VP, 256);
          umma::bulk_store(reinterpret_cast<float*>(a.dw) + (tok * g.Hv + hv) * 128, WB + tid * WP, 512);
          umma::bulk_commit();
          if (pass + 1 < VW / 128) umma::bulk_wait_read<0>();      // the staging rows are reused by the next pass
        }
      }
    } else
    {
      constexpr int PV = VW / 8;
      const int x = myrow, t = t0 + x;
      const bool live = t < g.L;
      const size_t tok = (size_t)b * g.L + t;
      const int steps_per_head = g.V / 32;            // warp steps that cover one value head
      float sw = 0.f;
      const size_t tokr = live ? tok : (size_t)b * g.L + t0;      // row read when this one does not exist
#pragma unroll 4
      for (int it = 0; it < PV / 4; ++it) {
        const int p = it * 4 + lgrp;
        const int col0 = h * VW + 8 * p, hv = col0 / g.V, cv = col0 - hv * g.V;
        float vv[8], ww[8], dy[8], dv8[8], dw8[8];
        load8(a.v, tokr * g.Hv * g.V + col0, qdt, vv);
        if (wC == 1) {
          const float w1 = ldf_ro(a.w, tokr * g.wH + g.w_head(hv), gdt);
#pragma unroll
          for (int i = 0; i < 8; ++i) ww[i] = w1;
        } else {
          load8(a.w, (tokr * g.wH + g.w_head(hv)) * wC + cv, gdt, ww);
        }
        umma::unpack8(reinterpret_cast<const uint4*>(smraw)[p * 128 + x], dy);
        if (live) {
          const size_t vrow = tok * g.Hv * g.V + col0;
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            float wa = ww[i], dwv = dy[i] * vv[i];
            if (fuse) { wa = 1.f / (1.f + expf(-ww[i])); dwv *= wa * (1.f - wa); }
            dv8[i] = dy[i] * wa;
            dw8[i] = dwv;
            sw += dwv;
          }
          out8(a.dv, vrow, qdt, dv8);
          if (wC != 1) out8(a.dw, (tok * g.Hv + hv) * wC + cv, a.dw_dt, dw8);
        }
        if (wC == 1 && (it + 1) % steps_per_head == 0) {
          sw += __shfl_xor_sync(0xffffffffu, sw, 8);
          sw += __shfl_xor_sync(0xffffffffu, sw, 16);
          if (live && lgrp == 0) stf(a.dw, tok * g.Hv + hv, sw, a.dw_dt);
          sw = 0.f;
        }
      }
    }
    __syncthreads();

    DN_MARK(7);
    // ---- L. rows, normalisers, cumulative decay
    row_norms_8x4(r, myrow, lgrp, rq_s, rk_s);
    lambda_scan_512(r, seg_s, LAM, TOTL, reset_s);
    __syncthreads();
    if (bulk_v) {                                          // dv, dw have left their staging rows (reused below);
      if (tid < C) umma::bulk_wait_read<0>();              // the copies had the whole of phase L to do so
      __syncthreads();
    }

    // where phase E finds dbeta', dq', dk': 0 = fp32 panels in the scratch; 1 = the accumulators T1 | T2 | T3 in tensor
    // memory, still to be scaled by f, f, 1/f; 2 = the same unscaled
    int tm_src = 0;
    if constexpr (CF::scalar_gates) {
      // ---- D + H for one scalar decay and one scalar beta per (token, head).  With f_ij = e^{lam_i - lam_j}
      //      (exact, <= 1 on the entries that survive the masks) and b_i the activated erase gate,
      //        dbeta'_i = sum_j (dA_ij f_ij) k_j            dq'_i = sum_{j<i} (dM_ij f_ij) k_j
      //        dk'_j    = sum_i (dA_ij f_ij b_i) k_i + sum_{i>j} (dM_ij f_ij) q_i
      //      i.e. four products on the plain bf16 images of k_hat and q_hat: no levels, no diagonal pass.
      //      The image of dA f is used twice, the second time with its rows scaled by b_i.
      DN_MARK(8);
      {
        const int x = myrow;
        const bool live = x < r.rows_valid;
        if (lgrp == 0) dlend_b_s[x] = live ? ldf_ro(r.b, r.b_row0 + (size_t)x * r.b_pitch, DN_F32) : 0.f;
#pragma unroll 2
        for (int it = 0; it < 4; ++it) {
          const int p = it * 4 + lgrp;
          float qh[8], kh[8];
          qhat8(r, x, p, qh);
          khat8(r, x, p, kh);
          I_KR[p * 128 + x] = umma::pack8(kh);
          I_QK[p * 128 + x] = umma::pack8(qh);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {                    // images of dA f and dM f (strictly lower; the diagonal of dM goes through E)
        const int e = u * NT + tid, p = e >> 7, x = e & 127;
        const bool any = 8 * p < x;                    // the piece has entries below the diagonal
        const float4 a0 = umma::ld_keep4_pred(DA4 + p4v(x, 8 * p), any), a1 = umma::ld_keep4_pred(DA4 + p4v(x, 8 * p + 4), any);
        const float4 m0 = umma::ld_keep4_pred(DM4 + p4v(x, 8 * p), any), m1 = umma::ld_keep4_pred(DM4 + p4v(x, 8 * p + 4), any);
        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w}, mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        const float lx = LAM[x * LP] * DN_LOG2E;
        float oa[8], om[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const int j = 8 * p + i;
          const float f = umma::ex2_fast(fminf(lx - LAM[j * LP] * DN_LOG2E, 0.f));
          oa[i] = av[i] * f;                           // (dA is zero on and above the diagonal and across documents)
          om[i] = j < x ? mv[i] * f : 0.f;
        }
        I_DA[e] = umma::pack8(oa);
        I_DM[e] = umma::pack8(om);
      }
      umma::pre_issue_sync();
      umma::issue<128, false, true>(cx, I_DA, I_KR, C, 0, false);          // (dA f)   k_hat
      umma::issue<128, false, true>(cx, I_DM, I_KR, C, 128, false);        // (dM f)   k_hat
      umma::commit_wait(cx);
      DN_MARK(9);
      // T1, T2 stay in tensor memory (columns [0, 256)): phase E reads them there
      umma::tc_fence_before();
#pragma unroll
      for (int u = 0; u < 4; ++u) {                    // rows of the dA f image scaled by b_i
        const int e = u * NT + tid, x = e & 127;
        float v8[8];
        umma::unpack8(I_DA[e], v8);
        const float bx = dlend_b_s[x];
#pragma unroll
        for (int i = 0; i < 8; ++i) v8[i] *= bx;
        I_DA[e] = umma::pack8(v8);
      }
      umma::pre_issue_sync();
      umma::issue<128, true, true>(cx, I_DA, I_KR, C, 256, false);         // (dA f b)^T k_hat
      umma::issue<128, true, true>(cx, I_DM, I_QK, C, 256, true);          // + (dM f)^T q_hat
      umma::commit_wait(cx);
      DN_MARK(10);
      tm_src = 2;                                      // T3 at columns [256, 384), no scaling
      umma::tc_fence_before();
      __syncthreads();
    } else {
    // ---- Channel-wise decay, moderate in every channel of every document of the chunk (the same test as
    //      in the forward prepass): D + H collapse to four products as in the scalar case.  With m_c the
    //      midpoint of a document's cumulative decay and f_ic = e^{Lam_ic - m_c}, all within
    //      e^{+-FAST_HALF_RANGE},
    //        dbeta'_i = f_i * sum_j dA_ij (k_j / f_j)          dq'_i = f_i * sum_{j<i} dM_ij (k_j / f_j)
    //        dk'_j    = (1 / f_j) * sum_i (dA_ij (beta_i f_i) + [i>j] dM_ij (q_i f_i))
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
      DN_MARK(8);
      // log2 of f for (row x, channels 8p..8p+7)
      auto log2f8 = [&](int x, int p, float (&d)[8]) {
        const float* lx = LAM + x * LP + 8 * p;
        const float* ls = LAM + ds_s[x] * LP + 8 * p;
        const float* le = LAM + de_s[x] * LP + 8 * p;
        const float4 a0 = *reinterpret_cast<const float4*>(lx), a1 = *reinterpret_cast<const float4*>(lx + 4);
        const float4 s0 = *reinterpret_cast<const float4*>(ls), s1 = *reinterpret_cast<const float4*>(ls + 4);
        const float4 e0 = *reinterpret_cast<const float4*>(le), e1 = *reinterpret_cast<const float4*>(le + 4);
        const float l8[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const float m8[8] = {s0.x + e0.x, s0.y + e0.y, s0.z + e0.z, s0.w + e0.w, s1.x + e1.x, s1.y + e1.y, s1.z + e1.z, s1.w + e1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) d[i] = (l8[i] - 0.5f * m8[i]) * DN_LOG2E;
      };
      uint4 bt[4];                                     // this thread's pieces of the beta f image, for the second round
      {
        const int x = myrow;
#pragma unroll
        for (int it = 0; it < 4; ++it) {               // images of k / f (slot KR) and q f (slot QK)
          const int p = it * 4 + lgrp;
          float qh[8], kh[8], ba[8], d[8];
          qhat8(r, x, p, qh);
          khat8(r, x, p, kh);
          bact8(r, x, p, ba);
          log2f8(x, p, d);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float f = umma::ex2_fast(d[i]);
            ba[i] = (ba[i] * kh[i]) * f;
            kh[i] *= umma::ex2_fast(-d[i]);
            qh[i] *= f;
          }
          I_KR[p * 128 + x] = umma::pack8(kh);
          I_QK[p * 128 + x] = umma::pack8(qh);
          bt[it] = umma::pack8(ba);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {                    // images of dA and of the strictly lower part of dM
        const int e = u * NT + tid, p = e >> 7, x = e & 127;
        const bool any = 8 * p < x;
        const float4 a0 = umma::ld_keep4_pred(DA4 + p4v(x, 8 * p), any), a1 = umma::ld_keep4_pred(DA4 + p4v(x, 8 * p + 4), any);
        const float4 m0 = umma::ld_keep4_pred(DM4 + p4v(x, 8 * p), any), m1 = umma::ld_keep4_pred(DM4 + p4v(x, 8 * p + 4), any);
        const float mv[8] = {m0.x, m0.y, m0.z, m0.w, m1.x, m1.y, m1.z, m1.w};
        float om[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) om[i] = 8 * p + i < x ? mv[i] : 0.f;
        I_DA[e] = make_uint4(umma::pack2(a0.x, a0.y), umma::pack2(a0.z, a0.w), umma::pack2(a1.x, a1.y), umma::pack2(a1.z, a1.w));
        I_DM[e] = umma::pack8(om);
      }
      umma::pre_issue_sync();
      umma::issue<128, false, true>(cx, I_DA, I_KR, C, 0, false);          // dA (k / f)
      umma::issue<128, false, true>(cx, I_DM, I_KR, C, 128, false);        // dM (k / f)
      umma::commit_wait(cx);
      DN_MARK(9);
      // the k / f image has been consumed: beta f takes its slot for the second pair of products
#pragma unroll
      for (int it = 0; it < 4; ++it) I_KR[(it * 4 + lgrp) * 128 + myrow] = bt[it];
      // f T1 = dbeta', f T2 = dq' are read from tensor memory by phase E (columns [0, 256))
      umma::tc_fence_before();
      umma::pre_issue_sync();
      umma::issue<128, true, true>(cx, I_DA, I_KR, C, 256, false);         // dA^T (beta f)
      umma::issue<128, true, true>(cx, I_DM, I_QK, C, 256, true);          // + dM^T (q f)
      umma::commit_wait(cx);
      DN_MARK(10);
      tm_src = 1;                                      // T3 / f = dk' at columns [256, 384)
      umma::tc_fence_before();
      __syncthreads();
    } else {
    DN_MARK(8);
    // ---- D. diagonal 16x16 blocks, exact.  The blocks of dA and dM are staged in shared memory
    //         (all lanes of a warp read the same entry), and so are k_hat, q_hat and beta of 64 rows
    //         at a time (fp32, one global round trip per half); one thread per (block, channel)
    //         then walks the rows i of its block and, for every earlier row j, adds to dbeta'_i,
    //         dq'_i (scalars) and dk'_j (one register per j), reading shared memory only.
    //         This pass initialises DBP / DQP / DKP; the levels of phase H add to them.
    {
      constexpr int CP = 132;                                        // row pitch of the caches
      float* KC = reinterpret_cast<float*>(smraw + OFF_IMG);         // [64][CP] k_hat
      float* QC = KC + 64 * CP;                                      // q_hat
      float* BC = QC + 64 * CP;                                      // beta = b_act * k_hat
      float4* DG4 = reinterpret_cast<float4*>(BC + 64 * CP);         // [2][8 blocks][16 rows][4]
      for (int e = tid; e < 512; e += NT) {
        const int blk = e >> 6, q4 = (e >> 4) & 3, row = e & 15;
        DG4[(blk * 16 + row) * 4 + q4] = umma::ld_keep4(DA4 + p4v(blk * 16 + row, blk * 16 + 4 * q4));
        DG4[512 + (blk * 16 + row) * 4 + q4] = umma::ld_keep4(DM4 + p4v(blk * 16 + row, blk * 16 + 4 * q4));
      }
#pragma unroll 1
      for (int half = 0; half < 2; ++half) {
#pragma unroll
        for (int it = 0; it < 2; ++it) {
          const int w = it * 16 + warp, xr = (w & 7) * 8 + (lane & 7), p = (w >> 3) * 4 + lgrp, x = half * 64 + xr;
          float kh[8], qh[8], ba[8];
          khat8(r, x, p, kh);
          qhat8(r, x, p, qh);
          bact8(r, x, p, ba);
#pragma unroll
          for (int i = 0; i < 8; ++i) ba[i] *= kh[i];
          *reinterpret_cast<float4*>(KC + xr * CP + 8 * p) = make_float4(kh[0], kh[1], kh[2], kh[3]);
          *reinterpret_cast<float4*>(KC + xr * CP + 8 * p + 4) = make_float4(kh[4], kh[5], kh[6], kh[7]);
          *reinterpret_cast<float4*>(QC + xr * CP + 8 * p) = make_float4(qh[0], qh[1], qh[2], qh[3]);
          *reinterpret_cast<float4*>(QC + xr * CP + 8 * p + 4) = make_float4(qh[4], qh[5], qh[6], qh[7]);
          *reinterpret_cast<float4*>(BC + xr * CP + 8 * p) = make_float4(ba[0], ba[1], ba[2], ba[3]);
          *reinterpret_cast<float4*>(BC + xr * CP + 8 * p + 4) = make_float4(ba[4], ba[5], ba[6], ba[7]);
        }
        __syncthreads();
        DN_MARK(20 + 3 * half);
        if (tm_cache && ((warp & 3) >> 1) == half) {
          // the level sweep reads k_hat, q_hat and beta from tensor memory instead of global memory:
          // thread = row (its own lane), the four warps of a lane quarter take 32 channels each
          const int xr = (warp & 3) * 32 + lane - 64 * half, cg0 = (warp >> 2) * 32;
          const uint32_t tl = cx.tmem + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int c0 = cg0 + 8 * j;
            float kq[8], be8[8];
            const float4 k0 = *reinterpret_cast<const float4*>(KC + xr * CP + c0), k1 = *reinterpret_cast<const float4*>(KC + xr * CP + c0 + 4);
            const float4 q0 = *reinterpret_cast<const float4*>(QC + xr * CP + c0), q1 = *reinterpret_cast<const float4*>(QC + xr * CP + c0 + 4);
            const float4 b0 = *reinterpret_cast<const float4*>(BC + xr * CP + c0), b1 = *reinterpret_cast<const float4*>(BC + xr * CP + c0 + 4);
            const float kk[8] = {k0.x, k0.y, k0.z, k0.w, k1.x, k1.y, k1.z, k1.w}, qq[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
            for (int i = 0; i < 8; ++i)                 // both are exactly representable in bf16 here
              kq[i] = __uint_as_float((__float_as_uint(kk[i]) >> 16) | (__float_as_uint(qq[i]) & 0xffff0000u));
            be8[0] = b0.x; be8[1] = b0.y; be8[2] = b0.z; be8[3] = b0.w; be8[4] = b1.x; be8[5] = b1.y; be8[6] = b1.z; be8[7] = b1.w;
            umma::tmem_st8(tl + COL_KQ + c0, kq);
            umma::tmem_st8(tl + COL_BE + c0, be8);
          }
          umma::tmem_wait_st();
        }
        {
          const int lb = tid >> 7, blk = half * 4 + lb, r0 = blk * 16, c = tid & 127;
          const float* kc = KC + lb * 16 * CP + c;
          const float* qc = QC + lb * 16 * CP + c;
          const float* bc = BC + lb * 16 * CP + c;
          float lam[16], kh[16], sk[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            lam[i] = LAM[(r0 + i) * LP + c] * DN_LOG2E;
            kh[i] = kc[i * CP];
            sk[i] = 0.f;
          }
          umma::st_keep1(DBP + p4f(r0, c), 0.f);
          umma::st_keep1(DQP + p4f(r0, c), 0.f);
          // rolled over the rows (the body is executed 15 times, which keeps the code small enough
          // to stay in the instruction cache): rows 1..7 see columns j < i <= 7, rows 8..15 see
          // columns 0..7 unconditionally and columns 8..14 while j < i
#pragma unroll 1
          for (int i = 1; i < 8; ++i) {
            float sb, sq;
            diag_row<0, 7>(i, LAM[(r0 + i) * LP + c] * DN_LOG2E, lam, kh, sk, DG4 + (r0 + i) * 4, DG4 + 512 + (r0 + i) * 4, bc[i * CP], qc[i * CP], sb, sq);
            umma::st_keep1(DBP + p4f(r0 + i, c), sb);
            umma::st_keep1(DQP + p4f(r0 + i, c), sq);
          }
#pragma unroll 1
          for (int i = 8; i < 16; ++i) {
            float sb, sq;
            diag_row<8, 7>(i, LAM[(r0 + i) * LP + c] * DN_LOG2E, lam, kh, sk, DG4 + (r0 + i) * 4, DG4 + 512 + (r0 + i) * 4, bc[i * CP], qc[i * CP], sb, sq);
            umma::st_keep1(DBP + p4f(r0 + i, c), sb);
            umma::st_keep1(DQP + p4f(r0 + i, c), sq);
          }
#pragma unroll
          for (int j = 0; j < 16; ++j) umma::st_keep1(DKP + p4f(r0 + j, c), sk[j]);
        }
        DN_MARK(21 + 3 * half);
        __syncthreads();
        DN_MARK(22 + 3 * half);
      }
    }

    DN_MARK(9);
    // ---- H. three levels
    auto build = [&](int lv) {
      const int s = 16 << lv;
      static_assert(IMG == 4 * NT, "four pieces per thread");
#pragma unroll
      for (int half = 0; half < 2; ++half) {           // dA_s, dM_s: the entries this level owns
        float4 a0[2], a1[2], m0[2], m1[2];
        bool own[2];
#pragma unroll
        for (int u = 0; u < 2; ++u) {                  // predicated, branch-free loads: only the level's own entries
          const int e = (2 * half + u) * NT + tid, p = e >> 7, x = e & 127;
          const int bi = x >> 4, bj = p >> 1;
          own[u] = bj < bi && owner_level(bi, bj) == lv;
          a0[u] = umma::ld_keep4_pred(DA4 + p4v(x, 8 * p), own[u]); a1[u] = umma::ld_keep4_pred(DA4 + p4v(x, 8 * p + 4), own[u]);
          m0[u] = umma::ld_keep4_pred(DM4 + p4v(x, 8 * p), own[u]); m1[u] = umma::ld_keep4_pred(DM4 + p4v(x, 8 * p + 4), own[u]);
        }
#pragma unroll
        for (int u = 0; u < 2; ++u) {
          const int e = (2 * half + u) * NT + tid;
          uint4 va = make_uint4(umma::pack2(a0[u].x, a0[u].y), umma::pack2(a0[u].z, a0[u].w), umma::pack2(a1[u].x, a1[u].y), umma::pack2(a1[u].z, a1[u].w));
          uint4 vm = make_uint4(umma::pack2(m0[u].x, m0[u].y), umma::pack2(m0[u].z, m0[u].w), umma::pack2(m1[u].x, m1[u].y), umma::pack2(m1[u].z, m1[u].w));
          I_DA[e] = va;
          I_DM[e] = vm;
        }
      }
      if (tm_cache) {
        const int x = (warp & 3) * 32 + lane;
        const uint32_t tl = cx.tmem + ((uint32_t)((warp & 3) * 32) << 16);
#pragma unroll 2
        for (int j = 0; j < 4; ++j) {
          const int p = (warp >> 2) * 4 + j;
          float kq[8], be8[8], kh[8], qh[8];
          umma::tmem_ld8(tl + COL_KQ + 8 * p, kq);
          umma::tmem_ld8(tl + COL_BE + 8 * p, be8);
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            kh[i] = __uint_as_float(__float_as_uint(kq[i]) << 16);
            qh[i] = __uint_as_float(__float_as_uint(kq[i]) & 0xffff0000u);
          }
          build_level_from_beta(kh, be8, qh, LAM, s, x, p, I_KR, I_QK);
        }
      } else {
#pragma unroll 2
        for (int it = 0; it < 4; ++it) build_level_piece(r, LAM, s, myrow, it * 4 + lgrp, I_KR, I_QK);
      }
    };
    auto drain_level = [&](int lv) {
      const int s = 16 << lv;
      const int quarter = warp & 3, group = warp >> 2;
      const int x = quarter * 32 + lane, ref = level_ref(x, s);
      const bool lower = x >= ref;
      const uint32_t tbase = cx.tmem + ((uint32_t)(quarter * 32) << 16);
      // one code path for both roles: a lower row adds rowfac * T1 to dbeta' and rowfac * T2 to dq',
      // an upper row adds colfac * (T1 + T2) to dk'
      float4* const pb = lower ? DBP4 : DKP4;
      const float* const la = LAM + (lower ? x : ref) * LP;
      const float* const lb = LAM + (lower ? ref : x) * LP;
#pragma unroll 1
      for (int cc = 0; cc < 32; cc += 16) {
        const int col = group * 32 + cc;
        float4 ob[4], oq[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) { ob[i] = umma::ld_keep4(pb + p4v(x, col + 4 * i)); oq[i] = umma::ld_keep4_pred(DQP4 + p4v(x, col + 4 * i), lower); }
        float t1[16], t2[16];
        if (!cx.dead) {
          umma::tmem_ld16(tbase + col, t1);
          umma::tmem_ld16(tbase + 128 + col, t2);
        } else {
#pragma unroll
          for (int i = 0; i < 16; ++i) t1[i] = t2[i] = 0.f;
        }
        float f[16];
        decay8(la + col, lb + col, *reinterpret_cast<float(*)[8]>(f));
        decay8(la + col + 8, lb + col + 8, *reinterpret_cast<float(*)[8]>(f + 8));
#pragma unroll
        for (int i = 0; i < 16; ++i) t1[i] = lower ? t1[i] : t1[i] + t2[i];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          ob[i].x = fmaf(t1[4 * i], f[4 * i], ob[i].x); ob[i].y = fmaf(t1[4 * i + 1], f[4 * i + 1], ob[i].y);
          ob[i].z = fmaf(t1[4 * i + 2], f[4 * i + 2], ob[i].z); ob[i].w = fmaf(t1[4 * i + 3], f[4 * i + 3], ob[i].w);
          oq[i].x = fmaf(t2[4 * i], f[4 * i], oq[i].x); oq[i].y = fmaf(t2[4 * i + 1], f[4 * i + 1], oq[i].y);
          oq[i].z = fmaf(t2[4 * i + 2], f[4 * i + 2], oq[i].z); oq[i].w = fmaf(t2[4 * i + 3], f[4 * i + 3], oq[i].w);
          umma::st_keep4(pb + p4v(x, col + 4 * i), ob[i]);
          if (lower) umma::st_keep4(DQP4 + p4v(x, col + 4 * i), oq[i]);
        }
      }
      umma::tc_fence_before();
    };
    // one rolled loop, one call site each: build(lv) and drain(lv - 1) share a barrier interval (the
    // images are free once the products of lv - 1 have completed), then the products of lv are issued
#pragma unroll 1
    for (int lv = 0; lv <= 3; ++lv) {
      if (lv < 3) build(lv);
      if (lv > 0) drain_level(lv - 1);
      if (lv < 3) {
        umma::pre_issue_sync();
        umma::issue<128, false, true>(cx, I_DA, I_KR, C, 0, false);        // dA_s   KR
        umma::issue<128, true, true>(cx, I_DA, I_KR, C, 0, true);          // dA_s^T KR
        umma::issue<128, false, true>(cx, I_DM, I_QK, C, 128, false);      // dM_s   QK
        umma::issue<128, true, true>(cx, I_DM, I_QK, C, 128, true);        // dM_s^T QK
        umma::commit_wait(cx);
        DN_MARK(10 + lv);
      }
    }
    __syncthreads();
    }
    }

    DN_MARK(13);
    // ---- E. combination.  Thread mapping of a tensor-memory drain: warp w owns rows 32 (w % 4) + lane
    //         and the 32 channels [32 (w / 4), +32), walked in four pieces of 8.  dbeta', dq', dk' come
    //         straight from the accumulators of the two product rounds when the chunk took a single-Gram
    //         route (tm_src != 0), else from the scratch panels.  dLambda and dke*ke go to shared memory,
    //         d b is written.  The l2norm adjoint needs each row's <q_n, dq_n> and <k_n, dk_n>, whose
    //         four partial sums sit in four warps: they meet in shared memory; until then a thread
    //         parks its d q_n, d k_n, q_n, k_n in the tensor-memory columns it has just read (and in
    //         [384, 512)), so nothing goes through global memory twice.
    {
      umma::tc_fence_after();
      const int fq = warp & 3, fg = warp >> 2;
      const uint32_t tb = cx.tmem + ((uint32_t)(fq * 32) << 16) + (uint32_t)(fg * 32);
      const int x = fq * 32 + lane, t = t0 + x;
      const bool live = x < r.rows_valid;
      const bool first = seg_s[x] == seg0, last = seg_s[x] == segL;
      const float dmii = umma::ld_keep1(DM + p4f(x, x));
      const float rq = rq_s[x], rk = rk_s[x];
      const size_t tok = (size_t)b * g.L + t;
      const size_t outb = (tok * g.H + h) * r.bC;
      const size_t outqk = (tok * g.H + h) * K;
      const bool tm_live = tm_src != 0 && !cx.dead;
      float dq_dot = 0.f, dk_dot = 0.f, sb2 = 0.f;
#pragma unroll 1
      for (int it = 0; it < 4; ++it) {
        const int p = fg * 4 + it;
        float qr[8], kr[8], ba[8], braw[8], dbp[8], dqp[8], dkp[8], dx[8], dqe[8], dke[8];
        raw_q8(r, x, p, qr);
        raw_k8(r, x, p, kr);
        bact8(r, x, p, ba);
        if (!fuse && guard) raw_gate8(r.b, r.b_row0, r.b_pitch, r.bC, r.gate_dt, live ? x : 0, p, braw);
        if (tm_src != 0) {
          if (tm_live) {
            umma::tmem_ld8(tb + it * 8, dbp);
            umma::tmem_ld8(tb + 128 + it * 8, dqp);
            umma::tmem_ld8(tb + 256 + it * 8, dkp);
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) dbp[i] = dqp[i] = dkp[i] = 0.f;
          }
        } else {
          ld2x4(DBP4 + p4v(x, 8 * p), dbp);
          ld2x4(DQP4 + p4v(x, 8 * p), dqp);
          ld2x4(DKP4 + p4v(x, 8 * p), dkp);
        }
        ld2x4(DX4 + p4v(x, 8 * p), dx);
        ld2x4(DQE4 + p4v(x, 8 * p), dqe);
        ld2x4(DKE4 + p4v(x, 8 * p), dke);
        float lam[8], lend[8], odl[8], odk[8], odb[8];
        *reinterpret_cast<float4*>(lam) = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p);
        *reinterpret_cast<float4*>(lam + 4) = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p + 4);
        *reinterpret_cast<float4*>(lend) = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p);
        *reinterpret_cast<float4*>(lend + 4) = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p + 4);
        if (tm_src == 1) {                                       // f = e^{Lambda - the document's midpoint}
          const float* ls = LAM + ds_s[x] * LP + 8 * p;
          const float* le = LAM + de_s[x] * LP + 8 * p;
          const float4 s0 = *reinterpret_cast<const float4*>(ls), s1 = *reinterpret_cast<const float4*>(ls + 4);
          const float4 e0 = *reinterpret_cast<const float4*>(le), e1 = *reinterpret_cast<const float4*>(le + 4);
          const float m8[8] = {s0.x + e0.x, s0.y + e0.y, s0.z + e0.z, s0.w + e0.w, s1.x + e1.x, s1.y + e1.y, s1.z + e1.z, s1.w + e1.w};
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float d = (lam[i] - 0.5f * m8[i]) * DN_LOG2E;
            const float f = umma::ex2_fast(d);
            dbp[i] *= f; dqp[i] *= f; dkp[i] *= umma::ex2_fast(-d);
          }
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float qh = (qr[i] * rq) * r.scale, kh = kr[i];
          if (r.round_in) qh = bf16r(qh);
          if (l2) { kh *= rk; if (r.round_in) kh = bf16r(kh); }
          const float el = umma::exp_neg(fminf(lam[i], 0.f)), eke = umma::exp_neg(fminf(lend[i] - lam[i], 0.f));
          const float be = ba[i] * kh;
          const float X = first ? be * el : 0.f, qe = first ? qh * el : 0.f, ke = last ? kh * eke : 0.f;
          const float dbeta = dbp[i] + (first ? dx[i] * el : 0.f);
          const float dq = dqp[i] + dmii * kh + (first ? dqe[i] * el : 0.f);
          const float dk = dkp[i] + dmii * qh + (last ? dke[i] * eke : 0.f) + dbeta * ba[i];
          odl[i] = be * dbp[i] + qh * dqp[i] - kh * dkp[i] + dx[i] * X + dqe[i] * qe;
          odk[i] = dke[i] * ke;
          float dbv = dbeta * kh;                               // d b_act
          if (fuse) dbv *= ba[i] * (1.f - ba[i]);               // through the sigmoid
          else if (guard) dbv *= braw[i] > 0.f ? 1.f : (braw[i] == 0.f ? 0.5f : 0.f);   // through max(b, 0)
          odb[i] = dbv;
          sb2 += dbv;
          dqp[i] = dq * g.scale;                                // d q_n (before the l2norm adjoint)
          dkp[i] = dk;
          qr[i] *= rq;                                          // q_n, k_n
          kr[i] *= rk;
          dq_dot = fmaf(qr[i], dqp[i], dq_dot);
          dk_dot = fmaf(kr[i], dkp[i], dk_dot);
        }
        umma::tmem_st8(tb + 128 + it * 8, dqp);
        umma::tmem_st8(tb + 256 + it * 8, dkp);
        umma::tmem_st8(tb + it * 8, qr);
        umma::tmem_st8(tb + 384 + it * 8, kr);
        *reinterpret_cast<float4*>(DLs + x * LP + 8 * p) = make_float4(odl[0], odl[1], odl[2], odl[3]);
        *reinterpret_cast<float4*>(DLs + x * LP + 8 * p + 4) = make_float4(odl[4], odl[5], odl[6], odl[7]);
        *reinterpret_cast<float4*>(DKs + x * LP + 8 * p) = make_float4(odk[0], odk[1], odk[2], odk[3]);
        *reinterpret_cast<float4*>(DKs + x * LP + 8 * p + 4) = make_float4(odk[4], odk[5], odk[6], odk[7]);
        if (live && r.bC != 1) out8(a.db, outb + 8 * p, a.db_dt, odb);
      }
      // the four channel groups of a row meet here (added in a fixed order)
      TOT[fg * 128 + x] = dq_dot;
      TOT[512 + fg * 128 + x] = dk_dot;
      TOT[1024 + fg * 128 + x] = sb2;
      umma::tmem_wait_st();
      __syncthreads();
      dq_dot = (TOT[x] + TOT[128 + x]) + (TOT[256 + x] + TOT[384 + x]);
      dk_dot = (TOT[512 + x] + TOT[640 + x]) + (TOT[768 + x] + TOT[896 + x]);
      if (r.bC == 1 && fg == 0 && live)
        stf(a.db, outb, (TOT[1024 + x] + TOT[1152 + x]) + (TOT[1280 + x] + TOT[1408 + x]), a.db_dt);
#pragma unroll 2
      for (int it = 0; it < 4; ++it) {
        const int p = fg * 4 + it;
        float qn[8], kn[8], dqn[8], dkn[8];
        umma::tmem_ld8(tb + 128 + it * 8, dqn);
        umma::tmem_ld8(tb + 256 + it * 8, dkn);
        umma::tmem_ld8(tb + it * 8, qn);
        umma::tmem_ld8(tb + 384 + it * 8, kn);
        if (l2) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            dqn[i] = rq * (dqn[i] - qn[i] * dq_dot);
            dkn[i] = rk * (dkn[i] - kn[i] * dk_dot);
          }
        }
        if (live) {
          out8(a.dq, outqk + 8 * p, a.dq_dt, dqn);
          out8(a.dk, outqk + 8 * p, a.dq_dt, dkn);
        }
      }
      umma::tc_fence_before();
    }
    __syncthreads();

    DN_MARK(14);
    // ---- R. dg_t = sum_{i >= t, same doc} dLambda_i + the Lambda_end path (prefix sum of dke*ke over
    //         earlier rows of the last document, plus the carried-state term).  Thread (channel c,
    //         quarter qd) scans 32 rows in registers; the quarters are chained through shared memory.
    {
      const int c = tid & 127, qd = tid >> 7, x0 = qd * 32;
      float v[32];
      float run = 0.f, ksum = 0.f;
      int nb = -1;                                  // lowest row (largest index) after which a document ends
#pragma unroll
      for (int i = 31; i >= 0; --i) {
        const int x = x0 + i;
        if (i < 31 && seg_s[x] != seg_s[x + 1]) { run = 0.f; if (nb < 0) nb = i; }
        run += DLs[x * LP + c];
        v[i] = run;
        if (seg_s[x] == segL) ksum += DKs[x * LP + c];
      }
      TOT[qd * 128 + c] = run;                      // sum from the quarter's first row to its first document end
      TOT[512 + qd * 128 + c] = ksum;
      if (c == 0) reset_s[4 + qd] = nb >= 0;
      __syncthreads();
      // what flows in from the rows below this quarter
      float carry = 0.f;
      for (int q2 = 3; q2 > qd; --q2) {
        const bool joins = seg_s[q2 * 32] == seg_s[q2 * 32 - 1];      // quarter q2 continues the document above it
        const float inner = reset_s[4 + q2] ? 0.f : carry;              // what passed through all of q2
        carry = joins ? TOT[q2 * 128 + c] + inner : 0.f;
      }
      float acc = dlend_s[c];
      for (int q2 = 0; q2 < qd; ++q2) acc += TOT[512 + q2 * 128 + c];
#pragma unroll
      for (int i = 0; i < 32; ++i) {
        const int x = x0 + i;
        float o = v[i] + (i > nb ? carry : 0.f);
        if (seg_s[x] == segL) { o += acc; acc += DKs[x * LP + c]; }
        DLs[x * LP + c] = o;
      }
    }
    __syncthreads();

    DN_MARK(15);
    // ---- dg: one warp per row, 4 channels per lane
    {
      const int hg = g.gate_head(h, g.gH);
#pragma unroll 4
      for (int i = warp; i < C; i += NT / 32) {
        const bool live = t0 + i < g.L;
        const int t = live ? t0 + i : t0;              // a row past the end reads row 0 and writes nothing
        const size_t tok = (size_t)b * g.L + t;
        const size_t rowg = (tok * g.gH + hg) * r.gC, outg = (tok * g.H + h) * r.gC;
        const float4 dl = *reinterpret_cast<const float4*>(DLs + i * LP + 4 * lane);
        float dgv[4] = {dl.x, dl.y, dl.z, dl.w}, gr[4];
        if (r.gC == 1) { gr[0] = gr[1] = gr[2] = gr[3] = ldf_ro(a.gg, rowg, gdt); }
        else if (gdt == DN_BF16) {
          const uint2 u = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.gg) + rowg + 4 * lane));
          gr[0] = __uint_as_float(u.x << 16); gr[1] = __uint_as_float(u.x & 0xffff0000u);
          gr[2] = __uint_as_float(u.y << 16); gr[3] = __uint_as_float(u.y & 0xffff0000u);
        } else {
          const float4 u = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.gg) + rowg + 4 * lane));
          gr[0] = u.x; gr[1] = u.y; gr[2] = u.z; gr[3] = u.w;
        }
        float sg = 0.f;
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          if (fuse) {
            const float gexp = -expf(fminf(gr[u], 5.f));
            const bool pass = gr[u] <= 5.f && (!guard || gexp < -1e-6f);
            dgv[u] = pass ? dgv[u] * gexp : 0.f;
          } else {
            dgv[u] = (guard ? gr[u] < -1e-6f : gr[u] <= 0.f) ? dgv[u] : 0.f;      // through min(min(g, 0), -1e-6)
          }
          sg += dgv[u];
        }
        if (r.gC == 1) { sg = warp_sum(sg); if (lane == 0 && live) stf(a.dg, outg, sg, a.dg_dt); }
        else if (!live) { }
        else if (a.dg_dt == DN_BF16)
          *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.dg) + outg + 4 * lane) = make_uint2(umma::pack2(dgv[0], dgv[1]), umma::pack2(dgv[2], dgv[3]));
        else
          *reinterpret_cast<float4*>(reinterpret_cast<float*>(a.dg) + outg + 4 * lane) = make_float4(dgv[0], dgv[1], dgv[2], dgv[3]);
      }
    }

    DN_MARK(16);
    __syncthreads();
#ifdef DN_PHASE_TIMING
    DN_MARK(17);
    if (blockIdx.x == 0 && tid == 0 && e_item == 0) {
      for (int i = 1; i < 18; ++i) printf("mark %d -> %d: %lld\n", i - 1, i, g_phase_marks[i] - g_phase_marks[i - 1]);
      printf("item total %lld\n", g_phase_marks[17] - g_phase_marks[0]);
      printf("D: stage0 %lld compute0(warp0) %lld wait0 %lld stage1 %lld compute1 %lld wait1 %lld\n", g_phase_marks[20] - g_phase_marks[8],
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

size_t prepass_bwd_tc_scratch_per_cta(const Geo&) { return (size_t)6 * C * K + (size_t)2 * C * C; }

int launch_prepass_bwd_tc(PrepassBwdArgs& a, size_t scratch_floats, cudaStream_t st) {
  const Geo& g = a.g;
  if (a.c_end <= 0) { a.c_begin = 0; a.c_end = g.NC; }
  a.items = g.B * g.H * (a.c_end - a.c_begin);
  if (a.items <= 0) return DN_OK;
  a.scratch_per_cta = prepass_bwd_tc_scratch_per_cta(g);
  a.err = device_error_ptr();
  const int grid = a.items < sm_count() ? a.items : sm_count();
  if (scratch_floats < (size_t)grid * a.scratch_per_cta) return DN_ERR_SCRATCH_TOO_SMALL;
  const size_t lam_phase = (size_t)C * LP * 4 + 4 * 32768;
  size_t smem = bwd_tc_image_bytes(g.Vw);
  if (smem < lam_phase) smem = lam_phase;
  if (smem < (size_t)3 * C * LP * 4 + 6144) smem = (size_t)3 * C * LP * 4 + 6144;
  auto go = [&](auto kernel) {
    cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    kernel<<<grid, NT, smem, st>>>(a);
  };
  const int mode = input_mode(g);
  auto al16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; };
  a.bulk_v = mode == 0 && g.V == 128 && a.dw_dt == DN_F32 && al16(a.v) && al16(a.w) && al16(a.dv) && al16(a.dw);
  if (g.Vw == 256) {
    if (mode == 0) go(prepass_bwd_tc_kernel<256, 0>); else if (mode == 1) go(prepass_bwd_tc_kernel<256, 1>); else if (mode == 3) go(prepass_bwd_tc_kernel<256, 3>); else if (mode == 4) go(prepass_bwd_tc_kernel<256, 4>); else go(prepass_bwd_tc_kernel<256, 2>);
  } else {
    if (mode == 0) go(prepass_bwd_tc_kernel<128, 0>); else if (mode == 1) go(prepass_bwd_tc_kernel<128, 1>); else if (mode == 3) go(prepass_bwd_tc_kernel<128, 3>); else if (mode == 4) go(prepass_bwd_tc_kernel<128, 4>); else go(prepass_bwd_tc_kernel<128, 2>);
  }
  return launch_status();
}

}  // namespace dn
