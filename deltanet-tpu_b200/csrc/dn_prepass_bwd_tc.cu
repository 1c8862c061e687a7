// Chunk-parallel backward on the tcgen05 tensor cores (bf16 precision, chunk = K = 128, value
// width 128 or 256): the adjoint of the state step's value-width contractions, of the prepass
// (reference: src/deltanet_tpu/gdn2.py:243-493, 750-762) and of the fused prologue (558-575).
//
// Per (batch, exec head, chunk), 512 threads, one CTA per SM:
//   G. nine matrix products (bwd_gemms_tc): V_new, dqe, dM, dW, dke, dX, dY, dA.
//   L. the cumulative log-decay of the chunk in shared memory.
//   H. adjoints of A and M through the same three-level factorisation as the forward: per level
//        dbeta' += rowfac * (dA_s kc),  dq' += rowfac * (dM_s kc),
//        dk'    += colfac * (dA_s^T rb + dM_s^T rq)
//      where dA_s / dM_s keep only the entries the level owns, kc / rb / rq are the level's scaled
//      operand images and rowfac / colfac the same exp(Lam - Lam_ref) factors (all <= 1).
//   D. the 16x16 diagonal blocks, exact, one thread per (block, channel).
//   C. combination into dLambda, d q_hat, d k_hat, d b; R. dg by a within-document reverse
//      cumulative sum; W. row pass (gate adjoints, l2norm adjoint, writes); V. dv and dw.
#include "dn_chunkprep.cuh"
#include "dn_kernels.cuh"
#include "dn_prepass_bwd_tc.cuh"

namespace dn {
namespace {

using namespace prep;
constexpr int NT = 512;

template <int VW>
__global__ void __launch_bounds__(NT, 1) prepass_bwd_tc_kernel(PrepassBwdArgs a) {
  extern __shared__ __align__(128) uint8_t smraw[];
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_base;
  __shared__ int seg_s[C];
  __shared__ float rq_s[C], rk_s[C], dlend_s[K];
  const Geo& g = a.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int OFF_IMG = C * LP * 4;
  float* LAM = reinterpret_cast<float*>(smraw);
  uint4* I_DA = reinterpret_cast<uint4*>(smraw + OFF_IMG);
  uint4* I_DM = I_DA + IMG;
  uint4* I_KR = I_DM + IMG;                 // kc, then rb
  uint4* I_RQ = I_KR + IMG;
  float* DLs = reinterpret_cast<float*>(smraw + OFF_IMG);          // dLambda (pitch LP), over the images
  float* DKs = DLs + C * LP;                                        // dke*ke   (pitch LP)

  const size_t CK = (size_t)C * K, CV = (size_t)C * VW, CC = (size_t)C * C;
  float* sc = a.scratch + (size_t)blockIdx.x * a.scratch_per_cta;
  float* DQE = sc;          float* DKE = DQE + CK;   float* DX = DKE + CK;
  float* DBP = DX + CK;     float* DQP = DBP + CK;   float* DKP = DQP + CK;
  float* DY = DKP + CK;     float* DM = DY + CV;     float* DA = DM + CC;

  if (tid == 0) { umma::mbar_init(&mma_bar, 1); umma::fence_mbar_init(); }
  if (warp == 0) umma::tmem_alloc(&tmem_base, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &mma_bar, 0u, a.err, false};

  const bool l2 = g.flags & DN_QK_L2NORM, fuse = g.flags & DN_FUSE_PROLOGUE;
  const bool guard = g.flags & DN_STABILITY_GUARD;
  const bool trunc = g.flags & DN_TRUNC_DT_BF16;

  for (int item = blockIdx.x; item < a.items; item += gridDim.x) {
    const int c_idx = item % g.NC, h = (item / g.NC) % g.H, b = item / (g.NC * g.H);
    const int t0 = c_idx * C;
    const size_t ibase = (size_t)item;
    for (int i = tid; i < C; i += NT) seg_s[i] = seg_at(a.seg, b, t0 + i, g.L);
    bool is_new, all_same;
    chunk_flags(a.seg, g, b, c_idx, is_new, all_same);
    const float* S = a.res.states + ibase * K * VW;
    const float* dH = a.dH + ibase * K * VW;
    // dLambda_end from the carried state: [one doc] sum_v dH*S*exp(Lambda_end)   (gdn2.py:759-762)
    for (int kk = warp; kk < K; kk += NT / 32) {
      float s = 0.f;
      for (int j = lane; j < VW; j += 32) s += dH[(size_t)kk * VW + j] * S[(size_t)kk * VW + j];
      s = warp_sum(s);
      if (lane == 0) dlend_s[kk] = all_same ? s * expf(fminf(a.res.lam_end[ibase * K + kk], 0.f)) : 0.f;
    }
    __syncthreads();
    const int seg0 = seg_s[0], segL = seg_s[C - 1];

    // ---- G. the matrix products
    {
      BwdTcIo io;
      io.W = reinterpret_cast<const __nv_bfloat16*>(a.res.W) + ibase * CK;
      io.U = reinterpret_cast<const __nv_bfloat16*>(a.res.U) + ibase * CV;
      io.S = S; io.dH = dH; io.dV = a.dV + ibase * CV; io.T = a.res.T + ibase * CC;
      io.d_out = a.d_out; io.qkv_dt = g.qkv_dt;
      io.dO_off = ((size_t)b * g.L + t0) * g.Hv * g.V + (size_t)h * VW;
      io.dO_pitch = (size_t)g.Hv * g.V;
      io.rows_valid = g.L - t0 < C ? g.L - t0 : C;
      io.DQE = DQE; io.DKE = DKE; io.DX = DX; io.DY = DY; io.DM = DM; io.DA = DA;
      io.seg_s = seg_s; io.trunc = trunc;
      bwd_gemms_tc<VW, NT>(cx, smraw, io);
    }

    // ---- L. rows, normalisers, cumulative decay; zero the accumulators of phase H
    const Rows r = make_rows(g, a.q, a.k, a.gg, a.b, b, h, t0, rq_s, rk_s);
    row_norms<NT>(r, rq_s, rk_s);
    for (int e = tid; e < 3 * C * K / 4; e += NT) reinterpret_cast<float4*>(DBP)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    __syncthreads();
    build_lambda<NT>(r, seg_s, LAM);

    // ---- H. three levels
    for (int lv = 0; lv < 3; ++lv) {
      const int s = 16 << lv;
      for (int e = tid; e < IMG; e += NT) {            // dA_s, dM_s: the entries this level owns
        const int p = e >> 7, x = e & 127;
        const int bi = x >> 4, bj = p >> 1;
        uint4 va = make_uint4(0, 0, 0, 0), vm = va;
        if (bj < bi && owner_level(bi, bj) == lv) {
          va = umma::ld8_f32(DA + x * C + 8 * p);
          vm = umma::ld8_f32(DM + x * C + 8 * p);
        }
        I_DA[e] = va;
        I_DM[e] = vm;
      }
      build_level<NT>(r, LAM, s, nullptr, I_RQ, I_KR);               // kc and rq
      umma::pre_issue_sync();
      umma::issue<128, false, true>(cx, I_DA, I_KR, C, 0, false);    // dA_s kc
      umma::issue<128, false, true>(cx, I_DM, I_KR, C, 128, false);  // dM_s kc
      umma::commit_wait(cx);
      build_level<NT>(r, LAM, s, I_KR, nullptr, nullptr);            // rb over kc
      umma::pre_issue_sync();
      umma::issue<128, true, true>(cx, I_DA, I_KR, C, 256, false);   // dA_s^T rb
      umma::issue<128, true, true>(cx, I_DM, I_RQ, C, 256, true);    //  + dM_s^T rq
      umma::commit_wait(cx);
      {
        const int quarter = warp & 3, group = warp >> 2;
        const int x = quarter * 32 + lane, ref = level_ref(x, s);
        const bool lower = x >= ref;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        for (int c = 0; c < 32; c += 16) {
          const int col = group * 32 + c;
          float vb[16], vq[16], vk[16];
          if (!cx.dead) {
            umma::tmem_ld16(cx.tmem + lane_base + col, vb);
            umma::tmem_ld16(cx.tmem + lane_base + 128 + col, vq);
            umma::tmem_ld16(cx.tmem + lane_base + 256 + col, vk);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) vb[i] = vq[i] = vk[i] = 0.f;
          }
          float f0[8], f1[8];
          if (lower) {
            decay8(LAM + x * LP + col, LAM + ref * LP + col, f0);
            decay8(LAM + x * LP + col + 8, LAM + ref * LP + col + 8, f1);
            float4* db = reinterpret_cast<float4*>(DBP + x * K + col);
            float4* dq = reinterpret_cast<float4*>(DQP + x * K + col);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float* f = i < 2 ? f0 + 4 * i : f1 + 4 * (i - 2);
              float4 ob = db[i], oq = dq[i];
              ob.x += vb[4 * i] * f[0]; ob.y += vb[4 * i + 1] * f[1]; ob.z += vb[4 * i + 2] * f[2]; ob.w += vb[4 * i + 3] * f[3];
              oq.x += vq[4 * i] * f[0]; oq.y += vq[4 * i + 1] * f[1]; oq.z += vq[4 * i + 2] * f[2]; oq.w += vq[4 * i + 3] * f[3];
              db[i] = ob;
              dq[i] = oq;
            }
          } else {
            decay8(LAM + ref * LP + col, LAM + x * LP + col, f0);
            decay8(LAM + ref * LP + col + 8, LAM + x * LP + col + 8, f1);
            float4* dk = reinterpret_cast<float4*>(DKP + x * K + col);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
              const float* f = i < 2 ? f0 + 4 * i : f1 + 4 * (i - 2);
              float4 ok = dk[i];
              ok.x += vk[4 * i] * f[0]; ok.y += vk[4 * i + 1] * f[1]; ok.z += vk[4 * i + 2] * f[2]; ok.w += vk[4 * i + 3] * f[3];
              dk[i] = ok;
            }
          }
        }
        umma::tc_fence_before();
      }
      __syncthreads();
    }

    // ---- D. diagonal 16x16 blocks, exact: one thread per (block, channel).  Row side first
    //         (dbeta'_i, dq'_i: one output row at a time, inner loop over the earlier rows j), then
    //         the column side (dk'_j, inner loop over the later rows i).
    for (int task = tid; task < 8 * K; task += NT) {
      const int r0 = (task >> 7) * 16, c = task & 127;
      float lam[16], kh[16], be[16], qh[16];
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const int x = r0 + i;
        lam[i] = LAM[x * LP + c] * DN_LOG2E;
        float kv = 0.f, qv = 0.f, bv = 0.f;
        if (x < r.rows_valid) {
          kv = ldf(r.k, r.qk_row0 + (size_t)x * r.qk_pitch + c, r.qkv_dt);
          qv = ldf(r.q, r.qk_row0 + (size_t)x * r.qk_pitch + c, r.qkv_dt);
          bv = ldf(r.b, r.b_row0 + (size_t)x * r.b_pitch + (r.bC == 1 ? 0 : c), r.gate_dt);
          if (l2) { kv *= rk_s[x]; if (r.round_in) kv = bf16r(kv); }
          qv = (qv * rq_s[x]) * r.scale;
          if (r.round_in) qv = bf16r(qv);
          if (fuse) bv = 1.f / (1.f + expf(-bv));
        }
        kh[i] = kv; qh[i] = qv; be[i] = bv * kv;
      }
#pragma unroll 1
      for (int i = 1; i < 16; ++i) {
        const float li = LAM[(r0 + i) * LP + c] * DN_LOG2E;
        const float* da = DA + (r0 + i) * C + r0;
        const float* dm = DM + (r0 + i) * C + r0;
        float sb = 0.f, sq = 0.f;
#pragma unroll
        for (int j = 0; j < 15; ++j) {
          if (j < i) {
            const float ek = exp2f(fminf(li - lam[j], 0.f)) * kh[j];
            sb = fmaf(da[j], ek, sb);
            sq = fmaf(dm[j], ek, sq);
          }
        }
        DBP[(r0 + i) * K + c] += sb;
        DQP[(r0 + i) * K + c] += sq;
      }
#pragma unroll 1
      for (int j = 0; j < 15; ++j) {
        const float lj = LAM[(r0 + j) * LP + c] * DN_LOG2E;
        float sk = 0.f;
#pragma unroll
        for (int i = 1; i < 16; ++i) {
          if (i > j) {
            const float e = exp2f(fminf(lam[i] - lj, 0.f));
            sk = fmaf(fmaf(DA[(r0 + i) * C + r0 + j], be[i], DM[(r0 + i) * C + r0 + j] * qh[i]), e, sk);
          }
        }
        DKP[(r0 + j) * K + c] += sk;
      }
    }
    __syncthreads();

    // ---- C. combine (pieces of 8 channels): dLambda and dke*ke to shared memory; d q_hat, d k_hat,
    //         d b_act in place over DQP, DKP, DBP
    for (int e = tid; e < IMG; e += NT) {
      const int x = e >> 4, p = e & 15;
      float qh[8], kh[8], ba[8];
      qhat8(r, x, p, qh);
      khat8(r, x, p, kh);
      bact8(r, x, p, ba);
      const bool first = seg_s[x] == seg0, last = seg_s[x] == segL;
      const float dmii = DM[x * C + x];
      float4* pDB = reinterpret_cast<float4*>(DBP + x * K + 8 * p);
      float4* pDQ = reinterpret_cast<float4*>(DQP + x * K + 8 * p);
      float4* pDK = reinterpret_cast<float4*>(DKP + x * K + 8 * p);
      const float4* pDX = reinterpret_cast<const float4*>(DX + x * K + 8 * p);
      const float4* pQE = reinterpret_cast<const float4*>(DQE + x * K + 8 * p);
      const float4* pKE = reinterpret_cast<const float4*>(DKE + x * K + 8 * p);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        float4 vdb = pDB[hh], vdq = pDQ[hh], vdk = pDK[hh];
        const float4 vdx = pDX[hh], vqe = pQE[hh], vke = pKE[hh];
        const float4 vl = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p + 4 * hh);
        const float4 vle = *reinterpret_cast<const float4*>(LAM + (C - 1) * LP + 8 * p + 4 * hh);
        float dbp[4] = {vdb.x, vdb.y, vdb.z, vdb.w}, dqp[4] = {vdq.x, vdq.y, vdq.z, vdq.w}, dkp[4] = {vdk.x, vdk.y, vdk.z, vdk.w};
        const float dx[4] = {vdx.x, vdx.y, vdx.z, vdx.w}, dqe[4] = {vqe.x, vqe.y, vqe.z, vqe.w}, dke[4] = {vke.x, vke.y, vke.z, vke.w};
        const float lam[4] = {vl.x, vl.y, vl.z, vl.w}, lend[4] = {vle.x, vle.y, vle.z, vle.w};
        float odl[4], odk[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const int ci = 4 * hh + i;
          const float el = expf(fminf(lam[i], 0.f)), eke = expf(fminf(lend[i] - lam[i], 0.f));
          const float be = ba[ci] * kh[ci];
          const float X = first ? be * el : 0.f, qe = first ? qh[ci] * el : 0.f, ke = last ? kh[ci] * eke : 0.f;
          const float dbeta = dbp[i] + (first ? dx[i] * el : 0.f);
          const float dq = dqp[i] + dmii * kh[ci] + (first ? dqe[i] * el : 0.f);
          const float dk = dkp[i] + dmii * qh[ci] + (last ? dke[i] * eke : 0.f) + dbeta * ba[ci];
          odl[i] = be * dbp[i] + qh[ci] * dqp[i] - kh[ci] * dkp[i] + dx[i] * X + dqe[i] * qe;
          odk[i] = dke[i] * ke;
          dbp[i] = dbeta * kh[ci];     // d b_act
          dqp[i] = dq;
          dkp[i] = dk;
        }
        pDB[hh] = make_float4(dbp[0], dbp[1], dbp[2], dbp[3]);
        pDQ[hh] = make_float4(dqp[0], dqp[1], dqp[2], dqp[3]);
        pDK[hh] = make_float4(dkp[0], dkp[1], dkp[2], dkp[3]);
        *reinterpret_cast<float4*>(DLs + x * LP + 8 * p + 4 * hh) = make_float4(odl[0], odl[1], odl[2], odl[3]);
        *reinterpret_cast<float4*>(DKs + x * LP + 8 * p + 4 * hh) = make_float4(odk[0], odk[1], odk[2], odk[3]);
      }
    }
    __syncthreads();
    // ---- R. dg_t = sum_{i >= t, same doc} dLambda_i + the Lambda_end path (prefix sum of dke*ke over
    //         earlier rows of the last document, plus the carried-state term)
    if (tid < K) {
      const int c = tid;
      float run = 0.f;
      for (int i = C - 1; i >= 0; --i) {
        if (i < C - 1 && seg_s[i] != seg_s[i + 1]) run = 0.f;
        run += DLs[i * LP + c];
        DLs[i * LP + c] = run;
      }
      float acc = dlend_s[c];
      for (int i = 0; i < C; ++i) {
        if (seg_s[i] != segL) continue;
        DLs[i * LP + c] += acc;
        acc += DKs[i * LP + c];
      }
    }
    __syncthreads();
    // ---- W. row pass: gate adjoints, l2norm adjoint, writes (one warp per row, 4 channels per lane)
    const int hq = h / g.qk_div;
    const int hg = g.gate_head(h, g.gH), hb = g.gate_head(h, g.bH);
    for (int i = warp; i < C; i += NT / 32) {
      const int t = t0 + i;
      if (t >= g.L) continue;
      const size_t rowg = ((size_t)(b * (size_t)g.L + t) * g.gH + hg) * g.gC;
      const size_t outg = ((size_t)(b * (size_t)g.L + t) * g.H + h) * g.gC;
      const size_t outb = ((size_t)(b * (size_t)g.L + t) * g.H + h) * g.bC;
      const size_t rowqk = ((size_t)(b * (size_t)g.L + t) * g.Hk + hq) * K;
      const size_t outqk = ((size_t)(b * (size_t)g.L + t) * g.H + h) * K;
      const float rq = rq_s[i], rk = rk_s[i];
      float sg = 0.f, sb2 = 0.f, qn[4], kn[4], dqn[4], dkn[4], dq_dot = 0.f, dk_dot = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = lane + 32 * u;
        const float gr = ldf(a.gg, rowg + (g.gC == 1 ? 0 : c), g.gate_dt);
        float dgv = DLs[i * LP + c], dbv = DBP[i * K + c];
        if (fuse) {
          const float gexp = -expf(fminf(gr, 5.f));
          const bool pass = gr <= 5.f && (!guard || gexp < -1e-6f);
          dgv = pass ? dgv * gexp : 0.f;
          float bb = ldf(r.b, r.b_row0 + (size_t)i * r.b_pitch + (r.bC == 1 ? 0 : c), r.gate_dt);
          bb = 1.f / (1.f + expf(-bb));
          dbv = dbv * (bb * (1.f - bb));
        } else {
          dgv = gr <= 0.f ? dgv : 0.f;
        }
        if (g.gC == 1) sg += dgv; else stf(a.dg, outg + c, dgv, a.dg_dt);
        if (g.bC == 1) sb2 += dbv; else stf(a.db, outb + c, dbv, a.db_dt);
        qn[u] = ldf(a.q, rowqk + c, g.qkv_dt) * rq;
        kn[u] = ldf(a.k, rowqk + c, g.qkv_dt) * rk;
        dqn[u] = DQP[i * K + c] * g.scale;
        dkn[u] = DKP[i * K + c];
        dq_dot += qn[u] * dqn[u];
        dk_dot += kn[u] * dkn[u];
      }
      if (g.gC == 1) { sg = warp_sum(sg); if (lane == 0) stf(a.dg, outg, sg, a.dg_dt); }
      if (g.bC == 1) { sb2 = warp_sum(sb2); if (lane == 0) stf(a.db, outb, sb2, a.db_dt); }
      if (l2) { dq_dot = warp_sum(dq_dot); dk_dot = warp_sum(dk_dot); }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int c = lane + 32 * u;
        stf(a.dq, outqk + c, l2 ? rq * (dqn[u] - qn[u] * dq_dot) : dqn[u], a.dq_dt);
        stf(a.dk, outqk + c, l2 ? rk * (dkn[u] - kn[u] * dk_dot) : dkn[u], a.dq_dt);
      }
    }
    // ---- V. dv = dY * w_act, dw = dY * v (+ sigmoid adjoint; summed over a value head's columns
    //         when w is one scalar per head)
    constexpr int PV = VW / 8;
    const int pieces_per_head = g.V / 8;
    for (int e = tid; e < C * PV; e += NT) {
      const int x = e / PV, p = e - x * PV, t = t0 + x;
      float sw = 0.f;
      const int col0 = h * VW + 8 * p, hv = col0 / g.V, cv = col0 - hv * g.V;
      if (t < g.L) {
        const size_t vrow = (size_t)(b * (size_t)g.L + t) * g.Hv * g.V + col0;
        const size_t wrow = ((size_t)(b * (size_t)g.L + t) * g.wH + g.w_head(hv)) * g.wC;
        float vv[8], ww[8], dv8[8], dw8[8];
        load8(a.v, vrow, g.qkv_dt, vv);
        if (g.wC == 1) {
          const float w1 = ldf(a.w, wrow, g.gate_dt);
#pragma unroll
          for (int i = 0; i < 8; ++i) ww[i] = w1;
        } else {
          load8(a.w, wrow + cv, g.gate_dt, ww);
        }
        const float4 y0 = *reinterpret_cast<const float4*>(DY + (size_t)x * VW + 8 * p), y1 = *reinterpret_cast<const float4*>(DY + (size_t)x * VW + 8 * p + 4);
        const float dy[8] = {y0.x, y0.y, y0.z, y0.w, y1.x, y1.y, y1.z, y1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          float wa = ww[i], dwv = dy[i] * vv[i];
          if (fuse) { wa = 1.f / (1.f + expf(-ww[i])); dwv *= wa * (1.f - wa); }
          dv8[i] = dy[i] * wa;
          dw8[i] = dwv;
          sw += dwv;
        }
        if (g.qkv_dt == DN_BF16) *reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.dv) + vrow) = umma::pack8(dv8);
        else {
          float4* d = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.dv) + vrow);
          d[0] = make_float4(dv8[0], dv8[1], dv8[2], dv8[3]);
          d[1] = make_float4(dv8[4], dv8[5], dv8[6], dv8[7]);
        }
        if (g.wC != 1) {
          const size_t outw = ((size_t)(b * (size_t)g.L + t) * g.Hv + hv) * g.wC + cv;
#pragma unroll
          for (int i = 0; i < 8; ++i) stf(a.dw, outw + i, dw8[i], a.dw_dt);
        }
      }
      if (g.wC == 1) {
        for (int o = pieces_per_head >> 1; o > 0; o >>= 1) sw += __shfl_xor_sync(0xffffffffu, sw, o);
        if (t < g.L && (p % pieces_per_head) == 0)
          stf(a.dw, (size_t)(b * (size_t)g.L + t) * g.Hv + hv, sw, a.dw_dt);
      }
    }
    __syncthreads();
  }
  umma::tc_fence_before();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, 512);
}

}  // namespace

size_t prepass_bwd_tc_scratch_per_cta(const Geo& g) {
  return (size_t)6 * C * K + (size_t)C * g.Vw + (size_t)2 * C * C;
}

int launch_prepass_bwd_tc(PrepassBwdArgs& a, size_t scratch_floats, cudaStream_t st) {
  const Geo& g = a.g;
  a.items = g.B * g.H * g.NC;
  a.scratch_per_cta = prepass_bwd_tc_scratch_per_cta(g);
  a.err = device_error_ptr();
  const int grid = a.items < 148 ? a.items : 148;
  if (scratch_floats < (size_t)grid * a.scratch_per_cta) return DN_ERR_SCRATCH_TOO_SMALL;
  const size_t lam_phase = (size_t)C * LP * 4 + 4 * 32768;
  size_t smem = bwd_tc_image_bytes(g.Vw);
  if (smem < lam_phase) smem = lam_phase;
  if (smem < (size_t)3 * C * LP * 4) smem = (size_t)3 * C * LP * 4;
  if (g.Vw == 256) {
    cudaFuncSetAttribute(prepass_bwd_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    prepass_bwd_tc_kernel<256><<<grid, NT, smem, st>>>(a);
  } else {
    cudaFuncSetAttribute(prepass_bwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    prepass_bwd_tc_kernel<128><<<grid, NT, smem, st>>>(a);
  }
  return cudaGetLastError() == cudaSuccess ? DN_OK : DN_ERR_CUDA_LAUNCH;
}

}  // namespace dn
