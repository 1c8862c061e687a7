// Chunk-parallel backward, fp32 SIMT formulation.
//
// Per (batch, exec head, chunk) it forms the cotangents that the reference's state-backward
// kernel emits per chunk (src/deltanet_tpu/gdn2.py:750-762: dW, dM, dqe, dke, dLambda_end --
// contractions over the value width that need only the chunk's entry state S, the state
// cotangent dH it receives and dV) and then applies the adjoint of the prepass
// (gdn2.py:243-493) and of the fused prologue (gdn2.py:558-575, and the wrapper-level
// l2norm / scale / g-clamp the reference leaves to autodiff, gdn2.py:1970-1971, 2113-2122).
//
// Formulation notes (same result up to rounding):
//  * dA = -T^T dT T^T with dT = dW X^T + dU Y^T collapses to dA = -(dX W^T + dY U^T) with
//    dX = T^T dW, dY = T^T dU, because W = T X and U = T Y; dT is never formed.
//  * the adjoints of A and M are evaluated pair by pair with exact exponents, and
//    dLambda = beta*dbeta' + q*dq' - k*dk' (primes: the parts coming through A and M) plus the
//    terms through X, qe, ke and Lambda_end; dg is the within-document reverse cumulative sum.
//  * all clamps exp(min(x,0)) are inactive by construction (the cumulative decay is
//    monotone inside a document), so their subgradients are 1.
#include "dn_kernels.cuh"

namespace dn {


// fp32 SIMT products (the tensor-core variant lives in dn_prepass_bwd_tc.cu).
__global__ void __launch_bounds__(DN_THREADS, 1) prepass_bwd_kernel(PrepassBwdArgs a) {
  extern __shared__ __align__(128) float smem[];
  const Geo& g = a.g;
  const int C = g.C, K = g.K, Vw = g.Vw;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* tile = smem;                      // SIMT GEMM staging
  float* rq_s = tile + GEMM_SMEM_FLOATS;   // C
  float* rk_s = rq_s + C;                  // C
  float* dlend_s = rk_s + C;               // K
  int* seg_s = reinterpret_cast<int*>(dlend_s + K);   // C
  int* dstart_s = seg_s + C;               // C first row of the row's document inside the chunk

  const size_t CK = (size_t)C * K, CV = (size_t)C * Vw, CC = (size_t)C * C;
  float* sc = a.scratch + (size_t)blockIdx.x * a.scratch_per_cta;
  float* QH = sc;            float* KH = QH + CK;      float* LAM = KH + CK;
  float* GB = LAM + CK;      float* BA = GB + CK;      float* DW = BA + CK;
  float* DQE = DW + CK;      float* DKE = DQE + CK;    float* DX = DKE + CK;
  float* DBP = DX + CK;      float* DQP = DBP + CK;    float* DKP = DQP + CK;
  float* DLAM = DKP + CK;    float* VN = DLAM + CK;    float* DY = VN + CV;
  float* DM = DY + CV;       float* DA = DM + CC;

  const bool l2 = g.flags & DN_QK_L2NORM, fuse = g.flags & DN_FUSE_PROLOGUE;
  const bool guard = g.flags & DN_STABILITY_GUARD;
  const bool round_in = !fuse && g.qkv_dt == DN_BF16;
  const bool sbf = g.state_bf16(), ibf = g.bf16_mode(), trunc = ibf && (g.flags & DN_TRUNC_DT_BF16);
  const int pre = g.pre_dt;

  for (int item = blockIdx.x; item < a.items; item += gridDim.x) {
    const int c_idx = item % g.NC, h = (item / g.NC) % g.H, b = item / (g.NC * g.H);
    const int t0 = c_idx * C;
    const int hq = h / g.qk_div;
    const int hg = g.gate_head(h, g.gH), hb = g.gate_head(h, g.bH);
    for (int i = tid; i < C; i += DN_THREADS) seg_s[i] = seg_at(a.seg, b, t0 + i, g.L);
    __syncthreads();
    if (tid < C) {
      int s = tid;
      while (s > 0 && seg_s[s - 1] == seg_s[tid]) --s;
      dstart_s[tid] = s;
    }
    const int seg0 = seg_s[0], segL = seg_s[C - 1];
    bool is_new, all_same;
    chunk_flags(a.seg, g, b, c_idx, is_new, all_same);
    const size_t ibase = (size_t)item;
    const float* S = a.res.states + ibase * K * Vw;
    const float* dH = a.dH + ibase * K * Vw;
    const float* dV = a.dV + ibase * CV;
    const float* T = a.res.T + ibase * CC;
    const size_t bW = ibase * CK, bU = ibase * CV;

    // ---- prologue (as in the forward prepass), keeping the row norms and the activated b
    const int per = K / 32;
    for (int i = warp; i < C; i += DN_THREADS / 32) {
      const int t = t0 + i;
      const bool valid = t < g.L;
      const size_t rowqk = ((size_t)(b * (size_t)g.L + t) * g.Hk + hq) * K;
      float qv[4], kv[4], sq = 0.f, sk = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        qv[u] = kv[u] = 0.f;
        if (u < per && valid) {
          qv[u] = ldf(a.q, rowqk + lane + 32 * u, g.qkv_dt);
          kv[u] = ldf(a.k, rowqk + lane + 32 * u, g.qkv_dt);
        }
        sq += qv[u] * qv[u];
        sk += kv[u] * kv[u];
      }
      sq = warp_sum(sq);
      sk = warp_sum(sk);
      const float rq = l2 ? rsqrtf(sq + 1e-6f) : 1.f, rk = l2 ? rsqrtf(sk + 1e-6f) : 1.f;
      if (lane == 0) { rq_s[i] = rq; rk_s[i] = rk; }
      const size_t rowg = ((size_t)(b * (size_t)g.L + t) * g.gH + hg) * g.gC;
      const size_t rowb = ((size_t)(b * (size_t)g.L + t) * g.bH + hb) * g.bC;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (u >= per) break;
        const int c = lane + 32 * u;
        float qh = (qv[u] * rq) * g.scale, kh = l2 ? kv[u] * rk : kv[u];
        if (round_in) { qh = bf16r(qh); if (l2) kh = bf16r(kh); }
        float ga = 0.f, ba = 0.f;
        if (valid) {
          float gr = ldf(a.gg, rowg + (g.gC == 1 ? 0 : c), g.gate_dt);
          float br = ldf(a.b, rowb + (g.bC == 1 ? 0 : c), g.gate_dt);
          if (fuse) {
            ga = -expf(fminf(gr, 5.f));
            if (guard) ga = fminf(ga, -1e-6f);
            ba = 1.f / (1.f + expf(-br));
          } else {
            ga = gr <= 0.f ? gr : 0.f;
            ba = br;
            if (guard) { ga = fminf(ga, -1e-6f); ba = fmaxf(ba, 0.f); }      // gdn2.py:1972-1974
          }
        }
        QH[i * K + c] = qh;
        KH[i * K + c] = kh;
        LAM[i * K + c] = ga;
        BA[i * K + c] = ba;
        GB[i * K + c] = ba * kh;
      }
    }
    __syncthreads();
    if (tid < K) {
      float run = 0.f;
      int prev = seg_s[0];
      for (int i = 0; i < C; ++i) {
        const int s = seg_s[i];
        if (s != prev) run = 0.f;
        prev = s;
        run += LAM[i * K + tid];
        LAM[i * K + tid] = run;
      }
    }
    // dLambda_end from the carried state: [one doc] sum_v dH*S*exp(Lambda_end)   (gdn2.py:759-762)
    for (int kk = warp; kk < K; kk += DN_THREADS / 32) {
      float s = 0.f;
      for (int j = lane; j < Vw; j += 32) s += dH[(size_t)kk * Vw + j] * S[(size_t)kk * Vw + j];
      s = warp_sum(s);
      if (lane == 0) dlend_s[kk] = all_same ? s * expf(fminf(a.res.lam_end[ibase * K + kk], 0.f)) : 0.f;
    }
    __syncthreads();

    // ---- V_new = U - W S
    cta_gemm<true, true>(C, Vw, K,
        [&](int i, int kk) { return ldf(a.res.W, bW + rix(g.img, i, kk, K), pre); },
        [&](int kk, int j) { float s = S[(size_t)kk * Vw + j]; return sbf ? bf16r(s) : s; },
        [&](int i, int j, float acc) { VN[i * Vw + j] = ldf(a.res.U, bU + rix(g.img, i, j, Vw), pre) - acc; },
        tile);
    auto dO_at = [&](int i, int j) -> float {
      const int t = t0 + i;
      return t < g.L ? ldf(a.d_out, ((size_t)b * g.L + t) * g.Hv * g.V + (size_t)h * Vw + j, g.qkv_dt) : 0.f;
    };
    // ---- dW = -dV S^T, dqe = dO S^T, dke = V_new dH^T, dM = dO V_new^T
    cta_gemm<true, false>(C, K, Vw,
        [&](int i, int kk) { float x = dV[(size_t)i * Vw + kk]; return sbf ? bf16r(x) : x; },
        [&](int kk, int j) { float s = S[(size_t)j * Vw + kk]; return sbf ? bf16r(s) : s; },
        [&](int i, int j, float acc) { DW[i * K + j] = -acc; }, tile);
    cta_gemm<true, false>(C, K, Vw,
        [&](int i, int kk) { float x = dO_at(i, kk); return sbf ? bf16r(x) : x; },
        [&](int kk, int j) { float s = S[(size_t)j * Vw + kk]; return sbf ? bf16r(s) : s; },
        [&](int i, int j, float acc) { DQE[i * K + j] = acc; }, tile);
    cta_gemm<true, false>(C, K, Vw,
        [&](int i, int kk) { float x = VN[i * Vw + kk]; return sbf ? bf16r(x) : x; },
        [&](int kk, int j) { float x = dH[(size_t)j * Vw + kk]; return sbf ? bf16r(x) : x; },
        [&](int i, int j, float acc) { DKE[i * K + j] = acc; }, tile);
    cta_gemm<true, false>(C, C, Vw,
        [&](int i, int kk) { float x = dO_at(i, kk); return ibf ? bf16r(x) : x; },
        [&](int kk, int j) { float x = VN[j * Vw + kk]; return ibf ? bf16r(x) : x; },
        [&](int i, int j, float acc) { DM[i * C + j] = (i >= j && seg_s[i] == seg_s[j]) ? acc : 0.f; }, tile);
    // ---- dX = T^T dW, dY = T^T dV
    cta_gemm<false, true>(C, K, C,
        [&](int i, int kk) { float t = g.img ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(T)[rix(true, kk, i, C)]) : T[(size_t)kk * C + i]; return ibf ? bf16r(t) : t; },
        [&](int kk, int j) { float x = DW[kk * K + j]; return ibf ? bf16r(x) : x; },
        [&](int i, int j, float acc) { DX[i * K + j] = trunc ? bf16r(acc) : acc; }, tile);
    cta_gemm<false, true>(C, Vw, C,
        [&](int i, int kk) { float t = g.img ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(T)[rix(true, kk, i, C)]) : T[(size_t)kk * C + i]; return ibf ? bf16r(t) : t; },
        [&](int kk, int j) { float x = dV[(size_t)kk * Vw + j]; return ibf ? bf16r(x) : x; },
        [&](int i, int j, float acc) { DY[i * Vw + j] = trunc ? bf16r(acc) : acc; }, tile);
    // ---- dA = -(dX W^T + dY U^T), strictly lower and same document
    cta_gemm<true, false>(C, C, K + Vw,
        [&](int i, int kk) { return kk < K ? DX[i * K + kk] : DY[i * Vw + (kk - K)]; },
        [&](int kk, int j) {
          return kk < K ? ldf(a.res.W, bW + rix(g.img, j, kk, K), pre)
                        : ldf(a.res.U, bU + rix(g.img, j, kk - K, Vw), pre);
        },
        [&](int i, int j, float acc) { DA[i * C + j] = (i > j && seg_s[i] == seg_s[j]) ? -acc : 0.f; }, tile);

    // ---- adjoints of A and M, pair by pair.  Row side: dbeta', dq'.  Column side: dk'.
    // The diagonal pair (i == i) has exponent 0: it feeds dq and dk but not dLambda, and is
    // kept out of the dLambda products so that they do not leave a rounding residue.
    for (int e = tid; e < C * K; e += DN_THREADS) {
      const int i = e / K, c = e - i * K;
      const float li = LAM[e] * DN_LOG2E;
      float sb = 0.f, sq = 0.f;
      for (int j = dstart_s[i]; j < i; ++j) {
        const float ek = KH[j * K + c] * exp2f(fminf(li - LAM[j * K + c] * DN_LOG2E, 0.f));
        sb = fmaf(DA[i * C + j], ek, sb);
        sq = fmaf(DM[i * C + j], ek, sq);
      }
      DLAM[e] = GB[e] * sb + QH[e] * sq;
      DBP[e] = sb;
      DQP[e] = fmaf(DM[i * C + i], KH[e], sq);
    }
    for (int e = tid; e < C * K; e += DN_THREADS) {
      const int j = e / K, c = e - j * K;
      const float lj = LAM[e] * DN_LOG2E;
      float sk = 0.f;
      for (int i = j + 1; i < C && seg_s[i] == seg_s[j]; ++i) {
        const float ex = exp2f(fminf(LAM[i * K + c] * DN_LOG2E - lj, 0.f));
        sk = fmaf(fmaf(DA[i * C + j], GB[i * K + c], DM[i * C + j] * QH[i * K + c]), ex, sk);
      }
      DLAM[e] -= KH[e] * sk;
      DKP[e] = fmaf(DM[j * C + j], QH[e], sk);
    }
    __syncthreads();

    // ---- combine: dLambda, d q_hat, d k_hat, d b_act  (in place over DLAM, DQP, DKP, DBP)
    for (int e = tid; e < C * K; e += DN_THREADS) {
      const int i = e / K, c = e - i * K;
      const float lam = LAM[e], el = expf(fminf(lam, 0.f));
      const float eke = expf(fminf(LAM[(C - 1) * K + c] - lam, 0.f));
      const bool first = seg_s[i] == seg0, last = seg_s[i] == segL;
      const float qh = QH[e], kh = KH[e], be = GB[e];
      const float X = first ? be * el : 0.f, qe = first ? qh * el : 0.f, ke = last ? kh * eke : 0.f;
      const float dbp = DBP[e], dqp = DQP[e], dkp = DKP[e];
      const float dx = DX[e], dqe = DQE[e], dke = DKE[e];
      const float dbeta = dbp + (first ? dx * el : 0.f);
      const float dq = dqp + (first ? dqe * el : 0.f);
      const float dk = dkp + (last ? dke * eke : 0.f) + dbeta * BA[e];
      DLAM[e] += dx * X + dqe * qe;
      DKE[e] = dke * ke;          // enters dg as a prefix sum over earlier rows (below)
      DQP[e] = dq;
      DKP[e] = dk;
      DBP[e] = dbeta * kh;        // d b_act
    }
    __syncthreads();
    // ---- dg_t = sum_{i >= t, same doc} dLambda_i  +  the Lambda_end path.  A row i of the last
    // document reaches the chunk end through every later g, so the ke term adds the prefix sum
    // of dke*ke over EARLIER rows (the equivalent "-dke*ke at row i, +sum at the last row" form
    // cancels only up to rounding); the carried-state term dLambda_end reaches every row.
    if (tid < K) {
      const int c = tid;
      float run = 0.f;
      for (int i = C - 1; i >= 0; --i) {
        if (i < C - 1 && seg_s[i] != seg_s[i + 1]) run = 0.f;
        run += DLAM[i * K + c];
        DLAM[i * K + c] = run;
      }
      float acc = dlend_s[c];              // zero unless the chunk is one document
      for (int i = 0; i < C; ++i) {
        if (seg_s[i] != segL) continue;
        DLAM[i * K + c] += acc;
        acc += DKE[i * K + c];
      }
    }
    __syncthreads();
    // ---- write dg, db (per row: gate adjoints, optional channel reduction)
    for (int i = warp; i < C; i += DN_THREADS / 32) {
      const int t = t0 + i;
      if (t >= g.L) continue;
      const size_t rowg = ((size_t)(b * (size_t)g.L + t) * g.gH + hg) * g.gC;
      const size_t outg = ((size_t)(b * (size_t)g.L + t) * g.H + h) * g.gC;   // exec-head granularity
      const size_t outb = ((size_t)(b * (size_t)g.L + t) * g.H + h) * g.bC;
      float sg = 0.f, sb2 = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (u >= per) break;
        const int c = lane + 32 * u;
        const float gr = ldf(a.gg, rowg + (g.gC == 1 ? 0 : c), g.gate_dt);
        float dgv = DLAM[i * K + c], dbv = DBP[i * K + c];
        if (fuse) {
          const float gexp = -expf(fminf(gr, 5.f));
          const bool pass = gr <= 5.f && (!guard || gexp < -1e-6f);
          dgv = pass ? dgv * gexp : 0.f;
          const float ba = BA[i * K + c];
          dbv = dbv * (ba * (1.f - ba));
        } else {
          dgv = (guard ? gr < -1e-6f : gr <= 0.f) ? dgv : 0.f;
          if (guard) {                                             // through max(b, 0)
            const size_t rowb = ((size_t)(b * (size_t)g.L + t) * g.bH + hb) * g.bC;
            const float br = ldf(a.b, rowb + (g.bC == 1 ? 0 : c), g.gate_dt);
            dbv *= br > 0.f ? 1.f : (br == 0.f ? 0.5f : 0.f);
          }
        }
        if (g.gC == 1) sg += dgv; else stf(a.dg, outg + c, dgv, a.dg_dt);
        if (g.bC == 1) sb2 += dbv; else stf(a.db, outb + c, dbv, a.db_dt);
      }
      if (g.gC == 1) { sg = warp_sum(sg); if (lane == 0) stf(a.dg, outg, sg, a.dg_dt); }
      if (g.bC == 1) { sb2 = warp_sum(sb2); if (lane == 0) stf(a.db, outb, sb2, a.db_dt); }
      // ---- dq, dk through scale and l2norm
      const size_t rowqk = ((size_t)(b * (size_t)g.L + t) * g.Hk + hq) * K;
      const size_t outqk = ((size_t)(b * (size_t)g.L + t) * g.H + h) * K;    // exec-head granularity
      const float rq = rq_s[i], rk = rk_s[i];
      float qn[4], kn[4], dqn[4], dkn[4], dq_dot = 0.f, dk_dot = 0.f;
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        qn[u] = kn[u] = dqn[u] = dkn[u] = 0.f;
        if (u >= per) continue;
        const int c = lane + 32 * u;
        qn[u] = ldf(a.q, rowqk + c, g.qkv_dt) * rq;
        kn[u] = ldf(a.k, rowqk + c, g.qkv_dt) * rk;
        dqn[u] = DQP[i * K + c] * g.scale;
        dkn[u] = DKP[i * K + c];
        dq_dot += qn[u] * dqn[u];
        dk_dot += kn[u] * dkn[u];
      }
      if (l2) { dq_dot = warp_sum(dq_dot); dk_dot = warp_sum(dk_dot); }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        if (u >= per) break;
        const int c = lane + 32 * u;
        const float dqr = l2 ? rq * (dqn[u] - qn[u] * dq_dot) : dqn[u];
        const float dkr = l2 ? rk * (dkn[u] - kn[u] * dk_dot) : dkn[u];
        stf(a.dq, outqk + c, dqr, a.dq_dt);
        stf(a.dk, outqk + c, dkr, a.dq_dt);
      }
    }
    // ---- dv = dY * w_act, dw = dY * v (+ sigmoid adjoint, optional column reduction)
    const int nvh = Vw / g.V;      // value heads inside this exec head
    for (int rv = warp; rv < C * nvh; rv += DN_THREADS / 32) {
      const int i = rv / nvh, vh = rv - i * nvh, t = t0 + i;
      if (t >= g.L) continue;
      const int hv = h * g.G + vh;
      const size_t rowv = ((size_t)b * g.L + t) * g.Hv * g.V + (size_t)hv * g.V;
      const size_t roww = ((size_t)(b * (size_t)g.L + t) * g.wH + g.w_head(hv)) * g.wC;
      const size_t outw = ((size_t)(b * (size_t)g.L + t) * g.Hv + hv) * g.wC;  // value-head granularity
      float sw = 0.f;
      for (int cv = lane; cv < g.V; cv += 32) {
        const float dy = DY[i * Vw + vh * g.V + cv];
        const float vv = ldf(a.v, rowv + cv, g.qkv_dt);
        float wr = ldf(a.w, roww + (g.wC == 1 ? 0 : cv), g.gate_dt);
        float wa = wr, dwv = dy * vv;
        if (fuse) { wa = 1.f / (1.f + expf(-wr)); dwv *= wa * (1.f - wa); }
        stf(a.dv, rowv + cv, dy * wa, g.qkv_dt);
        if (g.wC == 1) sw += dwv; else stf(a.dw, outw + cv, dwv, a.dw_dt);
      }
      if (g.wC == 1) { sw = warp_sum(sw); if (lane == 0) stf(a.dw, outw, sw, a.dw_dt); }
    }
    __syncthreads();
  }
}

size_t prepass_bwd_scratch_per_cta(const Geo& g) {
  return (size_t)13 * g.C * g.K + (size_t)2 * g.C * g.Vw + (size_t)2 * g.C * g.C;
}

bool prepass_bwd_tc_eligible(const Geo& g) { return g.img && !(g.flags & DN_STATE_FP32_MM); }

int launch_prepass_bwd(PrepassBwdArgs& a, size_t scratch_floats, cudaStream_t st) {
  const Geo& g = a.g;
  a.items = g.B * g.H * g.NC;
  a.scratch_per_cta = prepass_bwd_scratch_per_cta(g);
  const bool tc = prepass_bwd_tc_eligible(g);
  a.err = device_error_ptr();
  if (tc) return launch_prepass_bwd_tc(a, scratch_floats, st);
  const int max_ctas = 2 * sm_count();
  int grid = a.items < max_ctas ? a.items : max_ctas;
  if (scratch_floats < (size_t)grid * a.scratch_per_cta) return DN_ERR_SCRATCH_TOO_SMALL;
  const size_t smem = (GEMM_SMEM_FLOATS + (size_t)4 * g.C + g.K) * sizeof(float);
  prepass_bwd_kernel<<<grid, DN_THREADS, smem, st>>>(a);
  return launch_status();
}

}  // namespace dn
