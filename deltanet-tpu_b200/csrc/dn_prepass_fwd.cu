// Prepass forward, fp32 SIMT formulation (any supported C, K, V; both precisions).
//
// Per (batch, exec head, chunk) it produces what the reference's prepass kernel body
// produces (src/deltanet_tpu/gdn2.py:115-240): the cumulative log-decay, the strictly
// lower matrix A and the lower matrix M with document masks, T = (I+A)^-1,
// W = T (beta e^Lambda), U = T (w*v), the masked q/k factors and Lambda_end -- with the
// prologue (l2norm, scale, gate activations, g clamp) fused in front.
//
// Differences in formulation (same result up to rounding):
//  * the cumulative decay restarts at document changes (the reference's
//    mask_lambda_by_doc variant, gdn2.py:150-155), so exponents only ever span one document;
//  * A and M are evaluated pair by pair with exact exponents exp(Lambda_i - Lambda_j) <= 1
//    instead of the 32x32 factorisation;
//  * T is obtained by substitution on 16x16 diagonal blocks followed by block merges
//    T21 = -T22 A21 T11, instead of the polynomial + Newton-Schulz scheme (gdn2.py:67-111).
#include "dn_kernels.cuh"

namespace dn {

__device__ __forceinline__ void tri_unrank(int m, int& bi, int& bj) {
  int r = (int)((sqrtf(8.f * (float)m + 1.f) - 1.f) * 0.5f);
  while (r * (r + 1) / 2 > m) --r;
  while ((r + 1) * (r + 2) / 2 <= m) ++r;
  bi = r;
  bj = m - r * (r + 1) / 2;
}

__global__ void __launch_bounds__(DN_THREADS, 1) prepass_fwd_kernel(PrepassFwdArgs a) {
  extern __shared__ __align__(16) float smem[];
  const Geo& g = a.g;
  const int C = g.C, K = g.K, Vw = g.Vw;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* As = smem;                    // C*C
  float* Ts = As + C * C;              // C*C
  float* Tm = Ts + C * C;              // C*C (merge temporary); panels alias Ts/Tm
  const int PS = 33;
  float* pan = Ts;                     // 4 panels of C*33
  float* tile = smem + a.smem_tile_off;
  int* seg_s = reinterpret_cast<int*>(tile + GEMM_SMEM_FLOATS);

  float* sc = a.scratch + (size_t)blockIdx.x * a.scratch_per_cta;
  float* QH = sc;
  float* KH = QH + C * K;
  float* LAM = KH + C * K;
  float* GB = LAM + C * K;
  float* X = GB + C * K;
  float* Y = X + C * K;

  const bool l2 = g.flags & DN_QK_L2NORM, fuse = g.flags & DN_FUSE_PROLOGUE;
  const bool guard = g.flags & DN_STABILITY_GUARD;
  const bool round_in = !fuse && g.qkv_dt == DN_BF16;

  for (int item = blockIdx.x; item < a.items; item += gridDim.x) {
    const int c_idx = item % g.NC, h = (item / g.NC) % g.H, b = item / (g.NC * g.H);
    const int t0 = c_idx * C;
    const int hq = h / g.qk_div;
    const int hg = g.gate_head(h, g.gH), hb = g.gate_head(h, g.bH);
    for (int i = tid; i < C; i += DN_THREADS) seg_s[i] = seg_at(a.seg, b, t0 + i, g.L);
    __syncthreads();
    const int seg0 = seg_s[0], segL = seg_s[C - 1];

    // ---- 1. prologue, one warp per row
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
        GB[i * K + c] = ba * kh;
      }
    }
    __syncthreads();

    // ---- 2. cumulative log-decay down the rows, restarting at document changes
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
    __syncthreads();

    // ---- 3. masked factors: X = [first doc] beta e^Lam, qe, ke, Lambda_end, Y = w*v
    const size_t ibase = (size_t)item;
    for (int e = tid; e < C * K; e += DN_THREADS) {
      const int i = e / K, c = e - i * K;
      const float lam = LAM[e], el = expf(fminf(lam, 0.f));
      const bool first = seg_s[i] == seg0, last = seg_s[i] == segL;
      X[e] = first ? GB[e] * el : 0.f;
      const float lend = LAM[(C - 1) * K + c];
      stf(a.res.qe, ibase * C * K + e, first ? QH[e] * el : 0.f, g.pre_dt);
      stf(a.res.ke, ibase * C * K + e, last ? KH[e] * expf(fminf(lend - lam, 0.f)) : 0.f, g.pre_dt);
      if (i == C - 1) a.res.lam_end[ibase * K + c] = lam;
    }
    for (int e = tid; e < C * Vw; e += DN_THREADS) {
      const int i = e / Vw, j = e - i * Vw;
      const int t = t0 + i;
      float y = 0.f;
      if (t < g.L) {
        const int col = h * Vw + j, hv = col / g.V, cv = col - hv * g.V;
        const float vv = ldf(a.v, (size_t)(b * (size_t)g.L + t) * g.Hv * g.V + col, g.qkv_dt);
        float wr = ldf(a.w, ((size_t)(b * (size_t)g.L + t) * g.wH + g.w_head(hv)) * g.wC + (g.wC == 1 ? 0 : cv), g.gate_dt);
        if (fuse) wr = 1.f / (1.f + expf(-wr));
        y = wr * vv;
      }
      Y[e] = y;
    }
    for (int e = tid; e < C * C; e += DN_THREADS) As[e] = 0.f;
    __syncthreads();

    // ---- 4. A and M, pair by pair in 4x4 micro-blocks, channels in panels of 32
    const int nb = C / 4, nmb = nb * (nb + 1) / 2;
    float* pL = pan;
    float* pK = pL + C * PS;
    float* pB = pK + C * PS;
    float* pQ = pB + C * PS;
    for (int slot = 0; slot * DN_THREADS < nmb; ++slot) {
      const int m = tid + slot * DN_THREADS;
      int bi = 0, bj = 0;
      const bool act = m < nmb;
      if (act) tri_unrank(m, bi, bj);
      float accA[4][4], accM[4][4];
#pragma unroll
      for (int r = 0; r < 4; ++r)
#pragma unroll
        for (int s = 0; s < 4; ++s) accA[r][s] = accM[r][s] = 0.f;
      for (int p = 0; p < K / 32; ++p) {
        __syncthreads();                    // As zero-fill / previous panel consumers done
        for (int e = tid; e < C * 32; e += DN_THREADS) {
          const int i = e >> 5, c = e & 31, src = i * K + p * 32 + c;
          pL[i * PS + c] = LAM[src] * DN_LOG2E;
          pK[i * PS + c] = KH[src];
          pB[i * PS + c] = GB[src];
          pQ[i * PS + c] = QH[src];
        }
        __syncthreads();
        if (act) {
          for (int c = 0; c < 32; ++c) {
            float Li[4], Bi[4], Qi[4], Lj[4], Kj[4];
#pragma unroll
            for (int r = 0; r < 4; ++r) {
              Li[r] = pL[(4 * bi + r) * PS + c];
              Bi[r] = pB[(4 * bi + r) * PS + c];
              Qi[r] = pQ[(4 * bi + r) * PS + c];
              Lj[r] = pL[(4 * bj + r) * PS + c];
              Kj[r] = pK[(4 * bj + r) * PS + c];
            }
#pragma unroll
            for (int r = 0; r < 4; ++r)
#pragma unroll
              for (int s = 0; s < 4; ++s) {
                const float kk = Kj[s] * exp2f(fminf(Li[r] - Lj[s], 0.f));
                accA[r][s] = fmaf(Bi[r], kk, accA[r][s]);
                accM[r][s] = fmaf(Qi[r], kk, accM[r][s]);
              }
          }
        }
      }
      __syncthreads();                      // panels (aliasing Ts/Tm) no longer read
      if (act) {
#pragma unroll
        for (int r = 0; r < 4; ++r)
#pragma unroll
          for (int s = 0; s < 4; ++s) {
            const int i = 4 * bi + r, j = 4 * bj + s;
            const bool same = seg_s[i] == seg_s[j];
            As[i * C + j] = (i > j && same) ? accA[r][s] : 0.f;
            stf(a.res.M, ibase * C * C + i * C + j, (i >= j && same) ? accM[r][s] : 0.f, g.pre_dt);
          }
      }
    }
    // upper micro-blocks of M are zero
    for (int e = tid; e < C * C; e += DN_THREADS) {
      const int i = e / C, j = e - i * C;
      if ((j >> 2) > (i >> 2)) stf(a.res.M, ibase * C * C + e, 0.f, g.pre_dt);
    }
    for (int e = tid; e < C * C; e += DN_THREADS) { Ts[e] = 0.f; }
    __syncthreads();

    // ---- 5. T = (I + A)^-1: 16x16 diagonal blocks by substitution, then block merges
    if (tid < C) {
      const int j = tid, blk0 = j & ~15;
      Ts[j * C + j] = 1.f;
      for (int i = j + 1; i < blk0 + 16; ++i) {
        float s = 0.f;
        for (int m = j; m < i; ++m) s = fmaf(As[i * C + m], Ts[m * C + j], s);
        Ts[i * C + j] = -s;
      }
    }
    __syncthreads();
    for (int s = 16; s < C; s <<= 1) {
      const int total = C * s / 2;
      for (int e = tid; e < total; e += DN_THREADS) {
        const int p = e / (s * s), rem = e - p * s * s, il = rem / s, jl = rem - il * s;
        const int i = 2 * p * s + s + il, j = 2 * p * s + jl, mend = 2 * p * s + s;
        float acc = 0.f;
        for (int m = j; m < mend; ++m) acc = fmaf(As[i * C + m], Ts[m * C + j], acc);
        Tm[i * C + j] = acc;
      }
      __syncthreads();
      for (int e = tid; e < total; e += DN_THREADS) {
        const int p = e / (s * s), rem = e - p * s * s, il = rem / s, jl = rem - il * s;
        const int i = 2 * p * s + s + il, j = 2 * p * s + jl, m0 = 2 * p * s + s;
        float acc = 0.f;
        for (int m = m0; m <= i; ++m) acc = fmaf(Ts[i * C + m], Tm[m * C + j], acc);
        Ts[i * C + j] = -acc;
      }
      __syncthreads();
    }
    if (a.res.T)
      for (int e = tid; e < C * C; e += DN_THREADS) a.res.T[ibase * C * C + e] = Ts[e];

    // ---- 6. W = T X, U = T Y (operands rounded to bf16 in bf16 precision, gdn2.py:226-230)
    const bool bf = g.bf16_mode();
    {
      void* Wd = a.res.W;
      const int pre = g.pre_dt;
      const size_t base = ibase * C * K;
      cta_gemm<true, true>(C, K, C,
          [&](int i, int kk) { float t = Ts[i * C + kk]; return bf ? bf16r(t) : t; },
          [&](int kk, int j) { float x = X[kk * K + j]; return bf ? bf16r(x) : x; },
          [&](int i, int j, float acc) { stf(Wd, base + (size_t)i * K + j, acc, pre); }, tile);
    }
    {
      void* Ud = a.res.U;
      const int pre = g.pre_dt;
      const size_t base = ibase * C * Vw;
      cta_gemm<true, true>(C, Vw, C,
          [&](int i, int kk) { float t = Ts[i * C + kk]; return bf ? bf16r(t) : t; },
          [&](int kk, int j) { float y = Y[kk * Vw + j]; return bf ? bf16r(y) : y; },
          [&](int i, int j, float acc) { stf(Ud, base + (size_t)i * Vw + j, acc, pre); }, tile);
    }
    __syncthreads();
  }
}

size_t prepass_fwd_scratch_per_cta(const Geo& g) { return (size_t)5 * g.C * g.K + (size_t)g.C * g.Vw; }

int launch_prepass_fwd(const Geo& g, const void* q, const void* k, const void* v, const void* gg,
                       const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                       float* scratch, size_t scratch_floats, cudaStream_t st) {
  if (prepass_fwd_tc_eligible(g))
    return launch_prepass_fwd_tc(g, q, k, v, gg, b, w, seg, res, scratch, scratch_floats, st);
  PrepassFwdArgs a;
  a.g = g; a.q = q; a.k = k; a.v = v; a.gg = gg; a.b = b; a.w = w; a.seg = seg; a.res = res;
  a.items = g.B * g.H * g.NC;
  a.scratch_per_cta = prepass_fwd_scratch_per_cta(g);
  int grid = a.items < sm_count() ? a.items : sm_count();
  if (scratch_floats < (size_t)grid * a.scratch_per_cta) return DN_ERR_SCRATCH_TOO_SMALL;
  a.scratch = scratch;
  a.smem_tile_off = 3 * g.C * g.C;
  if (4 * g.C * 33 > 2 * g.C * g.C) a.smem_tile_off = g.C * g.C + 4 * g.C * 33;
  size_t smem = ((size_t)a.smem_tile_off + GEMM_SMEM_FLOATS + g.C) * sizeof(float);
  cudaFuncSetAttribute(prepass_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  prepass_fwd_kernel<<<grid, DN_THREADS, smem, st>>>(a);
  return launch_status();
}

}  // namespace dn
