// Inter-chunk recurrence, fp32 SIMT formulation: the forward chain (with or without the
// output) and the reverse chain of the state cotangent.
//
// The recurrence is independent per value column, so one CTA carries a (K x VS) slice of
// the state of one (batch, exec head) through all chunks; a grid of (Vw/VS, H, B) CTAs
// covers the job.  Forward, per chunk (src/deltanet_tpu/gdn2.py:585-652):
//     S      <- 0 at a document start (or the initial state at chunk 0)
//     V_new   = U - W S
//     O       = qe S + M V_new
//     S      <- [chunk is one document] exp(Lambda_end) * S + ke^T V_new
// Reverse, per chunk (the V-column-independent part of gdn2.py:698-769):
//     dV      = M^T dO + ke dH
//     dH     <- [one document] exp(Lambda_end) * dH + qe^T dO - W^T dV ; 0 at a document start
// The contractions over the value width (dW, dM, dqe, dke, dLambda_end) are left to the
// chunk-parallel backward kernel, which gets dV and the per-chunk dH from here.
#include "dn_kernels.cuh"

namespace dn {

constexpr int VS = 64;   // value columns per CTA

__device__ __forceinline__ size_t native_state_index(const Geo& g, int b, int h, int k, int jj) {
  const int hv = h * g.G + jj / g.V, cv = jj % g.V;   // exec column jj -> (value head, column)
  return (((size_t)b * g.Hv + hv) * g.K + k) * g.V + cv;
}

template <bool WITH_OUT>
__global__ void __launch_bounds__(DN_THREADS) state_fwd_kernel(StateArgs a) {
  extern __shared__ __align__(16) float smem[];
  const Geo& g = a.g;
  const int C = g.C, K = g.K, Vw = g.Vw;
  const int h = blockIdx.y, b = blockIdx.z;
  // slices past the value width carry the transition columns (see StateArgs::P_out)
  const bool trans = (int)blockIdx.x * VS >= Vw;
  const int v0 = trans ? 0 : blockIdx.x * VS, p0 = trans ? blockIdx.x * VS - Vw : 0;
  const int tid = threadIdx.x;
  float* S = smem;               // K*VS
  float* Vn = S + K * VS;        // C*VS
  float* tile = Vn + C * VS;
  const bool sbf = g.state_bf16(), ibf = g.bf16_mode();
  const int pre = g.pre_dt;

  for (int c = 0; c < g.NC; ++c) {
    bool is_new, all_same;
    chunk_flags(a.seg, g, b, c, is_new, all_same);
    if (c == 0 || is_new) {
      for (int e = tid; e < K * VS; e += DN_THREADS) {
        float s0 = 0.f;
        if (c == 0 && !is_new && trans) s0 = (e / VS == p0 + e % VS) ? 1.f : 0.f;
        else if (c == 0 && !is_new && a.init_state)
          s0 = a.init_state[native_state_index(g, b, h, e / VS, v0 + e % VS)];
        S[e] = s0;
      }
      __syncthreads();
    }
    const size_t item = ((size_t)b * g.H + h) * g.NC + c;
    if (a.states && !trans)
      for (int e = tid; e < K * VS; e += DN_THREADS)
        a.states[item * K * Vw + (size_t)(e / VS) * Vw + v0 + e % VS] = S[e];

    const size_t bW = item * C * K, bU = item * C * Vw, bM = item * C * C;
    // V_new = U - W S
    cta_gemm<true, true>(C, VS, K,
        [&](int i, int kk) { return ldf(a.res.W, bW + rix(g.img, i, kk, K), pre); },
        [&](int kk, int j) { float s = S[kk * VS + j]; return sbf ? bf16r(s) : s; },
        [&](int i, int j, float acc) {
          const float u = (a.res.U && !trans) ? ldf(a.res.U, bU + rix(g.img, i, v0 + j, Vw), pre) : 0.f;   // transition columns: U = 0
          Vn[i * VS + j] = u - acc;
        },
        tile);
    if (WITH_OUT && !trans) {
      // O = [qe | M] [S ; V_new]
      cta_gemm<true, true>(C, VS, K + C,
          [&](int i, int kk) {
            return kk < K ? ldf(a.res.qe, bW + rix(g.img, i, kk, K), pre)
                          : ldf(a.res.M, bM + rix(g.img, i, kk - K, C), pre);
          },
          [&](int kk, int j) {
            if (kk < K) { float s = S[kk * VS + j]; return sbf ? bf16r(s) : s; }
            float x = Vn[(kk - K) * VS + j];
            return ibf ? bf16r(x) : x;
          },
          [&](int i, int j, float acc) {
            const int t = c * C + i;
            if (t < g.L) stf(a.out, ((size_t)b * g.L + t) * g.Hv * g.V + (size_t)h * Vw + v0 + j, acc, g.qkv_dt);
          },
          tile);
    }
    // S <- decay * S + ke^T V_new
    cta_gemm<false, true>(K, VS, C,
        [&](int i, int kk) { return ldf(a.res.ke, bW + rix(g.img, kk, i, K), pre); },
        [&](int kk, int j) { float x = Vn[kk * VS + j]; return sbf ? bf16r(x) : x; },
        [&](int i, int j, float acc) {
          float carried = 0.f;
          if (all_same) carried = S[i * VS + j] * expf(fminf(a.res.lam_end[item * K + i], 0.f));
          S[i * VS + j] = carried + acc;
        },
        tile);
    if (a.until_independent && !all_same) break;       // (uniform over the CTA: the flags depend on the chunk only)
    if (a.until_independent && c + 1 < g.NC) {
      bool nn, na;
      chunk_flags(a.seg, g, b, c + 1, nn, na);
      if (nn) break;
    }
  }
  if (a.until_independent) return;                     // the caller has the final state from the shard's affine summary
  if (trans) {
    for (int e = tid; e < K * VS; e += DN_THREADS)
      if (p0 + e % VS < K) a.P_out[(((size_t)b * g.H + h) * K + e / VS) * K + p0 + e % VS] = S[e];
  } else if (a.final_state)
    for (int e = tid; e < K * VS; e += DN_THREADS)
      a.final_state[native_state_index(g, b, h, e / VS, v0 + e % VS)] = S[e];
}

__global__ void __launch_bounds__(DN_THREADS) state_bwd_kernel(StateArgs a) {
  extern __shared__ __align__(16) float smem[];
  const Geo& g = a.g;
  const int C = g.C, K = g.K, Vw = g.Vw;
  const int v0 = blockIdx.x * VS, h = blockIdx.y, b = blockIdx.z;
  const int tid = threadIdx.x;
  float* dH = smem;              // K*VS
  float* dOs = dH + K * VS;      // C*VS
  float* dVs = dOs + C * VS;     // C*VS
  float* tile = dVs + C * VS;
  const bool sbf = g.state_bf16(), ibf = g.bf16_mode();
  const int pre = g.pre_dt;

  for (int e = tid; e < K * VS; e += DN_THREADS)
    dH[e] = a.d_final ? a.d_final[native_state_index(g, b, h, e / VS, v0 + e % VS)] : 0.f;
  __syncthreads();

  for (int c = g.NC - 1; c >= 0; --c) {
    bool is_new, all_same;
    chunk_flags(a.seg, g, b, c, is_new, all_same);
    const size_t item = ((size_t)b * g.H + h) * g.NC + c;
    const size_t bW = item * C * K, bM = item * C * C;
    for (int e = tid; e < C * VS; e += DN_THREADS) {
      const int i = e / VS, j = e - i * VS, t = c * C + i;
      dOs[e] = t < g.L ? ldf(a.d_out, ((size_t)b * g.L + t) * g.Hv * g.V + (size_t)h * Vw + v0 + j, g.qkv_dt) : 0.f;
    }
    for (int e = tid; e < K * VS; e += DN_THREADS)
      a.dH[item * K * Vw + (size_t)(e / VS) * Vw + v0 + e % VS] = dH[e];
    __syncthreads();
    // dV = M^T dO + ke dH
    cta_gemm<false, true>(C, VS, C + K,
        [&](int i, int kk) {
          return kk < C ? ldf(a.res.M, bM + rix(g.img, kk, i, C), pre)
                        : ldf(a.res.ke, bW + rix(g.img, i, kk - C, K), pre);
        },
        [&](int kk, int j) {
          if (kk < C) { float x = dOs[kk * VS + j]; return ibf ? bf16r(x) : x; }
          float x = dH[(kk - C) * VS + j];
          return sbf ? bf16r(x) : x;
        },
        [&](int i, int j, float acc) {
          dVs[i * VS + j] = acc;
          a.dV[item * C * Vw + (size_t)i * Vw + v0 + j] = acc;
        },
        tile);
    // dH <- decay * dH + qe^T dO - W^T dV, cleared at a document start
    cta_gemm<false, true>(K, VS, 2 * C,
        [&](int i, int kk) {
          return kk < C ? ldf(a.res.qe, bW + rix(g.img, kk, i, K), pre)
                        : -ldf(a.res.W, bW + rix(g.img, kk - C, i, K), pre);
        },
        [&](int kk, int j) {
          float x = kk < C ? dOs[kk * VS + j] : dVs[(kk - C) * VS + j];
          return sbf ? bf16r(x) : x;
        },
        [&](int i, int j, float acc) {
          float carried = 0.f;
          if (all_same) carried = dH[i * VS + j] * expf(fminf(a.res.lam_end[item * K + i], 0.f));
          dH[i * VS + j] = is_new ? 0.f : carried + acc;
        },
        tile);
    if (a.until_independent && (is_new || !all_same)) break;
  }
  if (a.until_independent) return;                     // the caller has d_init from the shard's affine summary
  if (a.d_init)
    for (int e = tid; e < K * VS; e += DN_THREADS)
      a.d_init[native_state_index(g, b, h, e / VS, v0 + e % VS)] = dH[e];
}

static size_t state_smem(const Geo& g, bool bwd) {
  size_t fl = (size_t)g.K * VS + (size_t)g.C * VS * (bwd ? 2 : 1) + GEMM_SMEM_FLOATS;
  return fl * sizeof(float);
}

int launch_state_fwd(const StateArgs& a, cudaStream_t st) {
  const Geo& g = a.g;
  if (state_tc_eligible(g) && !force_simt()) return launch_state_fwd_tc(a, st);
  dim3 grid(g.Vw / VS + (a.P_out ? (g.K + VS - 1) / VS : 0), g.H, g.B);
  size_t smem = state_smem(g, false);
  // (the attribute is per device: set on every launch, like the tensor-core launchers do)
  if (a.out) {
    cudaFuncSetAttribute(state_fwd_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    state_fwd_kernel<true><<<grid, DN_THREADS, smem, st>>>(a);
  } else {
    cudaFuncSetAttribute(state_fwd_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    state_fwd_kernel<false><<<grid, DN_THREADS, smem, st>>>(a);
  }
  return launch_status();
}

int launch_state_bwd(const StateArgs& a, cudaStream_t st) {
  const Geo& g = a.g;
  if (state_tc_eligible(g) && !force_simt()) return launch_state_bwd_tc(a, st);
  dim3 grid(g.Vw / VS, g.H, g.B);
  size_t smem = state_smem(g, true);
  cudaFuncSetAttribute(state_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  state_bwd_kernel<<<grid, DN_THREADS, smem, st>>>(a);
  return launch_status();
}

}  // namespace dn
