// Small integer / reduction kernels around the main path.
#include "dn_kernels.cuh"

#include <cstdlib>

namespace dn {

bool force_simt() {
  static const bool v = [] { const char* e = std::getenv("DN_FORCE_SIMT"); return e && e[0] == '1'; }();
  return v;
}

// One CTA per batch row: out[t] = first_is_new + number of id changes in raw[1..t]
// (the reference's canonicalisation, src/deltanet_tpu/gdn2.py:2081-2094).
__global__ void __launch_bounds__(256) canonical_segments_kernel(const int32_t* raw, const int32_t* first_is_new,
                                                                  int32_t* out, int L) {
  __shared__ int part[256];
  const int b = blockIdx.x, tid = threadIdx.x;
  const int32_t* r = raw + (size_t)b * L;
  int32_t* o = out + (size_t)b * L;
  const int per = (L + 255) / 256, lo = tid * per, hi = min(L, lo + per);
  int cnt = 0;
  for (int t = max(lo, 1); t < hi; ++t) cnt += r[t] != r[t - 1];
  part[tid] = cnt;
  __syncthreads();
  if (tid == 0) {
    int run = first_is_new ? first_is_new[b] : 0;
    for (int i = 0; i < 256; ++i) { int c = part[i]; part[i] = run; run += c; }
  }
  __syncthreads();
  int run = part[tid];
  for (int t = lo; t < hi; ++t) {
    if (t > 0) run += r[t] != r[t - 1];
    o[t] = run;
  }
}

int launch_canonical_segments(const int32_t* raw, const int32_t* first_is_new, int32_t* out,
                              int B, int L, cudaStream_t st) {
  canonical_segments_kernel<<<B, 256, 0, st>>>(raw, first_is_new, out, L);
  return cudaGetLastError() == cudaSuccess ? DN_OK : DN_ERR_CUDA_LAUNCH;
}

// out[row][ho][c] = sum over gi of in[row][ho*groups + gi][c], added in a fixed order.
__global__ void __launch_bounds__(256) group_sum_kernel(const float* in, void* out, int out_dt, size_t total,
                                                        int heads_out, int groups, int cols) {
  for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
    const int c = (int)(e % cols);
    const size_t rh = e / cols;
    const int ho = (int)(rh % heads_out);
    const size_t row = rh / heads_out;
    const float* p = in + ((row * heads_out + ho) * groups) * cols + c;
    float s = 0.f;
    for (int gi = 0; gi < groups; ++gi) s += p[(size_t)gi * cols];
    stf(out, e, s, out_dt);
  }
}

int launch_group_sum(const float* in, void* out, int out_dt, size_t rows, int heads_out, int groups,
                     int cols, cudaStream_t st) {
  const size_t total = rows * heads_out * cols;
  size_t blocks = (total + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  group_sum_kernel<<<(unsigned)blocks, 256, 0, st>>>(in, out, out_dt, total, heads_out, groups, cols);
  return cudaGetLastError() == cudaSuccess ? DN_OK : DN_ERR_CUDA_LAUNCH;
}

// One CTA per (batch, value head): S_out = op(P) S_in + Q with the CTA-wide fp32 GEMM.
__global__ void __launch_bounds__(DN_THREADS) sp_apply_kernel(const float* P, const float* S_in, const float* Q,
                                                              float* S_out, int H, int G, int K, int V, int transpose) {
  __shared__ __align__(16) float tile[GEMM_SMEM_FLOATS];
  const int hv = blockIdx.x % (H * G), b = blockIdx.x / (H * G), h = hv / G;
  const float* p = P + ((size_t)b * H + h) * K * K;
  const size_t so = ((size_t)b * H * G + hv) * K * V;
  const float* si = S_in + so;
  const float* q = Q ? Q + so : nullptr;
  float* o = S_out + so;
  if (transpose)
    cta_gemm<false, true>(K, V, K, [&](int i, int kk) { return p[kk * K + i]; }, [&](int kk, int j) { return si[kk * V + j]; },
                          [&](int i, int j, float acc) { o[i * V + j] = acc + (q ? q[i * V + j] : 0.f); }, tile);
  else
    cta_gemm<true, true>(K, V, K, [&](int i, int kk) { return p[i * K + kk]; }, [&](int kk, int j) { return si[kk * V + j]; },
                         [&](int i, int j, float acc) { o[i * V + j] = acc + (q ? q[i * V + j] : 0.f); }, tile);
}

int launch_sp_apply(const float* P, const float* S_in, const float* Q, float* S_out, int B, int H, int G,
                    int K, int V, int transpose, cudaStream_t st) {
  sp_apply_kernel<<<B * H * G, DN_THREADS, 0, st>>>(P, S_in, Q, S_out, H, G, K, V, transpose);
  return cudaGetLastError() == cudaSuccess ? DN_OK : DN_ERR_CUDA_LAUNCH;
}

}  // namespace dn
