// Small integer / reduction kernels around the main path.
#include "dn_kernels.cuh"

#include <cstdlib>
#include <mutex>

namespace dn {

int sm_count() {
  static int table[64] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = __atomic_load_n(&table[dev], __ATOMIC_RELAXED);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n < 1) { cudaGetLastError(); n = 148; }
    __atomic_store_n(&table[dev], n, __ATOMIC_RELAXED);
  }
  return n;
}

namespace { long long g_launches = 0; }
int launch_status() {
  if (cudaGetLastError() != cudaSuccess) return DN_ERR_CUDA_LAUNCH;
  __atomic_fetch_add(&g_launches, 1, __ATOMIC_RELAXED);
  return DN_OK;
}
long long launches_total() { return __atomic_load_n(&g_launches, __ATOMIC_RELAXED); }

// ---- the error word ------------------------------------------------------------------------------
// Kernels whose bounded waits give up store 1 into one int.  The int lives in a page of this
// library's own static host memory that is pinned and mapped into the device address space on first
// use (registering existing memory allocates nothing), so the host can look at it WITHOUT
// synchronising: every entry point checks it before it enqueues anything.  If the page cannot be
// registered the word falls back to a __device__ variable, which only dn_device_error() (a
// synchronising call) can read.
namespace {
alignas(4096) int g_err_page[1024];
__device__ int g_err_fallback = 0;
std::once_flag g_err_once;
bool g_err_mapped = false;
void err_setup() {
  g_err_mapped = cudaHostRegister(g_err_page, sizeof(g_err_page), cudaHostRegisterPortable | cudaHostRegisterMapped) == cudaSuccess;
  if (!g_err_mapped) cudaGetLastError();
}
}  // namespace

int* device_error_ptr() {
  std::call_once(g_err_once, err_setup);
  int* p = nullptr;
  if (g_err_mapped && cudaHostGetDevicePointer(reinterpret_cast<void**>(&p), g_err_page, 0) == cudaSuccess && p) return p;
  cudaGetLastError();
  p = nullptr;
  cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_err_fallback);
  return p;
}

int peek_device_error() { return g_err_mapped ? __atomic_load_n(&g_err_page[0], __ATOMIC_RELAXED) : 0; }

int read_device_error() {
  cudaDeviceSynchronize();
  int v = 0;
  if (cudaMemcpyFromSymbol(&v, g_err_fallback, sizeof(int)) != cudaSuccess) { cudaGetLastError(); v = 0; }
  return (v || peek_device_error()) ? 1 : 0;
}

void reset_device_error() {
  __atomic_store_n(&g_err_page[0], 0, __ATOMIC_RELAXED);
  const int zero = 0;
  if (cudaMemcpyToSymbol(g_err_fallback, &zero, sizeof(int)) != cudaSuccess) cudaGetLastError();
}

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
  return launch_status();
}

// Canonical ids straight from cumulative sequence lengths: token t belongs to document d with
// cu[d] <= t < cu[d+1] (binary search per token); the same ids for every batch row, plus
// first_is_new[b].  Tokens at or past cu[n_cu-1] take the last document.
__global__ void __launch_bounds__(256) cu_seqlens_segments_kernel(const int32_t* cu, int n_cu, const int32_t* first_is_new,
                                                                  int32_t* out, int B, int L) {
  const size_t total = (size_t)B * L;
  for (size_t e = (size_t)blockIdx.x * 256 + threadIdx.x; e < total; e += (size_t)gridDim.x * 256) {
    const int t = (int)(e % L), b = (int)(e / L);
    int lo = 0, hi = n_cu - 1;                          // invariant: cu[lo] <= t, and t < cu[hi] or hi is the end
    while (hi - lo > 1) {
      const int mid = (lo + hi) >> 1;
      if (cu[mid] <= t) lo = mid; else hi = mid;
    }
    out[e] = lo + (first_is_new ? first_is_new[b] : 0);
  }
}

int launch_cu_seqlens_segments(const int32_t* cu, int n_cu, const int32_t* first_is_new, int32_t* out,
                               int B, int L, cudaStream_t st) {
  size_t blocks = ((size_t)B * L + 255) / 256;
  if (blocks > (size_t)sm_count() * 8) blocks = (size_t)sm_count() * 8;
  cu_seqlens_segments_kernel<<<(unsigned)blocks, 256, 0, st>>>(cu, n_cu, first_is_new, out, B, L);
  return launch_status();
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
  if (blocks > (size_t)sm_count() * 16) blocks = (size_t)sm_count() * 16;
  group_sum_kernel<<<(unsigned)blocks, 256, 0, st>>>(in, out, out_dt, total, heads_out, groups, cols);
  return launch_status();
}

// One CTA per 64 x 64 tile of a (batch, value head)'s S_out = op(P) S_in + Q (K, V multiples of 64): the
// kernel sits on the serial path between two ranks' transfers, so it is spread over many SMs.
__global__ void __launch_bounds__(DN_THREADS) sp_apply_kernel(const float* P, const float* S_in, const float* Q,
                                                              float* S_out, const uint8_t* keep, int H, int G, int K, int V,
                                                              int transpose) {
  __shared__ __align__(16) float tile[GEMM_SMEM_FLOATS];
  const int tn = V / GT, tiles = (K / GT) * tn;
  const int tq = blockIdx.x % tiles, bhv = blockIdx.x / tiles;
  const int m0 = (tq / tn) * GT, n0 = (tq % tn) * GT;
  const int hv = bhv % (H * G), b = bhv / (H * G), h = hv / G;
  const float* p = P + ((size_t)b * H + h) * K * K;
  const size_t so = ((size_t)b * H * G + hv) * K * V;
  const float* si = S_in + so + n0;
  const float* q = Q ? Q + so : nullptr;
  float* o = S_out + so;
  const bool kept = !keep || keep[b] != 0;            // a dropped batch row ends as zeros
  auto store = [&](int i, int j, float acc) {
    const size_t e = (size_t)(m0 + i) * V + n0 + j;
    o[e] = kept ? acc + (q ? q[e] : 0.f) : 0.f;
  };
  if (transpose)
    cta_gemm<false, true>(GT, GT, K, [&](int i, int kk) { return p[kk * K + m0 + i]; }, [&](int kk, int j) { return si[kk * V + j]; }, store, tile);
  else
    cta_gemm<true, true>(GT, GT, K, [&](int i, int kk) { return p[(m0 + i) * K + kk]; }, [&](int kk, int j) { return si[kk * V + j]; }, store, tile);
}

int launch_sp_apply(const float* P, const float* S_in, const float* Q, float* S_out, const uint8_t* keep, int B, int H,
                    int G, int K, int V, int transpose, cudaStream_t st) {
  if (K % GT || V % GT) return DN_ERR_BAD_SHAPE;
  sp_apply_kernel<<<B * H * G * (K / GT) * (V / GT), DN_THREADS, 0, st>>>(P, S_in, Q, S_out, keep, H, G, K, V, transpose);
  return launch_status();
}

}  // namespace dn
