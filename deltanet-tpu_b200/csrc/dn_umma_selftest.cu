// Diagnostic kernel: one 128 x N x Kc GEMM through the tcgen05 building blocks, for every
// combination of operand majors.  Used by the tests to pin the descriptor encodings.
#include "dn_kernels.cuh"
#include "dn_umma.cuh"

namespace dn {

template <int N, bool A_MN, bool B_MN>
__global__ void __launch_bounds__(256, 1) umma_selftest_kernel(const __nv_bfloat16* A, const __nv_bfloat16* B,
                                                               float* D, int Kc, int* err) {
  extern __shared__ __align__(128) uint8_t sm[];
  __shared__ uint64_t bar;
  __shared__ uint32_t tmem_base;
  uint4* sA = reinterpret_cast<uint4*>(sm);
  uint4* sB = reinterpret_cast<uint4*>(sm + 128 * Kc * 2);
  if (threadIdx.x == 0) { umma::mbar_init(&bar, 1); umma::fence_mbar_init(); }
  if (threadIdx.x < 32) umma::tmem_alloc(&tmem_base, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &bar, 0u, err, false};
  // A: K-major source is (128, Kc) row-major; MN-major source is (Kc, 128) row-major
  if (A_MN) umma::stage_operand<256>(sA, 128 / 8, Kc, [&](int p, int x) { return umma::ld8_bf16(A + (size_t)x * 128 + p * 8); });
  else      umma::stage_operand<256>(sA, Kc / 8, 128, [&](int p, int x) { return umma::ld8_bf16(A + (size_t)x * Kc + p * 8); });
  // B: K-major source is (N, Kc) row-major; MN-major source is (Kc, N) row-major
  if (B_MN) umma::stage_operand<256>(sB, N / 8, Kc, [&](int p, int x) { return umma::ld8_bf16(B + (size_t)x * N + p * 8); });
  else      umma::stage_operand<256>(sB, Kc / 8, N, [&](int p, int x) { return umma::ld8_bf16(B + (size_t)x * Kc + p * 8); });
  umma::issue_and_wait<N, A_MN, B_MN>(cx, sA, sB, Kc, 0, false);
  umma::drain<256, N>(cx, 0, [&](int row, int col, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 16; ++i) D[(size_t)row * N + col + i] = v[i];
  });
  __syncthreads();
  if (threadIdx.x < 32) umma::tmem_dealloc(tmem_base, 512);
}

template <int N>
static int launch_selftest(int a_mn, int b_mn, int Kc, const void* A, const void* B, float* D, int* err, cudaStream_t st) {
  const size_t smem = (size_t)(128 + N) * Kc * 2;
  auto go = [&](auto kern) {
    cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    kern<<<1, 256, smem, st>>>(reinterpret_cast<const __nv_bfloat16*>(A), reinterpret_cast<const __nv_bfloat16*>(B), D, Kc, err);
  };
  if (!a_mn && !b_mn) go(umma_selftest_kernel<N, false, false>);
  else if (!a_mn && b_mn) go(umma_selftest_kernel<N, false, true>);
  else if (a_mn && !b_mn) go(umma_selftest_kernel<N, true, false>);
  else go(umma_selftest_kernel<N, true, true>);
  return launch_status();
}

}  // namespace dn

extern "C" int dn_selftest_umma(int32_t a_mn, int32_t b_mn, int32_t N, int32_t Kc, const void* A, const void* B,
                                float* D, int32_t* err, void* stream) {
  if (!A || !B || !D || !err) return DN_ERR_NULL_POINTER;
  if (Kc % 16 || Kc < 16 || Kc > 256) return DN_ERR_BAD_SHAPE;
  cudaStream_t st = (cudaStream_t)stream;
  switch (N) {
    case 32: return dn::launch_selftest<32>(a_mn, b_mn, Kc, A, B, D, err, st);
    case 64: return dn::launch_selftest<64>(a_mn, b_mn, Kc, A, B, D, err, st);
    case 128: return dn::launch_selftest<128>(a_mn, b_mn, Kc, A, B, D, err, st);
    case 256: return dn::launch_selftest<256>(a_mn, b_mn, Kc, A, B, D, err, st);
    default: return DN_ERR_BAD_SHAPE;
  }
}
