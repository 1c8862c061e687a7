// The nine matrix products of the chunk-parallel backward on the tcgen05 tensor cores
// (bf16 precision, chunk = K = 128, value width VW in {128, 256}).
//
// Operand images live in four shared-memory slots (X, Y, Z of 128 x VW bf16, P of 128 x 128)
// that are refilled as the sequence advances; accumulators live in tensor memory (512 columns)
// and are drained one row per thread.  An image written once serves as a matrix and as its
// transpose (the descriptor says which), which is why S, V_new, dV, W and U are staged only once
// per use group:
//   1. V_new = U - W S                       A = W (P)          B = S (X); U (Z) read by the drain -> image Y
//   2. dqe   = dO S^T ; dM = dO V_new^T      A = dO (Z)         B = S (X), V_new (Y)
//   3. dW    = -dV S^T                       A = dV (Z)         B = S (X)         -> image P
//   4. dke   = V_new dH^T                    A = V_new (Y)      B = dH (X)
//   5. dX    = T^T dW ; dY = T^T dV          A = T^T (Y)        B = dW (P), dV (Z) -> images Y', X
//      (dY leaves the function as the image X: the caller forms dv, dw from it)
//   6. dA    = -(dX W^T + dY U^T)            A = dX (Y'), dY (X)   B = W (P), U (Z)
//
// Every operand except dO arrives as a bf16 operand image that its producer wrote in exactly this
// layout (W, U: forward prepass; the chunk-entry state S: forward chain; dV, dH: reverse chain; T:
// forward prepass), so staging is one bulk asynchronous copy per operand (cp.async.bulk, completion
// counted on an mbarrier), issued while the previous accumulator drains.  dO is
// the operator's row-major tensor: warps cover 8 rows x 4 pieces of 8 elements per step
// (stage_coords).  fp32 results go to the per-CTA scratch in a PANEL layout, [column / 4][row][4]: a
// thread that owns one row of tensor memory then writes 16 bytes next to its neighbours' and a warp
// store covers 512 contiguous bytes.
#pragma once
#include "dn_common.cuh"
#include "dn_umma.cuh"

namespace dn {

// float4 index of (row, col) in a panel-layout array (col a multiple of 4)
__device__ __forceinline__ int p4v(int row, int col) { return ((col >> 2) << 7) + row; }
// float index of (row, col) in a panel-layout array
__device__ __forceinline__ int p4f(int row, int col) { return ((((col >> 2) << 7) + row) << 2) + (col & 3); }

struct BwdTcIo {
  const __nv_bfloat16 *W, *U;          // this item's (128,128) and (128,VW) tiles, image layout
  const __nv_bfloat16 *S, *dH, *dV;    // this item's (128,VW) images: chunk-entry state, state cotangent, dV
  const __nv_bfloat16* T;              // this item's (128,128) image
  const float* dlend_part;             // this item's (slices, 128) partial sums of sum_v dH * S
  int slices;
  const float* lam_end;                // this item's (128) log-decay to the chunk end
  const void* d_out;                   // whole tensor
  int qkv_dt;
  size_t dO_off;                       // element offset of (row 0, column 0) of this item's dO block
  size_t dO_pitch;                     // elements between token rows
  int rows_valid;                      // rows of the chunk that exist (others read as 0)
  float *DQE, *DKE, *DX, *DM, *DA;       // fp32 results in scratch, panel layout
  float* dlend_s;                      // out (shared, 128): [one doc] exp(lam_end) * sum_v dH * S
  bool all_same;
  const int* seg_s;
  bool trunc;
};

// dO staging.  A warp covers 8 rows x 4 panels per step: its 32 global loads fall in 8 row
// segments of 128 B (fp32) or 64 B (bf16), and each quarter-warp writes 8 consecutive rows of one
// panel (128 contiguous bytes of shared memory).
template <int R>
__device__ __forceinline__ void stage_coords(int e, int& p, int& x) {
  const int lane = e & 31, w = e >> 5;
  x = (w % (R / 8)) * 8 + (lane & 7);
  p = (w / (R / 8)) * 4 + (lane >> 3);
}
// Operand images by bulk asynchronous copies: one thread announces the bytes on the mbarrier and
// issues one copy per image; everybody waits on the barrier (bounded) before the tensor core reads.
struct ImgLoader {
  uint64_t* bar;
  uint32_t phase;
  int* err;
  // (the proxy fence orders the CTA's earlier ordinary accesses to the slot before the copy engine's writes)
  __device__ __forceinline__ void expect(uint32_t bytes) {
    if (threadIdx.x == 0) { umma::fence_async_smem(); umma::mbar_expect_tx(bar, bytes); }
  }
  __device__ __forceinline__ void load(void* dst, const void* src, uint32_t bytes) {
    if (threadIdx.x == 0) umma::bulk_load(dst, src, bytes, bar);
  }
  __device__ __forceinline__ void wait() {
    if (!umma::mbar_wait(bar, phase)) umma::report_timeout(err);
    phase ^= 1u;
  }
};

// `after_products` is called by all threads once the last products have completed, i.e. when every operand
// slot except X is free again, and before the last accumulator is drained: the caller starts the copies
// of its next phase there, so that they travel during the drain.
template <int VW, int NT, class AfterProducts>
__device__ __forceinline__ void bwd_gemms_tc(umma::Ctx& cx, uint8_t* img, const BwdTcIo& io, ImgLoader& ld,
                                             AfterProducts after_products) {
  constexpr int SLOT = 128 * VW * 2;
  uint4* X = reinterpret_cast<uint4*>(img);
  uint4* Y = reinterpret_cast<uint4*>(img + SLOT);
  uint4* Z = reinterpret_cast<uint4*>(img + 2 * SLOT);
  uint4* P = reinterpret_cast<uint4*>(img + 3 * SLOT);
  uint4* Y2 = Y + 128 * 16;                       // second 32 KB of Y (VW = 256) or ...
  if (VW == 128) Y2 = reinterpret_cast<uint4*>(img + 3 * SLOT + 32768);   // ... an extra slot after P
  constexpr int PV = VW / 8;                      // panels along the value width
  const int* seg_s = io.seg_s;
  float4* DQE4 = reinterpret_cast<float4*>(io.DQE);
  float4* DKE4 = reinterpret_cast<float4*>(io.DKE);
  float4* DX4 = reinterpret_cast<float4*>(io.DX);
  float4* DM4 = reinterpret_cast<float4*>(io.DM);
  float4* DA4 = reinterpret_cast<float4*>(io.DA);

  DN_MARK(1);
  // ---- 1. V_new = U - W S: the product in tensor memory, U taken from its image by the drain
  constexpr uint32_t B_KK = 128 * 128 * 2, B_KV = 128 * VW * 2;     // bytes of a (128,128) / (128,VW) image
  ld.expect(B_KK + 2 * B_KV);
  ld.load(P, io.W, B_KK);
  ld.load(X, io.S, B_KV);
  ld.load(Z, io.U, B_KV);
  // dLambda_end = [one doc] exp(Lambda_end) sum_v dH * S  (gdn2.py:759-762) from the reverse chain's
  // per-slice partial sums, added in a fixed order
  if (threadIdx.x < 128) {
    float acc = 0.f;
    for (int sl = 0; sl < io.slices; ++sl) acc += __ldg(io.dlend_part + sl * 128 + threadIdx.x);
    io.dlend_s[threadIdx.x] = io.all_same ? acc * expf(fminf(__ldg(io.lam_end + threadIdx.x), 0.f)) : 0.f;
  }
  ld.wait();
  umma::pre_issue_sync();
  umma::issue<VW, false, true>(cx, P, X, 128, 0, false);
  umma::commit_wait(cx);
  umma::drain<NT, VW>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float u0[8], u1[8];
    umma::unpack8(Z[(col / 8) * 128 + row], u0);
    umma::unpack8(Z[(col / 8 + 1) * 128 + row], u1);
#pragma unroll
    for (int i = 0; i < 8; ++i) { u0[i] -= v[i]; u1[i] -= v[8 + i]; }
    Y[(col / 8) * 128 + row] = umma::pack8(u0);
    Y[(col / 8 + 1) * 128 + row] = umma::pack8(u1);
  });
  __syncthreads();                                // every row of U has been read before dO overwrites Z

  DN_MARK(2);
  // ---- 2. dqe = dO S^T, dM = dO V_new^T
  if (io.qkv_dt == DN_BF16) {
#pragma unroll
    for (int it = 0; it < PV * 128 / NT; ++it) {
      int p, x;
      stage_coords<128>(it * NT + threadIdx.x, p, x);
      if (x < io.rows_valid)
        umma::cp_async16(Z + p * 128 + x, reinterpret_cast<const __nv_bfloat16*>(io.d_out) + io.dO_off + (size_t)x * io.dO_pitch + 8 * p);
      else
        Z[p * 128 + x] = make_uint4(0, 0, 0, 0);
    }
    umma::cp_async_commit();
    umma::cp_async_wait<0>();
  } else {
#pragma unroll 8
    for (int it = 0; it < PV * 128 / NT; ++it) {
      int p, x;
      stage_coords<128>(it * NT + threadIdx.x, p, x);
      const bool live = x < io.rows_valid;
      uint4 val = umma::ld8_f32_ro(reinterpret_cast<const float*>(io.d_out) + io.dO_off + (size_t)(live ? x : 0) * io.dO_pitch + 8 * p);
      if (!live) val = make_uint4(0, 0, 0, 0);
      Z[p * 128 + x] = val;
    }
  }
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Z, X, VW, 256, false);
  umma::issue<128, false, false>(cx, Z, Y, VW, 384, false);
  umma::commit_wait(cx);
  ld.expect(B_KV);
  ld.load(Z, io.dV, B_KV);                           // dO has been consumed: dV for step 3 travels during the drains
  umma::drain<NT, 128>(cx, 256, [&](int row, int col, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::st_keep4(DQE4 + p4v(row, col + 4 * i), make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
  });
  umma::drain<NT, 128>(cx, 384, [&](int row, int col, const float (&v)[16]) {
    float m[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = (row >= col + i && seg_s[row] == seg_s[col + i]) ? v[i] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::st_keep4(DM4 + p4v(row, col + 4 * i), make_float4(m[4 * i], m[4 * i + 1], m[4 * i + 2], m[4 * i + 3]));
  });

  DN_MARK(3);
  // ---- 3. dW = -dV S^T (kept only as the operand image of step 5)
  ld.wait();
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Z, X, VW, 0, false);
  umma::commit_wait(cx);
  ld.expect(B_KV);
  ld.load(X, io.dH, B_KV);                           // S has been consumed: dH for step 4 travels during the drain
  umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float n[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) n[i] = -v[i];
    P[(col / 8) * 128 + row] = umma::pack8p(n);
    P[(col / 8 + 1) * 128 + row] = umma::pack8p(n + 8);
  });

  DN_MARK(4);
  // ---- 4. dke = V_new dH^T
  ld.wait();
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Y, X, VW, 128, false);
  umma::commit_wait(cx);
  ld.expect(B_KK);
  ld.load(Y, io.T, B_KK);                             // V_new has been consumed: T for step 5
  umma::drain<NT, 128>(cx, 128, [&](int row, int col, const float (&v)[16]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::st_keep4(DKE4 + p4v(row, col + 4 * i), make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]));
  });

  DN_MARK(5);
  // ---- 5. dX = T^T dW, dY = T^T dV
  ld.wait();
  umma::pre_issue_sync();
  umma::issue<128, true, true>(cx, Y, P, 128, 0, false);
  umma::issue<VW, true, true>(cx, Y, Z, 128, 256, false);
  umma::commit_wait(cx);
  ld.expect(B_KK + B_KV);
  ld.load(P, io.W, B_KK);                             // dW and dV have been consumed: W, U for step 6
  ld.load(Z, io.U, B_KV);
  umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float r[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = io.trunc ? bf16r(v[i]) : v[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::st_keep4(DX4 + p4v(row, col + 4 * i), make_float4(r[4 * i], r[4 * i + 1], r[4 * i + 2], r[4 * i + 3]));
    Y2[(col / 8) * 128 + row] = umma::pack8p(r);
    Y2[(col / 8 + 1) * 128 + row] = umma::pack8p(r + 8);
  });
  // dY is kept only as its bf16 image X: operand of step 6, and read again by the caller for dv, dw
  umma::drain<NT, VW>(cx, 256, [&](int row, int col, const float (&v)[16]) {
    X[(col / 8) * 128 + row] = umma::pack8p(v);
    X[(col / 8 + 1) * 128 + row] = umma::pack8p(v + 8);
  });

  DN_MARK(6);
  // ---- 6. dA = -(dX W^T + dY U^T), strictly lower and same document
  ld.wait();
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Y2, P, 128, 0, false);
  umma::issue<128, false, false>(cx, X, Z, VW, 0, true);
  umma::commit_wait(cx);
  after_products();
  umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float m[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = (row > col + i && seg_s[row] == seg_s[col + i]) ? -v[i] : 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) umma::st_keep4(DA4 + p4v(row, col + 4 * i), make_float4(m[4 * i], m[4 * i + 1], m[4 * i + 2], m[4 * i + 3]));
  });
  __syncthreads();
}

// bytes of operand images: VW=256: X,Y,Z (64 KB each) + P (32 KB); VW=128: X,Y,Z,P (32 KB each) + Y2 (32 KB)
__host__ __device__ constexpr int bwd_tc_image_bytes(int vw) { return vw == 256 ? 3 * 65536 + 32768 : 5 * 32768; }

}  // namespace dn
