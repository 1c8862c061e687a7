// The nine matrix products of the chunk-parallel backward on the tcgen05 tensor cores
// (bf16 precision, chunk = K = 128, value width VW in {128, 256}).
//
// Operand images live in four shared-memory slots (X, Y, Z of 128 x VW bf16, P of 128 x 128)
// that are refilled as the sequence advances; accumulators live in tensor memory (512 columns)
// and are drained one row per thread.  An image written once serves as a matrix and as its
// transpose (the descriptor says which), which is why S, V_new, dV, W and U are staged only once
// per use group:
//   1. V_new = U - W S                      A = W (P)        B = S (X)          -> image Y
//   2. dqe   = dO S^T ; dM = dO V_new^T      A = dO (Z)       B = S (X), V_new (Y)
//   3. dW    = -dV S^T                       A = dV (Z)       B = S (X)          -> image P
//   4. dke   = V_new dH^T                    A = V_new (Y)    B = dH (X)
//   5. dX    = T^T dW ; dY = T^T dV          A = T^T (Y)      B = dW (P), dV (Z) -> images Y', X
//   6. dA    = -(dX W^T + dY U^T)            A = dX (Y'), dY (X)   B = W (P), U (Z)
#pragma once
#include "dn_common.cuh"
#include "dn_umma.cuh"

namespace dn {

struct BwdTcIo {
  const __nv_bfloat16 *W, *U;          // this item's (128,128) and (128,VW) tiles
  const float *S, *dH, *dV, *T;        // this item's fp32 arrays: (128,VW), (128,VW), (128,VW), (128,128)
  const void* d_out;                   // whole tensor
  int qkv_dt;
  size_t dO_off;                       // element offset of (row 0, column 0) of this item's dO block
  size_t dO_pitch;                     // elements between token rows
  int rows_valid;                      // rows of the chunk that exist (others read as 0)
  float *DQE, *DKE, *DX, *DY, *DM, *DA;  // fp32 results in scratch
  const int* seg_s;
  bool trunc;
};

template <int R, int NT>
__device__ __forceinline__ void stage_f32(uint4* dst, const float* src, int pitch, int panels) {
  for (int e = threadIdx.x; e < panels * R; e += NT) {
    const int p = e / R, x = e - p * R;
    dst[e] = umma::ld8_f32(src + (size_t)x * pitch + 8 * p);
  }
}
template <int R, int NT>
__device__ __forceinline__ void stage_bf16(uint4* dst, const __nv_bfloat16* src, int pitch, int panels) {
  for (int e = threadIdx.x; e < panels * R; e += NT) {
    const int p = e / R, x = e - p * R;
    dst[e] = umma::ld8_bf16(src + (size_t)x * pitch + 8 * p);
  }
}

template <int VW, int NT>
__device__ __forceinline__ void bwd_gemms_tc(umma::Ctx& cx, uint8_t* img, const BwdTcIo& io) {
  constexpr int SLOT = 128 * VW * 2;
  uint4* X = reinterpret_cast<uint4*>(img);
  uint4* Y = reinterpret_cast<uint4*>(img + SLOT);
  uint4* Z = reinterpret_cast<uint4*>(img + 2 * SLOT);
  uint4* P = reinterpret_cast<uint4*>(img + 3 * SLOT);
  uint4* Y2 = Y + 128 * 16;                       // second 32 KB of Y (VW = 256) or ...
  if (VW == 128) Y2 = reinterpret_cast<uint4*>(img + 3 * SLOT + 32768);   // ... an extra slot after P
  constexpr int PV = VW / 8;                      // panels along the value width
  const int* seg_s = io.seg_s;

  // ---- 1. V_new = U - W S
  stage_bf16<128, NT>(P, io.W, 128, 16);
  stage_f32<128, NT>(X, io.S, VW, PV);
  umma::pre_issue_sync();
  umma::issue<VW, false, true>(cx, P, X, 128, 0, false);
  umma::commit_wait(cx);
  umma::drain<NT, VW>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float u0[8], u1[8];
    const uint4* up = reinterpret_cast<const uint4*>(io.U + (size_t)row * VW + col);
    umma::unpack8(up[0], u0);
    umma::unpack8(up[1], u1);
#pragma unroll
    for (int i = 0; i < 8; ++i) { u0[i] -= v[i]; u1[i] -= v[8 + i]; }
    Y[(col / 8) * 128 + row] = umma::pack8(u0);
    Y[(col / 8 + 1) * 128 + row] = umma::pack8(u1);
  });

  // ---- 2. dqe = dO S^T, dM = dO V_new^T
  for (int e = threadIdx.x; e < PV * 128; e += NT) {
    const int p = e / 128, x = e - p * 128;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (x < io.rows_valid) {
      const size_t off = io.dO_off + (size_t)x * io.dO_pitch + 8 * p;
      val = io.qkv_dt == DN_BF16 ? umma::ld8_bf16(reinterpret_cast<const __nv_bfloat16*>(io.d_out) + off)
                                 : umma::ld8_f32(reinterpret_cast<const float*>(io.d_out) + off);
    }
    Z[e] = val;
  }
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Z, X, VW, 256, false);
  umma::issue<128, false, false>(cx, Z, Y, VW, 384, false);
  umma::commit_wait(cx);
  umma::drain<NT, 128>(cx, 256, [&](int row, int col, const float (&v)[16]) {
    float4* d = reinterpret_cast<float4*>(io.DQE + row * 128 + col);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  });
  umma::drain<NT, 128>(cx, 384, [&](int row, int col, const float (&v)[16]) {
    float m[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = (row >= col + i && seg_s[row] == seg_s[col + i]) ? v[i] : 0.f;
    float4* d = reinterpret_cast<float4*>(io.DM + row * 128 + col);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = make_float4(m[4 * i], m[4 * i + 1], m[4 * i + 2], m[4 * i + 3]);
  });

  // ---- 3. dW = -dV S^T (kept only as the operand image of step 5)
  stage_f32<128, NT>(Z, io.dV, VW, PV);
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Z, X, VW, 0, false);
  umma::commit_wait(cx);
  umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = -v[i]; b[i] = -v[8 + i]; }
    P[(col / 8) * 128 + row] = umma::pack8(a);
    P[(col / 8 + 1) * 128 + row] = umma::pack8(b);
  });

  // ---- 4. dke = V_new dH^T
  stage_f32<128, NT>(X, io.dH, VW, PV);
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Y, X, VW, 128, false);
  umma::commit_wait(cx);
  umma::drain<NT, 128>(cx, 128, [&](int row, int col, const float (&v)[16]) {
    float4* d = reinterpret_cast<float4*>(io.DKE + row * 128 + col);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
  });

  // ---- 5. dX = T^T dW, dY = T^T dV
  stage_f32<128, NT>(Y, io.T, 128, 16);
  umma::pre_issue_sync();
  umma::issue<128, true, true>(cx, Y, P, 128, 0, false);
  umma::issue<VW, true, true>(cx, Y, Z, 128, 256, false);
  umma::commit_wait(cx);
  umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = io.trunc ? bf16r(v[i]) : v[i]; b[i] = io.trunc ? bf16r(v[8 + i]) : v[8 + i]; }
    float4* d = reinterpret_cast<float4*>(io.DX + row * 128 + col);
    d[0] = make_float4(a[0], a[1], a[2], a[3]); d[1] = make_float4(a[4], a[5], a[6], a[7]);
    d[2] = make_float4(b[0], b[1], b[2], b[3]); d[3] = make_float4(b[4], b[5], b[6], b[7]);
    Y2[(col / 8) * 128 + row] = umma::pack8(a);
    Y2[(col / 8 + 1) * 128 + row] = umma::pack8(b);
  });
  umma::drain<NT, VW>(cx, 256, [&](int row, int col, const float (&v)[16]) {
    float a[8], b[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) { a[i] = io.trunc ? bf16r(v[i]) : v[i]; b[i] = io.trunc ? bf16r(v[8 + i]) : v[8 + i]; }
    float4* d = reinterpret_cast<float4*>(io.DY + (size_t)row * VW + col);
    d[0] = make_float4(a[0], a[1], a[2], a[3]); d[1] = make_float4(a[4], a[5], a[6], a[7]);
    d[2] = make_float4(b[0], b[1], b[2], b[3]); d[3] = make_float4(b[4], b[5], b[6], b[7]);
    X[(col / 8) * 128 + row] = umma::pack8(a);
    X[(col / 8 + 1) * 128 + row] = umma::pack8(b);
  });

  // ---- 6. dA = -(dX W^T + dY U^T), strictly lower and same document
  stage_bf16<128, NT>(P, io.W, 128, 16);
  stage_bf16<128, NT>(Z, io.U, VW, PV);
  umma::pre_issue_sync();
  umma::issue<128, false, false>(cx, Y2, P, 128, 0, false);
  umma::issue<128, false, false>(cx, X, Z, VW, 0, true);
  umma::commit_wait(cx);
  umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
    float m[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) m[i] = (row > col + i && seg_s[row] == seg_s[col + i]) ? -v[i] : 0.f;
    float4* d = reinterpret_cast<float4*>(io.DA + row * 128 + col);
#pragma unroll
    for (int i = 0; i < 4; ++i) d[i] = make_float4(m[4 * i], m[4 * i + 1], m[4 * i + 2], m[4 * i + 3]);
  });
  __syncthreads();
}

// bytes of operand images: VW=256: X,Y,Z (64 KB each) + P (32 KB); VW=128: X,Y,Z,P (32 KB each) + Y2 (32 KB)
__host__ __device__ constexpr int bwd_tc_image_bytes(int vw) { return vw == 256 ? 3 * 65536 + 32768 : 5 * 32768; }

}  // namespace dn
