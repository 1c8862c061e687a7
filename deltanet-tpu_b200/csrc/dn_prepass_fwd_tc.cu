// Prepass forward on the tcgen05 tensor cores (bf16 precision, chunk = K = 128, value width
// 128 or 256).  Produces the same outputs as the fp32 formulation in dn_prepass_fwd.cu
// (reference body: src/deltanet_tpu/gdn2.py:115-240).
//
// A and M.  A_ij = sum_c beta_ic exp(Lam_ic - Lam_jc) k_jc cannot be one matrix product because
// the decay couples i, j and the channel c.  It is built hierarchically: at level s in {64,32,16}
// the chunk is cut into pairs of adjacent s-row blocks, and for a pair with rows I (lower block),
// columns J (upper block) and reference row r = first row of I
//     A[I,J] = (beta_I * exp(Lam_I - Lam_r)) (k_J * exp(Lam_r - Lam_J))^T ,
// with both scale factors <= 1 (the cumulative decay is monotone inside a document), so nothing
// can overflow however strong the decay.  Scaling EVERY row by its own pair's factors turns each
// level into ONE 128x128x128 MMA (per matrix); entries outside the level's blocks are finite
// garbage that the drain ignores (entry (i,j) belongs to the level of the highest bit in which
// i>>4 and j>>4 differ).  The 16x16 diagonal blocks are evaluated exactly, pair by pair, on the
// CUDA cores.  The reference does the same with 32-row blocks and one reference per block row
// (gdn2.py:162-197).
//
// T = (I+A)^-1 is obtained as in the fp32 formulation (substitution on 16x16 blocks + block
// merges, fp32 in shared memory); W = T X and U = T Y are tcgen05 MMAs on bf16 operands, which
// is also where the reference rounds to bf16 (gdn2.py:226-230).
//
// 512 threads per CTA, one CTA per SM, looping over (batch, exec head, chunk) items.  The
// cumulative decay stays in shared memory; q, k, b, g, v, w are read straight from the user's
// tensors in 16/32-byte pieces (no staging copy in global memory).
#include "dn_chunkprep.cuh"
#include "dn_kernels.cuh"

namespace dn {
namespace {

using namespace prep;
constexpr int NT = 512;
constexpr int OFF_IMG = C * LP * 4;                 // level images start after Lambda
constexpr int OFF_XI = 3 * 65536;                   // X image: survives the inverse

__device__ __forceinline__ void load4(const void* base, size_t off, int dt, float (&x)[4]) {
  if (dt == DN_BF16) {
    const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(base) + off);
    x[0] = __uint_as_float(u.x << 16); x[1] = __uint_as_float(u.x & 0xffff0000u);
    x[2] = __uint_as_float(u.y << 16); x[3] = __uint_as_float(u.y & 0xffff0000u);
  } else {
    const float4 a = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);
    x[0] = a.x; x[1] = a.y; x[2] = a.z; x[3] = a.w;
  }
}

// four channels (4*lane ..) of k_hat, q_hat, beta for chunk row x
__device__ __forceinline__ void row4(const Rows& r, int x, int lane, float (&kh)[4], float (&qh)[4], float (&be)[4],
                                     bool want_q) {
#pragma unroll
  for (int i = 0; i < 4; ++i) kh[i] = qh[i] = be[i] = 0.f;
  if (x >= r.rows_valid) return;
  const size_t off = r.qk_row0 + (size_t)x * r.qk_pitch + 4 * lane;
  load4(r.k, off, r.qkv_dt, kh);
  if (r.l2) {
#pragma unroll
    for (int i = 0; i < 4; ++i) { kh[i] *= r.rk[x]; if (r.round_in) kh[i] = bf16r(kh[i]); }
  }
  if (!want_q) return;
  load4(r.q, off, r.qkv_dt, qh);
#pragma unroll
  for (int i = 0; i < 4; ++i) { qh[i] = (qh[i] * r.rq[x]) * r.scale; if (r.round_in) qh[i] = bf16r(qh[i]); }
  if (r.bC == 1) {
    const float v = ldf(r.b, r.b_row0 + (size_t)x * r.b_pitch, r.gate_dt);
#pragma unroll
    for (int i = 0; i < 4; ++i) be[i] = v;
  } else {
    load4(r.b, r.b_row0 + (size_t)x * r.b_pitch + 4 * lane, r.gate_dt, be);
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (r.fuse) be[i] = 1.f / (1.f + expf(-be[i]));
    be[i] *= kh[i];
  }
}

template <int VW>
__global__ void __launch_bounds__(NT, 1) prepass_fwd_tc_kernel(PrepassFwdArgs a, int* err) {
  extern __shared__ __align__(128) uint8_t smraw[];
  __shared__ uint64_t mma_bar;
  __shared__ uint32_t tmem_base;
  __shared__ int seg_s[C];
  __shared__ float rq_s[C], rk_s[C];
  const Geo& g = a.g;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float* LAM = reinterpret_cast<float*>(smraw);
  uint4* RB = reinterpret_cast<uint4*>(smraw + OFF_IMG);
  uint4* RQ = RB + IMG;
  uint4* KC = RQ + IMG;
  uint4* XI = reinterpret_cast<uint4*>(smraw + OFF_XI);
  float* As = reinterpret_cast<float*>(smraw);
  float* Ts = As + C * C;
  float* Tm = Ts + C * C;
  uint4* TI = reinterpret_cast<uint4*>(smraw);
  uint4* YI = reinterpret_cast<uint4*>(Tm);

  float* Ag = a.scratch + (size_t)blockIdx.x * a.scratch_per_cta;     // A (fp32), masked

  if (tid == 0) { umma::mbar_init(&mma_bar, 1); umma::fence_mbar_init(); }
  if (warp == 0) umma::tmem_alloc(&tmem_base, 512);
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &mma_bar, 0u, err, false};

  __nv_bfloat16* Wg = reinterpret_cast<__nv_bfloat16*>(a.res.W);
  __nv_bfloat16* Ug = reinterpret_cast<__nv_bfloat16*>(a.res.U);
  __nv_bfloat16* Mg = reinterpret_cast<__nv_bfloat16*>(a.res.M);
  __nv_bfloat16* QEg = reinterpret_cast<__nv_bfloat16*>(a.res.qe);
  __nv_bfloat16* KEg = reinterpret_cast<__nv_bfloat16*>(a.res.ke);
  const bool fuse = g.flags & DN_FUSE_PROLOGUE;

  for (int item = blockIdx.x; item < a.items; item += gridDim.x) {
    const int c_idx = item % g.NC, h = (item / g.NC) % g.H, b = item / (g.NC * g.H);
    const int t0 = c_idx * C;
    const size_t ibase = (size_t)item;
    for (int i = tid; i < C; i += NT) seg_s[i] = seg_at(a.seg, b, t0 + i, g.L);
    const Rows r = make_rows(g, a.q, a.k, a.gg, a.b, b, h, t0, rq_s, rk_s);
    row_norms<NT>(r, rq_s, rk_s);
    __syncthreads();
    const int seg0 = seg_s[0], segL = seg_s[C - 1];
    build_lambda<NT>(r, seg_s, LAM);

    // ---- qe, ke, Lambda_end and the X = [first doc] beta e^Lam operand image
    for (int e = tid; e < IMG; e += NT) {
      const int x = e >> 4, p = e & 15;
      float qh[8], kh[8], lam[8], o[8];
      qhat8(r, x, p, qh);
      khat8(r, x, p, kh);
      const float4 l0 = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p), l1 = *reinterpret_cast<const float4*>(LAM + x * LP + 8 * p + 4);
      lam[0] = l0.x; lam[1] = l0.y; lam[2] = l0.z; lam[3] = l0.w; lam[4] = l1.x; lam[5] = l1.y; lam[6] = l1.z; lam[7] = l1.w;
      const bool first = seg_s[x] == seg0, last = seg_s[x] == segL;
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = first ? qh[i] * expf(fminf(lam[i], 0.f)) : 0.f;
      *reinterpret_cast<uint4*>(QEg + ibase * C * K + (size_t)x * K + 8 * p) = umma::pack8(o);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = last ? kh[i] * expf(fminf(LAM[(C - 1) * LP + 8 * p + i] - lam[i], 0.f)) : 0.f;
      *reinterpret_cast<uint4*>(KEg + ibase * C * K + (size_t)x * K + 8 * p) = umma::pack8(o);
      if (x == C - 1) {
#pragma unroll
        for (int i = 0; i < 8; ++i) a.res.lam_end[ibase * K + 8 * p + i] = lam[i];
      }
      float be[8];
      bact8(r, x, p, be);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = first ? be[i] * kh[i] * expf(fminf(lam[i], 0.f)) : 0.f;
      XI[p * 128 + x] = umma::pack8(o);
    }

    // ---- A and M, level by level: three images, two MMAs, one predicated drain per level
    for (int lv = 0; lv < 3; ++lv) {
      build_level<NT>(r, LAM, 16 << lv, RB, RQ, KC);
      umma::pre_issue_sync();
      umma::issue<128, false, false>(cx, RB, KC, K, 0, false);
      umma::issue<128, false, false>(cx, RQ, KC, K, 128, false);
      umma::commit_wait(cx);
      {
        const int quarter = warp & 3, group = warp >> 2;
        const int row = quarter * 32 + lane, bi = row >> 4, bi0 = quarter * 2;
        const uint32_t lane_base = (uint32_t)(quarter * 32) << 16;
        for (int c = 0; c < 32; c += 16) {
          const int col = group * 32 + c, bj = col >> 4;
          // warp-uniform skip: neither of the warp's two row blocks has this piece at this level
          const bool own0 = bj < bi0 && owner_level(bi0, bj) == lv, own1 = bj < bi0 + 1 && owner_level(bi0 + 1, bj) == lv;
          const bool upper = lv == 0 && bj > bi0;                  // zero fill, once
          if (!own0 && !own1 && !upper) continue;
          float va[16], vm[16];
          if (!cx.dead && (own0 || own1)) {
            umma::tmem_ld16(cx.tmem + lane_base + col, va);
            umma::tmem_ld16(cx.tmem + lane_base + 128 + col, vm);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) va[i] = vm[i] = 0.f;
          }
          const bool mine = bj < bi && owner_level(bi, bj) == lv;
          const bool zero_fill = lv == 0 && bj > bi;
          if (!mine && !zero_fill) continue;
          float oa[16], om[16];
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const bool keep = mine && seg_s[row] == seg_s[col + i];
            oa[i] = keep ? va[i] : 0.f;
            om[i] = keep ? vm[i] : 0.f;
          }
          float4* da = reinterpret_cast<float4*>(Ag + row * C + col);
#pragma unroll
          for (int i = 0; i < 4; ++i) da[i] = make_float4(oa[4 * i], oa[4 * i + 1], oa[4 * i + 2], oa[4 * i + 3]);
          float lo[8], hi[8];
#pragma unroll
          for (int i = 0; i < 8; ++i) { lo[i] = om[i]; hi[i] = om[8 + i]; }
          uint4* dm = reinterpret_cast<uint4*>(Mg + ibase * C * C + (size_t)row * C + col);
          dm[0] = umma::pack8(lo);
          dm[1] = umma::pack8(hi);
        }
        umma::tc_fence_before();
      }
      __syncthreads();
    }

    // ---- 16x16 diagonal blocks, exact: two warps per block (alternate rows), lanes own 4 channels
    {
      const int r0 = (warp >> 1) * 16;
      for (int i = warp & 1; i < 16; i += 2) {
        const int ri = r0 + i;
        float ki[4], qi[4], bi4[4];
        row4(r, ri, lane, ki, qi, bi4, true);
        const float4 li = *reinterpret_cast<const float4*>(LAM + ri * LP + 4 * lane);
        float arow = 0.f, mrow = 0.f;                  // lane j (< 16) keeps entry (ri, r0 + j)
        for (int j = 0; j <= i; ++j) {
          const int rj = r0 + j;
          float kj[4], dq[4], db[4];
          row4(r, rj, lane, kj, dq, db, false);
          const float4 lj = *reinterpret_cast<const float4*>(LAM + rj * LP + 4 * lane);
          const float e0 = kj[0] * exp2f(fminf(li.x - lj.x, 0.f) * DN_LOG2E), e1 = kj[1] * exp2f(fminf(li.y - lj.y, 0.f) * DN_LOG2E);
          const float e2 = kj[2] * exp2f(fminf(li.z - lj.z, 0.f) * DN_LOG2E), e3 = kj[3] * exp2f(fminf(li.w - lj.w, 0.f) * DN_LOG2E);
          float pa = bi4[0] * e0 + bi4[1] * e1 + bi4[2] * e2 + bi4[3] * e3;
          float pm = qi[0] * e0 + qi[1] * e1 + qi[2] * e2 + qi[3] * e3;
          pa = warp_sum(pa);
          pm = warp_sum(pm);
          const bool same = seg_s[ri] == seg_s[rj];
          if (lane == j) { arow = (j < i && same) ? pa : 0.f; mrow = same ? pm : 0.f; }
        }
        if (lane < 16) {
          Ag[ri * C + r0 + lane] = arow;
          Mg[ibase * C * C + (size_t)ri * C + r0 + lane] = __float2bfloat16_rn(mrow);
        }
      }
    }
    __syncthreads();

    // ---- T = (I + A)^-1 in fp32: substitution on the diagonal blocks, then block merges
    for (int e = tid; e < C * C / 4; e += NT) {
      reinterpret_cast<float4*>(As)[e] = reinterpret_cast<const float4*>(Ag)[e];
      reinterpret_cast<float4*>(Ts)[e] = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
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
      for (int e = tid; e < total; e += NT) {
        const int p = e / (s * s), rem = e - p * s * s, il = rem / s, jl = rem - il * s;
        const int i = 2 * p * s + s + il, j = 2 * p * s + jl, mend = 2 * p * s + s;
        float acc = 0.f;
        for (int m = j; m < mend; ++m) acc = fmaf(As[i * C + m], Ts[m * C + j], acc);
        Tm[i * C + j] = acc;
      }
      __syncthreads();
      for (int e = tid; e < total; e += NT) {
        const int p = e / (s * s), rem = e - p * s * s, il = rem / s, jl = rem - il * s;
        const int i = 2 * p * s + s + il, j = 2 * p * s + jl, m0 = 2 * p * s + s;
        float acc = 0.f;
        for (int m = m0; m <= i; ++m) acc = fmaf(Ts[i * C + m], Tm[m * C + j], acc);
        Ts[i * C + j] = -acc;
      }
      __syncthreads();
    }
    if (a.res.T)
      for (int e = tid; e < C * C / 4; e += NT)
        reinterpret_cast<float4*>(a.res.T + ibase * C * C)[e] = reinterpret_cast<const float4*>(Ts)[e];

    // ---- W = T X, U = T Y on the tensor cores
    for (int e = tid; e < IMG; e += NT) {                       // T as K-major A: piece (p = j/8, x = i)
      const int p = e >> 7, x = e & 127;
      TI[e] = umma::ld8_f32(Ts + x * C + 8 * p);
    }
    for (int e = tid; e < (VW / 8) * 128; e += NT) {            // Y = w*v as MN-major B
      const int p = e >> 7, x = e & 127, t = t0 + x;
      float f[8];
      zero8(f);
      if (t < g.L) {
        const int col0 = h * VW + 8 * p, hv = col0 / g.V, cv = col0 - hv * g.V;
        float vv[8], ww[8];
        load8(a.v, (size_t)(b * (size_t)g.L + t) * g.Hv * g.V + col0, g.qkv_dt, vv);
        const size_t wrow = ((size_t)(b * (size_t)g.L + t) * g.wH + g.w_head(hv)) * g.wC;
        if (g.wC == 1) {
          const float w1 = ldf(a.w, wrow, g.gate_dt);
#pragma unroll
          for (int i = 0; i < 8; ++i) ww[i] = w1;
        } else {
          load8(a.w, wrow + cv, g.gate_dt, ww);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const float wa = fuse ? 1.f / (1.f + expf(-ww[i])) : ww[i];
          f[i] = wa * vv[i];
        }
      }
      YI[p * 128 + x] = umma::pack8(f);
    }
    umma::pre_issue_sync();
    umma::issue<128, false, true>(cx, TI, XI, C, 0, false);
    umma::issue<VW, false, true>(cx, TI, YI, C, 128, false);
    umma::commit_wait(cx);
    umma::drain<NT, 128>(cx, 0, [&](int row, int col, const float (&v)[16]) {
      float lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
      uint4* d = reinterpret_cast<uint4*>(Wg + ibase * C * K + (size_t)row * K + col);
      d[0] = umma::pack8(lo);
      d[1] = umma::pack8(hi);
    });
    umma::drain<NT, VW>(cx, 128, [&](int row, int col, const float (&v)[16]) {
      float lo[8], hi[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) { lo[i] = v[i]; hi[i] = v[8 + i]; }
      uint4* d = reinterpret_cast<uint4*>(Ug + ibase * C * VW + (size_t)row * VW + col);
      d[0] = umma::pack8(lo);
      d[1] = umma::pack8(hi);
    });
    __syncthreads();
  }
  umma::tc_fence_before();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, 512);
}

}  // namespace

bool prepass_fwd_tc_eligible(const Geo& g) {
  return g.prec == DN_PREC_BF16 && g.C == 128 && g.K == 128 && (g.Vw == 128 || g.Vw == 256);
}

size_t prepass_fwd_tc_scratch_per_cta() { return (size_t)C * C; }

int launch_prepass_fwd_tc(const Geo& g, const void* q, const void* k, const void* v, const void* gg,
                          const void* b, const void* w, const int32_t* seg, const dn_residuals& res,
                          float* scratch, size_t scratch_floats, cudaStream_t st) {
  PrepassFwdArgs a;
  a.g = g; a.q = q; a.k = k; a.v = v; a.gg = gg; a.b = b; a.w = w; a.seg = seg; a.res = res;
  a.items = g.B * g.H * g.NC;
  a.scratch_per_cta = prepass_fwd_tc_scratch_per_cta();
  a.smem_tile_off = 0;
  const int grid = a.items < 148 ? a.items : 148;
  if (scratch_floats < (size_t)grid * a.scratch_per_cta) return DN_ERR_SCRATCH_TOO_SMALL;
  a.scratch = scratch;
  const size_t smem = 3 * 65536 + 32768;
  int* err = device_error_ptr();
  if (g.Vw == 256) {
    cudaFuncSetAttribute(prepass_fwd_tc_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    prepass_fwd_tc_kernel<256><<<grid, NT, smem, st>>>(a, err);
  } else {
    cudaFuncSetAttribute(prepass_fwd_tc_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    prepass_fwd_tc_kernel<128><<<grid, NT, smem, st>>>(a, err);
  }
  return cudaGetLastError() == cudaSuccess ? DN_OK : DN_ERR_CUDA_LAUNCH;
}

}  // namespace dn
