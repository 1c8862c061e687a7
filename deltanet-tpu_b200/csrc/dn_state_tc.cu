// Inter-chunk recurrence on the tcgen05 tensor cores (bf16 precision, chunk = K = 128).
//
// Same math and same CTA decomposition as the fp32 formulation in dn_state.cu: one CTA carries
// a (128 x VS) column slice of the state of one (batch, exec head) through all chunks.  Here
//   * the fp32 master copy of the slice lives in registers, one state row per thread
//     (128 threads), and a bf16 copy in shared memory is the MMA operand -- the reference rounds
//     the state to bf16 for these products as well (src/deltanet_tpu/gdn2.py:627-632);
//   * the four 128x128 bf16 tiles of a chunk (W, qe, M, ke) are operand images in global memory and
//     arrive one chunk ahead by one bulk copy each (mbarrier completion), each buffer refilled as
//     soon as the MMA reading it has completed (row-major tiles of the fp32-residual layout: 16-byte
//     cp.async copies); passes that need no outputs fetch W and ke only;
//   * every product is a 128 x VS x 128 tcgen05.mma with the accumulator in tensor memory,
//     read back one row per thread.  A 128x128 tile image in shared memory serves both as the
//     operand (K-major descriptor) and as its transpose (MN-major descriptor), so ke^T, M^T,
//     qe^T and W^T need no data movement.
// Every wait on the MMA barrier is bounded; on a timeout the CTA stops issuing tensor work,
// raises the library's error word and runs to its end.
#include "dn_kernels.cuh"
#include "dn_umma.cuh"

namespace dn {

namespace {

constexpr int TILE_U4 = 128 * 16;   // a 128x128 bf16 tile in 16-byte units

__device__ __forceinline__ size_t native_state_index_tc(const Geo& g, int b, int h, int k, int jj) {
  const int hv = h * g.G + jj / g.V, cv = jj % g.V;
  return (((size_t)b * g.Hv + hv) * g.K + k) * g.V + cv;
}

// Thread `row` copies its share of a (128,128) bf16 tile into the panel image: its 256-byte row of
// a row-major tile, or (img) piece `row` of each of the 16 panels of a tile that already lies in
// global memory as the image -- then a warp's 32 copies are 512 contiguous bytes.
__device__ __forceinline__ void copy_tile_async(uint4* dst, const __nv_bfloat16* src, int row, bool img) {
  if (img) {
    const uint4* s = reinterpret_cast<const uint4*>(src) + row;
#pragma unroll
    for (int p = 0; p < 16; ++p) umma::cp_async16(dst + p * 128 + row, s + p * 128);
  } else {
    const uint4* s = reinterpret_cast<const uint4*>(src + (size_t)row * 128);
#pragma unroll
    for (int p = 0; p < 16; ++p) umma::cp_async16(dst + p * 128 + row, s + p);
  }
}

// A (128,128) bf16 tile that lies in global memory as its operand image: one bulk copy, issued by
// one thread, completion counted on an mbarrier (image layout only).
__device__ __forceinline__ void bulk_tile(uint4* dst, const __nv_bfloat16* src, uint64_t* bar) {
  umma::bulk_load(dst, src, TILE_U4 * 16, bar);
}

template <int VS>
__device__ __forceinline__ void stage_rows(uint4* dst, int row, const float (&x)[VS], float sign = 1.f) {
#pragma unroll
  for (int p = 0; p < VS / 8; ++p) {
    float t[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) t[i] = sign * x[p * 8 + i];
    dst[p * 128 + row] = umma::pack8(t);
  }
}

// issue the loads of one accumulator row (VS columns) without waiting; read_wait() before use
template <int VS>
__device__ __forceinline__ void read_acc_nowait(const umma::Ctx& cx, uint32_t col, int warp, float (&x)[VS]) {
  if (!cx.dead) {
#pragma unroll
    for (int c = 0; c < VS; c += 32) umma::tmem_ld32_nowait(cx.tmem + ((uint32_t)(warp * 32) << 16) + col + c, x + c);
  } else {
#pragma unroll
    for (int i = 0; i < VS; ++i) x[i] = 0.f;
  }
}
__device__ __forceinline__ void read_wait(const umma::Ctx& cx) { if (!cx.dead) umma::tmem_wait_ld(); }
template <int VS>
__device__ __forceinline__ void read_acc(const umma::Ctx& cx, uint32_t col, int warp, float (&x)[VS]) {
  read_acc_nowait<VS>(cx, col, warp, x);
  read_wait(cx);
}

// Document flags of the chunks a chain walks, kept in shared memory 128 chunks at a time (plus one of
// look-ahead) so that no step of the chain waits for the segment ids: thread i fills entry i.
// dir = +1: entry i is chunk top + i; dir = -1: chunk top - i.  Bit 0: the chunk starts a document; bit 1:
// the chunk is one document.  Ends with a __syncthreads().
__device__ __forceinline__ void fill_flags(uint8_t* fl, const int32_t* seg, const Geo& g, int b, int top, int dir,
                                           int lo, int hi) {
  for (int i = threadIdx.x; i < 129; i += blockDim.x) {
    const int c = top + dir * i;
    uint8_t f = 0;
    if (c >= lo && c < hi) {
      bool n, s;
      chunk_flags(seg, g, b, c, n, s);
      f = (n ? 1 : 0) | (s ? 2 : 0);
    }
    fl[i] = f;
  }
  __syncthreads();
}

__host__ __device__ constexpr uint32_t tmem_cols(int vs) { return 3 * vs <= 128 ? 128u : (3 * vs <= 256 ? 256u : 512u); }

template <int VS, bool WITH_OUT>
__global__ void __launch_bounds__(128, 1) state_fwd_tc_kernel(StateArgs a) {
  extern __shared__ __align__(128) uint8_t sm[];
  __shared__ uint64_t bar, tb[2];                       // MMA completion; tile arrival: W | qe, M, ke
  __shared__ uint32_t tmem_base;
  __shared__ uint8_t fl_s[132];
  const Geo& g = a.g;
  constexpr int C = 128, K = 128;
  const int Vw = g.Vw, h = blockIdx.y, b = blockIdx.z;
  // slices past the value width carry the transition columns (see StateArgs::P_out)
  const bool trans = (int)blockIdx.x * VS >= Vw;
  const int v0 = trans ? 0 : blockIdx.x * VS, p0 = trans ? blockIdx.x * VS - Vw : 0;
  const int row = threadIdx.x, warp = row >> 5;
  uint4* sW = reinterpret_cast<uint4*>(sm);
  uint4* sQE = sW + TILE_U4;
  uint4* sM = sQE + TILE_U4;
  uint4* sKE = sM + TILE_U4;
  uint4* sS = sKE + TILE_U4;
  uint4* sVn = sS + (VS / 8) * 128;
  if (row == 0) { umma::mbar_init(&bar, 1); umma::mbar_init(&tb[0], 1); umma::mbar_init(&tb[1], 1); umma::fence_mbar_init(); }
  if (warp == 0) umma::tmem_alloc(&tmem_base, tmem_cols(VS));
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &bar, 0u, a.err, false};
  constexpr uint32_t colP = 0, colO = VS, colS = 2 * VS;
  const bool img = g.img;
  uint32_t tph[2] = {0u, 0u};
  auto tile_wait = [&](int i) {                         // bounded, like every wait here
    if (!umma::mbar_wait(&tb[i], tph[i])) umma::report_timeout(a.err);
    tph[i] ^= 1u;
  };

  const __nv_bfloat16* Wg = reinterpret_cast<const __nv_bfloat16*>(a.res.W);
  const __nv_bfloat16* QEg = reinterpret_cast<const __nv_bfloat16*>(a.res.qe);
  const __nv_bfloat16* KEg = reinterpret_cast<const __nv_bfloat16*>(a.res.ke);
  const __nv_bfloat16* Mg = reinterpret_cast<const __nv_bfloat16*>(a.res.M);
  const __nv_bfloat16* Ug = trans ? nullptr : reinterpret_cast<const __nv_bfloat16*>(a.res.U);
  float* const states = trans ? nullptr : a.states;
  const size_t item0 = ((size_t)b * g.H + h) * g.NC;

  const int cb = a.c_begin, ce = a.c_end;               // chunk range of this launch
  float* carry = a.carry ? a.carry + (((size_t)b * g.H + h) * K + row) * Vw + v0 : nullptr;
  auto fetch_W = [&](size_t it_) {
    if (img) {
      if (row == 0) { umma::mbar_expect_tx(&tb[0], TILE_U4 * 16); bulk_tile(sW, Wg + it_ * C * K, &tb[0]); }
    } else {
      copy_tile_async(sW, Wg + it_ * C * K, row, false);
    }
    umma::cp_async_commit();
  };
  // (a pass without outputs needs neither qe nor M: half the bytes a chunk step pulls through L2, which
  // is what bounds the step)
  const bool need_out_tiles = WITH_OUT && !trans;
  // With skip_provisional the outputs of the chunks that still depend on the state this launch started from
  // are left to the pass that follows with the true state (it rewrites exactly those chunks): `indep` turns
  // true after the first chunk that holds a document boundary or precedes one.  Uniform over the CTA.
  bool indep = !a.skip_provisional;
  auto fetch_QMK = [&](size_t it_, bool with_out) {
    if (img) {
      if (row == 0) {
        umma::mbar_expect_tx(&tb[1], (with_out ? 3 : 1) * TILE_U4 * 16);
        if (with_out) {
          bulk_tile(sQE, QEg + it_ * C * K, &tb[1]);
          bulk_tile(sM, Mg + it_ * C * C, &tb[1]);
        }
        bulk_tile(sKE, KEg + it_ * C * K, &tb[1]);
      }
    } else {
      if (with_out) {
        copy_tile_async(sQE, QEg + it_ * C * K, row, false);
        copy_tile_async(sM, Mg + it_ * C * C, row, false);
      }
      copy_tile_async(sKE, KEg + it_ * C * K, row, false);
    }
    umma::cp_async_commit();
  };
  fetch_W(item0 + cb);
  fetch_QMK(item0 + cb, need_out_tiles && indep);

  float S[VS];
#pragma unroll
  for (int j = 0; j < VS; ++j) S[j] = cb > 0 ? carry[j] : 0.f;

  // This thread's row of U (VS columns) and of Lambda_end for one chunk, fetched one chunk ahead of use
  // (right after the previous chunk's copy has been consumed), so the chain never waits for them.
  uint4 ureg[VS / 8];
  float lam_cur;
  auto fetch_row = [&](size_t it_) {
    if (Ug) {
      if (g.img) {
        const uint4* up = reinterpret_cast<const uint4*>(Ug + it_ * C * Vw) + (size_t)(v0 / 8) * 128 + row;
#pragma unroll
        for (int p = 0; p < VS / 8; ++p) ureg[p] = __ldg(up + p * 128);
      } else {
        const uint4* up = reinterpret_cast<const uint4*>(Ug + it_ * C * Vw + (size_t)row * Vw + v0);
#pragma unroll
        for (int p = 0; p < VS / 8; ++p) ureg[p] = __ldg(up + p);
      }
    } else {                                            // transition columns / U == NULL: U = 0
#pragma unroll
      for (int p = 0; p < VS / 8; ++p) ureg[p] = make_uint4(0, 0, 0, 0);
    }
    lam_cur = __ldg(a.res.lam_end + it_ * K + row);
  };
  fetch_row(item0 + cb);

  for (int c = cb; c < ce; ++c) {
    const size_t item = item0 + c;
    const int fo = (c - cb) & 127;
    if (fo == 0) fill_flags(fl_s, a.seg, g, b, c, 1, cb, ce);
    const bool is_new = fl_s[fo] & 1, all_same = fl_s[fo] & 2;
    const bool nis_new = fl_s[fo + 1] & 1;              // (zero past the end of the range)
    if (c == 0 && !is_new && trans) {
#pragma unroll
      for (int j = 0; j < VS; ++j) S[j] = row == p0 + j ? 1.f : 0.f;
    } else if (c == 0 && !is_new && a.init_state) {
#pragma unroll
      for (int j = 0; j < VS; ++j) S[j] = a.init_state[native_state_index_tc(g, b, h, row, v0 + j)];
    } else if (is_new) {
#pragma unroll
      for (int j = 0; j < VS; ++j) S[j] = 0.f;
    }
    if (states && !g.img) {
      float4* dst = reinterpret_cast<float4*>(states + item * K * Vw + (size_t)row * Vw + v0);
#pragma unroll
      for (int j = 0; j < VS / 4; ++j) dst[j] = make_float4(S[4 * j], S[4 * j + 1], S[4 * j + 2], S[4 * j + 3]);
    }
    stage_rows<VS>(sS, row, S);
    if (states && g.img) {                              // the same bf16 rows, as an operand image for the backward
      uint4* simg = reinterpret_cast<uint4*>(const_cast<__nv_bfloat16*>(states_img(g, states)) + item * K * Vw) + (size_t)(v0 / 8) * 128 + row;
#pragma unroll
      for (int p = 0; p < VS / 8; ++p) simg[p * 128] = sS[p * 128 + row];
    }
    const float dec = all_same ? expf(fminf(lam_cur, 0.f)) : 0.f;
    // the last chunk this CTA walks: the end of the range, or (until_independent) the point after which
    // nothing depends on the state the chain started from.  Uniform over the CTA (the flags depend on the
    // chunk only).  Nothing is prefetched past it, so no copy is in flight when the CTA leaves.
    const bool last = c + 1 >= ce || (a.until_independent && (!all_same || nis_new));

    if (img) tile_wait(0); else umma::cp_async_wait<1>();      // this chunk's W has landed
    umma::pre_issue_sync();
    umma::issue<VS, false, true>(cx, sW, sS, K, colP, false);          // P = W S
    umma::commit_wait(cx);
    if (!last) fetch_W(item + 1); else umma::cp_async_commit();

    float vn[VS];
    read_acc<VS>(cx, colP, warp, vn);
#pragma unroll
    for (int p = 0; p < VS / 8; ++p) {
      float u[8];
      umma::unpack8(ureg[p], u);
#pragma unroll
      for (int i = 0; i < 8; ++i) vn[p * 8 + i] = u[i] - vn[p * 8 + i];      // V_new = U - W S
    }
    if (!last) fetch_row(item + 1);
    stage_rows<VS>(sVn, row, vn);

    if (img) tile_wait(1); else umma::cp_async_wait<1>();      // this chunk's qe, M, ke have landed
    umma::pre_issue_sync();
    const bool outc = need_out_tiles && indep;                         // this chunk's outputs are wanted
    indep = indep || !all_same || nis_new;                             // ... and the next chunk's
    if (outc) {
      umma::issue<VS, false, true>(cx, sQE, sS, K, colO, false);       // O  = qe S
      umma::issue<VS, false, true>(cx, sM, sVn, C, colO, true);        //    + M V_new
    }
    umma::issue<VS, true, true>(cx, sKE, sVn, C, colS, false);         // ke^T V_new
    umma::commit_wait(cx);
    if (!last) fetch_QMK(item + 1, need_out_tiles && indep); else umma::cp_async_commit();

    float sn[VS];
    if (outc) {
      float o[VS];
      read_acc_nowait<VS>(cx, colO, warp, o);
      read_acc_nowait<VS>(cx, colS, warp, sn);
      read_wait(cx);
      const int t = c * C + row;
      if (t < g.L) {
        const size_t off = ((size_t)b * g.L + t) * g.Hv * g.V + (size_t)h * Vw + v0;
        if (g.qkv_dt == DN_BF16) {
          uint4* dst = reinterpret_cast<uint4*>(reinterpret_cast<__nv_bfloat16*>(a.out) + off);
#pragma unroll
          for (int p = 0; p < VS / 8; ++p) {
            float t8[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) t8[i] = o[p * 8 + i];
            dst[p] = umma::pack8(t8);
          }
        } else {
          float4* dst = reinterpret_cast<float4*>(reinterpret_cast<float*>(a.out) + off);
#pragma unroll
          for (int j = 0; j < VS / 4; ++j) dst[j] = make_float4(o[4 * j], o[4 * j + 1], o[4 * j + 2], o[4 * j + 3]);
        }
      }
    }
    if (!outc) read_acc<VS>(cx, colS, warp, sn);
#pragma unroll
    for (int j = 0; j < VS; ++j) S[j] = fmaf(dec, S[j], sn[j]);       // S <- decay * S + ke^T V_new
    umma::tc_fence_before();
    if (last) break;
  }
  if (a.until_independent) {
    // nothing to hand on: the caller has the final state from the shard's affine summary
  } else if (trans) {
    float* dst = a.P_out + (((size_t)b * g.H + h) * K + row) * K + p0;
#pragma unroll
    for (int j = 0; j < VS; ++j) dst[j] = S[j];
  } else if (ce < g.NC) {
#pragma unroll
    for (int j = 0; j < VS; ++j) carry[j] = S[j];
  } else if (a.final_state) {
#pragma unroll
    for (int j = 0; j < VS; ++j) a.final_state[native_state_index_tc(g, b, h, row, v0 + j)] = S[j];
  }
  umma::cp_async_wait<0>();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, tmem_cols(VS));
}

template <int VS>
__global__ void __launch_bounds__(128, 1) state_bwd_tc_kernel(StateArgs a) {
  extern __shared__ __align__(128) uint8_t sm[];
  __shared__ uint64_t bar, tb[2];                       // MMA completion; tile arrival: M, ke | qe, W
  __shared__ uint32_t tmem_base;
  __shared__ uint8_t fl_s[132];
  const Geo& g = a.g;
  constexpr int C = 128, K = 128;
  const int Vw = g.Vw, v0 = blockIdx.x * VS, h = blockIdx.y, b = blockIdx.z;
  const int row = threadIdx.x, warp = row >> 5;
  uint4* sM = reinterpret_cast<uint4*>(sm);
  uint4* sKE = sM + TILE_U4;
  uint4* sQE = sKE + TILE_U4;
  uint4* sW = sQE + TILE_U4;
  uint4* sdO = sW + TILE_U4;
  uint4* sdH = sdO + (VS / 8) * 128;
  uint4* sdV = sdH + (VS / 8) * 128;
  uint4* sSl = sdV + (VS / 8) * 128 + row;              // this thread's row of S (image path, bf16): piece j at sSl[j * 128]
  const bool img = g.img;
  if (row == 0) { umma::mbar_init(&bar, 1); umma::mbar_init(&tb[0], 1); umma::mbar_init(&tb[1], 1); umma::fence_mbar_init(); }
  uint32_t tph[2] = {0u, 0u};
  auto tile_wait = [&](int i) {                         // bounded, like every wait here
    if (!umma::mbar_wait(&tb[i], tph[i])) umma::report_timeout(a.err);
    tph[i] ^= 1u;
  };
  if (warp == 0) umma::tmem_alloc(&tmem_base, tmem_cols(VS));
  umma::tc_fence_before();
  __syncthreads();
  umma::tc_fence_after();
  umma::Ctx cx{tmem_base, &bar, 0u, a.err, false};
  constexpr uint32_t colV = 0, colH = VS;

  const __nv_bfloat16* Wg = reinterpret_cast<const __nv_bfloat16*>(a.res.W);
  const __nv_bfloat16* QEg = reinterpret_cast<const __nv_bfloat16*>(a.res.qe);
  const __nv_bfloat16* KEg = reinterpret_cast<const __nv_bfloat16*>(a.res.ke);
  const __nv_bfloat16* Mg = reinterpret_cast<const __nv_bfloat16*>(a.res.M);
  const size_t item0 = ((size_t)b * g.H + h) * g.NC;
  const int cb = a.c_begin, ce = a.c_end;               // chunk range of this launch, walked from ce - 1 down
  float* carry = a.carry ? a.carry + (((size_t)b * g.H + h) * K + row) * Vw + v0 : nullptr;
  const size_t last = item0 + ce - 1;

  // image path: the thread's own row of the chunk-entry state (its bf16 image, the only copy kept)
  // travels with M and ke, one chunk ahead, into a private strip of shared memory; it is needed for
  // dLambda_end = sum_v dH * S
  auto copy_S_row = [&](size_t it_) {
    const uint4* src = reinterpret_cast<const uint4*>(states_img(g, a.res.states) + it_ * K * Vw) + (size_t)(v0 / 8) * 128 + row;
#pragma unroll
    for (int j = 0; j < VS / 8; ++j) umma::cp_async16(sSl + j * 128, src + j * 128);
  };
  // image path: whole tiles by bulk copies on tb[], the S row by this thread's own cp.async group;
  // otherwise everything by cp.async groups (two per chunk)
  auto fetch_MK = [&](size_t it_) {
    if (img) {
      if (row == 0) {
        umma::mbar_expect_tx(&tb[0], 2 * TILE_U4 * 16);
        bulk_tile(sM, Mg + it_ * C * C, &tb[0]);
        bulk_tile(sKE, KEg + it_ * C * K, &tb[0]);
      }
      copy_S_row(it_);
    } else {
      copy_tile_async(sM, Mg + it_ * C * C, row, false);
      copy_tile_async(sKE, KEg + it_ * C * K, row, false);
    }
    umma::cp_async_commit();
  };
  auto fetch_QW = [&](size_t it_) {
    if (img) {
      if (row == 0) {
        umma::mbar_expect_tx(&tb[1], 2 * TILE_U4 * 16);
        bulk_tile(sQE, QEg + it_ * C * K, &tb[1]);
        bulk_tile(sW, Wg + it_ * C * K, &tb[1]);
      }
    } else {
      copy_tile_async(sQE, QEg + it_ * C * K, row, false);
      copy_tile_async(sW, Wg + it_ * C * K, row, false);
    }
    umma::cp_async_commit();
  };
  fetch_MK(last);
  fetch_QW(last);

  float dH[VS];
#pragma unroll
  for (int j = 0; j < VS; ++j)
    dH[j] = ce < g.NC ? carry[j] : (a.d_final ? a.d_final[native_state_index_tc(g, b, h, row, v0 + j)] : 0.f);

  // This thread's row of dO of one chunk as raw 16-byte vectors (token c*C+row; zero past the end).
  // They are fetched one chunk ahead so that the chain never waits for them.
  constexpr int NV = VS / 8;                            // bf16 vectors per row slice; fp32 needs 2 * NV
  uint4 raw[2 * NV];
  const bool dobf = g.qkv_dt == DN_BF16;
  auto fetch_dO = [&](int c) {
    const int t = c * C + row;
    const bool live = c >= cb && t < g.L;
    const size_t off = ((size_t)b * g.L + (live ? t : 0)) * g.Hv * g.V + (size_t)h * Vw + v0;
    if (dobf) {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(a.d_out) + off);
#pragma unroll
      for (int p = 0; p < NV; ++p) raw[p] = live ? __ldg(src + p) : make_uint4(0, 0, 0, 0);
    } else {
      const uint4* src = reinterpret_cast<const uint4*>(reinterpret_cast<const float*>(a.d_out) + off);
#pragma unroll
      for (int p = 0; p < 2 * NV; ++p) raw[p] = live ? __ldg(src + p) : make_uint4(0, 0, 0, 0);
    }
  };
  fetch_dO(ce - 1);

  for (int c = ce - 1; c >= cb; --c) {
    const size_t item = item0 + c;
    const int fo = (ce - 1 - c) & 127;
    if (fo == 0) fill_flags(fl_s, a.seg, g, b, c, -1, cb, ce);
    const bool is_new = fl_s[fo] & 1, all_same = fl_s[fo] & 2;
    // dO of this chunk, rounded to bf16 as the reference does (gdn2.py:731)
    float dO[VS];
    if (dobf) {
#pragma unroll
      for (int p = 0; p < NV; ++p) {
        float t8[8];
        umma::unpack8(raw[p], t8);
#pragma unroll
        for (int i = 0; i < 8; ++i) dO[p * 8 + i] = t8[i];
      }
    } else {
#pragma unroll
      for (int p = 0; p < 2 * NV; ++p) {
        dO[4 * p] = __uint_as_float(raw[p].x); dO[4 * p + 1] = __uint_as_float(raw[p].y);
        dO[4 * p + 2] = __uint_as_float(raw[p].z); dO[4 * p + 3] = __uint_as_float(raw[p].w);
      }
    }
    // the last chunk this CTA walks: the start of the range, or (until_independent) the point below which
    // nothing depends on the cotangent the chain started from.  Uniform over the CTA; nothing is
    // prefetched past it.
    const bool last = c <= cb || (a.until_independent && (is_new || !all_same));
    fetch_dO(last ? cb - 1 : c - 1);                    // in flight during this chunk's products (zeros past the end)
    stage_rows<VS>(sdO, row, dO);
    stage_rows<VS>(sdH, row, dH);
    if (img) {                                           // dH as a bf16 operand image
      uint4* dst = reinterpret_cast<uint4*>(a.dH) + item * (K * Vw / 8) + (size_t)(v0 / 8) * 128 + row;
#pragma unroll
      for (int p = 0; p < VS / 8; ++p) dst[p * 128] = sdH[p * 128 + row];
    } else {
      float4* dst = reinterpret_cast<float4*>(a.dH + item * K * Vw + (size_t)row * Vw + v0);
#pragma unroll
      for (int j = 0; j < VS / 4; ++j) dst[j] = make_float4(dH[4 * j], dH[4 * j + 1], dH[4 * j + 2], dH[4 * j + 3]);
    }
    const float dec = all_same ? expf(fminf(__ldg(a.res.lam_end + item * K + row), 0.f)) : 0.f;

    umma::cp_async_wait<1>();                           // M, ke of this chunk (cp.async path); the S row (image path)
    if (img) tile_wait(0);
    if (img) {                                          // partial sum of dLambda_end over this CTA's columns
      float part = 0.f;
#pragma unroll
      for (int j = 0; j < VS / 8; ++j) {
        float sv[8];
        umma::unpack8(sSl[j * 128], sv);
#pragma unroll
        for (int i = 0; i < 8; ++i) part = fmaf(dH[8 * j + i], sv[i], part);
      }
      dlend_part(g, a.dH)[(item * gridDim.x + blockIdx.x) * K + row] = part;
    }
    umma::pre_issue_sync();
    umma::issue<VS, true, true>(cx, sM, sdO, C, colV, false);          // dV  = M^T dO
    umma::issue<VS, false, true>(cx, sKE, sdH, K, colV, true);         //     + ke dH
    umma::commit_wait(cx);
    if (!last) fetch_MK(item - 1); else umma::cp_async_commit();

    float dv[VS];
    read_acc<VS>(cx, colV, warp, dv);
    if (img) {                                           // dV as a bf16 operand image
      uint4* dst = reinterpret_cast<uint4*>(a.dV) + item * (C * Vw / 8) + (size_t)(v0 / 8) * 128 + row;
#pragma unroll
      for (int p = 0; p < VS / 8; ++p) {
        float t8[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) t8[i] = dv[p * 8 + i];
        dst[p * 128] = umma::pack8(t8);
      }
    } else {
      float4* dst = reinterpret_cast<float4*>(a.dV + item * C * Vw + (size_t)row * Vw + v0);
#pragma unroll
      for (int j = 0; j < VS / 4; ++j) dst[j] = make_float4(dv[4 * j], dv[4 * j + 1], dv[4 * j + 2], dv[4 * j + 3]);
    }
    stage_rows<VS>(sdV, row, dv, -1.f);                 // staged negated: the product below is -W^T dV

    if (img) tile_wait(1); else umma::cp_async_wait<1>();      // qe, W of this chunk
    umma::pre_issue_sync();
    umma::issue<VS, true, true>(cx, sQE, sdO, C, colH, false);         // qe^T dO
    umma::issue<VS, true, true>(cx, sW, sdV, C, colH, true);           // - W^T dV
    umma::commit_wait(cx);
    if (!last) fetch_QW(item - 1); else umma::cp_async_commit();

    float dn_[VS];
    read_acc<VS>(cx, colH, warp, dn_);
#pragma unroll
    for (int j = 0; j < VS; ++j) dH[j] = is_new ? 0.f : fmaf(dec, dH[j], dn_[j]);
    umma::tc_fence_before();
    if (last) break;
  }
  if (a.until_independent) {
    // nothing to hand on: the caller has d_init from the shard's affine summary
  } else if (cb > 0) {
#pragma unroll
    for (int j = 0; j < VS; ++j) carry[j] = dH[j];
  } else if (a.d_init) {
#pragma unroll
    for (int j = 0; j < VS; ++j) a.d_init[native_state_index_tc(g, b, h, row, v0 + j)] = dH[j];
  }
  umma::cp_async_wait<0>();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem_base, tmem_cols(VS));
}

int pick_vs(const Geo& g) {
  const int chains = g.B * g.H;
  if (g.Vw % 64 == 0 && chains * (g.Vw / 64) >= sm_count()) return 64;
  return 32;
}

template <int VS>
size_t tc_smem(bool bwd) {
  return (size_t)4 * TILE_U4 * 16 + (size_t)(bwd ? 3 : 2) * (VS / 8) * 128 * 16 + (bwd ? (size_t)128 * VS * 2 : 0);
}

template <int VS>
int launch_fwd_vs(const StateArgs& a, cudaStream_t st) {
  dim3 grid((a.g.Vw + (a.P_out ? a.g.K : 0)) / VS, a.g.H, a.g.B);
  const size_t smem = tc_smem<VS>(false);
  if (a.out) {
    cudaFuncSetAttribute(state_fwd_tc_kernel<VS, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    state_fwd_tc_kernel<VS, true><<<grid, 128, smem, st>>>(a);
  } else {
    cudaFuncSetAttribute(state_fwd_tc_kernel<VS, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    state_fwd_tc_kernel<VS, false><<<grid, 128, smem, st>>>(a);
  }
  return launch_status();
}

template <int VS>
int launch_bwd_vs(const StateArgs& a, cudaStream_t st) {
  dim3 grid(a.g.Vw / VS, a.g.H, a.g.B);
  const size_t smem = tc_smem<VS>(true);
  cudaFuncSetAttribute(state_bwd_tc_kernel<VS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  state_bwd_tc_kernel<VS><<<grid, 128, smem, st>>>(a);
  return launch_status();
}

}  // namespace

bool state_tc_eligible(const Geo& g) {
  return g.prec == DN_PREC_BF16 && !(g.flags & DN_STATE_FP32_MM) && g.C == 128 && g.K == 128 && g.Vw % 32 == 0;
}

static StateArgs with_range(const StateArgs& in) {
  StateArgs a = in;
  if (a.c_end <= 0) { a.c_begin = 0; a.c_end = a.g.NC; }
  a.err = device_error_ptr();
  return a;
}

int launch_state_fwd_tc(const StateArgs& in, cudaStream_t st) {
  const StateArgs a = with_range(in);
  // with the transition columns aboard, 64-column slices keep one (batch, head)'s Vw + K columns in few
  // enough CTAs to run in one wave; the chain's time is its per-chunk latency, not the slice width
  const int vs = (a.P_out && a.g.Vw % 64 == 0) ? 64 : pick_vs(a.g);
  switch (vs) {
    case 64: return launch_fwd_vs<64>(a, st);
    default: return launch_fwd_vs<32>(a, st);
  }
}

int launch_state_bwd_tc(const StateArgs& in, cudaStream_t st) {
  const StateArgs a = with_range(in);
  // image path: slices of 32 columns (the dLambda_end partial sums are laid out per slice of 32, and the
  // S strip of a 64-column slice would not fit in shared memory)
  switch (a.g.img ? 32 : pick_vs(a.g)) {
    case 64: return launch_bwd_vs<64>(a, st);
    default: return launch_bwd_vs<32>(a, st);
  }
}

}  // namespace dn
