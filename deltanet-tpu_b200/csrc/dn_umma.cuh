// tcgen05 (5th-gen tensor core) building blocks for sm_100a, in inline PTX:
// TMEM allocation, shared-memory matrix descriptors, single-thread MMA issue, commit to an
// mbarrier with a BOUNDED wait, TMEM loads, and on top of them `umma_gemm`, a CTA-wide
// bf16 x bf16 -> fp32 GEMM whose operands are gathered by the CTA's threads into shared memory
// and whose 128 x N result is handed to an epilogue functor straight from tensor memory.
//
// Shared-memory operand layout (no swizzle, the "interleaved" canonical layout): an operand
// tile is a sequence of PANELS; a panel is `inner` rows of 16 bytes (8 bf16 elements):
//   K-major operand  (rows x Kc, contraction index contiguous in the source):
//       panel p = k/8, inner index = row         -> byte offset (p*rows + row)*16
//       descriptor: LBO (between the two k-groups of one MMA) = rows*16, SBO (8-row groups) = 128
//   MN-major operand (rows x Kc, row index contiguous in the source, i.e. a transposed view):
//       panel p = row/8, inner index = k         -> byte offset (p*Kc + k)*16
//       descriptor: LBO (k groups of 8) = 128, SBO (between row groups) = Kc*16
// One tcgen05.mma consumes 16 values of the contraction index: two K-major panels, or 256
// bytes of every MN-major panel.
#pragma once
#include <cuda_bf16.h>
#include <stdint.h>

namespace dn {
namespace umma {

constexpr uint32_t SPIN_LIMIT = 1u << 22;   // bounded wait: ~tens of ms, then the kernel bails out

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// A bounded wait gave up: raise the library's error word (a plain store; the word may live in host
// memory that the device reaches over the bus).
__device__ __forceinline__ void report_timeout(int* err) {
  if (err) { *reinterpret_cast<volatile int*>(err) = 1; __threadfence_system(); }
}

// ---- mbarrier ----------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// Returns false if the phase did not complete within SPIN_LIMIT polls.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity) {
  const uint32_t a = smem_u32(bar);
  for (uint32_t it = 0; it < SPIN_LIMIT; ++it) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(a), "r"(parity) : "memory");
    if (ok) return true;
  }
  return false;
}

// ---- bulk asynchronous copies (contiguous ranges; addresses and sizes multiples of 16 bytes) -------
// global -> shared, completion counted in bytes on an mbarrier that was told what to expect
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_load(void* dst, const void* src, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(dst)), "l"(src), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
// shared -> global, tracked per issuing thread in bulk groups
__device__ __forceinline__ void bulk_store(void* dst, const void* src, uint32_t bytes) {
  asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(src)), "r"(bytes) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// wait until at most N of this thread's bulk groups still READ shared memory
template <int N>
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory"); }

// Asks the memory system to bring a contiguous global range into L2 (no destination, nothing to wait
// for).  Skipped unless address and size are multiples of 16 bytes.
__device__ __forceinline__ void prefetch_l2(const void* p, uint32_t bytes) {
  if (((reinterpret_cast<uintptr_t>(p) | bytes) & 15u) == 0 && bytes)
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}

// ---- fences ------------------------------------------------------------------------------
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// ---- tensor memory -----------------------------------------------------------------------
// Executed by one full warp.  ncols: power of two in [32, 512].  The base address lands in *dst (smem).
__device__ __forceinline__ void tmem_alloc(uint32_t* dst, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst)), "r"(ncols) : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// 32 lanes x 16 consecutive 32-bit columns: thread i of the warp gets lane (base lane + i).
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// 32 lanes x 32 consecutive 32-bit columns, issued without waiting: follow one or several of these with
// tmem_wait_ld() before the values are used.
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, float* v) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,"
      "%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
        "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
        "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
        "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr));
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// Tensor memory as per-thread scratch: 8 consecutive 32-bit columns of the calling thread's own lane
// (lane = base lane + thread index in the warp).  Warp-collective; a warp may only touch the lane
// quarter 32 * (warp % 4).  A store must be followed by tmem_wait_st() before the data is read back.
__device__ __forceinline__ void tmem_st8(uint32_t taddr, const float (&v)[8]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
      ::"r"(taddr), "r"(__float_as_uint(v[0])), "r"(__float_as_uint(v[1])), "r"(__float_as_uint(v[2])),
        "r"(__float_as_uint(v[3])), "r"(__float_as_uint(v[4])), "r"(__float_as_uint(v[5])),
        "r"(__float_as_uint(v[6])), "r"(__float_as_uint(v[7])) : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld8(uint32_t taddr, float (&v)[8]) {
  uint32_t r[8];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
      : "r"(taddr));
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 8; ++i) v[i] = __uint_as_float(r[i]);
}

// ---- descriptors -------------------------------------------------------------------------
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr >> 4) & 0x3FFF);
  d |= (uint64_t)((lbo_bytes >> 4) & 0x3FFF) << 16;
  d |= (uint64_t)((sbo_bytes >> 4) & 0x3FFF) << 32;
  d |= (uint64_t)1 << 46;                 // descriptor version for this architecture
  return d;                               // base offset 0, layout type 0 (no swizzle)
}
// bf16 x bf16 -> fp32, M = 128, N columns; majors: 0 = K-major, 1 = MN-major.
__host__ __device__ constexpr uint32_t instr_desc(int N, int a_mn, int b_mn) {
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)a_mn << 15) | ((uint32_t)b_mn << 16) |
         ((uint32_t)(N >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
}
__device__ __forceinline__ void mma_bf16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
  asm volatile(
      "{\n\t.reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
      ::"r"(d_tmem), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void mma_commit(uint64_t* bar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// ---- asynchronous 16-byte global -> shared copies (generic proxy; follow with fence_async_smem) -------
__device__ __forceinline__ void cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(smem_u32(dst)), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int PENDING>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(PENDING) : "memory"); }

// ---- per-CTA scratch that should stay in L2 -----------------------------------------------------
// Loads and stores of the fp32 scratch a CTA writes and reads back within one work item: through L2 only
// (no L1), with an evict-last L2 policy, so that the streaming inputs and outputs of the kernel, which
// are touched once, do not push the scratch out to HBM between its write and its read.
__device__ __forceinline__ uint64_t keep_policy() {
  uint64_t p;
  asm("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
  return p;
}
__device__ __forceinline__ void st_keep4(float4* p, float4 v) {
  asm volatile("st.global.cg.L2::cache_hint.v4.f32 [%0], {%1,%2,%3,%4}, %5;"
               ::"l"(p), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w), "l"(keep_policy()) : "memory");
}
__device__ __forceinline__ void st_keep1(float* p, float v) {
  asm volatile("st.global.cg.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(p), "f"(v), "l"(keep_policy()) : "memory");
}
__device__ __forceinline__ float4 ld_keep4(const float4* p) {
  float4 v;
  asm volatile("ld.global.cg.L2::cache_hint.v4.f32 {%0,%1,%2,%3}, [%4], %5;"
               : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "l"(p), "l"(keep_policy()) : "memory");
  return v;
}
__device__ __forceinline__ float ld_keep1(const float* p) {
  float v;
  asm volatile("ld.global.cg.L2::cache_hint.f32 %0, [%1], %2;" : "=f"(v) : "l"(p), "l"(keep_policy()) : "memory");
  return v;
}
// the same 16-byte load skipped (zeros returned) when `pred` is false: no branch
__device__ __forceinline__ float4 ld_keep4_pred(const float4* p, bool pred) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q ld.global.cg.L2::cache_hint.v4.f32 {%0, %1, %2, %3}, [%4], %6;\n\t}"
      : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w) : "l"(p), "r"((int)pred), "l"(keep_policy()) : "memory");
  return v;
}

// ---- predicated loads ------------------------------------------------------------------------
// 16-byte global load through L2 only, skipped (zeros returned) when `pred` is false: no branch, so
// the loads of an unrolled group stay back to back
__device__ __forceinline__ float4 ldcg_pred(const float4* p, bool pred) {
  float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
  asm volatile(
      "{\n\t.reg .pred q;\n\t"
      "setp.ne.b32 q, %5, 0;\n\t"
      "@q ld.global.cg.v4.f32 {%0, %1, %2, %3}, [%4];\n\t}"
      : "+f"(v.x), "+f"(v.y), "+f"(v.z), "+f"(v.w) : "l"(p), "r"((int)pred) : "memory");
  return v;
}

// ---- packing helpers ---------------------------------------------------------------------
__device__ __forceinline__ uint32_t pack2(float a, float b) {
  __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
  return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ uint4 pack8(const float (&x)[8]) {
  return make_uint4(pack2(x[0], x[1]), pack2(x[2], x[3]), pack2(x[4], x[5]), pack2(x[6], x[7]));
}
__device__ __forceinline__ uint4 pack8p(const float* x) {
  return make_uint4(pack2(x[0], x[1]), pack2(x[2], x[3]), pack2(x[4], x[5]), pack2(x[6], x[7]));
}
// 2^x for x <= 0 on the special-function unit, results below the normal range flushed to 0
__device__ __forceinline__ float ex2_fast(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
// e^x for x <= 0 through the same unit (relative error ~1e-6 at |x| ~ 10: bf16-precision paths only)
__device__ __forceinline__ float exp_neg(float x) { return ex2_fast(x * 1.4426950408889634f); }
__device__ __forceinline__ uint4 ld8_f32(const float* p) {       // 8 consecutive floats -> 8 bf16
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  return make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
}
__device__ __forceinline__ uint4 ld8_bf16(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
// The same two loads through the read-only path: only for data written by EARLIER launches.  The
// compiler may move these above shared-memory stores, which is what lets a staging loop keep
// several loads in flight.
__device__ __forceinline__ uint4 ld8_f32_ro(const float* p) {
  const float4 a = __ldg(reinterpret_cast<const float4*>(p)), b = __ldg(reinterpret_cast<const float4*>(p + 4));
  return make_uint4(pack2(a.x, a.y), pack2(a.z, a.w), pack2(b.x, b.y), pack2(b.z, b.w));
}
__device__ __forceinline__ void unpack8(uint4 u, float (&x)[8]) {
  const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) { x[2 * i] = __uint_as_float(w[i] << 16); x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u); }
}

// Per-CTA tensor-core context: TMEM base, the completion barrier and its phase, an error flag.
struct Ctx {
  uint32_t tmem;        // base address of the allocation (lane 0, first column)
  uint64_t* bar;        // mbarrier the MMAs commit to
  uint32_t phase;       // parity of the next completion
  int* err;             // global error word: set to 1 if a bounded wait gave up
  bool dead;            // this CTA stopped issuing work after a timeout
};

// Fill one operand: panels x inner 16-byte rows, produced by ld(panel, inner) -> uint4 (8 bf16).
template <int THREADS, class LD>
__device__ __forceinline__ void stage_operand(uint4* dst, int panels, int inner, LD ld) {
  const int total = panels * inner;
  for (int e = threadIdx.x; e < total; e += THREADS) {
    const int p = e / inner, x = e - p * inner;
    dst[e] = ld(p, x);
  }
}

// Make operand writes of all threads visible to the tensor core and order TMEM accesses: call
// once by every thread after staging and before `issue`.
__device__ __forceinline__ void pre_issue_sync() {
  fence_async_smem();                  // operand writes (generic proxy) -> visible to the MMA (async proxy)
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
}

// Issue (one thread) the MMAs of D[128 x N] (+)= A[128 x Kc] B[N x Kc]^T on staged operands.
template <int N, bool A_MN, bool B_MN>
__device__ __forceinline__ void issue(const Ctx& cx, const void* sA, const void* sB, int Kc, uint32_t tmem_col,
                                      bool accumulate) {
  if (threadIdx.x != 0 || cx.dead) return;
  const uint32_t a0 = smem_u32(sA), b0 = smem_u32(sB);
  constexpr uint32_t idesc = instr_desc(N, A_MN ? 1 : 0, B_MN ? 1 : 0);
  const uint32_t a_lbo = A_MN ? 128u : 128u * 16u, a_sbo = A_MN ? (uint32_t)Kc * 16u : 128u;
  const uint32_t b_lbo = B_MN ? 128u : (uint32_t)N * 16u, b_sbo = B_MN ? (uint32_t)Kc * 16u : 128u;
  const uint32_t a_step = A_MN ? 256u : 2u * 128u * 16u, b_step = B_MN ? 256u : 2u * (uint32_t)N * 16u;
  for (int ks = 0; ks < Kc / 16; ++ks)
    mma_bf16(cx.tmem + tmem_col, smem_desc(a0 + ks * a_step, a_lbo, a_sbo), smem_desc(b0 + ks * b_step, b_lbo, b_sbo),
             idesc, (accumulate || ks > 0) ? 1u : 0u);
}

// Commit everything issued so far (one thread) and make every thread wait for it, boundedly.
__device__ __forceinline__ void commit_wait(Ctx& cx) {
  if (threadIdx.x == 0 && !cx.dead) mma_commit(cx.bar);
  if (!cx.dead && !mbar_wait(cx.bar, cx.phase)) {
    cx.dead = true;
    report_timeout(cx.err);
  }
  cx.phase ^= 1u;
  tc_fence_after();
}

template <int N, bool A_MN, bool B_MN>
__device__ __forceinline__ void issue_and_wait(Ctx& cx, const void* sA, const void* sB, int Kc, uint32_t tmem_col,
                                               bool accumulate) {
  pre_issue_sync();
  issue<N, A_MN, B_MN>(cx, sA, sB, Kc, tmem_col, accumulate);
  commit_wait(cx);
}

// Hand D[128 x N] (fp32, tensor memory) to epi(row, col0, v[16]) in 16-column pieces.
// THREADS must be 128 (each warp reads its own lane quarter, all columns) or 256 (the second
// warp group takes the upper half of the columns).
template <int THREADS, int N, class EPI>
__device__ __forceinline__ void drain(const Ctx& cx, uint32_t tmem_col, EPI epi) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int quarter = warp & 3, group = warp >> 2;
  constexpr int GROUPS = THREADS / 128;
  constexpr int PER = N / GROUPS;
  const int row = quarter * 32 + lane;
#pragma unroll 1
  for (int c = 0; c < PER; c += 16) {
    const int col = group * PER + c;
    float v[16];
    if (!cx.dead) tmem_ld16(cx.tmem + ((uint32_t)(quarter * 32) << 16) + tmem_col + col, v);
    else {
#pragma unroll
      for (int i = 0; i < 16; ++i) v[i] = 0.f;
    }
    epi(row, col, v);
  }
  tc_fence_before();
}

}  // namespace umma
}  // namespace dn
