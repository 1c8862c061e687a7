// XLA FFI handlers over the C ABI: what JAX calls when deltanet_b200.jax_op lowers its custom calls.
//
// OPTIONAL translation unit.  It needs the XLA FFI headers that ship inside jaxlib
// (jax.ffi.include_dir()); build_ffi.sh compiles it into libdeltanet_b200_ffi.so only where
// `python -c "import jax.ffi"` succeeds, and nothing else in the library depends on it.  The image
// this library is developed and tested on has no jaxlib, so this file has not been compiled there:
// the C ABI underneath is what the tests exercise (through ctypes).
//
// One handler per operator-level entry point, matching the reference's custom-VJP boundary
// (src/deltanet_tpu/gdn2.py:1461-1477 forward, 1496-1766 backward) and its decode step (2289-2490):
//   dn_ffi_chunk_fwd   operands q,k,v,g,b,w,seg,init   results out,final_state,residuals,scratch
//   dn_ffi_chunk_bwd   operands q,k,v,g,b,w,seg,init,residuals,d_out,d_final   results dq..dw,d_init,scratch
//   dn_ffi_decode_step operands q,k,v,g,b,w,state,reset   results out,new_state
// Static configuration arrives as attributes (the reference closes over the same values: they are its
// cache key, gdn2.py:1446-1460).  Workspace is requested from XLA as an extra result buffer, so the
// handlers allocate nothing; they only enqueue on the stream XLA hands them and return a status.
#include <cuda_runtime_api.h>

#include <cstdint>
#include <string>

#include "xla/ffi/api/ffi.h"

#include "../../include/deltanet_b200.h"

namespace ffi = xla::ffi;

namespace {

int dtype_code(ffi::DataType t) {
  if (t == ffi::DataType::F32) return DN_F32;
  if (t == ffi::DataType::BF16) return DN_BF16;
  return -1;
}

// gate layout (heads, cols) from a (B,L,H) or (B,L,H,C) buffer
void gate_layout(const ffi::AnyBuffer& x, int first_head_dim, int32_t* heads, int32_t* cols) {
  auto d = x.dimensions();
  *heads = static_cast<int32_t>(d[first_head_dim]);
  *cols = d.size() > static_cast<size_t>(first_head_dim + 1) ? static_cast<int32_t>(d[first_head_dim + 1]) : 1;
}

ffi::Error status(int rc, const char* what) {
  if (rc == DN_OK) return ffi::Error::Success();
  return ffi::Error(rc == DN_ERR_CUDA_LAUNCH || rc == DN_ERR_DEVICE_WAIT ? ffi::ErrorCode::kInternal : ffi::ErrorCode::kInvalidArgument,
                    std::string(what) + ": " + dn_status_string(rc));
}

ffi::Error make_shape(const ffi::AnyBuffer& q, const ffi::AnyBuffer& v, const ffi::AnyBuffer& g, const ffi::AnyBuffer& b,
                      const ffi::AnyBuffer& w, int64_t chunk, int64_t precision, int64_t flags, float scale, dn_shape* s) {
  auto qd = q.dimensions();
  auto vd = v.dimensions();
  if (qd.size() != 4 || vd.size() != 4) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "q, k, v must be rank 4");
  s->B = static_cast<int32_t>(qd[0]); s->L = static_cast<int32_t>(qd[1]);
  s->Hk = static_cast<int32_t>(qd[2]); s->K = static_cast<int32_t>(qd[3]);
  s->Hv = static_cast<int32_t>(vd[2]); s->V = static_cast<int32_t>(vd[3]);
  s->chunk = static_cast<int32_t>(chunk);
  gate_layout(g, 2, &s->g_heads, &s->g_cols);
  gate_layout(b, 2, &s->b_heads, &s->b_cols);
  gate_layout(w, 2, &s->w_heads, &s->w_cols);
  s->qkv_dtype = dtype_code(q.element_type());
  s->gate_dtype = dtype_code(g.element_type());
  if (s->qkv_dtype < 0 || s->gate_dtype < 0) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "unsupported dtype");
  s->precision = static_cast<int32_t>(precision);
  s->flags = static_cast<uint32_t>(flags);
  s->scale = scale;
  return ffi::Error::Success();
}

// ---- forward --------------------------------------------------------------------------------------
ffi::Error ChunkFwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer g,
                        ffi::AnyBuffer b, ffi::AnyBuffer w, ffi::AnyBuffer seg, ffi::AnyBuffer init,
                        ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> final_state,
                        ffi::Result<ffi::AnyBuffer> residuals, ffi::Result<ffi::AnyBuffer> scratch, int64_t chunk,
                        int64_t precision, int64_t flags, float scale, bool keep_residuals) {
  dn_shape s{};
  if (auto e = make_shape(q, v, g, b, w, chunk, precision, flags, scale, &s); e.failure()) return e;
  dn_residuals res{};
  const dn_residuals* rp = nullptr;
  if (keep_residuals) {
    if (int rc = dn_residual_carve(&s, residuals->untyped_data(), &res)) return status(rc, "dn_residual_carve");
    rp = &res;
  } else {
    s.flags |= DN_INFERENCE;
  }
  const float* init_p = (s.flags & DN_HAS_INIT) ? reinterpret_cast<const float*>(init.untyped_data()) : nullptr;
  return status(dn_chunk_fwd(&s, q.untyped_data(), k.untyped_data(), v.untyped_data(), g.untyped_data(), b.untyped_data(),
                             w.untyped_data(), reinterpret_cast<const int32_t*>(seg.untyped_data()), init_p,
                             out->untyped_data(), reinterpret_cast<float*>(final_state->untyped_data()), rp,
                             scratch->untyped_data(), scratch->size_bytes(), stream),
                "dn_chunk_fwd");
}

// ---- backward -------------------------------------------------------------------------------------
ffi::Error ChunkBwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer g,
                        ffi::AnyBuffer b, ffi::AnyBuffer w, ffi::AnyBuffer seg, ffi::AnyBuffer init,
                        ffi::AnyBuffer residuals, ffi::AnyBuffer d_out, ffi::AnyBuffer d_final,
                        ffi::Result<ffi::AnyBuffer> dq, ffi::Result<ffi::AnyBuffer> dk, ffi::Result<ffi::AnyBuffer> dv,
                        ffi::Result<ffi::AnyBuffer> dg, ffi::Result<ffi::AnyBuffer> db, ffi::Result<ffi::AnyBuffer> dw,
                        ffi::Result<ffi::AnyBuffer> d_init, ffi::Result<ffi::AnyBuffer> scratch, int64_t chunk,
                        int64_t precision, int64_t flags, float scale, bool recompute_states) {
  dn_shape s{};
  if (auto e = make_shape(q, v, g, b, w, chunk, precision, flags, scale, &s); e.failure()) return e;
  dn_residuals res{};
  const dn_residuals* rp = nullptr;
  if (!recompute_states) {
    if (int rc = dn_residual_carve(&s, const_cast<void*>(residuals.untyped_data()), &res)) return status(rc, "dn_residual_carve");
    rp = &res;
  }
  const bool has_init = s.flags & DN_HAS_INIT;
  return status(dn_chunk_bwd(&s, q.untyped_data(), k.untyped_data(), v.untyped_data(), g.untyped_data(), b.untyped_data(),
                             w.untyped_data(), reinterpret_cast<const int32_t*>(seg.untyped_data()),
                             has_init ? reinterpret_cast<const float*>(init.untyped_data()) : nullptr, rp,
                             d_out.untyped_data(), reinterpret_cast<const float*>(d_final.untyped_data()),
                             dq->untyped_data(), dk->untyped_data(), dv->untyped_data(), dg->untyped_data(),
                             db->untyped_data(), dw->untyped_data(),
                             has_init ? reinterpret_cast<float*>(d_init->untyped_data()) : nullptr,
                             scratch->untyped_data(), scratch->size_bytes(), stream),
                "dn_chunk_bwd");
}

// ---- decode ---------------------------------------------------------------------------------------
ffi::Error DecodeStepImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v, ffi::AnyBuffer g,
                          ffi::AnyBuffer b, ffi::AnyBuffer w, ffi::AnyBuffer state, ffi::AnyBuffer reset,
                          ffi::Result<ffi::AnyBuffer> out, ffi::Result<ffi::AnyBuffer> new_state, int64_t flags, float scale,
                          float stability_tau, bool has_reset) {
  auto qd = q.dimensions();
  auto vd = v.dimensions();
  if (qd.size() != 3 || vd.size() != 3) return ffi::Error(ffi::ErrorCode::kInvalidArgument, "decode q, k, v must be rank 3");
  dn_decode_shape s{};
  s.B = static_cast<int32_t>(qd[0]); s.Hk = static_cast<int32_t>(qd[1]); s.K = static_cast<int32_t>(qd[2]);
  s.Hv = static_cast<int32_t>(vd[1]); s.V = static_cast<int32_t>(vd[2]);
  gate_layout(g, 1, &s.g_heads, &s.g_cols);
  gate_layout(b, 1, &s.b_heads, &s.b_cols);
  gate_layout(w, 1, &s.w_heads, &s.w_cols);
  s.qkv_dtype = dtype_code(q.element_type());
  s.gate_dtype = dtype_code(g.element_type());
  s.state_in_dtype = dtype_code(state.element_type());
  s.state_out_dtype = dtype_code(new_state->element_type());
  if (s.qkv_dtype < 0 || s.gate_dtype < 0 || s.state_in_dtype < 0 || s.state_out_dtype < 0)
    return ffi::Error(ffi::ErrorCode::kInvalidArgument, "unsupported dtype");
  s.flags = static_cast<uint32_t>(flags);
  s.scale = scale;
  s.stability_tau = stability_tau;
  return status(dn_decode_step(&s, q.untyped_data(), k.untyped_data(), v.untyped_data(), g.untyped_data(), b.untyped_data(),
                               w.untyped_data(), state.untyped_data(),
                               has_reset ? reinterpret_cast<const uint8_t*>(reset.untyped_data()) : nullptr,
                               out->untyped_data(), new_state->untyped_data(), stream),
                "dn_decode_step");
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    dn_ffi_chunk_fwd, ChunkFwdImpl,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()      // q, k, v
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()      // g, b, w
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()                            // seg, init
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Attr<int64_t>("chunk").Attr<int64_t>("precision").Attr<int64_t>("flags").Attr<float>("scale")
        .Attr<bool>("keep_residuals"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    dn_ffi_chunk_bwd, ChunkBwdImpl,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()      // residuals, d_out, d_final
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()                            // d_init, scratch
        .Attr<int64_t>("chunk").Attr<int64_t>("precision").Attr<int64_t>("flags").Attr<float>("scale")
        .Attr<bool>("recompute_states"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(
    dn_ffi_decode_step, DecodeStepImpl,
    ffi::Ffi::Bind()
        .Ctx<ffi::PlatformStream<cudaStream_t>>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
        .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()                            // state, reset
        .Ret<ffi::AnyBuffer>().Ret<ffi::AnyBuffer>()
        .Attr<int64_t>("flags").Attr<float>("scale").Attr<float>("stability_tau").Attr<bool>("has_reset"));
