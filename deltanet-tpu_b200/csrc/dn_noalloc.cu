// dn_prepass_fwd_static: the forward prepass for callers that cannot allocate device memory.
//
// Some hosts of this library cannot hand it a scratch buffer: a runtime that forbids
// allocation inside its custom-call handlers and was not asked for scratch when the call was
// built, a real-time serving loop that has pinned its whole memory plan, a sandboxed plugin
// with no access to the CUDA allocator.  For them this one entry point carries its own
// scratch: a fixed array that lives in the library image on every GPU that loads it, from load
// to process exit.  The caller still passes all inputs and outputs.
#include <mutex>

#include "dn_kernels.cuh"

#define DN_STATIC_SCRATCH_BYTES (32u << 20)

// File-scope device array.  In host code this name is only a handle for the symbol, never a
// device address: the address is looked up once per device with cudaGetSymbolAddress below.
static __device__ __align__(256) unsigned char dn_static_scratch[DN_STATIC_SCRATCH_BYTES];

namespace {
constexpr int kMaxDevices = 64;
std::mutex g_lock;
void* g_scratch_ptr[kMaxDevices] = {};

// Device address of the array on the CURRENT device (looked up on first use, per device).
int static_scratch(void** out) {
  int dev = -1;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return DN_ERR_CUDA_LAUNCH;
  std::lock_guard<std::mutex> guard(g_lock);
  if (!g_scratch_ptr[dev]) {
    void* p = nullptr;
    if (cudaGetSymbolAddress(&p, dn_static_scratch) != cudaSuccess || !p) return DN_ERR_CUDA_LAUNCH;
    g_scratch_ptr[dev] = p;
  }
  *out = g_scratch_ptr[dev];
  return DN_OK;
}
}  // namespace

extern "C" {

size_t dn_static_scratch_bytes(void) { return DN_STATIC_SCRATCH_BYTES; }

int dn_prepass_fwd_static(const dn_shape* s, const void* q, const void* k, const void* v,
                          const void* g_, const void* b, const void* w, const int32_t* seg,
                          const dn_residuals* res, void* stream) {
  dn::Geo g;
  int rc = dn::make_geo(s, &g);
  if (rc) return rc;
  if (dn::peek_device_error()) return DN_ERR_DEVICE_WAIT;
  if (!q || !k || !v || !g_ || !b || !w || !res) return DN_ERR_NULL_POINTER;
  if (!res->W || !res->U || !res->M || !res->qe || !res->ke || !res->lam_end) return DN_ERR_NULL_POINTER;
  // what the launcher will ask for: one scratch block per CTA, at most one CTA per SM
  const size_t items = (size_t)g.B * g.H * g.NC, ctas = items < (size_t)dn::sm_count() ? items : (size_t)dn::sm_count();
  const bool tc = dn::prepass_fwd_tc_eligible(g);
  const size_t per_cta = tc ? dn::prepass_fwd_tc_scratch_per_cta() : dn::prepass_fwd_scratch_per_cta(g);
  const size_t need = ctas * per_cta * sizeof(float);
  if (need > DN_STATIC_SCRATCH_BYTES) return DN_ERR_STATIC_SCRATCH_EXCEEDED;
  void* scratch = nullptr;
  if ((rc = static_scratch(&scratch))) return rc;
  return dn::launch_prepass_fwd(g, q, k, v, g_, b, w, seg, *res, reinterpret_cast<float*>(scratch),
                                DN_STATIC_SCRATCH_BYTES / sizeof(float), (cudaStream_t)stream);
}

}  // extern "C"
