// fb_bwd_noalloc: first-order attention backward for callers that must not allocate.
//
// The ordinary route to dq, dk, dv is two calls: fb_bwd_row_stats writes dpsum = rowsum(dO * O)
// into a scratch vector the CALLER allocates (heads_q * total_q floats), then fb_hvp_bwd consumes
// it. Some callers have no way to provide that vector: a runtime that reserved the whole device
// up front and only hands out fixed, pre-planned buffers; a latency-critical callback where a
// cudaMalloc / cudaFree pair would synchronise the device; a plain C host that binds this ABI and
// has no device allocator of its own. For them this file keeps the scratch vector inside the
// library, as a fixed-size array in device memory, and offers one entry point that runs both
// steps on it. Nothing in this path calls cudaMalloc, cudaFree or any allocating routine.
//
// Limits and rules (also in include/flashback_b200.h):
//   * heads_q * total_q <= FB_NOALLOC_MAX_STAT_FLOATS (1,048,576 floats = 4 MiB). Every GPU that
//     loads the library holds these 4 MiB until the process exits. Larger problems are refused
//     with FB_ERR_TOO_LARGE.
//   * The first call on each device looks up the array's device address (once per device, with
//     that device current). Make that first call outside any stream capture.
//   * All calls share the one array and it keeps whatever the previous call left. The kernels here
//     overwrite every element they later read, so nothing has to be cleared; but two calls whose
//     kernels overlap on the GPU (different streams, no ordering between them) race on the array.
#include "../../include/flashback_b200.h"
#include "fb_params.h"

#include <cuda_runtime.h>
#include <mutex>

namespace {

// In host code this name is only a handle for the CUDA runtime, NOT a device address: passing
// `g_stat_scratch` itself to a kernel would make the kernel use a host pointer. The real device
// address comes from cudaGetSymbolAddress, per device, below.
static __device__ __align__(256) float g_stat_scratch[FB_NOALLOC_MAX_STAT_FLOATS];

constexpr int kMaxDevices = 64;
float* g_scratch_addr[kMaxDevices];  // device address of g_stat_scratch on each device, nullptr = not looked up yet
std::mutex g_setup_mutex;

// Device address of the scratch array on the CURRENT device (looked up on first use). A failing
// CUDA call is recorded like in the other entry points (fb_last_cuda_error()).
int scratch_for_current_device(float** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fb::record_cuda(e);
  if (dev < 0 || dev >= kMaxDevices) return FB_ERR_ARCH;
  std::lock_guard<std::mutex> lock(g_setup_mutex);
  if (!g_scratch_addr[dev]) {
    float* p = nullptr;
    e = cudaGetSymbolAddress(reinterpret_cast<void**>(&p), g_stat_scratch);
    if (e != cudaSuccess) return fb::record_cuda(e);
    if (!p) return FB_ERR_CUDA;
    g_scratch_addr[dev] = p;
  }
  *out = g_scratch_addr[dev];
  return FB_OK;
}

}  // namespace

extern "C" int fb_bwd_noalloc(const fb_bwd_noalloc_args* a, fb_stream_t stream) {
  fb::set_launch_count(0);
  if (!a) return FB_ERR_NULL_ARG;
  const fb_problem& pr = a->prob;
  if (pr.heads_q <= 0 || pr.total_q < 0) return FB_ERR_SHAPE;
  if ((long long)pr.heads_q * (long long)pr.total_q > (long long)FB_NOALLOC_MAX_STAT_FLOATS) return FB_ERR_TOO_LARGE;
  int s = fb::check_problem(pr);
  if (s != FB_OK) return s;
  if (!a->lse) return FB_ERR_NULL_ARG;
  // architecture first: on a device this library has no code for, the symbol look-up below would fail
  // with a less telling error
  int* status_word = nullptr;
  s = fb::device_setup(&status_word);
  if (s != FB_OK) return s;
  float* dpsum = nullptr;
  s = scratch_for_current_device(&dpsum);
  if (s != FB_OK) return s;

  fb_stats_args st = {};
  st.prob = pr;
  st.out = a->out;
  st.dout = a->dout;
  st.dpsum = dpsum;
  s = fb_bwd_row_stats(&st, stream);
  if (s != FB_OK) { fb::set_launch_count(0); return s; }
  const int stat_launches = fb_last_launch_count();

  fb_hvp_args h = {};
  h.prob = pr;
  h.q = a->q; h.k = a->k; h.v = a->v; h.dout = a->dout;
  h.lse = a->lse;
  h.dpsum = dpsum;
  h.dq = a->dq; h.dk = a->dk; h.dv = a->dv;
  s = fb_hvp_bwd(&h, stream);
  // fb_last_launch_count() after this call = the row-statistics launch + the backward's launches
  fb::set_launch_count(s == FB_OK ? stat_launches + fb_last_launch_count() : 0);
  return s;
}
