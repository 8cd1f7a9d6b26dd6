// C-ABI entry points (include/flashback_b200.h): argument validation, parameter-block
// construction and dispatch to the tensor-core (tcgen05) or CUDA-core kernels.
// There is no CPU path: on a machine without an sm_100 device every compute entry point
// returns FB_ERR_ARCH / FB_ERR_CUDA.
#include "../../include/flashback_b200.h"
#include "fb_params.h"

#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

namespace fb {

__device__ int g_device_status = 0;

namespace {

thread_local int tl_launches = 0;
thread_local char tl_cuda_error[256] = "";

constexpr int kMaxDevices = 64;
// Per-device facts, looked up once. The entry points may be called from several host threads at
// once (autograd runs backward passes on worker threads), so the look-up takes a mutex and the
// "known" flag is published last, with release ordering, after the pointer it guards.
// (cudaDeviceReset invalidates these cached device addresses; the library does not support it.)
std::atomic<int> g_arch_major[kMaxDevices];  // 0 = not looked up yet
int* g_status_ptr[kMaxDevices];              // device address of g_device_status per device
std::mutex g_setup_mutex;

}  // namespace

int record_cuda(cudaError_t e) {
  snprintf(tl_cuda_error, sizeof(tl_cuda_error), "%s: %s", cudaGetErrorName(e), cudaGetErrorString(e));
  return FB_ERR_CUDA;
}

void set_launch_count(int n) { tl_launches = n; }

// Per-device lazy set-up: architecture check and the address of the status word.
int device_setup(int** status_ptr) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return record_cuda(e);
  if (dev < 0 || dev >= kMaxDevices) return FB_ERR_ARCH;
  int major = g_arch_major[dev].load(std::memory_order_acquire);
  if (major == 0) {
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    major = g_arch_major[dev].load(std::memory_order_relaxed);
    if (major == 0) {
      e = cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev);
      if (e != cudaSuccess) return record_cuda(e);
      int* sp = nullptr;
      if (major == 10) {
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&sp), g_device_status);
        if (e != cudaSuccess) return record_cuda(e);
      }
      g_status_ptr[dev] = sp;
      g_arch_major[dev].store(major, std::memory_order_release);
    }
  }
  if (major != 10) return FB_ERR_ARCH;
  *status_ptr = g_status_ptr[dev];
  return FB_OK;
}

namespace {

// Environment switches are read once, before any thread can race on them.
struct EnvSwitches {
  bool force_simt;
  int debug;
  EnvSwitches() {
    const char* s = getenv("FLASHBACK_FORCE_SIMT");
    force_simt = s && s[0] == '1';
    const char* d = getenv("FLASHBACK_DEBUG");
    debug = d ? atoi(d) : 0;
  }
};
const EnvSwitches g_env;

bool env_force_simt() { return g_env.force_simt; }

}  // namespace

int check_problem(const fb_problem& pr) {
  if (pr.dtype != FB_BF16 && pr.dtype != FB_F16 && pr.dtype != FB_F32) return FB_ERR_DTYPE;
  if (pr.head_dim != 64 && pr.head_dim != 128) return FB_ERR_HEAD_DIM;
  if (pr.heads_q <= 0 || pr.heads_kv <= 0 || pr.heads_q % pr.heads_kv != 0) return FB_ERR_HEADS;
  if (pr.batch <= 0 || pr.seqlen_q < 0 || pr.seqlen_k < 0 || pr.total_q < 0 || pr.total_k < 0) return FB_ERR_SHAPE;
  if ((pr.cu_seqlens_q == nullptr) != (pr.cu_seqlens_k == nullptr)) return FB_ERR_MODE;
  if (!pr.cu_seqlens_q) {
    if (pr.total_q != (int64_t)pr.batch * pr.seqlen_q || pr.total_k != (int64_t)pr.batch * pr.seqlen_k) return FB_ERR_SHAPE;
  }
  if (pr.total_q >= (1ll << 31) || pr.total_k >= (1ll << 31)) return FB_ERR_TOO_LARGE;
  if (pr.batch > 65535 || pr.heads_q > 65535) return FB_ERR_TOO_LARGE;
  const int split = (pr.flags >> 8) & 15;
  if (split != 0 && split != 1 && split != 2 && split != 4 && split != 8) return FB_ERR_MODE;
  int prev_row = 0, prev_shift = INT32_MAX;
  bool ended = false;
  const int seg_len = (pr.flags & FB_FLAG_SEG_KEYS) ? pr.seqlen_k : pr.seqlen_q;
  for (int t = 0; t < 4; ++t) {  // row segments: dense causal, breaks on owner-tile boundaries, positions growing with the row
    if (pr.seg_rows[t] == 0 && pr.seg_shift[t] == 0) { ended = true; continue; }
    if (!pr.causal || pr.cu_seqlens_q) return FB_ERR_MODE;
    if (ended || pr.seg_rows[t] <= prev_row || pr.seg_rows[t] > seg_len || pr.seg_rows[t] % 128 != 0) return FB_ERR_SHAPE;
    if (pr.seg_shift[t] < 0 || pr.seg_shift[t] > prev_shift) return FB_ERR_SHAPE;
    prev_row = pr.seg_rows[t];
    prev_shift = pr.seg_shift[t];
  }
  return FB_OK;
}

namespace {

// Required tensor: non-NULL, 16-byte aligned, strides multiples of 8 elements (16 bytes for
// 16-bit types; what TMA and the vector accesses need).
int check_tensor(const fb_tensor& t, bool required) {
  if (!t.ptr) return required ? FB_ERR_NULL_ARG : FB_OK;
  if (reinterpret_cast<uintptr_t>(t.ptr) % 16 != 0) return FB_ERR_ALIGNMENT;
  if (t.row_stride % 8 != 0 || t.head_stride % 8 != 0 || t.row_stride <= 0 || t.head_stride <= 0) return FB_ERR_ALIGNMENT;
  return FB_OK;
}

SeqT cvt(const fb_tensor& t) { return SeqT{t.ptr, t.row_stride, t.head_stride}; }

void fill_problem(Params& p, const fb_problem& pr) {
  memset(&p, 0, sizeof(p));
  p.dtype = pr.dtype;
  p.B = pr.batch; p.Hq = pr.heads_q; p.Hkv = pr.heads_kv; p.D = pr.head_dim;
  p.Sq = pr.seqlen_q; p.Sk = pr.seqlen_k; p.causal = pr.causal ? 1 : 0;
  p.Tq = pr.total_q; p.Tk = pr.total_k;
  for (int t = 0; t < 4 && pr.seg_rows[t] > 0; ++t) { p.seg_rows[t] = pr.seg_rows[t]; p.seg_shift[t] = pr.seg_shift[t]; p.seg_n = t + 1; }
  p.seg_keys = (p.seg_n > 0 && (pr.flags & FB_FLAG_SEG_KEYS)) ? 1 : 0;
  p.cu_q = pr.cu_seqlens_q; p.cu_k = pr.cu_seqlens_k;
  p.scale = pr.softmax_scale;
  p.debug = g_env.debug;
  p.group = (pr.flags & FB_FLAG_TILE_MAJOR) ? 1 : ((pr.flags >> 12) & 0xfff);  // 0 = chosen by the launcher
  p.split = (pr.flags >> 8) & 15;  // 0 = chosen by the launcher
  p.kv_f32 = (pr.flags & FB_FLAG_KV_OUT_F32) ? 1 : 0;
  p.kv_accum = (pr.flags & FB_FLAG_KV_ACCUMULATE) ? 1 : 0;
  p.kv_accum_rows = INT64_MAX;
  p.wait_budget = 0;
}

bool use_tensor_cores(const fb_problem& pr) {
  return pr.dtype != FB_F32 && !(pr.flags & FB_FLAG_FORCE_SIMT) && !env_force_simt();
}

// key segments: only the kernels that own key rows (dK/dV side) take them
bool has_key_segments(const fb_problem& pr) { return (pr.flags & FB_FLAG_SEG_KEYS) && pr.seg_rows[0] > 0; }

#define FB_TRY(expr) do { int _s = (expr); if (_s != FB_OK) return _s; } while (0)

}  // namespace
}  // namespace fb

using namespace fb;

extern "C" int fb_jvp_fwd(const fb_jvp_args* a, fb_stream_t stream) {
  tl_launches = 0;
  if (!a) return FB_ERR_NULL_ARG;
  FB_TRY(check_problem(a->prob));
  const bool tangent = a->q_dot.ptr || a->k_dot.ptr || a->v_dot.ptr;
  if (tangent && !(a->q_dot.ptr && a->k_dot.ptr && a->v_dot.ptr)) return FB_ERR_MODE;
  FB_TRY(check_tensor(a->q, true)); FB_TRY(check_tensor(a->k, true)); FB_TRY(check_tensor(a->v, true));
  FB_TRY(check_tensor(a->q_dot, tangent)); FB_TRY(check_tensor(a->k_dot, tangent)); FB_TRY(check_tensor(a->v_dot, tangent));
  FB_TRY(check_tensor(a->out, true));
  FB_TRY(check_tensor(a->out_dot, tangent));
  if (!a->lse) return FB_ERR_NULL_ARG;
  if (tangent && !a->z1) return FB_ERR_NULL_ARG;
  if (a->lse_known && !tangent) return FB_ERR_MODE;
  if (has_key_segments(a->prob)) return FB_ERR_MODE;
  FB_TRY(check_tensor(a->dout, false)); FB_TRY(check_tensor(a->dout_dot, false));
  if (a->dout_dot.ptr && !(a->dout.ptr && tangent)) return FB_ERR_MODE;
  if (a->dout.ptr && (!a->dpsum || (tangent && !a->ddot))) return FB_ERR_NULL_ARG;
  if (a->prob.total_q == 0) return FB_OK;

  Params p;
  fill_problem(p, a->prob);
  FB_TRY(device_setup(&p.status));
  p.q = cvt(a->q); p.k = cvt(a->k); p.v = cvt(a->v);
  p.qd = cvt(a->q_dot); p.kd = cvt(a->k_dot); p.vd = cvt(a->v_dot);
  p.o = cvt(a->out); p.od = cvt(a->out_dot);
  p.lse = a->lse; p.z1 = a->z1;
  p.dout = cvt(a->dout); p.doutd = cvt(a->dout_dot);
  p.dpsum = a->dpsum; p.ddot = a->ddot;
  p.lse_known = a->lse_known ? 1 : 0;
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int n = use_tensor_cores(a->prob) ? launch_tc_fwd(p, s) : launch_simt_fwd(p, s);
  if (n < 0) { if (n == FB_ERR_CUDA) record_cuda(cudaGetLastError()); return n; }
  tl_launches = n;
  return FB_OK;
}

extern "C" int fb_bwd_row_stats(const fb_stats_args* a, fb_stream_t stream) {
  tl_launches = 0;
  if (!a) return FB_ERR_NULL_ARG;
  FB_TRY(check_problem(a->prob));
  FB_TRY(check_tensor(a->out, true)); FB_TRY(check_tensor(a->dout, true));
  FB_TRY(check_tensor(a->out_dot, false)); FB_TRY(check_tensor(a->dout_dot, false));
  if (!a->dpsum) return FB_ERR_NULL_ARG;
  if (a->out_dot.ptr && !a->ddot) return FB_ERR_NULL_ARG;
  if (a->dout_dot.ptr && !a->out_dot.ptr) return FB_ERR_MODE;
  if (a->prob.total_q == 0) return FB_OK;
  Params p;
  fill_problem(p, a->prob);
  FB_TRY(device_setup(&p.status));
  p.o = cvt(a->out); p.dout = cvt(a->dout); p.od = cvt(a->out_dot); p.doutd = cvt(a->dout_dot);
  p.dpsum = a->dpsum; p.ddot = a->out_dot.ptr ? a->ddot : nullptr;
  int n = launch_row_stats(p, reinterpret_cast<cudaStream_t>(stream));
  if (n < 0) { if (n == FB_ERR_CUDA) record_cuda(cudaGetLastError()); return n; }
  tl_launches = n;
  return FB_OK;
}

static int hvp_bwd_impl(const fb_hvp_args* a, const fb_kv_scatter* sc, fb_stream_t stream) {
  tl_launches = 0;
  if (!a) return FB_ERR_NULL_ARG;
  FB_TRY(check_problem(a->prob));
  const bool tangent = a->q_dot.ptr || a->k_dot.ptr || a->v_dot.ptr;
  if (tangent && !(a->q_dot.ptr && a->k_dot.ptr && a->v_dot.ptr)) return FB_ERR_MODE;
  const bool want_dot = a->dq_dot.ptr || a->dk_dot.ptr || a->dv_dot.ptr;
  if (want_dot && !tangent) return FB_ERR_MODE;
  if (a->dout_dot.ptr && !tangent) return FB_ERR_MODE;
  FB_TRY(check_tensor(a->q, true)); FB_TRY(check_tensor(a->k, true)); FB_TRY(check_tensor(a->v, true));
  FB_TRY(check_tensor(a->dout, true));
  FB_TRY(check_tensor(a->q_dot, tangent)); FB_TRY(check_tensor(a->k_dot, tangent)); FB_TRY(check_tensor(a->v_dot, tangent));
  FB_TRY(check_tensor(a->dout_dot, false));
  FB_TRY(check_tensor(a->dq, false)); FB_TRY(check_tensor(a->dk, false)); FB_TRY(check_tensor(a->dv, false));
  FB_TRY(check_tensor(a->dq_dot, false)); FB_TRY(check_tensor(a->dk_dot, false)); FB_TRY(check_tensor(a->dv_dot, false));
  if (!a->lse || !a->dpsum) return FB_ERR_NULL_ARG;
  if (tangent && (!a->z1 || !a->ddot)) return FB_ERR_NULL_ARG;
  if (has_key_segments(a->prob) && (a->dq.ptr || a->dq_dot.ptr)) return FB_ERR_MODE;
  if (a->prob.flags & (FB_FLAG_KV_OUT_F32 | FB_FLAG_KV_ACCUMULATE)) {
    // float32 / accumulating dK,dV-side outputs: tensor-core kernels only, and accumulation needs float32
    if (!use_tensor_cores(a->prob)) return FB_ERR_MODE;
    if ((a->prob.flags & FB_FLAG_KV_ACCUMULATE) && !(a->prob.flags & FB_FLAG_KV_OUT_F32)) return FB_ERR_MODE;
  }
  if (a->prob.total_q == 0 || a->prob.total_k == 0) return FB_OK;

  Params p;
  fill_problem(p, a->prob);
  FB_TRY(device_setup(&p.status));
  p.q = cvt(a->q); p.k = cvt(a->k); p.v = cvt(a->v); p.dout = cvt(a->dout);
  // Tangent inputs only matter if a directional derivative is requested.
  if (want_dot) { p.qd = cvt(a->q_dot); p.kd = cvt(a->k_dot); p.vd = cvt(a->v_dot); p.doutd = cvt(a->dout_dot); }
  p.lse = const_cast<float*>(a->lse); p.dpsum = const_cast<float*>(a->dpsum);
  p.z1 = const_cast<float*>(a->z1); p.ddot = const_cast<float*>(a->ddot);
  p.dq = cvt(a->dq); p.dk = cvt(a->dk); p.dv = cvt(a->dv);
  p.dqd = cvt(a->dq_dot); p.dkd = cvt(a->dk_dot); p.dvd = cvt(a->dv_dot);
  if (sc) {
    // scatter mode: float32 results of the dK/dV kernels go to the owners of the key rows
    if (!p.kv_f32 || a->prob.batch != 1 || a->prob.cu_seqlens_q) return FB_ERR_MODE;
    if (sc->n_peers < 1 || sc->n_peers > 8 || sc->rows_per_peer <= 0 || sc->rows_per_peer % 128 != 0) return FB_ERR_SHAPE;
    if ((int64_t)sc->n_peers * sc->rows_per_peer < a->prob.seqlen_k) return FB_ERR_SHAPE;
    if (sc->row_stride <= 0 || sc->head_stride <= 0 || sc->row_stride % 4 != 0 || sc->head_stride % 4 != 0) return FB_ERR_ALIGNMENT;
    void* const* lists[4] = {sc->dk, sc->dv, sc->dk_dot, sc->dv_dot};
    const void* wanted[4] = {a->dk.ptr, a->dv.ptr, a->dk_dot.ptr, a->dv_dot.ptr};
    for (int o = 0; o < 4; ++o)
      for (int i = 0; i < sc->n_peers; ++i) {
        if (wanted[o] && !lists[o][i]) return FB_ERR_NULL_ARG;
        if (reinterpret_cast<uintptr_t>(lists[o][i]) % 16 != 0) return FB_ERR_ALIGNMENT;
        p.scat[o][i] = lists[o][i];
      }
    if (sc->accumulate_rows < 0 || sc->accumulate_rows % 128 != 0) return FB_ERR_SHAPE;
    if (sc->accumulate_rows > 0) p.kv_accum_rows = sc->accumulate_rows;
    p.scat_n = sc->n_peers; p.scat_rows = sc->rows_per_peer;
    p.scat_row_stride = sc->row_stride; p.scat_head_stride = sc->head_stride;
  }
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  int n = use_tensor_cores(a->prob) ? launch_tc_bwd(p, s) : launch_simt_bwd(p, s);
  if (n < 0) { if (n == FB_ERR_CUDA) record_cuda(cudaGetLastError()); return n; }
  tl_launches = n;
  return FB_OK;
}

extern "C" int fb_hvp_bwd(const fb_hvp_args* a, fb_stream_t stream) { return hvp_bwd_impl(a, nullptr, stream); }

extern "C" int fb_hvp_bwd_scatter(const fb_hvp_args* a, const fb_kv_scatter* sc, fb_stream_t stream) {
  if (!sc) { tl_launches = 0; return FB_ERR_NULL_ARG; }
  return hvp_bwd_impl(a, sc, stream);
}

extern "C" int fb_sum_slots(const float* slots, int32_t n_slots, int64_t slot_stride, int64_t count, int64_t period, const int64_t* valid,
                            float* out, fb_stream_t stream) {
  tl_launches = 0;
  if (!slots || !out) return FB_ERR_NULL_ARG;
  if (n_slots < 1 || n_slots > 8 || count < 0 || slot_stride < count || period < 0) return FB_ERR_SHAPE;
  if (period % 4 != 0 || (period > 0 && count % period != 0)) return FB_ERR_SHAPE;
  if (valid)
    for (int s = 0; s < n_slots; ++s)
      if (valid[s] < 0 || valid[s] % 4 != 0) return FB_ERR_SHAPE;
  if (count % 4 != 0 || slot_stride % 4 != 0 || reinterpret_cast<uintptr_t>(slots) % 16 != 0 || reinterpret_cast<uintptr_t>(out) % 16 != 0)
    return FB_ERR_ALIGNMENT;
  if (count == 0) return FB_OK;
  int* status_word = nullptr;
  FB_TRY(device_setup(&status_word));
  int n = launch_sum_slots(slots, n_slots, slot_stride, count, period, valid, out, reinterpret_cast<cudaStream_t>(stream));
  if (n < 0) { if (n == FB_ERR_CUDA) record_cuda(cudaGetLastError()); return n; }
  tl_launches = n;
  return FB_OK;
}

extern "C" int fb_last_launch_count(void) { return tl_launches; }

extern "C" int fb_check_device_status(void) {
  int* sp = nullptr;
  FB_TRY(device_setup(&sp));
  cudaError_t e = cudaDeviceSynchronize();
  if (e != cudaSuccess) return record_cuda(e);
  int v = 0;
  e = cudaMemcpy(&v, sp, sizeof(int), cudaMemcpyDeviceToHost);
  if (e != cudaSuccess) return record_cuda(e);
  if (v != 0) {
    int zero = 0;
    cudaMemcpy(sp, &zero, sizeof(int), cudaMemcpyHostToDevice);
    snprintf(tl_cuda_error, sizeof(tl_cuda_error), "device status word = 0x%x (bits 0-2: a bounded wait gave up in the FWD/DQ/DKV kernel; bit 8: shared memory misaligned)", v);
    return FB_ERR_DEVICE_TIMEOUT;
  }
  return FB_OK;
}

extern "C" const char* fb_status_string(int status) {
  switch (status) {
    case FB_OK: return "ok";
    case FB_ERR_NULL_ARG: return "a required pointer is NULL";
    case FB_ERR_DTYPE: return "q, k, v must share a dtype in {float16, bfloat16, float32}";
    case FB_ERR_HEAD_DIM: return "head_dim must equal head_dim_v and be 64 or 128";
    case FB_ERR_HEADS: return "number of q heads must be divisible by number of kv heads";
    case FB_ERR_SHAPE: return "inconsistent problem sizes";
    case FB_ERR_ALIGNMENT: return "pointers must be 16-byte aligned and strides multiples of 8 elements";
    case FB_ERR_ARCH: return "flashback_b200 supports only sm_100 (Blackwell B200) GPUs";
    case FB_ERR_CUDA: return "CUDA call failed";
    case FB_ERR_MODE: return "inconsistent combination of optional tensors";
    case FB_ERR_TOO_LARGE: return "size exceeds a documented maximum";
    case FB_ERR_DEVICE_TIMEOUT: return "a bounded device-side wait gave up";
  }
  return "unknown status";
}

extern "C" const char* fb_last_cuda_error(void) { return tl_cuda_error; }

extern "C" int fb_version(void) { return 100; }

extern "C" int fb_debug_profile(long long* out16) { return out16 ? read_profile(out16) : FB_ERR_NULL_ARG; }

extern "C" int fb_debug_wait_timeout(const fb_jvp_args* a, long long budget_cycles, fb_stream_t stream) {
  tl_launches = 0;
  if (!a) return FB_ERR_NULL_ARG;
  FB_TRY(check_problem(a->prob));
  if (a->prob.dtype != FB_BF16 || a->prob.head_dim != 64) return FB_ERR_MODE;
  if (budget_cycles < 1000 || budget_cycles > 2000000000ll) return FB_ERR_MODE;
  FB_TRY(check_tensor(a->q, true)); FB_TRY(check_tensor(a->k, true)); FB_TRY(check_tensor(a->v, true));
  FB_TRY(check_tensor(a->out, true));
  if (!a->lse) return FB_ERR_NULL_ARG;
  if (a->prob.total_q == 0) return FB_OK;
  Params p;
  fill_problem(p, a->prob);
  FB_TRY(device_setup(&p.status));
  p.q = cvt(a->q); p.k = cvt(a->k); p.v = cvt(a->v); p.o = cvt(a->out);
  p.lse = a->lse;
  p.wait_budget = budget_cycles;
  int n = launch_tc_fwd_wait_hook(p, reinterpret_cast<cudaStream_t>(stream));
  if (n < 0) { if (n == FB_ERR_CUDA) record_cuda(cudaGetLastError()); return n; }
  tl_launches = n;
  return FB_OK;
}

extern "C" size_t fb_workspace_bytes(const fb_problem* pr, int which) {
  if (!pr || which != 0 || pr->heads_q <= 0 || pr->total_q < 0) return 0;
  return (size_t)pr->heads_q * (size_t)pr->total_q * sizeof(float);
}

extern "C" size_t fb_abi_sizeof(int which) {
  switch (which) {
    case 0: return sizeof(fb_tensor);
    case 1: return sizeof(fb_problem);
    case 2: return sizeof(fb_jvp_args);
    case 3: return sizeof(fb_stats_args);
    case 4: return sizeof(fb_hvp_args);
    case 5: return sizeof(fb_bwd_noalloc_args);
    case 6: return sizeof(fb_kv_scatter);
  }
  return 0;
}
