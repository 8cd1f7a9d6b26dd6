// Internal kernel parameter block shared by the CUDA-core (SIMT) and tensor-core (tcgen05)
// kernels. Built by api.cu from the public C structs in include/flashback_b200.h.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/flashback_b200.h"

namespace fb {

struct SeqT {
  void* ptr;
  int64_t row_stride;
  int64_t head_stride;
};

struct Params {
  int dtype;
  int B, Hq, Hkv, D;
  int Sq, Sk;  // dense: per-sequence rows; varlen: max lengths
  int causal;
  // row segments (dense causal only; seg_n = 0: off) of the query rows, or with seg_keys of the key rows:
  // seg_n break rows, ascending; the rows below break s (and not below an earlier one) sit seg_shift[s]
  // positions earlier than bottom-right alignment puts them, the rows from the last break on do not
  int seg_n, seg_keys, seg_rows[4], seg_shift[4];
  int64_t Tq, Tk;
  const int32_t* cu_q;
  const int32_t* cu_k;
  float scale;
  int lse_known;
  // inputs
  SeqT q, k, v, qd, kd, vd, dout, doutd;
  // forward outputs (inputs of the backward / of lse_known mode)
  SeqT o, od;
  float *lse, *z1, *dpsum, *ddot;
  // backward outputs
  SeqT dq, dk, dv, dqd, dkd, dvd;
  // device status word (bounded-wait timeouts)
  int* status;
  int debug;  // FLASHBACK_DEBUG bits (kernel bring-up switches; 0 in normal use)
  // dK/dV-side outputs (dk, dv, dkd, dvd) as float32 tensors, optionally added to what they already hold
  int kv_f32, kv_accum;
  // dK/dV-side results scattered to the owners of the key rows (fb_hvp_bwd_scatter): key row r of output o
  // goes to scat[o][r / scat_rows] at row r % scat_rows; o = 0 dk, 1 dv, 2 dk_dot, 3 dv_dot. The
  // destinations may be another GPU's memory (plain stores over NVLink). scat_n = 0: off.
  void* scat[4][8];
  int scat_n, scat_rows;
  int64_t scat_row_stride, scat_head_stride;
  int64_t kv_accum_rows;  // kv_accum applies to key rows below this only
  // launch geometry of the tensor-core kernels (filled in by their launcher)
  int tma_out;            // 1: full owner tiles leave (and the forward's dO rows enter) through shared memory + TMA
  int ntiles;             // owner tiles per sequence
  int split;              // dK/dV kernels: CTAs (one cluster) sharing an owner tile, each a slice of its streamed blocks
  int group;              // (head, batch) pairs per scheduling group, see TcCta::setup (0 on entry = chosen by the launcher)
  long long wait_budget;  // clock budget of one bounded wait (test hook instantiation only)
};

struct SeqInfo {
  int q0, k0;    // first global row of this sequence
  int sq, sk;    // its lengths
};

__device__ __forceinline__ SeqInfo seq_info(const Params& p, int b) {
  SeqInfo s;
  if (p.cu_q) { s.q0 = p.cu_q[b]; s.sq = p.cu_q[b + 1] - s.q0; } else { s.q0 = b * p.Sq; s.sq = p.Sq; }
  if (p.cu_k) { s.k0 = p.cu_k[b]; s.sk = p.cu_k[b + 1] - s.k0; } else { s.k0 = b * p.Sk; s.sk = p.Sk; }
  return s;
}

// Shift of sequence-local row `row` of the segmented side (fb_problem.seg_rows / seg_shift).
__device__ __forceinline__ int seg_shift_of(const Params& p, int row) {
  int shift = 0;
  for (int t = p.seg_n - 1; t >= 0; --t)
    if (row < p.seg_rows[t]) shift = p.seg_shift[t];
  return shift;
}
// Causal masking: key j is visible to query row i (both sequence-local) iff j <= i + pair_off(p, s, i, j):
// bottom-right aligned, corrected by the shift of the segment the query (or, with key segments, the key) lies in.
__device__ __forceinline__ int pair_off(const Params& p, const SeqInfo& s, int i, int j) {
  return s.sk - s.sq + (p.seg_keys ? seg_shift_of(p, j) : -seg_shift_of(p, i));
}
// The same for a whole query row (query segments or none; kernels that own query rows do not take key segments).
__device__ __forceinline__ int causal_off(const Params& p, const SeqInfo& s, int i) {
  return s.sk - s.sq - (p.seg_keys ? 0 : seg_shift_of(p, i));
}
// First query row that sees key row j (positions grow with the row index, across the segment breaks too).
__device__ __forceinline__ int first_query_of_key(const Params& p, const SeqInfo& s, int j) {
  const int off = s.sk - s.sq;
  if (p.seg_keys) return max(0, j - (off + seg_shift_of(p, j)));
  int lo = 0;
  for (int t = 0; t < p.seg_n; ++t) {
    const int i = max(lo, j - (off - p.seg_shift[t]));
    if (i < p.seg_rows[t]) return i;
    lo = p.seg_rows[t];
  }
  return max(lo, j - off);
}

template <typename T> __device__ __forceinline__ float to_f(T x);
template <> __device__ __forceinline__ float to_f<float>(float x) { return x; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <> __device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }

template <typename T> __device__ __forceinline__ T from_f(float x);
template <> __device__ __forceinline__ float from_f<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <> __device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

// host-side launchers (each returns the number of kernels enqueued, or a negative fb_status)
int launch_simt_fwd(const Params& p, cudaStream_t stream);
int launch_simt_bwd(const Params& p, cudaStream_t stream);
int launch_row_stats(const Params& p, cudaStream_t stream);
int launch_tc_fwd(const Params& p, cudaStream_t stream);
int launch_tc_bwd(const Params& p, cudaStream_t stream);
int launch_tc_fwd_wait_hook(const Params& p, cudaStream_t stream);  // test instantiation, see fb_debug_wait_timeout
int launch_sum_slots(const float* slots, int n_slots, int64_t slot_stride, int64_t count, int64_t period, const int64_t* valid, float* out,
                     cudaStream_t stream);
int read_profile(long long* out16);

// shared host helpers (api.cu)
int check_problem(const fb_problem& pr);
int record_cuda(cudaError_t e);        // remembers the error text for fb_last_cuda_error(); returns FB_ERR_CUDA
int device_setup(int** status_ptr);    // architecture check + device address of the status word (cached per device)
void set_launch_count(int n);          // what fb_last_launch_count() reports for this thread

}  // namespace fb
