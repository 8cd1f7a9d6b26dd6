/*
 * flashback_b200.h — C ABI of the B200 (sm_100a) softmax-attention JVP-forward /
 * HVP-backward library (libflashback_b200.so).
 *
 * This is the operator boundary a host framework binds. In the reference the same
 * boundary is the TVM-FFI callable returned by cute.compile and invoked as
 *     cache[key](*tensor_args, softmax_scale, cu_seqlens_q, cu_seqlens_k)
 * (flashback_cute/interface.py:99-119), with the argument orders of
 * _jvp_fwd (interface.py:122-148) and _hvp_bwd (interface.py:151-175), plus FA4's
 * _bwd_preprocess (call site interface.py:230-236).
 *
 * Conventions
 *   - All pointers are DEVICE pointers on the device that is current when the call is
 *     made. The library never allocates or frees device memory (except where an entry
 *     point says otherwise); workspaces, if any, are passed in by the caller.
 *   - Sequence tensors are "rows x heads x head_dim" with the batch folded into rows:
 *     a dense (B, S, H, D) tensor is passed as B*S rows (batch stride must equal
 *     S * row_stride); a varlen (T, H, D) tensor as T rows. The last dimension is
 *     contiguous. Strides are in ELEMENTS.
 *   - Row statistics (lse, z1, dpsum, ddot) are float32 arrays of shape
 *     [heads_q][total_q] (index h * total_q + global_row).
 *   - Causal masking is bottom-right aligned: key j is visible to query i iff
 *     j <= i + (seqlen_k - seqlen_q), per sequence (tests/reference.py:24-28).
 *   - Every entry point returns FB_OK (0) or a negative fb_status; nothing aborts.
 *     Kernels are enqueued on `stream` and the call returns without synchronising.
 */
#ifndef FLASHBACK_B200_H
#define FLASHBACK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct CUstream_st* fb_stream_t; /* = cudaStream_t */

typedef enum {
  FB_OK = 0,
  FB_ERR_NULL_ARG = -1,       /* a required pointer is NULL */
  FB_ERR_DTYPE = -2,          /* dtype not in {bf16, f16, f32} (TypeError in the reference, interface.py:365-366) */
  FB_ERR_HEAD_DIM = -3,       /* head_dim not in {64, 128} (NotImplementedError, interface.py:367-368) */
  FB_ERR_HEADS = -4,          /* heads_q % heads_kv != 0 (ValueError, interface.py:369-370) */
  FB_ERR_SHAPE = -5,          /* negative / inconsistent sizes */
  FB_ERR_ALIGNMENT = -6,      /* pointer not 16-byte aligned or stride not a multiple of 8 elements */
  FB_ERR_ARCH = -7,           /* current device is not sm_100 (NotImplementedError, interface.py:363-364) */
  FB_ERR_CUDA = -8,           /* a CUDA runtime/driver call failed; see fb_last_cuda_error() */
  FB_ERR_MODE = -9,           /* inconsistent combination of optional tensors */
  FB_ERR_TOO_LARGE = -10,     /* size exceeds a documented maximum */
  FB_ERR_DEVICE_TIMEOUT = -11 /* a bounded device-side wait gave up (reported by fb_check_device_status) */
} fb_status;

typedef enum { FB_BF16 = 0, FB_F16 = 1, FB_F32 = 2 } fb_dtype;

/* One sequence tensor (q-like: heads_q heads, kv-like: heads_kv heads). */
typedef struct {
  void* ptr;           /* NULL = tensor absent (where the entry point allows it) */
  int64_t row_stride;  /* elements between consecutive rows (= H*D when contiguous) */
  int64_t head_stride; /* elements between consecutive heads (= D when contiguous) */
} fb_tensor;

/* Problem geometry shared by all entry points (replaces the shapes the reference reads
 * off its torch tensors, interface.py:189-204). */
typedef struct {
  int32_t dtype;      /* fb_dtype of every sequence tensor */
  int32_t batch;      /* number of sequences */
  int32_t heads_q;
  int32_t heads_kv;
  int32_t head_dim;   /* 64 or 128 */
  int32_t seqlen_q;   /* dense: rows per sequence; varlen: max_seqlen_q */
  int32_t seqlen_k;   /* dense: rows per sequence; varlen: max_seqlen_k */
  int32_t causal;     /* 0 / 1 */
  int64_t total_q;    /* rows in q-like tensors (dense: batch*seqlen_q) */
  int64_t total_k;    /* rows in kv-like tensors */
  const int32_t* cu_seqlens_q; /* device int32[batch+1] or NULL (dense) */
  const int32_t* cu_seqlens_k; /* device int32[batch+1] or NULL (dense) */
  float softmax_scale;
  int32_t flags;      /* FB_FLAG_* below; 0 = defaults */
  /* Row segments (dense causal problems only; all 0 = off). The QUERY rows of every sequence (the KEY
   * rows with FB_FLAG_SEG_KEYS) are cut at up to four break rows seg_rows[0] < seg_rows[1] < ... (unused
   * entries 0, at the end; the last break may be the row count itself); the rows below break s (and not
   * below an earlier one) sit seg_shift[s] positions EARLIER in the sequence than bottom-right alignment
   * puts them, rows from the last break on are not shifted. With query segments key j is visible to query
   * i iff j <= i + (seqlen_k - seqlen_q) - shift(i); with key segments iff j <= i + (seqlen_k - seqlen_q)
   * + shift(j). This makes the zig-zag chunks [a_0, b_0), [a_1, b_1), ... of a longer causal sequence
   * that one GPU holds ONE problem:
   *   - query segments: q-like tensors hold the chunks' rows one after the other, seqlen_q = their total,
   *     seqlen_k = the last chunk's end, break s = the local row where chunk s + 1 starts, seg_shift[s] =
   *     (local row where chunk s starts) + (seqlen_k - seqlen_q) - a_s (0 for the last chunk). All entry
   *     points; every kernel runs once over all chunks, the chunks' tiles balance each other inside one
   *     launch, and the dK/dV side sums the chunks inside the kernel.
   *   - key segments (fb_hvp_bwd with dk, dv, dk_dot, dv_dot outputs only): the k-like tensors hold the
   *     chunks' rows, the q-like tensors and row statistics ALL rows of the long sequence; break s = the
   *     local row where chunk s ends, seg_shift[s] = (seqlen_q - seqlen_k) + (local row where chunk s
   *     starts) - a_s. The GPU that holds those keys gets their complete dK, dV, dK_dot, dV_dot: nothing
   *     to sum across GPUs.
   * Breaks must be multiples of 128, shifts non-increasing and >= 0. (The reference is single-GPU and
   * has no counterpart.) */
  int32_t seg_rows[4];
  int32_t seg_shift[4];
} fb_problem;

/* Use the CUDA-core kernels even for 16-bit dtypes. */
#define FB_FLAG_FORCE_SIMT 1
/* Tensor-core kernels, order in which CTAs are scheduled. The (head, batch) pairs are taken in groups of
 * n; inside a group the heaviest tiles of every pair go first (which balances causal launches), and the
 * groups follow one another. n = 1 (FB_FLAG_TILE_MAJOR): all tiles of one pair before the next pair.
 * n = 0: chosen per launch (causal: all pairs in one group; otherwise 1). Tuning switches; results do
 * not depend on them. */
#define FB_FLAG_TILE_MAJOR 2
#define FB_FLAG_SCHED_GROUP(n) (((n) & 0xfff) << 12)
/* dK/dV kernels: number of CTAs (1, 2, 4 or 8; one thread-block cluster) that share a 128-row key tile,
 * each taking a slice of its query blocks; their partial sums are added in a fixed order inside the
 * kernel, so results are deterministic for a given value. 0 = chosen per launch from the grid size (more
 * than 1 only when the launch would otherwise have too few or too uneven CTAs for the GPU, e.g. the
 * per-GPU share of a problem partitioned over 8 GPUs). The reference's K2 always runs one CTA per
 * (key tile, query head) and reduce-adds (hvp_bwd_sm90.py:340-363). */
#define FB_FLAG_DKV_SPLIT(n) (((n) & 15) << 8)
/* fb_hvp_bwd, 16-bit problems on the tensor-core kernels: dk, dv, dk_dot, dv_dot point to FLOAT32 tensors
 * (strides in float32 elements), and with FB_FLAG_KV_ACCUMULATE the results are ADDED to what those
 * tensors hold instead of overwriting it (rows of a key tile no query sees still receive += 0). This is
 * how partial gradients of several query chunks are summed before a reduce-scatter without rounding
 * each partial to 16 bits (the reference sums GQA partials in fp32 accumulators for the same reason,
 * interface.py:215-227). dq and dq_dot are not affected. */
#define FB_FLAG_KV_OUT_F32 4
#define FB_FLAG_KV_ACCUMULATE 8
/* fb_problem.seg_rows / seg_shift describe the key rows instead of the query rows (see there). */
#define FB_FLAG_SEG_KEYS 16

/*
 * JVP forward. Replaces the reference's K1 launch `_jvp_fwd` (interface.py:122-148,
 * kernel jvp_fwd_sm90.py:307) and, in its tangent-free mode, FA4's `_flash_attn_fwd`
 * (call site interface.py:334-343).
 *
 *   O = softmax(c Q K^T) V,  LSE = logsumexp,
 *   O_dot = P_dot V + P V_dot,  S_dot = c (Q_dot K^T + Q K_dot^T),
 *   P_dot = P * (S_dot - z1),   z1 = rowsum(P * S_dot)
 *   optional row statistics for the backward: dpsum = rowsum(dO * O),
 *   ddot = rowsum(dO_dot * O + dO * O_dot)   (taken from fp32 values before rounding)
 *
 * Modes:
 *   - q_dot/k_dot/v_dot all NULL: plain forward (out, lse written; out_dot, z1 ignored).
 *   - lse_known != 0: `out` and `lse` are INPUTS (the reference's K1 situation: the
 *     forward already ran); only out_dot, z1 (and dpsum/ddot) are written.
 *   - dout.ptr != NULL: dpsum (and ddot when tangents are present) are written;
 *     dout_dot may be NULL (treated as zero — the reference's double backward).
 */
typedef struct {
  fb_problem prob;
  fb_tensor q, k, v;             /* in */
  fb_tensor q_dot, k_dot, v_dot; /* in, optional (all or none) */
  fb_tensor out;                 /* out (in when lse_known) */
  fb_tensor out_dot;             /* out, required with tangents */
  float* lse;                    /* out (in when lse_known), natural log, -inf on fully masked rows */
  float* z1;                     /* out, required with tangents */
  fb_tensor dout, dout_dot;      /* in, optional */
  float* dpsum;                  /* out, required when dout present */
  float* ddot;                   /* out, required when dout and tangents present */
  int32_t lse_known;
} fb_jvp_args;

int fb_jvp_fwd(const fb_jvp_args* args, fb_stream_t stream);

/*
 * Row statistics for the backward. Replaces FA4's `_bwd_preprocess` as the reference
 * calls it (interface.py:230-236): dpsum = rowsum(dO * O); additionally, when out_dot is
 * given, ddot = rowsum(dO_dot * O + dO * O_dot) (dout_dot may be NULL = zero).
 */
typedef struct {
  fb_problem prob;
  fb_tensor out, dout;         /* in */
  fb_tensor out_dot, dout_dot; /* in, optional */
  float* dpsum;                /* out */
  float* ddot;                 /* out, required when out_dot present */
} fb_stats_args;

int fb_bwd_row_stats(const fb_stats_args* args, fb_stream_t stream);

/*
 * HVP backward. Replaces the reference's K2 launch `_hvp_bwd` (interface.py:151-175,
 * kernel hvp_bwd_sm90.py:421) together with the fp32-accumulator post-processing that
 * follows it (interface.py:251-271) and, in its first-order mode, FA4's `_flash_attn_bwd`
 * (call site interface.py:303-309).
 *
 *   dP = dO V^T,  dS = P*(dP - dpsum),  dQ = c dS K,  dK = c dS^T Q,  dV = P^T dO
 *   dP_dot = dO V_dot^T + dO_dot V^T,  dS_dot = P_dot*(dP - dpsum) + P*(dP_dot - ddot)
 *   dQ_dot = c (dS_dot K + dS K_dot),  dK_dot = c (dS_dot^T Q + dS^T Q_dot),
 *   dV_dot = P_dot^T dO + P^T dO_dot
 *
 * Outputs are selected by non-NULL pointers: any subset of {dq, dk, dv} (first order)
 * and {dq_dot, dk_dot, dv_dot} (directional derivatives; these need q_dot/k_dot/v_dot,
 * z1 and ddot). dout_dot may be NULL (zero). Results are written in the problem dtype,
 * already scaled; accumulation across GQA query heads happens inside the kernel, so no
 * fp32 accumulator workspace or post-processing launch is needed, and the result does
 * not depend on launch order (deterministic).
 */
typedef struct {
  fb_problem prob;
  fb_tensor q, k, v, dout;                 /* in */
  fb_tensor q_dot, k_dot, v_dot, dout_dot; /* in, optional */
  const float* lse;                        /* in */
  const float* dpsum;                      /* in */
  const float* z1;                         /* in, with tangents */
  const float* ddot;                       /* in, with tangents */
  fb_tensor dq, dk, dv;                    /* out, optional */
  fb_tensor dq_dot, dk_dot, dv_dot;        /* out, optional */
} fb_hvp_args;

int fb_hvp_bwd(const fb_hvp_args* args, fb_stream_t stream);

/*
 * HVP backward whose dK/dV-side results are scattered to the GPUs that own the key rows: the fused
 * "kernel + exchange" step of a sequence-sharded backward (no counterpart in the reference, which is
 * single-GPU; there the partial dK/dV of the query heads meet in fp32 accumulators, interface.py:215-227).
 *
 * `args` as for fb_hvp_bwd, 16-bit problem, flags FB_FLAG_KV_OUT_F32 (| FB_FLAG_KV_ACCUMULATE): batch 1;
 * dk, dv, dk_dot, dv_dot name LOCAL float32 tensors that say which outputs are wanted and, with
 * FB_FLAG_KV_ACCUMULATE, hold partial sums that are added to this call's results. The sums are not
 * written back there: key row r of an output goes to dst[r / rows_per_peer], at row r % rows_per_peer
 * (strides row_stride / head_stride, in float32 elements). dst[i] is a device pointer the current device
 * can store to: its own memory or peer memory mapped into this process (for example a symmetric-memory
 * buffer); the kernels write it with plain 16-byte stores, tile by tile as results complete, so the
 * transfer over NVLink overlaps the remaining tiles' arithmetic. Ordering with the readers of those
 * buffers (a barrier across the GPUs after this call's stream work) is the caller's business.
 * rows_per_peer must be a multiple of 128; n_peers <= 8; seqlen_k <= n_peers * rows_per_peer.
 * accumulate_rows (with FB_FLAG_KV_ACCUMULATE; a multiple of 128, 0 = every row): only key rows below it
 * have a partial sum to add; the local tensors are not read beyond it (and need not be initialised there).
 */
typedef struct {
  int32_t n_peers;
  int32_t rows_per_peer;
  int64_t row_stride, head_stride;
  int64_t accumulate_rows;
  void* dk[8];
  void* dv[8];
  void* dk_dot[8];
  void* dv_dot[8];
} fb_kv_scatter;

int fb_hvp_bwd_scatter(const fb_hvp_args* args, const fb_kv_scatter* scatter, fb_stream_t stream);

/* out[i] = sum over the slots s < n_slots in which element i is valid, of slots[s * slot_stride + i], for
 * i < count (float32; count, slot_stride, period and valid[] multiples of 4; pointers 16-byte aligned;
 * n_slots <= 8): the owner's side of a sequence-sharded backward, adding up what the source GPUs left in
 * its memory. A slot is a sequence of blocks of `period` elements (period = 0: one block of `count`), and
 * source s wrote only the first valid[s] elements of each block (a source whose queries see only the
 * first keys of this owner's key block); `valid` is a HOST array of n_slots counts, or NULL when every
 * slot is complete. Deterministic (fixed order s = 0, 1, ..). */
int fb_sum_slots(const float* slots, int32_t n_slots, int64_t slot_stride, int64_t count, int64_t period, const int64_t* valid,
                 float* out, fb_stream_t stream);

/*
 * First-order backward without any allocation, for callers that cannot allocate device memory:
 * a runtime that reserved the whole GPU up front and hands out only pre-planned buffers, a
 * latency-critical callback where cudaMalloc/cudaFree would synchronise the device, or a plain
 * C host with no device allocator. It has no counterpart in the reference (there the scratch
 * vector is a torch allocation, flashback_cute/interface.py:205-209); it computes exactly what
 * fb_bwd_row_stats followed by fb_hvp_bwd (first-order mode) compute, with the intermediate
 * dpsum = rowsum(dO * O) kept in a fixed array inside the library instead of a caller buffer.
 *
 *   - Limit: heads_q * total_q <= FB_NOALLOC_MAX_STAT_FLOATS; otherwise FB_ERR_TOO_LARGE.
 *     Each GPU that loads the library holds the array (4 MiB) until the process exits.
 *   - The first call on a device looks up the array's device address; make that first call
 *     outside any stream capture.
 *   - All calls share the array, which keeps the previous call's contents (nothing needs
 *     clearing: every element read is first overwritten by the same call). Calls whose kernels
 *     overlap on the GPU race on it: keep them on one stream or order them with events.
 *   - Calls no cudaMalloc, cudaFree or other allocating routine. Inputs and outputs are still the
 *     caller's: q, k, v, out, dout, lse in; dq, dk, dv out (any of the three may be absent).
 */
#define FB_NOALLOC_MAX_STAT_FLOATS (1 << 20)

typedef struct {
  fb_problem prob;
  fb_tensor q, k, v, out, dout; /* in */
  const float* lse;             /* in, [heads_q][total_q] */
  fb_tensor dq, dk, dv;         /* out, optional */
} fb_bwd_noalloc_args;

int fb_bwd_noalloc(const fb_bwd_noalloc_args* args, fb_stream_t stream);

/* Number of kernels the most recent fb_* call on this thread enqueued (for launch accounting). */
int fb_last_launch_count(void);

/* Reads (and clears) the device-side status word of the current device after the caller has
 * synchronised the stream: FB_OK, or FB_ERR_DEVICE_TIMEOUT if a bounded wait in a kernel
 * gave up. Synchronises the device. While the word is set, the tensor-core kernels of later launches on
 * that device return without computing (a lost signal then costs one wait budget, not one per launch):
 * after a failure, collect the status with this call before relying on further results. */
int fb_check_device_status(void);

/* Text for a status code (static storage). Replaces the Python exception messages of
 * `_validate` (interface.py:362-370). */
const char* fb_status_string(int status);

/* Text of the last CUDA error recorded by this thread's most recent failing call. */
const char* fb_last_cuda_error(void);

/* Library ABI version: major*10000 + minor*100 + patch. */
int fb_version(void);

/* Diagnostics, only in a library built with -DFB_PROFILE (otherwise FB_ERR_MODE): with the environment
 * variable FLASHBACK_DEBUG=2 the tensor-core kernels record, for their first CTA, cycle totals per warp
 * role (16 int64 words; layout documented next to g_prof in csrc/tc_kernels.cu). This call synchronises
 * and copies them to host memory `out16`. */
int fb_debug_profile(long long* out16);

/* Test hook for the bounded-wait error path (no counterpart in the reference, whose kernels cannot
 * report a lost signal). Runs the plain forward (bf16, head_dim 64; q, k, v, out, lse of `args`) in an
 * instantiation whose TMA producer leaves out the loads of the second streamed block and whose waits
 * give up after `budget_cycles` SM clocks (1e3 .. 2e9). For seqlen_k > 64 the MMA warp's wait for that
 * block therefore runs out: the CTA stops issuing work, sets the device status word, releases its
 * resources and returns; CTAs that start afterwards see the word and return at once. Nothing faults or
 * hangs. fb_check_device_status() then reports FB_ERR_DEVICE_TIMEOUT (and clears the word); `out` and
 * `lse` hold no meaningful values. */
int fb_debug_wait_timeout(const fb_jvp_args* args, long long budget_cycles, fb_stream_t stream);

/* Bytes of caller-owned scratch for problem `p`. which = 0: ONE float32 row-statistic vector
 * (lse, z1, dpsum and ddot each have this size: heads_q * total_q floats). There is no other
 * workspace: the reference's fp32 accumulators dotq_accum / dotk_accum / dotv_accum and its 64-row
 * padding of the statistics (interface.py:195-227) have no counterpart here. Returns 0 for a null
 * or invalid problem or an unknown `which`. */
size_t fb_workspace_bytes(const fb_problem* p, int which);

/* sizeof() of the ABI structs as compiled into the library, for bindings to verify their own
 * layout: which = 0 fb_tensor, 1 fb_problem, 2 fb_jvp_args, 3 fb_stats_args, 4 fb_hvp_args,
 * 5 fb_bwd_noalloc_args, 6 fb_kv_scatter. */
size_t fb_abi_sizeof(int which);

#ifdef __cplusplus
}
#endif
#endif /* FLASHBACK_B200_H */
