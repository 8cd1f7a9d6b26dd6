// Tensor-core kernels (sm_100a): JVP forward and HVP backward of softmax attention with
// TMA-staged tiles, tcgen05 MMAs accumulating in TMEM and warp-specialised load / MMA /
// pointwise roles. One kernel template covers three work decompositions that share the same
// GEMM shapes:
//
//   KIND_FWD  owner = 128 query rows.  S-like tiles: S = Q K^T, S_dot = Q_dot K^T + Q K_dot^T.
//             Operands P, W = c P*S_dot.   O += P V,  O_dot += W V + P V_dot.
//             (replaces the reference's K1, jvp_fwd_sm90.py:792-842, plus the plain forward)
//   KIND_DQ   owner = 128 query rows.  S-like: S, dP = dO V^T, S_dot, dP_dot = dO V_dot^T + dO_dot V^T.
//             Operands dS, dS_dot.         dQ += dS K,  dQ_dot += dS_dot K + dS K_dot.
//   KIND_DKV  owner = 128 key rows, loops over the G query heads of the kv head and their
//             query blocks. S-like tiles are the transposes (K Q^T, ...). Operands P^T, dS^T,
//             P_dot^T, dS_dot^T.  dV += P^T dO, dK += dS^T Q, dV_dot += P_dot^T dO + P^T dO_dot,
//             dK_dot += dS_dot^T Q + dS^T Q_dot.
//             (KIND_DQ + KIND_DKV replace the reference's K2, hvp_bwd_sm90.py:1220-1526, its fp32
//              reduce-add accumulator and the post-processing launches, interface.py:251-271)
//
// In every kind the owner tile's operands stay resident in shared memory as the A side
// (K-major, 128-byte swizzle), the other side's 64-row tiles stream through a TMA pipeline and
// serve both as K-major B operands of the S-like GEMMs and as MN-major B operands of the output
// GEMMs; the pointwise warps (one thread per TMEM lane = owner row) turn the fp32 S-like tiles
// into 16-bit A operands written back into TMEM over the columns they came from. Kernels with
// spare TMEM columns also keep owner operands of N=64 S-like GEMMs there (Cfg::nATmem).
//
// Warp roles (128 + 128*NWG threads = whole warpgroups, so that registers can be moved between them):
// warpgroup 0 = the role warps: warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner (one elected lane
// each), warp 2 = DKV statistics stager, warp 3 idle; it gives most of its registers back (setmaxnreg) and
// the NWG pointwise / epilogue warpgroups that follow (warp % 4 selects the TMEM lane quadrant; each
// warpgroup takes an equal share of the streamed columns) take them. The reference does the same with
// its producer (24 registers) and MMA warpgroups (240), jvp_fwd_sm90.py:163,433,461.
#include "fb_params.h"
#include "ptx_sm100.cuh"
#include "../../include/flashback_b200.h"

#include <cuda.h>
#include <cstring>
#include <mutex>
#include <type_traits>

namespace fb {
namespace {

using namespace ptx;

constexpr int BM = 128;  // owner rows per CTA = TMEM lanes
constexpr int BN = 64;   // streamed rows per tile
constexpr int NWG = 2;                          // pointwise warpgroups
constexpr int kPwThreads = NWG * 128;
constexpr int kStatsWarp = 2;                   // DKV: warp that stages the streamed rows' statistics
constexpr int kRoleThreads = 128;               // warpgroup 0: producer, issuer, statistics stager, one idle warp
constexpr int kThreads = kRoleThreads + kPwThreads;
// Register budgets after the hand-over (setmaxnreg), for the kernels that use it (TcCta::kRealloc).
// A kernel of kThreads threads starts with kLaunchRegs registers per thread; `setmaxnreg.inc` WAITS (with no
// bound) until the registers it asks for are free, so the pointwise warpgroups may only ask for what the
// role warpgroup has given back: budgets that merely sum to the 64 K register file (96 / 208, 80 / 216)
// hung the kernel in an experiment, the launch allocation of the other warps being what it is.
constexpr int kLaunchRegs = 168;  // 65536 / 384 threads, rounded down to the allocation unit of 8
constexpr int kRoleRegs = 104, kPwRegs = 200;
static_assert(kRoleThreads * (kLaunchRegs - kRoleRegs) >= kPwThreads * (kPwRegs - kLaunchRegs),
              "the pointwise warpgroups would wait forever for registers nobody releases");
constexpr int kSmemLimit = 232448;  // 227 KB opt-in maximum per CTA
constexpr int kMiscBytes = 3072;    // barriers + TMEM slot + abort flag + DKV row statistics (2 buffers); FWD: x2, row-max exchange
constexpr float kLog2e = 1.4426950408889634f;
constexpr float kRescaleThreshold = 8.f;  // log2 units: rescale accumulators when the row max grew by > 2^8
// Experiment, off by default: every kPolyPeriod-th pair of exponentials computed on the FMA pipe
// (ex2_poly2) instead of the special-function unit (16 ex2 per clock and SM), in the kernels whose
// pointwise warps are the critical path. Measured on B200 with -DFB_EXP2_POLY=4 / =2 (all parity gates
// still pass): non-causal B8 H32 S4096 D64 whole step 14.1 -> 15.3 / 16.3 ms, first-order dK/dV at
// S8192 D128 2.01 -> 2.22 / 2.53 ms. The pointwise warps are bound by instruction issue and the FP32
// pipe, not by the special-function unit, so ten extra instructions per pair cost more than the ex2
// they replace (the reference found the same on Hopper, flashback_cute/interface.py:46-47).
#ifndef FB_EXP2_POLY
#define FB_EXP2_POLY 0
#endif
constexpr int kPolyPeriod = FB_EXP2_POLY;

enum { KIND_FWD = 0, KIND_DQ = 1, KIND_DKV = 2 };
// T_OUT0..3: the kernel's outputs, owner-tile boxes (FWD: O, O_dot; DQ: dQ, dQ_dot; DKV: dK, dV, dK_dot, dV_dot)
enum { T_Q = 0, T_K, T_V, T_DO, T_QD, T_KD, T_VD, T_DOD, T_OUT0, T_OUT1, T_OUT2, T_OUT3, T_COUNT };
constexpr int kStageOff = 8192;  // epilogue staging tiles in the (by then free) tile area, past the small exchange arrays

// Bring-up profile of the first CTA, compiled in with -DFB_PROFILE only (then switched on by
// FLASHBACK_DEBUG bit 1): cycle totals per role, read back with fb_debug_profile().  [0] kernel cycles  [1] n_it  [2] MMA: wait streamed tiles  [3] MMA: wait operands
// [4] MMA: issue  [5] pointwise: wait S-like tiles  [6] pointwise: work  [7] producer: wait empty
// [8] MMA: S-like GEMM issue  [9] pointwise: TMEM load waits  [10] pointwise: publish
#ifdef FB_PROFILE
__device__ long long g_prof[16];
constexpr bool kProfile = true;
// Per-CTA timeline of the last launch (globaltimer ns): [0] entry  [1] set-up done  [2] owner tiles loaded
// [3] first MMAs issued  [4] last MMAs issued  [5] accumulators complete  [6] epilogue done  [7] exit;
// g_trace_meta = SM id | iterations << 32. Read back with fb_debug_trace() (profile builds only).
constexpr int kTraceCtas = 16384;
__device__ unsigned long long g_trace[kTraceCtas][8];
__device__ unsigned long long g_trace_meta[kTraceCtas];
__device__ __forceinline__ unsigned long long trace_now() {
  unsigned long long t;
  asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
  return t;
}
#define FB_TRACE(slot) do { if (blockIdx.x < kTraceCtas) g_trace[blockIdx.x][slot] = trace_now(); } while (0)
#else
#define FB_TRACE(slot) do { } while (0)
__device__ long long g_prof[1];  // never written: every `prof` branch below is dead code in this build
constexpr bool kProfile = false;
#endif

struct TmaMaps {
  CUtensorMap m[T_COUNT];
};

constexpr int ceil_pow2(int x) {
  int p = 32;
  while (p < x) p *= 2;
  return p;
}

// Compile-time shape of one instantiation.
//   FWD: FIRST = accumulate O with online softmax (false = LSE known, O is an input).
//   DQ/DKV: FIRST = first-order outputs, TANGENT = directional-derivative outputs, DOD = dO_dot given.
template <int KIND, int D, bool TANGENT, bool FIRST, bool DOD>
struct Cfg {
  static constexpr bool kFwd = KIND == KIND_FWD;
  static constexpr int nOuter = kFwd ? (TANGENT ? 2 : 1)
                                     : (KIND == KIND_DQ ? (2 + (TANGENT ? 1 : 0) + ((TANGENT && DOD) ? 1 : 0)) : (TANGENT ? 4 : 2));
  // Streamed operands travel in two groups with their own pipelines. g0 is released early, g1 after
  // the last output GEMM of the block:
  //   FWD: g0 = {K, Kd} (free once the S-like GEMMs are done)        g1 = {V, Vd}
  //   DQ : g0 = {V, Vd} (free once the S-like GEMMs are done)        g1 = {K, Kd}
  //   DKV: first order: g1 = {Q, dO};  with tangents: g0 = {dO, dOd} (free after the dV_dot GEMMs, which are
  //        issued early), g1 = {Q, Qd}
  static constexpr int nG0 = KIND == KIND_DKV ? (TANGENT ? (DOD ? 2 : 1) : 0) : (TANGENT ? 2 : 1);
  static constexpr int nG1 = KIND == KIND_DKV ? 2 : (TANGENT ? 2 : 1);
  static constexpr int nS = kFwd ? (TANGENT ? 2 : 1) : (TANGENT ? 4 : 2);
  static constexpr int nAcc = (KIND == KIND_DKV ? 2 : 1) * ((FIRST ? 1 : 0) + (TANGENT ? 1 : 0));
  static constexpr int accCols = nAcc * D;
  static constexpr int ST = (accCols + 2 * nS * BN <= 512) ? 2 : 1;  // TMEM stages of the S-like tiles
  static_assert(accCols + ST * nS * BN <= 512, "TMEM budget exceeded");
  // Owner-side operands of N=64 S-like GEMMs also live in TMEM as 16-bit A operands when columns are
  // left over (LSE-known forward: Q_dot; plain forward: Q; first-order dQ: Q and dO): an N=64 MMA with
  // A in shared memory is limited to 48 clk by the operand bandwidth, with A in TMEM it runs in 32.
  // Not used where it measured slower or flat: the N=128 pair GEMMs (full rate from shared memory
  // already) and the two-phase dQ kernel with tangents (K2's dQ part: 2.95 -> 3.12 ms).
  // aOuter(j) = owner tile index of the j-th such operand.
  static constexpr int aCols = D / 2;
  static constexpr int nAWant = kFwd ? 1 : ((KIND == KIND_DQ && !TANGENT) ? 2 : 0);
  static constexpr int nAFit = (512 - accCols - ST * nS * BN) / aCols;
  static constexpr int nATmem = nAWant < nAFit ? nAWant : nAFit;
  __host__ __device__ static constexpr int aOuter(int j) { return kFwd ? (TANGENT ? 1 : 0) : j; }
  __host__ __device__ static constexpr int aSlot(int outer) {  // -1: operand `outer` is read from shared memory
    for (int j = 0; j < nATmem; ++j)
      if (aOuter(j) == outer) return j;
    return -1;
  }
  static constexpr int aBase = accCols + ST * nS * BN;
  static constexpr int tmemCols = ceil_pow2(aBase + nATmem * aCols);
  static constexpr int outerTile = BM * D * 2;
  static constexpr int innerTile = BN * D * 2;
  static constexpr int outerBytes = nOuter * outerTile;
  static constexpr int g0Bytes = nG0 * innerTile;
  static constexpr int g1Bytes = nG1 * innerTile;
  static constexpr int miscBytes = kMiscBytes;
  static constexpr int tileBudget = kSmemLimit - miscBytes;
  // Shared-memory stages. With two TMEM stages the S-like GEMMs of block i+1 are issued before the
  // output GEMMs of block i, so g0 needs two stages and a g1 that also feeds S-like GEMMs three;
  // with one TMEM stage one (g0) and two (g1) suffice. Spare shared memory deepens the pipelines.
  static constexpr int SS0min = nG0 == 0 ? 0 : (ST == 2 ? 2 : 1);
  static constexpr int SS1min = (ST == 2 && !kFwd) ? 3 : 2;
  static constexpr int base0 = outerBytes + SS0min * g0Bytes + SS1min * g1Bytes;
  static_assert(base0 <= tileBudget, "shared memory budget exceeded");
  // With one TMEM stage (two-phase schedule) the S-like GEMMs of block i+1 are issued before the last
  // output GEMMs of block i release their g1 stage, so a third g1 stage is worth more than a second g0
  // stage; with two TMEM stages it is the other way round.
  static constexpr bool g1First = ST == 1;
  static constexpr int SS1a = (g1First && SS1min < 3 && base0 + g1Bytes <= tileBudget) ? 3 : SS1min;
  static constexpr int base1 = outerBytes + SS0min * g0Bytes + SS1a * g1Bytes;
  static constexpr int SS0 = (nG0 > 0 && SS0min < 2 && base1 + g0Bytes <= tileBudget) ? 2 : SS0min;
  static constexpr int base2 = outerBytes + SS0 * g0Bytes + SS1a * g1Bytes;
  static constexpr int SS1 = (SS1a < 3 && base2 + g1Bytes <= tileBudget) ? 3 : SS1a;
  static constexpr int tileBytes = outerBytes + SS0 * g0Bytes + SS1 * g1Bytes;
  static constexpr int smemBytes = tileBytes + miscBytes;
};

// Barrier slots inside the misc area.
enum {
  BAR_OUTER = 0,
  BAR_FULL = 1,     // [group][stage] -> 1 + g*3 + s
  BAR_EMPTY = 7,    // 7 + g*3 + s
  BAR_S_FULL = 13,  // 13 + st
  BAR_P_FULL = 15,  // 15 + st
  BAR_PV_DONE = 17,
  BAR_ACC_DONE = 18,
  BAR_ST_EMPTY = 19,  // 19 + buffer: DKV statistics buffer released by the pointwise warps
  BAR_A_READY = 21,   // owner operands copied into TMEM
  BAR_S2_FULL = 22,   // 22 + phase: two-phase kernels, second tile of the pair (S_dot / dP_dot) complete
  BAR_P_HALF = 24,    // two-phase kernels: dS written (dS_dot still to come)
  BAR_COUNT = 25
};

template <typename T> __device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <> __device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <> __device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
template <typename T> __device__ __forceinline__ float2 unpack2(uint32_t u);
template <> __device__ __forceinline__ float2 unpack2<__nv_bfloat16>(uint32_t u) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162*>(&u));
}
template <> __device__ __forceinline__ float2 unpack2<__half>(uint32_t u) {
  return __half22float2(*reinterpret_cast<__half2*>(&u));
}

// Row pointer (this thread's own row) into a sequence tensor, or nullptr.
template <typename T>
__device__ __forceinline__ T* row_ptr(const SeqT& t, int head, int64_t row) {
  return t.ptr ? reinterpret_cast<T*>(t.ptr) + (int64_t)head * t.head_stride + row * t.row_stride : nullptr;
}
// 32 consecutive 16-bit elements (64 bytes) of a row.
template <typename T>
__device__ __forceinline__ void store32(T* rowp, int col0, const float (&v)[32]) {
  uint4* dst = reinterpret_cast<uint4*>(rowp + col0);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 u;
    u.x = pack2<T>(v[8 * i + 0], v[8 * i + 1]);
    u.y = pack2<T>(v[8 * i + 2], v[8 * i + 3]);
    u.z = pack2<T>(v[8 * i + 4], v[8 * i + 5]);
    u.w = pack2<T>(v[8 * i + 6], v[8 * i + 7]);
    dst[i] = u;
  }
}
// 32 consecutive float32 elements (128 bytes) of a row: v (+ what `srcp` holds, if given) -> dstp.
// dstp may point into another GPU's memory (plain 16-byte stores).
__device__ __forceinline__ void store32_f32(float* dstp, const float* srcp, int col0, const float (&v)[32]) {
  float4* dst = reinterpret_cast<float4*>(dstp + col0);
  const float4* src = reinterpret_cast<const float4*>(srcp + col0);
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    float4 u = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
    if (srcp) {
      const float4 o = src[i];
      u.x += o.x; u.y += o.y; u.z += o.z; u.w += o.w;
    }
    dst[i] = u;
  }
}
template <typename T>
__device__ __forceinline__ void load32(const T* rowp, int col0, float (&v)[32]) {
  const uint4* src = reinterpret_cast<const uint4*>(rowp + col0);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    uint4 u = src[i];
    float2 a = unpack2<T>(u.x), b = unpack2<T>(u.y), c = unpack2<T>(u.z), d = unpack2<T>(u.w);
    v[8 * i + 0] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = b.x; v[8 * i + 3] = b.y;
    v[8 * i + 4] = c.x; v[8 * i + 5] = c.y; v[8 * i + 6] = d.x; v[8 * i + 7] = d.y;
  }
}

// The MMA-issuing thread is the serial resource of the CTA: descriptors are built once per operand
// and only their start-address field (low word, units of 16 bytes) is advanced per instruction.
__device__ __forceinline__ uint32_t kmajor_desc(uint32_t saddr) { return smem_desc_lo(saddr, 16); }
// MN-major B operand: `chunk_bytes` = distance between the two 64-column halves of a head_dim-128 tile
__device__ __forceinline__ uint32_t mnmajor_desc(uint32_t saddr, uint32_t chunk_bytes) { return smem_desc_lo(saddr, chunk_bytes); }

// D[tmem: 128 x N] (+)= A[smem, K-major, BM x D] * B[smem, K-major, N x D]^T. BCH = bytes between the
// 64-element head_dim chunks of B (streamed tiles of a group are interleaved chunk by chunk, so a
// pair {X, X_dot} is also one 128-row operand).
template <int D, int BCH>
__device__ __forceinline__ void gemm_ss(uint32_t d_tmem, uint32_t adesc, uint32_t bdesc, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int chunk = kk >> 2, sub = kk & 3;
    mma_ss(d_tmem, adesc + (uint32_t)((chunk * (BM * 128) + sub * 32) >> 4), bdesc + (uint32_t)((chunk * BCH + sub * 32) >> 4),
           idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}
// D[tmem: 128 x D] (+)= A[tmem: 128 x BN, 16-bit] * B[smem, MN-major: BN rows (K) x D (N)]
// The 8 packed 16-bit columns of K-step kk sit at column 16*kk of the fp32 tile they replace.
template <int D>
__device__ __forceinline__ void gemm_ts(uint32_t d_tmem, uint32_t a_tmem, uint32_t bdesc, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk)
    mma_ts(d_tmem, a_tmem + kk * 16, bdesc + (uint32_t)((kk * 16 * 128) >> 4), idesc, (accumulate || kk > 0) ? 1u : 0u);
}
// gemm_ss with the owner operand read from TMEM: D[tmem: 128 x N] (+)= A[tmem: 128 x D, 16-bit, K-step kk
// at column 8*kk] * B[smem, K-major, N x D]^T
template <int D, int BCH>
__device__ __forceinline__ void gemm_ts_kmajor(uint32_t d_tmem, uint32_t a_tmem, uint32_t bdesc, uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int kk = 0; kk < D / 16; ++kk) {
    const int chunk = kk >> 2, sub = kk & 3;
    mma_ts(d_tmem, a_tmem + kk * 8, bdesc + (uint32_t)((chunk * BCH + sub * 32) >> 4), idesc, (accumulate || kk > 0) ? 1u : 0u);
  }
}

// ------------------------------------------------------------------------------------------------
// One CTA = one 128-row owner tile of one (batch, head). Its state and the code of its warp roles
// live in one struct, one member function per role:
//
//   setup()          every thread    tile geometry, mbarriers, TMEM allocation
//   producer()       warp 0 (*)      TMA loads: the owner tiles once, then the streamed stages
//   issuer()         warp 1 (*)      every tcgen05.mma (pipelined or two-phase schedule)
//   stats_stager()   warp 2          DKV only: per-row statistics of the streamed query rows
//   pointwise()      warps 4-11      softmax / dS arithmetic between the GEMMs (pw_*_block), epilogue_*
//   teardown()       every thread    abort report, TMEM release
//                                    (*) one elected lane
//
// Every member function is force-inlined into the kernel, so the members are plain registers (or
// constants) of the calling thread; members that belong to one role are dead in the others.
// ------------------------------------------------------------------------------------------------
//
// HOOK = true is a test instantiation: its bounded waits use the budget passed in Params and its
// producer leaves out the loads of streamed block 1, so that a wait runs out and the CTA takes the
// abort path (status word set, nothing issued afterwards, resources released) without any fault.
template <typename T, int KIND, int D, bool TANGENT, bool FIRST, bool DOD, bool HOOK = false>
struct TcCta {
  using C = Cfg<KIND, D, TANGENT, FIRST, DOD>;
  static constexpr bool kFwd = KIND == KIND_FWD, kDq = KIND == KIND_DQ, kDkv = KIND == KIND_DKV;
  static constexpr int ST = C::ST, SS0 = C::SS0, SS1 = C::SS1, nS = C::nS;
  static constexpr int SS0d = SS0 > 0 ? SS0 : 1;
  static constexpr int fmt = sizeof(T) == 2 && std::is_same<T, __nv_bfloat16>::value ? 1 : 0;
  static constexpr uint32_t idesc_s = make_idesc(fmt, BM, BN, 0, 0);
  static constexpr uint32_t idesc_o = make_idesc(fmt, BM, D, 0, 1);
  static constexpr uint32_t idesc_s2 = make_idesc(fmt, BM, 2 * BN, 0, 0);  // a pair {X, X_dot} as one 128-row B operand
  // S-like tile slots. DQ with tangents keeps (S, S_dot) and (dP, dP_dot) adjacent so that each pair
  // comes out of one N=128 MMA chain.
  static constexpr int tS = 0, tDP = TANGENT ? 2 : 1, tSD = 1, tDPD = 3;
  // Backward kernels with tangents run each block in two phases (see issuer()).
  static constexpr bool kSplit = !kFwd && TANGENT;
  // Registers move from the role warps to the pointwise warpgroups in the forward and first-order kernels
  // (jvp_fwd 2.61 -> 2.45 ms, first-order dK/dV 2.02 -> 1.96 ms at S8192 D128). Not in the two-phase
  // kernels: their MMA-issuing thread is the serial resource and generated slower code under any smaller
  // budget (hvp_dkv_dot 3.85 -> 4.04 ms at 136 registers without a spill, spills below 128; with 32-bit
  // descriptor words the same hand-over no longer spills but is still 3.5 % slower there and flat in hvp_dq).
  static constexpr bool kRealloc = !kSplit;
  static constexpr int ch0 = (C::nG0 > 0 ? C::nG0 : 1) * BN * 128, ch1 = C::nG1 * BN * 128;  // chunk strides of the streamed groups
  static constexpr int HC = BN / NWG;  // streamed columns per pointwise warpgroup
  // Two-phase kernels: dP_dot takes a GEMM of its own (otherwise it comes out of the pair GEMM with dP)
  static constexpr bool hasSB2 = kDkv || DOD;
  // hand S over before S_dot is complete / hand dS over before dS_dot is computed (see issuer())
  // (dQ at head_dim 64 is bound by the pointwise warps, where the extra waits cost more than the
  // shorter round trips gain: 4.4 -> 5.2 ms on non-causal B8 H32 S4096; it keeps the one-step hand-over.)
  static constexpr bool kSplitA = kDkv || (DOD && D == 128), kHalfB = hasSB2 && (kDkv || D == 128);
  // exponentials partly on the FMA pipe: head_dim 64 (every kernel there is bound by the pointwise warps)
  // and the first-order dK/dV kernel
  static constexpr bool kPoly = kPolyPeriod > 0 && (D == 64 || (kDkv && !TANGENT));
  __device__ __forceinline__ static float2 exp2_pair(float2 e, int pair, bool no_mask) {
    if (kPoly && no_mask && (pair % (kPolyPeriod > 0 ? kPolyPeriod : 1)) == (kPolyPeriod - 1)) return ex2_poly2(e);
    return make_float2(ex2(e.x), ex2(e.y));
  }
  static_assert(!kDkv || kSplitA, "the DKV statistics warp signals on the barrier of the first S tile");

  // ---- CTA state (same value in every thread) ----
  const TmaMaps& maps;
  const Params& p;
  uint8_t* const smem;
  uint32_t sbase, bar0, tmem_base;
  volatile int* abort_flag;
  // DKV: per streamed query row, four statistics as separate arrays of NEGATED values
  // ([0] -lse*log2e, [1] -dpsum, [2] -z1, [3] -ddot) so that pairs of columns load as one float2
  float* stats_base;  // [2 buffers][4][BN]
  int warp, lane, head, G, off, own_len, r0;
  // Range of streamed blocks. DKV iterates over blocks x the query heads of the kv head; when the tile is
  // shared by a cluster (p.split > 1) this CTA takes iterations [it_base, it_base + n_it) of the n_total.
  int blk_begin, blk_count, n_it, n_total, it_base, part;
  SeqInfo si;
  bool prof;
  long long t_kernel0;

  // ---- pointwise-thread state ----
  int wg, row, cb, orow;  // warpgroup, owner row within the tile (= TMEM lane), first streamed column, row in the sequence
  uint32_t lane_off;      // this warp's TMEM lane quadrant
  bool row_ok;
  float scale2;
  int64_t srow;           // statistics index (FWD / DQ)
  float* xchg;            // FWD: [2 parities][NWG warpgroups][128 rows]
  float m_used, l_sum, z_sum;   // FWD (l_sum, z_sum: this warpgroup's columns only)
  float lse2, dps, z1v, ddt;    // LSE-known FWD and DQ
  long long pw_wait, pw_work, pw_ld0, pw_st;

  __device__ __forceinline__ TcCta(const TmaMaps& maps_, const Params& p_, uint8_t* smem_) : maps(maps_), p(p_), smem(smem_) {}

  // ---- addresses ----
  __device__ __forceinline__ uint32_t bar(int i) const { return bar0 + 8 * i; }
  __device__ __forceinline__ uint32_t outer_addr(int o) const { return sbase + o * C::outerTile; }
  // streamed operand i of group g, stage s: its head_dim chunk c is at + c * (group size * BN * 128)
  __device__ __forceinline__ uint32_t inner_addr(int g, int s, int i) const {
    return sbase + C::outerBytes + (g == 0 ? s * C::g0Bytes : SS0 * C::g0Bytes + s * C::g1Bytes) + i * (BN * 128);
  }
  __device__ __forceinline__ uint32_t acc_addr(int a) const { return tmem_base + a * D; }
  __device__ __forceinline__ uint32_t stile_addr(int st, int t) const { return tmem_base + C::accCols + (st * nS + t) * BN; }
  __device__ __forceinline__ uint32_t aop_addr(int j) const { return tmem_base + C::aBase + j * C::aCols; }

  // S-like GEMM with owner operand O (descriptor `adesc`) as A: from TMEM when it was staged there.
  template <int O, int BCH>
  __device__ __forceinline__ void s_gemm(uint32_t dst, uint32_t adesc, uint32_t bdesc, uint32_t idesc, bool accumulate) const {
    constexpr int slot = C::aSlot(O);
    if constexpr (slot >= 0) gemm_ts_kmajor<D, BCH>(dst, aop_addr(slot), bdesc, idesc, accumulate);
    else gemm_ss<D, BCH>(dst, adesc, bdesc, idesc, accumulate);
  }

  // Bounded wait of one thread. False = the wait (or an earlier one in this CTA) gave up: the caller
  // stops issuing work and heads for teardown.
  __device__ __forceinline__ bool wait1(int barrier, int parity) const {
    return mbar_wait(bar(barrier), parity, abort_flag, HOOK ? p.wait_budget : kWaitBudgetCycles);
  }
  // One lane per warp polls (mbarrier polling is shared-memory traffic that competes with the MMA
  // operand fetches); the rest of the warp waits at the warp barrier.
  __device__ __forceinline__ void warp_wait(int barrier, int parity) const {
    if (lane == 0) wait1(barrier, parity);
    __syncwarp();
  }
  __device__ __forceinline__ bool aborted() const { return *abort_flag != 0; }

  // First iteration of cluster part j (parts are contiguous, near-equal slices of the n_total iterations).
  __device__ __forceinline__ int part_begin(int j) const { return (int)(((long long)n_total * j) / p.split); }

  // ================================================= set-up =================================================
  // Returns false when this CTA has nothing to do (or cannot run); the whole CTA then leaves together.
  __device__ __forceinline__ bool setup() {
    // The swizzled tiles need 1024-byte alignment. Dynamic shared memory starts at a 1024-byte boundary
    // when the kernel has no static shared memory; if that ever fails to hold the kernel reports it.
    if (threadIdx.x == 0) FB_TRACE(0);
    sbase = smem_u32(smem);
    if (sbase & 1023u) {
      if (threadIdx.x == 0) atomicOr(p.status, 0x100);
      return false;
    }
    // A CTA of this launch (or of an earlier one whose status the host has not collected yet) already gave
    // up on a wait: do not start. The results of such a launch are void anyway, and a lost signal then
    // costs one wait budget per launch instead of one per wave of CTAs.
    // (Not when a cluster shares the tile: its CTAs read each other's shared memory and must stay together.)
    if (p.split == 1 && *reinterpret_cast<volatile int*>(p.status) != 0) return false;
    bar0 = sbase + C::tileBytes;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(smem + C::tileBytes + 8 * BAR_COUNT);
    abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    stats_base = reinterpret_cast<float*>(smem + C::tileBytes + 256);

    warp = threadIdx.x >> 5;
    lane = threadIdx.x & 31;
    // 1-D grid. The CTAs of a cluster (DKV with p.split > 1: consecutive block indices) share one owner
    // tile. The (head, batch) pairs are taken in groups of p.group; inside a group the tile index is the
    // slowest coordinate, so that under causal masking the heaviest tiles of every pair of the group are
    // scheduled first and its lightest ones last (longest-processing-time-first; the reference's K1 uses
    // an LPT scheduler for the same reason, jvp_fwd_sm90.py:236-264). p.group = 1 walks all tiles of one
    // pair before the next pair (best locality in L2, no balancing); p.group = all pairs balances the
    // whole launch.
    uint32_t lin = blockIdx.x;
    part = 0;
    if (kDkv) { part = (int)(lin % (uint32_t)p.split); lin /= (uint32_t)p.split; }
    const uint32_t nh = kDkv ? p.Hkv : p.Hq;
    const uint32_t pairs = nh * (uint32_t)p.B, gsz = (uint32_t)p.group;
    const uint32_t grp = lin / (gsz * (uint32_t)p.ntiles);
    const uint32_t rem = lin - grp * gsz * (uint32_t)p.ntiles;
    const uint32_t in_grp = min(gsz, pairs - grp * gsz);  // the last group may be smaller
    const int tidx = (int)(rem / in_grp);
    const uint32_t pair = grp * gsz + rem % in_grp;
    head = (int)(pair % nh);
    const int b = (int)(pair / nh);
    G = p.Hq / p.Hkv;
    // Varlen: the sequence bounds are read from global memory, which the previous kernel in the stream may
    // have written (a caller computing cu_seqlens on the device): synchronise with it first. Dense problems
    // read nothing here and synchronise at the end of set-up instead.
    if (p.cu_q) grid_dependency_wait();
    si = seq_info(p, b);
    own_len = kDkv ? si.sk : si.sq;
    // Causal: query tiles with the largest row index see the most keys, key tiles with the smallest one
    // the most queries; those go first.
    const int tile = (!kDkv && p.causal) ? p.ntiles - 1 - tidx : tidx;
    r0 = tile * BM;
    if (r0 >= own_len) return false;  // (the same decision in every CTA of a cluster)
    // Causal offset (key j visible to query i iff j <= i + off). A query tile lies inside one query segment
    // (the break is a multiple of BM), so its offset is fixed here; a key tile streams query blocks of both
    // segments and takes the offset per block (pointwise()).
    // (With key segments it is the other way round: a key tile's offset is fixed, and only the dK/dV kernels run.)
    off = kDkv ? si.sk - si.sq + (p.seg_keys ? seg_shift_of(p, r0) : 0) : causal_off(p, si, r0);

    blk_begin = 0;
    blk_count = 0;
    it_base = 0;
    if (!kDkv) {
      int kmax = si.sk;
      if (p.causal) kmax = max(0, min(si.sk, r0 + BM + off));
      blk_count = (kmax + BN - 1) / BN;
      n_total = blk_count;
      n_it = n_total;
    } else {
      const int nmb = (si.sq + BN - 1) / BN;
      if (p.causal) blk_begin = first_query_of_key(p, si, r0) / BN;
      blk_count = max(0, nmb - blk_begin);
      n_total = blk_count * G;
      it_base = part_begin(part);
      n_it = part_begin(part + 1) - it_base;
    }

    if (threadIdx.x == 0) {
      for (int i = 0; i < BAR_COUNT; ++i) {
        uint32_t count = 1u;
        if ((i >= BAR_P_FULL && i < BAR_P_FULL + 2) || (i >= BAR_ST_EMPTY && i < BAR_ST_EMPTY + 2) || i == BAR_A_READY || i == BAR_P_HALF) count = NWG * 4;  // one arrival per pointwise warp
        // DKV: the S-like tiles a block's pointwise work starts from are complete when the MMAs have
        // committed AND the statistics warp has staged the block's row statistics (one wait for both)
        if (kDkv && (i == BAR_S_FULL || (i == BAR_S_FULL + 1 && !kSplit))) count = 2u;
        mbar_init(bar(i), count);
      }
      *abort_flag = 0;
      fence_barrier_init();
      // The owner tiles are requested here, by the thread that has just initialised their barrier, so that they
      // travel while the rest of the set-up (TMEM allocation, the CTA-wide barrier) runs: 1-1.4 us of a 4-5 us
      // prologue per CTA, which counts where CTAs are short (S = 2048: 20-40 us each). They are global reads, so
      // the dependency on the previous kernel in the stream comes first (dense problems; varlen waited above).
      if (n_it > 0) {
        grid_dependency_wait();
        request_owner_tiles();
      }
    }
    if (warp == 1) {
      tmem_alloc(smem_u32(tmem_slot), C::tmemCols);
      tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    tmem_base = *tmem_slot;
#ifdef FB_PROFILE
    if (threadIdx.x == 0) {
      FB_TRACE(1);
      unsigned smid;
      asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
      if (blockIdx.x < kTraceCtas) g_trace_meta[blockIdx.x] = (unsigned long long)smid | ((unsigned long long)n_it << 32);
    }
#endif
    prof = kProfile && (p.debug & 2) && blockIdx.x == 0;
    t_kernel0 = prof ? clock64() : 0;
    // Programmatic dependent launch: everything above touches no global memory another kernel writes,
    // so it may overlap the tail of the previous kernel in the stream. From here on this grid reads that
    // kernel's results (and overwrites buffers it may still be reading).
    grid_launch_dependents();
    grid_dependency_wait();
    return true;
  }

  __device__ __forceinline__ void run_role() {
    if (warp < kRoleThreads / 32) {
      if constexpr (kRealloc) reg_dealloc<kRoleRegs>();
      if (n_it > 0 && warp == 0) {
        if (elect_one()) producer();
      } else if (n_it > 0 && warp == 1) {
        if (elect_one()) issuer();
      } else if (warp == kStatsWarp) {
        if constexpr (kDkv) stats_stager();
      }
    } else {
      if constexpr (kRealloc) reg_alloc<kPwRegs>();
      pointwise();
    }
  }

  // =============================================== TMA producer ===============================================
  // Loads streamed group g (its nG tiles, head_dim chunk by chunk) of block `it` into its next stage.
  // Returns false when the wait for a free stage gave up.
  template <int GRP>
  __device__ __forceinline__ bool load_group(int it, int in_row, int in_head, long long& pt_wait) {
    constexpr int g0_ids[3][2] = {{T_K, T_KD}, {T_V, T_VD}, {T_DO, T_DOD}};
    constexpr int g1_ids[3][2] = {{T_V, T_VD}, {T_K, T_KD}, {T_Q, (kDkv && TANGENT) ? T_QD : T_DO}};
    constexpr int nG = GRP == 0 ? C::nG0 : C::nG1;
    constexpr int SS = GRP == 0 ? SS0d : SS1;
    constexpr int bytes = GRP == 0 ? C::g0Bytes : C::g1Bytes;
    constexpr int ch = GRP == 0 ? ch0 : ch1;
    if (nG == 0) return true;
    const int s = it % SS, k = it / SS;
    const long long tw = prof ? clock64() : 0;
    if (!wait1(BAR_EMPTY + 3 * GRP + s, (k & 1) ^ 1)) return false;
    if (prof) pt_wait += clock64() - tw;
    if (HOOK && it == 1) return true;  // test instantiation: this stage never fills, the issuer's wait runs out
    mbar_expect_tx(bar(BAR_FULL + 3 * GRP + s), bytes);
#pragma unroll
    for (int i = 0; i < nG; ++i)
#pragma unroll
      for (int c = 0; c < D / 64; ++c)
        tma_load_3d(inner_addr(GRP, s, i) + c * ch, &maps.m[GRP == 0 ? g0_ids[KIND][i] : g1_ids[KIND][i]], bar(BAR_FULL + 3 * GRP + s),
                    c * 64, in_row, in_head);
    return true;
  }

  // The CTA's owner tiles (one thread, once, from setup()).
  __device__ __forceinline__ void request_owner_tiles() {
    constexpr int outer_ids[3][4] = {{T_Q, T_QD, 0, 0}, {T_Q, T_DO, T_QD, T_DOD}, {T_K, T_V, T_KD, T_VD}};
    for (int i = 0; i < T_COUNT; ++i) prefetch_tmap(&maps.m[i]);
    const int own_row = (kDkv ? si.k0 : si.q0) + r0;
    mbar_expect_tx(bar(BAR_OUTER), C::outerBytes);
#pragma unroll
    for (int o = 0; o < C::nOuter; ++o)
#pragma unroll
      for (int c = 0; c < D / 64; ++c)
        tma_load_3d(outer_addr(o) + c * (BM * 128), &maps.m[outer_ids[KIND][o]], bar(BAR_OUTER), c * 64, own_row, head);
  }

  __device__ __forceinline__ void producer() {
    long long pt_wait = 0;
    for (int it = 0; it < n_it; ++it) {
      int in_head, in_row;
      if (!kDkv) {
        in_head = head / G;
        in_row = si.k0 + it * BN;
      } else {
        const int gi = it_base + it, g = gi / blk_count, mb = blk_begin + (gi - g * blk_count);
        in_head = head * G + g;
        in_row = si.q0 + mb * BN;
      }
      // the group whose buffer frees first goes first; nothing more is loaded once a wait has given up
      if (kFwd) {
        if (!load_group<0>(it, in_row, in_head, pt_wait) || !load_group<1>(it, in_row, in_head, pt_wait)) break;
      } else {
        if (!load_group<1>(it, in_row, in_head, pt_wait) || !load_group<0>(it, in_row, in_head, pt_wait)) break;
      }
    }
    if (prof) g_prof[7] = pt_wait;
  }

  // ================================================ MMA issuer ================================================
  // One function with local helper lambdas. (Written as separate member functions the same code made
  // the issuing thread about 140 cycles per block slower in the output GEMMs, which the forward
  // kernels, bound by this thread and the tensor pipe, showed as a 5% longer run.)
  __device__ __forceinline__ void issuer() {
    // `live` turns false when a bounded wait gives up; no MMA is issued after that.
    bool live = wait1(BAR_OUTER, 0);
    if constexpr (C::nATmem > 0) live = live && wait1(BAR_A_READY, 0);
    if (!live) return;
    FB_TRACE(2);
    tc_fence_after();
    long long pr_in = 0, pr_p = 0, pr_is = 0;
    // Operand descriptors, built once: ka = owner-side tiles (K-major A); k0/m0 and k1/m1 = streamed
    // tiles of groups g0 / g1 (stage 0) as K-major B (S-like GEMMs) and MN-major B (output GEMMs).
    uint32_t ka[4], k0[2], m0[2], k1[2], m1[2];
#pragma unroll
    for (int i = 0; i < 4; ++i) ka[i] = kmajor_desc(outer_addr(i < C::nOuter ? i : 0));
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      k0[i] = kmajor_desc(inner_addr(0, 0, i < C::nG0 ? i : 0));
      m0[i] = mnmajor_desc(inner_addr(0, 0, i < C::nG0 ? i : 0), ch0);
      k1[i] = kmajor_desc(inner_addr(1, 0, i < C::nG1 ? i : 0));
      m1[i] = mnmajor_desc(inner_addr(1, 0, i < C::nG1 ? i : 0), ch1);
    }
    auto wait_full = [&](int g, int it) {
      const int ss = g == 0 ? SS0d : SS1;
      const long long tw = prof ? clock64() : 0;
      live = wait1(BAR_FULL + 3 * g + it % ss, (it / ss) & 1) && live;
      if (prof) pr_in += clock64() - tw;
    };
    // S-like GEMMs of block `it` into TMEM stage it % ST.
    auto issue_s = [&](int it) {
      const int s0 = it % SS0d, s1 = it % SS1, st = it % ST;
      const uint32_t o0 = (uint32_t)((s0 * C::g0Bytes) >> 4), o1 = (uint32_t)((s1 * C::g1Bytes) >> 4);
      const long long ts0 = prof ? clock64() : 0;
      if (kFwd) {
        wait_full(0, it);
        if (!live) return;
        if (TANGENT) {
          s_gemm<0, ch0>(stile_addr(st, 0), ka[0], k0[0] + o0, idesc_s2, false);  // [S | Q K_dot^T] = Q [K | K_dot]^T
          s_gemm<1, ch0>(stile_addr(st, 1), ka[1], k0[0] + o0, idesc_s, true);    // S_dot += Q_dot K^T
        } else {
          s_gemm<0, ch0>(stile_addr(st, 0), ka[0], k0[0] + o0, idesc_s, false);   // S = Q K^T
        }
        mma_commit(bar(BAR_EMPTY + s0));  // K / K_dot are only read by these GEMMs
      } else if (kDq) {
        // first-order dQ (kernels with tangents take the two-phase schedule): owner {Q, dO}; g1 = {K}; g0 = {V}
        wait_full(1, it);
        if (!live) return;
        s_gemm<0, ch1>(stile_addr(st, tS), ka[0], k1[0] + o1, idesc_s, false);   // S = Q K^T
        wait_full(0, it);
        if (!live) return;
        s_gemm<1, ch0>(stile_addr(st, tDP), ka[1], k0[0] + o0, idesc_s, false);  // dP = dO V^T
        mma_commit(bar(BAR_EMPTY + s0));  // V is only read by this GEMM
      } else {
        // first-order dK/dV: owner {K, V}; g1 = {Q, dO}
        wait_full(1, it);
        if (!live) return;
        gemm_ss<D, ch1>(stile_addr(st, 0), ka[0], k1[0] + o1, idesc_s, false);  // S^T = K Q^T
        gemm_ss<D, ch1>(stile_addr(st, 1), ka[1], k1[1] + o1, idesc_s, false);  // dP^T = V dO^T
      }
      mma_commit(bar(BAR_S_FULL + st));
      if (prof) pr_is += clock64() - ts0;
    };
    // Output GEMMs of block `it`: A operands are the 16-bit tiles the pointwise warps left in TMEM.
    auto issue_out = [&](int it) {
      const int s0 = it % SS0d, s1 = it % SS1, st = it % ST;
      const uint32_t o0 = (uint32_t)((s0 * C::g0Bytes) >> 4), o1 = (uint32_t)((s1 * C::g1Bytes) >> 4);
      const bool accu = it > 0;
      {
        const long long tw = prof ? clock64() : 0;
        live = wait1(BAR_P_FULL + st, (it / ST) & 1) && live;
        if (prof) pr_p += clock64() - tw;
      }
      if (!live) return;
      tc_fence_after();
      if (kFwd) {
        wait_full(1, it);
        if (!live) return;
        constexpr int aOd = FIRST ? 1 : 0;
        if (FIRST) gemm_ts<D>(acc_addr(0), stile_addr(st, 0), m1[0] + o1, idesc_o, accu);  // O += P V
        if (TANGENT) {
          gemm_ts<D>(acc_addr(aOd), stile_addr(st, 1), m1[0] + o1, idesc_o, accu);  // O_dot += W V
          gemm_ts<D>(acc_addr(aOd), stile_addr(st, 0), m1[1] + o1, idesc_o, true);  //        + P V_dot
        }
        mma_commit(bar(BAR_EMPTY + 3 + s1));
        mma_commit(bar(BAR_PV_DONE));
      } else if (kDq) {
        gemm_ts<D>(acc_addr(0), stile_addr(st, 0), m1[0] + o1, idesc_o, accu);  // dQ += dS K
        mma_commit(bar(BAR_EMPTY + 3 + s1));
      } else {
        gemm_ts<D>(acc_addr(0), stile_addr(st, 1), m1[0] + o1, idesc_o, accu);  // dK += dS^T Q
        gemm_ts<D>(acc_addr(1), stile_addr(st, 0), m1[1] + o1, idesc_o, accu);  // dV += P^T dO
        mma_commit(bar(BAR_EMPTY + 3 + s1));
      }
    };
    const long long tm0 = prof ? clock64() : 0;
    if constexpr (kSplit) {
      // Two-phase schedule for the backward kernels with tangents (one TMEM stage of four tiles):
      //   phase A tiles (S, S_dot) and phase B tiles (dP, dP_dot) are produced and consumed separately, so
      //   the pointwise work on one pair overlaps the GEMMs of the other:
      //     SA(i+1) runs under pointwise B(i);  outB(i) and SB(i+1) run under pointwise A(i+1).
      //   DKV additionally issues its dV_dot GEMMs (operands P^T, P_dot^T from phase A) before SA(i+1)
      //   overwrites those tiles.
      //   Each phase is handed over in two steps to shorten the MMA -> pointwise -> MMA round trips that
      //   bound the loop: the first tile of a pair (S, dP) is committed before the GEMM that completes
      //   the second one (S_dot, dP_dot) is issued, so the exp / dS arithmetic starts under that GEMM;
      //   and the output GEMMs that only need dS are issued (BAR_P_HALF) while dS_dot is still being
      //   computed.
      constexpr bool pairB = kDq || DOD;    // g0 holds a pair {X, X_dot}
      auto wait_pw = [&](int barrier, int it) {
        const long long tw = prof ? clock64() : 0;
        live = wait1(barrier, it & 1) && live;
        if (prof) pr_p += clock64() - tw;
        tc_fence_after();
      };
      auto issue_sa = [&](int it) {
        const uint32_t o1 = (uint32_t)(((it % SS1) * C::g1Bytes) >> 4);
        wait_full(1, it);
        if (!live) return;
        s_gemm<0, ch1>(stile_addr(0, tS), ka[0], k1[0] + o1, idesc_s2, false);  // [S | A Bd^T] = A [B | Bd]^T
        if (kSplitA) mma_commit(bar(BAR_S_FULL + 0));                           // S complete
        s_gemm<2, ch1>(stile_addr(0, tSD), ka[2], k1[0] + o1, idesc_s, true);   // S_dot += Ad B^T
        mma_commit(bar(BAR_S2_FULL + 0));
      };
      auto issue_sb = [&](int it) {
        const int s0 = it % SS0d;
        const uint32_t o0 = (uint32_t)((s0 * C::g0Bytes) >> 4);
        wait_full(0, it);
        if (!live) return;
        if (pairB) s_gemm<1, ch0>(stile_addr(0, tDP), ka[1], k0[0] + o0, idesc_s2, false);  // [dP | A Xd^T]
        else s_gemm<1, ch0>(stile_addr(0, tDP), ka[1], k0[0] + o0, idesc_s, false);         // dP
        mma_commit(bar(BAR_S_FULL + 1));                                                    // dP complete
        if (hasSB2) {
          s_gemm<3, ch0>(stile_addr(0, tDPD), ka[3], k0[0] + o0, idesc_s, pairB);  // dP_dot (+)= Ad X^T
          mma_commit(bar(BAR_S2_FULL + 1));
        }
        if (kDq) mma_commit(bar(BAR_EMPTY + s0));  // V / V_dot are only read by these GEMMs
      };
      issue_sa(0);
      issue_sb(0);
      FB_TRACE(3);
      for (int it = 0; it < n_it; ++it) {
        const int s0 = it % SS0d, s1 = it % SS1;
        const uint32_t o0 = (uint32_t)((s0 * C::g0Bytes) >> 4), o1 = (uint32_t)((s1 * C::g1Bytes) >> 4);
        const bool accu = it > 0;
        wait_pw(BAR_P_FULL + 0, it);  // phase A done: S / S_dot tiles read (DKV: P^T, P_dot^T written)
        if (!live) break;
        constexpr int aKd = (kDkv && FIRST) ? 2 : 0;  // DKV accumulators: {dK, dV}? then {dK_dot, dV_dot}
        constexpr int aQd = FIRST ? 1 : 0;            // DQ accumulators: {dQ}? then {dQ_dot}
        if (kDkv) {
          if (FIRST) gemm_ts<D>(acc_addr(1), stile_addr(0, tS), m0[0] + o0, idesc_o, accu);      // dV += P^T dO
          gemm_ts<D>(acc_addr(aKd + 1), stile_addr(0, tSD), m0[0] + o0, idesc_o, accu);          // dV_dot += P_dot^T dO
          if (DOD) gemm_ts<D>(acc_addr(aKd + 1), stile_addr(0, tS), m0[1] + o0, idesc_o, true);  //        + P^T dO_dot
          mma_commit(bar(BAR_EMPTY + s0));
        }
        if (it + 1 < n_it) issue_sa(it + 1);
        wait_pw(kHalfB ? BAR_P_HALF : BAR_P_FULL + 1, it);  // dS written over the dP tile
        if (!live) break;
        if (kDq) {
          if (FIRST) gemm_ts<D>(acc_addr(0), stile_addr(0, tDP), m1[0] + o1, idesc_o, accu);  // dQ += dS K
          gemm_ts<D>(acc_addr(aQd), stile_addr(0, tDP), m1[1] + o1, idesc_o, accu);          // dQ_dot += dS K_dot
        } else {
          if (FIRST) gemm_ts<D>(acc_addr(0), stile_addr(0, tDP), m1[0] + o1, idesc_o, accu);  // dK += dS^T Q
          gemm_ts<D>(acc_addr(aKd), stile_addr(0, tDP), m1[1] + o1, idesc_o, accu);          // dK_dot += dS^T Q_dot
        }
        if (kHalfB) wait_pw(BAR_P_FULL + 1, it);  // dS_dot written over the dP_dot tile
        if (!live) break;
        gemm_ts<D>(acc_addr(kDq ? aQd : aKd), stile_addr(0, tDPD), m1[0] + o1, idesc_o, true);  // dQ_dot += dS_dot K / dK_dot += dS_dot^T Q
        mma_commit(bar(BAR_EMPTY + 3 + s1));
        if (it + 1 < n_it) issue_sb(it + 1);
      }
    } else {
      issue_s(0);
      FB_TRACE(3);
      for (int it = 0; it < n_it && live; ++it) {
        if (ST == 2 && it + 1 < n_it) issue_s(it + 1);
        issue_out(it);
        if (ST == 1 && it + 1 < n_it) issue_s(it + 1);
      }
    }
    mma_commit(bar(BAR_ACC_DONE));
    FB_TRACE(4);
    if (prof) { g_prof[2] = pr_in; g_prof[3] = pr_p; g_prof[4] = clock64() - tm0 - pr_in - pr_p; g_prof[1] = n_it; g_prof[8] = pr_is; }
  }

  // ====================================== statistics stager (DKV only) ======================================
  // Streamed query rows of block `it`: -lse*log2e, -dpsum, -z1, -ddot into one of two shared-memory
  // buffers, handed to the pointwise warps through the block's S_FULL mbarrier (no separate wait, no
  // CTA-wide barrier in the main loop).
  // The global loads of block it+1 are issued before the wait for block it's buffer, so their latency
  // (longer than one block of pointwise work) is off the pointwise warps' critical path.
  // raw values (lse, dpsum, z1, ddot) of this lane's rows; rows past the sequence read as lse = +inf
  __device__ __forceinline__ void stats_load(int it, float4 (&v)[BN / 32]) const {
    const int gi = it_base + it, g = gi / blk_count, mb = blk_begin + (gi - g * blk_count);
#pragma unroll
    for (int r = 0; r < BN / 32; ++r) {
      const int i = mb * BN + lane + 32 * r;
      v[r] = make_float4(INFINITY, 0.f, 0.f, 0.f);
      if (i < si.sq) {
        const int64_t sr = (int64_t)(head * G + g) * p.Tq + si.q0 + i;
        v[r].x = p.lse[sr];
        v[r].y = p.dpsum[sr];
        if (TANGENT) { v[r].z = p.z1[sr]; v[r].w = p.ddot[sr]; }
      }
    }
  }
  __device__ __forceinline__ void stats_stager() {
    float4 cur[BN / 32], nxt[BN / 32];
    if (n_it > 0) stats_load(0, nxt);
    for (int it = 0; it < n_it; ++it) {
      const int sb_ = it & 1;
#pragma unroll
      for (int r = 0; r < BN / 32; ++r) cur[r] = nxt[r];
      if (it + 1 < n_it) stats_load(it + 1, nxt);
      warp_wait(BAR_ST_EMPTY + sb_, ((it >> 1) & 1) ^ 1);
      if (aborted()) break;
      float* dst = stats_base + sb_ * (4 * BN);
#pragma unroll
      for (int r = 0; r < BN / 32; ++r) {
        const int rr = lane + 32 * r;
        dst[rr] = (fabsf(cur[r].x) == INFINITY) ? -INFINITY : -cur[r].x * kLog2e;  // a fully masked row has lse = -inf
        dst[BN + rr] = -cur[r].y; dst[2 * BN + rr] = -cur[r].z; dst[3 * BN + rr] = -cur[r].w;
      }
      __syncwarp();
      if (lane == 0) {
        // Second arrival on the barrier the MMA issuer commits block `it`'s first S-like tiles to. Its
        // previous phase must be over: with two TMEM stages the wait above implies that (the pointwise
        // warps release a buffer after they consumed block it-2); with one stage wait for block it-1.
        if (ST == 1 && it > 0) wait1(BAR_S_FULL, (it - 1) & 1);
        mbar_arrive(bar(BAR_S_FULL + it % ST));
      }
    }
  }

  // ========================================= pointwise + epilogue =========================================
  // Two warpgroups (warps 4-7 and 8-11). Both cover all 128 TMEM lanes (thread -> lane = owner row);
  // warpgroup w handles streamed columns [32w, 32w+32) of every S-like tile and half of the
  // accumulator columns in the epilogue.

  // Hands a finished block to the issuer. One arrival per warp: 32 lanes arriving on one mbarrier
  // are 32 serialised shared-memory atomics.
  __device__ __forceinline__ void pw_publish(int barrier, int it, bool release_stats) {
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) {
      mbar_arrive(bar(barrier));
      if (kDkv && release_stats) mbar_arrive(bar(BAR_ST_EMPTY + (it & 1)));  // this warp is done with the block's statistics
    }
  }

  // Backward with tangents, one block, in four steps (see the issuer): A1 S -> P, A2 S_dot -> P_dot,
  // B1 dP -> dS, B2 dP_dot -> dS_dot. Packed f32x2 arithmetic throughout: two streamed columns per
  // instruction. `stats` = the block's staged statistics (DKV); [cmin, cmax] = this thread's visible
  // streamed-column range (block local), consulted when need_mask.
  __device__ __forceinline__ void pw_two_phase_block(int it, bool need_mask, int cmin, int cmax, const float* stats) {
    static_assert(NWG == 2, "the two-phase pointwise path assumes 32 streamed columns per thread");
    const long long t0 = prof ? clock64() : 0;
    long long waited = 0;
    auto wait_tiles = [&](int barrier) {
      const long long tw = prof ? clock64() : 0;
      warp_wait(barrier, it & 1);
      if (prof) waited += clock64() - tw;
      tc_fence_after();
    };
    float2 pv[HC / 2], pdv[HC / 2];  // P and P_dot of this thread's columns; after B1 pdv holds P_dot * (dP - D)
    const float2 sc2 = make_float2(scale2, scale2), sc1 = make_float2(p.scale, p.scale);
    // ---- A1: S -> P (kept in registers; DKV also needs it as an MMA operand) ----
    wait_tiles(kSplitA ? BAR_S_FULL + 0 : BAR_S2_FULL + 0);
    {
      uint32_t rs[HC];
      tmem_ld32(stile_addr(0, tS) + lane_off + cb, rs);
      tmem_ld_wait();
#pragma unroll
      for (int c2 = 0; c2 < HC / 2; ++c2) {
        const int col = cb + 2 * c2;
        float2 nl2 = make_float2(-lse2, -lse2);
        if (kDkv) nl2 = *reinterpret_cast<const float2*>(&stats[col]);
        const float2 e = __ffma2_rn(make_float2(__uint_as_float(rs[2 * c2]), __uint_as_float(rs[2 * c2 + 1])), sc2, nl2);
        float2 pe = exp2_pair(e, c2, !need_mask);
        if (need_mask) {
          if (col > cmax || col < cmin) pe.x = 0.f;
          if (col + 1 > cmax || col + 1 < cmin) pe.y = 0.f;
        }
        pv[c2] = pe;
      }
    }
    if (kDkv && (DOD || FIRST)) {
#pragma unroll
      for (int h = 0; h < HC / 16; ++h) {
        uint32_t pk[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) pk[c] = pack2<T>(pv[h * 8 + c].x, pv[h * 8 + c].y);
        tmem_st8(stile_addr(0, tS) + lane_off + cb + h * 16, pk);
      }
    }
    // ---- A2: S_dot -> P_dot ----
    if (kSplitA) wait_tiles(BAR_S2_FULL + 0);
    {
      uint32_t rsd[HC];
      tmem_ld32(stile_addr(0, tSD) + lane_off + cb, rsd);
      tmem_ld_wait();
#pragma unroll
      for (int c2 = 0; c2 < HC / 2; ++c2) {
        float2 nz = make_float2(-z1v, -z1v);
        if (kDkv) nz = *reinterpret_cast<const float2*>(&stats[2 * BN + cb + 2 * c2]);
        pdv[c2] = __fmul2_rn(pv[c2], __ffma2_rn(make_float2(__uint_as_float(rsd[2 * c2]), __uint_as_float(rsd[2 * c2 + 1])), sc1, nz));
      }
    }
    if (kDkv) {
#pragma unroll
      for (int h = 0; h < HC / 16; ++h) {
        uint32_t pk[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) pk[c] = pack2<T>(pdv[h * 8 + c].x, pdv[h * 8 + c].y);
        tmem_st8(stile_addr(0, tSD) + lane_off + cb + h * 16, pk);
      }
    }
    pw_publish(BAR_P_FULL + 0, it, false);
    // ---- B1: dP -> dS, written over the tile it came from ----
    wait_tiles(BAR_S_FULL + 1);
    {
      uint32_t rp[HC];
      tmem_ld32(stile_addr(0, tDP) + lane_off + cb, rp);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < HC / 16; ++h) {
        uint32_t o_ds[8];
#pragma unroll
        for (int c2 = 0; c2 < 8; ++c2) {
          const int i2 = h * 8 + c2;
          float2 ndp = make_float2(-dps, -dps);
          if (kDkv) ndp = *reinterpret_cast<const float2*>(&stats[BN + cb + 2 * i2]);
          const float2 a = __fadd2_rn(make_float2(__uint_as_float(rp[2 * i2]), __uint_as_float(rp[2 * i2 + 1])), ndp);
          const float2 ds = __fmul2_rn(pv[i2], a);
          pdv[i2] = __fmul2_rn(pdv[i2], a);  // first term of dS_dot
          o_ds[c2] = pack2<T>(ds.x, ds.y);
        }
        tmem_st8(stile_addr(0, tDP) + lane_off + cb + h * 16, o_ds);
      }
    }
    if (kHalfB) pw_publish(BAR_P_HALF, it, false);
    // ---- B2: dP_dot -> dS_dot ----
    if (hasSB2) wait_tiles(BAR_S2_FULL + 1);  // otherwise dP_dot came out of the pair GEMM together with dP
    {
      uint32_t rpd[HC];
      tmem_ld32(stile_addr(0, tDPD) + lane_off + cb, rpd);
      tmem_ld_wait();
#pragma unroll
      for (int h = 0; h < HC / 16; ++h) {
        uint32_t o_dsd[8];
#pragma unroll
        for (int c2 = 0; c2 < 8; ++c2) {
          const int i2 = h * 8 + c2;
          float2 ndd = make_float2(-ddt, -ddt);
          if (kDkv) ndd = *reinterpret_cast<const float2*>(&stats[3 * BN + cb + 2 * i2]);
          const float2 t = __fadd2_rn(make_float2(__uint_as_float(rpd[2 * i2]), __uint_as_float(rpd[2 * i2 + 1])), ndd);
          const float2 dsd = __ffma2_rn(pv[i2], t, pdv[i2]);
          o_dsd[c2] = pack2<T>(dsd.x, dsd.y);
        }
        tmem_st8(stile_addr(0, tDPD) + lane_off + cb + h * 16, o_dsd);
      }
    }
    pw_publish(BAR_P_FULL + 1, it, true);
    if (prof) { pw_wait += waited; pw_work += clock64() - t0 - waited; }
  }

  // FWD, one block: (online) softmax of this thread's HC columns of S, and W = c P * S_dot.
  __device__ __forceinline__ void pw_fwd_block(int it, int st, bool need_mask, int cmax) {
    uint32_t rs[HC], rsd[HC];
    if constexpr (HC == 32) {
      tmem_ld32(stile_addr(st, 0) + lane_off + cb, rs);
      if (TANGENT) tmem_ld32(stile_addr(st, 1) + lane_off + cb, rsd);
    } else {
      tmem_ld16(stile_addr(st, 0) + lane_off + cb, rs);
      if (TANGENT) tmem_ld16(stile_addr(st, 1) + lane_off + cb, rsd);
    }
    tmem_ld_wait();
    float pv[HC];
#pragma unroll
    for (int c = 0; c < HC; ++c) pv[c] = __uint_as_float(rs[c]);
    if (need_mask) {
#pragma unroll
      for (int c = 0; c < HC; ++c) if (cb + c > cmax) pv[c] = -INFINITY;
    }
    float moff;
    if (FIRST) {
      float mx[4] = {pv[0], pv[1], pv[2], pv[3]};
#pragma unroll
      for (int c = 4; c < HC; ++c) mx[c & 3] = fmaxf(mx[c & 3], pv[c]);
      float mloc = fmaxf(fmaxf(mx[0], mx[1]), fmaxf(mx[2], mx[3]));
      // row maximum over both warpgroups' columns (double-buffered by block parity). Only the NWG warps that
      // share a TMEM lane quadrant (the same 32 rows) exchange values, so they synchronise among themselves
      // (one named barrier per quadrant) instead of all pointwise warps waiting for the slowest of them.
      xchg[((it & 1) * NWG + wg) * 128 + row] = mloc;
      named_barrier_sync(4 + (warp & 3), NWG * 32);
#pragma unroll
      for (int o = 1; o < NWG; ++o) mloc = fmaxf(mloc, xchg[((it & 1) * NWG + ((wg + o) % NWG)) * 128 + row]);
      const float m_new = fmaxf(m_used, mloc);
      const bool grow = (m_new - m_used) * scale2 > kRescaleThreshold;  // false when both are -inf (NaN)
      float alpha = 1.f;
      if (grow) {
        alpha = (m_used == -INFINITY) ? 0.f : ex2((m_used - m_new) * scale2);
        m_used = m_new;
        l_sum *= alpha;
        z_sum *= alpha;
      }
      if (it > 0 && __any_sync(0xffffffffu, grow)) {
        // Accumulators must be quiescent: wait for the output GEMMs of block it-1. The two
        // warpgroups take alternate 32-column chunks of the accumulators.
        warp_wait(BAR_PV_DONE, (it - 1) & 1);
        tc_fence_after();
#pragma unroll 1
        for (int cc = wg; cc < C::accCols / 32; cc += NWG) {
          uint32_t a[32];
          tmem_ld32(tmem_base + lane_off + cc * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) a[c] = __float_as_uint(__uint_as_float(a[c]) * alpha);
          tmem_st32(tmem_base + lane_off + cc * 32, a);
        }
        tmem_st_wait();
      }
      moff = (m_used == -INFINITY) ? 0.f : m_used * scale2;
    } else {
      moff = lse2;
    }
    // packed f32x2 arithmetic: two columns per FMA / add
    const float2 sc2 = make_float2(scale2, scale2), nmoff = make_float2(-moff, -moff);
    float2 ls2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
    for (int c2 = 0; c2 < HC / 2; ++c2) {
      const float2 e = __ffma2_rn(make_float2(pv[2 * c2], pv[2 * c2 + 1]), sc2, nmoff);
      const float2 pe = exp2_pair(e, c2, !need_mask);
      pv[2 * c2] = pe.x;
      pv[2 * c2 + 1] = pe.y;
      ls2[c2 & 1] = __fadd2_rn(ls2[c2 & 1], pe);
    }
    l_sum += (ls2[0].x + ls2[0].y) + (ls2[1].x + ls2[1].y);
    // 16-bit operands go back over the fp32 columns they came from: the 8 packed columns of
    // K-step kk live at tile column 16*kk (inside this warpgroup's own column range).
#pragma unroll
    for (int h = 0; h < HC / 16; ++h) {
      uint32_t pk[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) pk[c] = pack2<T>(pv[h * 16 + 2 * c], pv[h * 16 + 2 * c + 1]);
      tmem_st8(stile_addr(st, 0) + lane_off + cb + h * 16, pk);
    }
    if (TANGENT) {
      const float2 sc1 = make_float2(p.scale, p.scale);
      float2 zs2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
      for (int h = 0; h < HC / 16; ++h) {
        uint32_t pk[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          const int e = h * 16 + 2 * c;
          const float2 w = __fmul2_rn(make_float2(pv[e], pv[e + 1]),
                                      __fmul2_rn(make_float2(__uint_as_float(rsd[e]), __uint_as_float(rsd[e + 1])), sc1));
          zs2[c & 1] = __fadd2_rn(zs2[c & 1], w);
          pk[c] = pack2<T>(w.x, w.y);
        }
        tmem_st8(stile_addr(st, 1) + lane_off + cb + h * 16, pk);
      }
      z_sum += (zs2[0].x + zs2[0].y) + (zs2[1].x + zs2[1].y);
    }
  }

  // First-order dQ / dK,dV, one block (kernels with tangents take pw_two_phase_block): 16 streamed
  // columns at a time from the S and dP tiles, the TMEM loads of the next group in flight while
  // the current one is processed.
  __device__ __forceinline__ void pw_bwd_block(int st, bool need_mask, int cmin, int cmax, const float* stats) {
    static_assert(!TANGENT, "first-order kernels only");
    constexpr int CW = 16;
    constexpr int NG = HC / CW;
    uint32_t bs[2][CW], bp[2][CW];
    auto issue = [&](int gi, int buf) {
      const uint32_t col = lane_off + cb + gi * CW;
      tmem_ld16(stile_addr(st, tS) + col, bs[buf]);
      tmem_ld16(stile_addr(st, tDP) + col, bp[buf]);
    };
    const long long tq0 = prof ? clock64() : 0;
    issue(0, 0);
    tmem_ld_wait();
    if (prof) pw_ld0 += clock64() - tq0;
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
      const int buf = gi & 1;
      if (gi + 1 < NG) issue(gi + 1, buf ^ 1);
      uint32_t o_p[CW / 2], o_ds[CW / 2];
      const float2 sc2 = make_float2(scale2, scale2);
#pragma unroll
      for (int c2 = 0; c2 < CW / 2; ++c2) {
        const int c = 2 * c2, col = cb + gi * CW + c;
        float2 nl2 = make_float2(-lse2, -lse2), ndp = make_float2(-dps, -dps);
        if (kDkv) {
          nl2 = *reinterpret_cast<const float2*>(&stats[col]);
          ndp = *reinterpret_cast<const float2*>(&stats[BN + col]);
        }
        const float2 e = __ffma2_rn(make_float2(__uint_as_float(bs[buf][c]), __uint_as_float(bs[buf][c + 1])), sc2, nl2);
        float2 pe = exp2_pair(e, c2, !need_mask);
        if (need_mask) {
          if (col > cmax || col < cmin) pe.x = 0.f;
          if (col + 1 > cmax || col + 1 < cmin) pe.y = 0.f;
        }
        const float2 a = __fadd2_rn(make_float2(__uint_as_float(bp[buf][c]), __uint_as_float(bp[buf][c + 1])), ndp);
        const float2 ds = __fmul2_rn(pe, a);
        o_p[c2] = pack2<T>(pe.x, pe.y);
        o_ds[c2] = pack2<T>(ds.x, ds.y);
      }
      // the packed columns of streamed columns [16*kk, 16*kk+16) live at tile column 16*kk
      const uint32_t pcol = lane_off + cb + gi * CW;
      if (kDq) {
        tmem_st8(stile_addr(st, tS) + pcol, o_ds);   // dS replaces S
      } else {
        tmem_st8(stile_addr(st, 0) + pcol, o_p);     // P^T replaces S^T
        tmem_st8(stile_addr(st, 1) + pcol, o_ds);    // dS^T replaces dP^T
      }
      if (gi + 1 < NG) {
        const long long tq2 = prof ? clock64() : 0;
        tmem_ld_wait();
        if (prof) pw_ld0 += clock64() - tq2;
      }
    }
  }

  // Copies the owner operands chosen by Cfg::aOuter from shared memory (K-major, 128-byte swizzle) into
  // TMEM as 16-bit A operands: each thread its own row, the warpgroups alternate 64-element chunks.
  __device__ __forceinline__ void stage_a_operands() {
    warp_wait(BAR_OUTER, 0);
#pragma unroll
    for (int j = 0; j < C::nATmem; ++j) {
      for (int c = wg; c < D / 64; c += NWG) {
        const uint8_t* src = smem + C::aOuter(j) * C::outerTile + c * (BM * 128) + row * 128;
        uint32_t v[32];
#pragma unroll
        for (int u = 0; u < 8; ++u) {  // logical 16-byte unit u of the row sits at unit u ^ (row % 8)
          const uint4 x = *reinterpret_cast<const uint4*>(src + ((u ^ (row & 7)) << 4));
          v[4 * u + 0] = x.x; v[4 * u + 1] = x.y; v[4 * u + 2] = x.z; v[4 * u + 3] = x.w;
        }
        tmem_st32(aop_addr(j) + lane_off + c * 32, v);
      }
    }
    tmem_st_wait();
    tc_fence_before();
    __syncwarp();
    if (lane == 0) mbar_arrive(bar(BAR_A_READY));
  }

  __device__ __forceinline__ void pointwise() {
    const int ct = threadIdx.x - kRoleThreads;
    wg = ct >> 7;
    row = (warp & 3) * 32 + lane;
    lane_off = (uint32_t)((warp & 3) * 32) << 16;
    cb = wg * HC;
    orow = r0 + row;
    row_ok = orow < own_len;
    scale2 = p.scale * kLog2e;
    srow = (int64_t)head * p.Tq + si.q0 + orow;
    xchg = reinterpret_cast<float*>(smem + C::tileBytes + 256);

    m_used = -INFINITY; l_sum = 0.f; z_sum = 0.f;
    lse2 = INFINITY; dps = 0.f; z1v = 0.f; ddt = 0.f;
    if ((kFwd && !FIRST) || kDq) {
      if (row_ok) {
        float lse = p.lse[srow];
        lse2 = (lse == -INFINITY) ? INFINITY : lse * kLog2e;
        if (kDq) {
          dps = p.dpsum[srow];
          if (TANGENT) { z1v = p.z1[srow]; ddt = p.ddot[srow]; }
        }
      }
    }
    pw_wait = 0; pw_work = 0; pw_ld0 = 0; pw_st = 0;
    if constexpr (C::nATmem > 0) {
      if (n_it > 0) stage_a_operands();
    }
    for (int it = 0; it < n_it; ++it) {
      const int st = it % ST;
      int blk;  // streamed block index within the sequence
      if (!kDkv) blk = it; else blk = blk_begin + (it_base + it) % blk_count;
      const int c0 = blk * BN;  // first streamed row of the block
      // Does this block need masking? (sequence tail, or causal diagonal crossing the tile)
      bool need_mask;
      int cmin = 0, cmax = BN - 1;  // this thread's visible streamed-column range [cmin, cmax] (block local)
      if (!kDkv) {
        need_mask = (c0 + BN > si.sk) || (p.causal && c0 + BN - 1 > r0 + off);
        int jmax = si.sk - 1;
        if (p.causal) jmax = min(jmax, orow + off);
        cmax = jmax - c0;
      } else {
        const int off_blk = off - (p.seg_keys ? 0 : seg_shift_of(p, c0));  // the block lies inside one query segment
        need_mask = p.causal && (r0 + BM - 1 - off_blk > c0);
        if (p.causal) cmin = orow - off_blk - c0;  // query i visible iff i >= key - off
      }
      const float* stats = stats_base + (it & 1) * (4 * BN);  // DKV: this block's staged statistics
      if constexpr (kSplit) {
        pw_two_phase_block(it, need_mask, cmin, cmax, stats);
      } else {
        const long long tw = prof ? clock64() : 0;
        warp_wait(BAR_S_FULL + st, (it / ST) & 1);
        const long long tw1 = prof ? clock64() : 0;
        pw_wait += tw1 - tw;
        tc_fence_after();
        if constexpr (kFwd) pw_fwd_block(it, st, need_mask, cmax);
        else pw_bwd_block(st, need_mask, cmin, cmax, stats);
        const long long tq1 = prof ? clock64() : 0;
        pw_publish(BAR_P_FULL + st, it, true);
        if (prof) { pw_work += clock64() - tw1; pw_st += clock64() - tq1; }
      }
    }
    if (prof && ct == 0) { g_prof[5] = pw_wait; g_prof[6] = pw_work; g_prof[9] = pw_ld0; g_prof[10] = pw_st; }

    if (n_it > 0) {
      warp_wait(BAR_ACC_DONE, 0);
      tc_fence_after();
    }
    if (ct == 0) FB_TRACE(5);
    // After ACC_DONE every MMA and TMA of this CTA has completed: the tile area is free scratch.
    // (After an abort the pointwise warps still run through every block and the epilogue, with waits that
    // return at once: they synchronise among themselves with named barriers, so they must all take the
    // same path. What they write then is void; the host learns of it from the status word.)
    if constexpr (kFwd) epilogue_fwd();
    else if (kDkv && p.split > 1) { if (part > 0) spill_partial(); }  // the cluster's first CTA adds the parts up: reduce_and_store()
    else epilogue_bwd();
    if (ct == 0) FB_TRACE(6);
    tc_fence_before();
  }

  // FWD epilogue: O = acc / l, O_dot = acc_dot / l - z1 O, and the row statistics lse, z1, dpsum, ddot.
  // 32 elements of this thread's row out of a staged / TMA-loaded tile (same swizzled layout as stage32)
  __device__ __forceinline__ void unstage32(const uint8_t* tile, int cc, float (&v)[32]) const {
    const uint8_t* rowp = tile + (cc >> 1) * (BM * 128) + row * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint4 u = *reinterpret_cast<const uint4*>(rowp + ((((cc & 1) * 4 + i) ^ (row & 7)) << 4));
      float2 a = unpack2<T>(u.x), b = unpack2<T>(u.y), c = unpack2<T>(u.z), d = unpack2<T>(u.w);
      v[8 * i + 0] = a.x; v[8 * i + 1] = a.y; v[8 * i + 2] = b.x; v[8 * i + 3] = b.y;
      v[8 * i + 4] = c.x; v[8 * i + 5] = c.y; v[8 * i + 6] = d.x; v[8 * i + 7] = d.y;
    }
  }

  // On a full tile the rows of dO / dO_dot (and of O when it is an input) come in by TMA into staging
  // slots 2, 3 (0), requested as soon as the accumulators are complete, and O / O_dot go out through slots
  // 0 / 1 and TMA stores; see epilogue_bwd.
  __device__ __forceinline__ void epilogue_fwd() {
    float* epi = reinterpret_cast<float*>(smem);  // [4][NWG warpgroups][128 rows]
    const int64_t grow_ = si.q0 + orow;
    const bool staged = (r0 + BM <= own_len) && p.tma_out;
    const bool tma_in = staged && (p.dout.ptr != nullptr || !FIRST);
    if (tma_in && threadIdx.x == kRoleThreads) {
      const int row0 = si.q0 + r0;
      const uint32_t bytes = ((FIRST ? 0 : 1) + (p.dout.ptr ? 1 : 0) + ((TANGENT && p.doutd.ptr) ? 1 : 0)) * C::outerTile;
      mbar_expect_tx(bar(BAR_OUTER), bytes);
#pragma unroll
      for (int c = 0; c < D / 64; ++c) {
        if (!FIRST) tma_load_3d(sbase + kStageOff + 0 * C::outerTile + c * (BM * 128), &maps.m[T_OUT0], bar(BAR_OUTER), c * 64, row0, head);
        if (p.dout.ptr) tma_load_3d(sbase + kStageOff + 2 * C::outerTile + c * (BM * 128), &maps.m[T_DO], bar(BAR_OUTER), c * 64, row0, head);
        if (TANGENT && p.doutd.ptr) tma_load_3d(sbase + kStageOff + 3 * C::outerTile + c * (BM * 128), &maps.m[T_DOD], bar(BAR_OUTER), c * 64, row0, head);
      }
    }
    bool in_ready = !tma_in;
    auto wait_in = [&]() {
      if (!in_ready) {
        warp_wait(BAR_OUTER, n_it > 0 ? 1 : 0);  // second use of the barrier when the main loop ran
        in_ready = true;
      }
    };
    if (FIRST || TANGENT) {
      epi[(0 * NWG + wg) * 128 + row] = l_sum;
      epi[(1 * NWG + wg) * 128 + row] = z_sum;
      named_barrier_sync(1, kPwThreads);
      l_sum = 0.f;
      z_sum = 0.f;
#pragma unroll
      for (int o = 0; o < NWG; ++o) {  // same order in every warpgroup: identical sums
        l_sum += epi[(0 * NWG + o) * 128 + row];
        z_sum += epi[(1 * NWG + o) * 128 + row];
      }
    }
    const float inv = FIRST ? (l_sum > 0.f ? 1.f / l_sum : 0.f) : 1.f;
    const float z1o = z_sum * inv;
    T* op = row_ptr<T>(p.o, head, grow_);
    T* odp = row_ptr<T>(p.od, head, grow_);
    const T* gp = row_ptr<T>(p.dout, head, grow_);
    const T* gdp = row_ptr<T>(p.doutd, head, grow_);
    float dsum = 0.f, ddsum = 0.f;
#pragma unroll 1
    for (int cc = wg; cc < D / 32; cc += NWG) {
      float o[32], od[32];
      if (FIRST) {
        if (n_it > 0) {
          uint32_t a[32];
          tmem_ld32(acc_addr(0) + lane_off + cc * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = __uint_as_float(a[c]) * inv;
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = 0.f;
        }
        if (staged) stage32(smem + kStageOff, cc, o);
        else if (row_ok) store32<T>(op, cc * 32, o);
      } else {
        if (staged) { wait_in(); unstage32(smem + kStageOff, cc, o); }
        else if (row_ok) load32<T>(op, cc * 32, o);
        else {
#pragma unroll
          for (int c = 0; c < 32; ++c) o[c] = 0.f;
        }
      }
      if (TANGENT) {
        if (n_it > 0) {
          uint32_t a[32];
          tmem_ld32(acc_addr(FIRST ? 1 : 0) + lane_off + cc * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) od[c] = __uint_as_float(a[c]) * inv - z1o * o[c];
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) od[c] = 0.f;
        }
        if (staged) stage32(smem + kStageOff + C::outerTile, cc, od);
        else if (row_ok) store32<T>(odp, cc * 32, od);
      }
      if (gp && row_ok) {
        float g[32];
        if (staged) { wait_in(); unstage32(smem + kStageOff + 2 * C::outerTile, cc, g); }
        else load32<T>(gp, cc * 32, g);
#pragma unroll
        for (int c = 0; c < 32; ++c) {
          dsum = fmaf(g[c], o[c], dsum);
          if (TANGENT) ddsum = fmaf(g[c], od[c], ddsum);
        }
        if (TANGENT && gdp) {
          if (staged) unstage32(smem + kStageOff + 3 * C::outerTile, cc, g);
          else load32<T>(gdp, cc * 32, g);
#pragma unroll
          for (int c = 0; c < 32; ++c) ddsum = fmaf(g[c], o[c], ddsum);
        }
      }
    }
    if (staged) {
      wait_in();  // (every warp passes the barrier's phase before the CTA goes on)
      const int out_of[4] = {0, 1, 0, 0};
      store_staged((FIRST ? 1u : 0u) | (TANGENT ? 2u : 0u), out_of, si.q0 + r0);
    }
    if (gp) {  // uniform across the grid
      epi[(2 * NWG + wg) * 128 + row] = dsum;
      epi[(3 * NWG + wg) * 128 + row] = ddsum;
      named_barrier_sync(2, kPwThreads);
      dsum = 0.f;
      ddsum = 0.f;
#pragma unroll
      for (int o = 0; o < NWG; ++o) {
        dsum += epi[(2 * NWG + o) * 128 + row];
        ddsum += epi[(3 * NWG + o) * 128 + row];
      }
    }
    if (row_ok && wg == 0) {
      if (FIRST) p.lse[srow] = l_sum > 0.f ? m_used * p.scale + logf(l_sum) : -INFINITY;
      if (TANGENT) p.z1[srow] = z1o;
      if (gp) {
        p.dpsum[srow] = dsum;
        if (TANGENT) p.ddot[srow] = ddsum;
      }
    }
  }

  // ---- a key tile shared by a cluster (DKV, p.split > 1) ----
  // Every CTA of the cluster accumulates its slice of the tile's streamed blocks in its own TMEM. CTAs
  // 1.. then write their fp32 accumulators into their own shared memory (free once the main loop is
  // over), the cluster synchronises, and CTA 0 adds them to its own in the fixed order 1, 2, .. through
  // distributed shared memory before the single store: deterministic, no atomics, no workspace.
  // Image layout: 16-byte units [(accumulator * D/32 + 32-column chunk) * 8 + unit][row], so that a warp
  // reads or writes 512 consecutive bytes.
  static_assert(!kDkv || C::nAcc * BM * D * 4 <= C::tileBytes, "accumulator image must fit the tile area");
  static constexpr int kStageSlots = kFwd ? (TANGENT ? 4 : 3) : C::nAcc;  // FWD: O, O_dot, dO, dO_dot
  static_assert(kStageOff + kStageSlots * C::outerTile <= C::tileBytes, "epilogue staging tiles must fit the tile area");
  __device__ __forceinline__ uint32_t image_off(int a_i, int cc, int u) const {
    return (uint32_t)((((a_i * (D / 32) + cc) * 8 + u) * BM + row) * 16);
  }
  __device__ __forceinline__ void spill_partial() {
    if (n_it == 0) return;  // CTA 0 derives the same from part_begin() and skips this part
#pragma unroll
    for (int a_i = 0; a_i < C::nAcc; ++a_i) {
#pragma unroll 1
      for (int cc = wg; cc < D / 32; cc += NWG) {
        uint32_t a[32];
        tmem_ld32(acc_addr(a_i) + lane_off + cc * 32, a);
        tmem_ld_wait();
#pragma unroll
        for (int u = 0; u < 8; ++u)
          *reinterpret_cast<uint4*>(smem + image_off(a_i, cc, u)) = make_uint4(a[4 * u], a[4 * u + 1], a[4 * u + 2], a[4 * u + 3]);
      }
    }
  }
  // Runs in every thread of every CTA of the cluster, after run_role().
  __device__ __forceinline__ void cluster_reduce() {
    __syncwarp();
    cluster_sync_all();  // the images of CTAs 1.. are complete and visible
    if (part == 0 && warp >= kRoleThreads / 32) {
      tc_fence_after();
      epilogue_bwd(true);
      tc_fence_before();
    }
    __syncwarp();
    cluster_sync_all();  // CTA 0 has read the images: their owners may exit
  }

  // DQ: accumulators {dQ?, dQ_dot?};  DKV: {dK, dV}? then {dK_dot, dV_dot}?
  // (TMEM loads are warp-collective, so row predicates apply to the global stores only.)
  // add_parts: this is CTA 0 of a cluster sharing the tile; add the other CTAs' accumulator images.
  // Writes this thread's 32 scaled values of a row into the staging tile (K-major, 128-byte swizzle: the
  // layout the TMA store expects): 64-column chunk cc/2, 16-byte units 4*(cc%2) .. +3 of the row.
  __device__ __forceinline__ void stage32(uint8_t* tile, int cc, const float (&v)[32]) const {
    uint8_t* rowp = tile + (cc >> 1) * (BM * 128) + row * 128;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      uint4 u;
      u.x = pack2<T>(v[8 * i + 0], v[8 * i + 1]);
      u.y = pack2<T>(v[8 * i + 2], v[8 * i + 3]);
      u.z = pack2<T>(v[8 * i + 4], v[8 * i + 5]);
      u.w = pack2<T>(v[8 * i + 6], v[8 * i + 7]);
      *reinterpret_cast<uint4*>(rowp + ((((cc & 1) * 4 + i) ^ (row & 7)) << 4)) = u;
    }
  }
  // One thread stores the staged tiles `mask` (bit a = staging slot a -> output map T_OUT0 + out_of[a]).
  __device__ __forceinline__ void store_staged(uint32_t mask, const int (&out_of)[4], int64_t row0) const {
    fence_proxy_async_smem();            // the generic-proxy writes above -> visible to the TMA engine
    named_barrier_sync(3, kPwThreads);
    if (threadIdx.x == kRoleThreads) {
#pragma unroll
      for (int a = 0; a < 4; ++a) {
        if (!(mask & (1u << a))) continue;
#pragma unroll
        for (int c = 0; c < D / 64; ++c)
          tma_store_3d(&maps.m[T_OUT0 + out_of[a]], sbase + kStageOff + a * C::outerTile + c * (BM * 128), c * 64, (int)row0, head);
      }
      bulk_commit_group();
      bulk_wait_group_read0();  // shared memory must outlive the reads
    }
  }

  // A full owner tile of 16-bit outputs goes out through shared memory and TMA stores (one coalesced bulk
  // store per 64-column chunk instead of 32 lanes x 16 bytes at row stride per instruction, which made the
  // epilogue LSU-bound); a tile that ends inside the sequence keeps the per-row stores with their row predicate.
  __device__ __forceinline__ void epilogue_bwd(bool add_parts = false) {
    const int64_t grow_ = (kDkv ? si.k0 : si.q0) + orow;
    constexpr int perSet = kDkv ? 2 : 1;
    const bool staged = (r0 + BM <= own_len) && !(kDkv && p.kv_f32) && p.tma_out;
    uint32_t staged_mask = 0;
    int out_of[4] = {0, 0, 0, 0};
#pragma unroll
    for (int a_i = 0; a_i < C::nAcc; ++a_i) {
      const int set = a_i / perSet, which = a_i % perSet;  // which: 0 = dQ / dK (scaled by c), 1 = dV
      const bool is_dot = FIRST ? (set == 1) : true;
      const SeqT& dst = kDq ? (is_dot ? p.dqd : p.dq) : (which == 0 ? (is_dot ? p.dkd : p.dk) : (is_dot ? p.dvd : p.dv));
      if (!dst.ptr) continue;  // uniform across the grid
      if (staged) { staged_mask |= 1u << a_i; out_of[a_i] = kDq ? (is_dot ? 1 : 0) : which + (is_dot ? 2 : 0); }
      T* dp_ = row_ptr<T>(dst, head, grow_);
      // dK/dV-side results may go out as float32 (strides then count floats), stored or accumulated: the
      // long-context driver sums the partial results of its query chunks that way, without a 16-bit round trip
      float* fp_ = (kDkv && p.kv_f32) ? reinterpret_cast<float*>(dst.ptr) + (int64_t)head * dst.head_stride + grow_ * dst.row_stride : nullptr;
      // ... and the sum may go to the GPU that owns this key row instead of back to `dst` (scatter mode)
      float* wp_ = fp_;
      if (kDkv && p.scat_n > 0) {
        const int64_t peer = grow_ / p.scat_rows;
        wp_ = reinterpret_cast<float*>(p.scat[(is_dot ? 2 : 0) + which][peer]) + (int64_t)head * p.scat_head_stride +
              (grow_ - peer * p.scat_rows) * p.scat_row_stride;
      }
      const float mul = (which == 0) ? p.scale : 1.f;
#pragma unroll 1
      for (int cc = wg; cc < D / 32; cc += NWG) {
        float v[32];
        if (n_it > 0) {
          uint32_t a[32];
          tmem_ld32(acc_addr(a_i) + lane_off + cc * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int c = 0; c < 32; ++c) v[c] = __uint_as_float(a[c]);
        } else {
#pragma unroll
          for (int c = 0; c < 32; ++c) v[c] = 0.f;
        }
        if constexpr (kDkv) {
          if (add_parts) {
#pragma unroll 1
            for (int j = 1; j < p.split; ++j) {
              if (part_begin(j + 1) == part_begin(j)) continue;  // that CTA had no blocks and wrote no image
              const uint32_t img = map_to_cta(sbase, (uint32_t)j);
#pragma unroll
              for (int u = 0; u < 8; ++u) {
                const float4 r = ld_cluster_f4(img + image_off(a_i, cc, u));
                v[4 * u] += r.x; v[4 * u + 1] += r.y; v[4 * u + 2] += r.z; v[4 * u + 3] += r.w;
              }
            }
          }
        }
#pragma unroll
        for (int c = 0; c < 32; ++c) v[c] *= mul;
        if (staged) stage32(smem + kStageOff + a_i * C::outerTile, cc, v);
        else if (row_ok) {
          if (kDkv && fp_) store32_f32(wp_, (p.kv_accum && grow_ < p.kv_accum_rows) ? fp_ : nullptr, cc * 32, v);
          else store32<T>(dp_, cc * 32, v);
        }
      }
    }
    if (staged) store_staged(staged_mask, out_of, (kDkv ? si.k0 : si.q0) + r0);
  }

  // ================================================ teardown ================================================
  __device__ __forceinline__ void teardown() {
    __syncwarp();  // the single-lane role branches must rejoin their warps before the CTA-wide barrier
    __syncthreads();
    if (prof && threadIdx.x == 0) g_prof[0] = clock64() - t_kernel0;
    if (*abort_flag) {
      if (threadIdx.x == 0) atomicOr(p.status, 1 << KIND);
      // give in-flight asynchronous copies / MMAs time to land before the CTA's resources are released
      for (int i = 0; i < 64; ++i) __nanosleep(20000);
      __syncthreads();
    }
    if (warp == 1) {
      tc_fence_after();
      tmem_dealloc(tmem_base, C::tmemCols);
    }
    if (threadIdx.x == 0) FB_TRACE(7);
  }
};

template <typename T, int KIND, int D, bool TANGENT, bool FIRST, bool DOD, bool HOOK = false>
__global__ void __launch_bounds__(kThreads, 1) tc_kernel(const __grid_constant__ TmaMaps maps, const __grid_constant__ Params p) {
  extern __shared__ __align__(1024) uint8_t smem[];
  TcCta<T, KIND, D, TANGENT, FIRST, DOD, HOOK> cta(maps, p, smem);
  if (!cta.setup()) return;
  cta.run_role();
  if constexpr (KIND == KIND_DKV) {
    if (p.split > 1) cta.cluster_reduce();
  }
  cta.teardown();
}

// ------------------------------------------------------------------------------------------------
// Host side: tensor maps and dispatch
// ------------------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn get_encode_fn() {
  static EncodeTiledFn fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* ptr = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &qres) == cudaSuccess &&
        qres == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(ptr);
  });
  return fn;
}

// (head_dim, rows, heads) view of a sequence tensor; box = 64 elements x box_rows rows x 1 head,
// 128-byte swizzle; rows past `rows` read as zero.
int encode_map(CUtensorMap* m, const SeqT& t, int dtype, int D, int64_t rows, int heads, int box_rows) {
  EncodeTiledFn enc = get_encode_fn();
  if (!enc) return FB_ERR_CUDA;
  cuuint64_t gdim[3] = {(cuuint64_t)D, (cuuint64_t)rows, (cuuint64_t)heads};
  cuuint64_t gstr[2] = {(cuuint64_t)t.row_stride * 2, (cuuint64_t)t.head_stride * 2};
  cuuint32_t box[3] = {64, (cuuint32_t)box_rows, 1};
  cuuint32_t estr[3] = {1, 1, 1};
  CUresult r = enc(m, dtype == FB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, t.ptr, gdim, gstr,
                   box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                   CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  return r == CUDA_SUCCESS ? FB_OK : FB_ERR_CUDA;
}

// Encoded tensor maps are kept in a small direct-mapped cache: a map is a pure function of (pointer,
// strides, extents, box, dtype), so an entry can never go stale, and a training loop presents the same
// buffers call after call (16 maps per backward, about 1 us each to encode). The reference rebuilds its
// TMA descriptors on every call (jvp_fwd_sm90.py:193-234).
struct MapKey {
  void* ptr;
  int64_t row_stride, head_stride, rows;
  int32_t heads, box_rows, dtype, D;
  bool operator==(const MapKey& o) const {
    return ptr == o.ptr && row_stride == o.row_stride && head_stride == o.head_stride && rows == o.rows && heads == o.heads &&
           box_rows == o.box_rows && dtype == o.dtype && D == o.D;
  }
};
struct MapSlot {
  MapKey key;
  CUtensorMap map;
  bool valid;
};
constexpr int kMapSlots = 1024;
MapSlot g_map_cache[kMapSlots];
std::mutex g_map_mutex;

size_t map_hash(const MapKey& k) {
  uint64_t h = reinterpret_cast<uint64_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
  h ^= (uint64_t)k.rows * 0xC2B2AE3D27D4EB4Full + (uint64_t)k.row_stride * 0x165667B19E3779F9ull + (uint64_t)k.head_stride * 31u;
  h ^= ((uint64_t)k.heads << 40) ^ ((uint64_t)k.box_rows << 20) ^ ((uint64_t)k.dtype << 8) ^ (uint64_t)k.D;
  h ^= h >> 29;
  return (size_t)(h % kMapSlots);
}

int make_map(CUtensorMap* m, const SeqT& t, int dtype, int D, int64_t rows, int heads, int box_rows) {
  if (!t.ptr) { memset(m, 0, sizeof(*m)); return FB_OK; }
  const MapKey key{t.ptr, t.row_stride, t.head_stride, rows, heads, box_rows, dtype, D};
  MapSlot& slot = g_map_cache[map_hash(key)];
  {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (slot.valid && slot.key == key) { *m = slot.map; return FB_OK; }
  }
  const int st = encode_map(m, t, dtype, D, rows, heads, box_rows);
  if (st == FB_OK) {
    std::lock_guard<std::mutex> lock(g_map_mutex);
    slot.key = key; slot.map = *m; slot.valid = true;
  }
  return st;
}

// kind: which kernel family the maps are for (decides the box of each side and the output maps)
int build_maps(TmaMaps& maps, const Params& p, int kind) {
  const bool q_side_outer = kind != KIND_DKV;
  const int qb = q_side_outer ? BM : BN, kb = q_side_outer ? BN : BM;
  int s;
  const SeqT none{nullptr, 0, 0};
  const SeqT* outs[4] = {&none, &none, &none, &none};
  if (kind == KIND_FWD) { outs[0] = &p.o; outs[1] = &p.od; }
  else if (kind == KIND_DQ) { outs[0] = &p.dq; outs[1] = &p.dqd; }
  else if (!p.kv_f32) { outs[0] = &p.dk; outs[1] = &p.dv; outs[2] = &p.dkd; outs[3] = &p.dvd; }
  for (int i = 0; i < 4; ++i)
    if ((s = make_map(&maps.m[T_OUT0 + i], *outs[i], p.dtype, p.D, q_side_outer ? p.Tq : p.Tk, q_side_outer ? p.Hq : p.Hkv, BM))) return s;
  if ((s = make_map(&maps.m[T_Q], p.q, p.dtype, p.D, p.Tq, p.Hq, qb))) return s;
  if ((s = make_map(&maps.m[T_DO], p.dout, p.dtype, p.D, p.Tq, p.Hq, qb))) return s;
  if ((s = make_map(&maps.m[T_QD], p.qd, p.dtype, p.D, p.Tq, p.Hq, qb))) return s;
  if ((s = make_map(&maps.m[T_DOD], p.doutd, p.dtype, p.D, p.Tq, p.Hq, qb))) return s;
  if ((s = make_map(&maps.m[T_K], p.k, p.dtype, p.D, p.Tk, p.Hkv, kb))) return s;
  if ((s = make_map(&maps.m[T_V], p.v, p.dtype, p.D, p.Tk, p.Hkv, kb))) return s;
  if ((s = make_map(&maps.m[T_KD], p.kd, p.dtype, p.D, p.Tk, p.Hkv, kb))) return s;
  if ((s = make_map(&maps.m[T_VD], p.vd, p.dtype, p.D, p.Tk, p.Hkv, kb))) return s;
  return FB_OK;
}

// Per-device facts the launcher needs, looked up once (under a mutex: the entry points may be called
// from several host threads, e.g. autograd worker threads).
struct DeviceFacts {
  bool known;
  int sm_count;
};
DeviceFacts g_dev[64];
std::mutex g_launch_mutex;

int device_sm_count(int dev) {
  if (dev < 0 || dev >= 64) return 148;
  std::lock_guard<std::mutex> lock(g_launch_mutex);
  if (!g_dev[dev].known) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    g_dev[dev].sm_count = n;
    g_dev[dev].known = true;
  }
  return g_dev[dev].sm_count;
}

// How many CTAs (one cluster) share a key tile of the dK/dV kernels. One CTA per key tile loops over all
// G query heads and all visible query blocks; with few (batch, kv-head) groups per GPU - the
// (batch, kv-head) partition of a problem over several GPUs - that leaves fewer CTAs than SMs, and under
// causal masking the first key tile carries twice the mean work. When the heaviest CTA would exceed
// three quarters of the mean load of an SM (no order of scheduling can balance that), or there are
// fewer CTAs than SMs, the tile's blocks are split over the two CTAs of a cluster. Measured on the 1/8
// share of the causal B2 Hq32 Hkv8 S8192 problem (B1 Hq8 Hkv2): tangent kernel 0.91 ms with one CTA per
// tile, 0.48 with two, 0.52 with four, 0.82 with eight (every extra CTA reloads the owner tile and pays
// its own prologue and epilogue, and larger clusters are harder to place); on the 1/2 share and the
// whole problem one CTA per tile is fastest. (The reference's K2 grid is one CTA per (key tile, QUERY
// head), hvp_bwd_sm90.py:340-363, reduce-adding into fp32 accumulators; here the parts are added up
// through distributed shared memory instead.)
int choose_split(const Params& p, int ntiles, int sm_count) {
  if (p.split > 0) return p.split <= 8 ? p.split : 8;  // forced through fb_problem.flags
  const long long ctas = (long long)ntiles * p.Hkv * p.B;
  const long long blocks = (p.Sq + BN - 1) / BN;
  const long long heaviest = blocks * (p.Hq / p.Hkv);
  const long long total = p.causal ? ctas * heaviest / 2 : ctas * heaviest;
  const double mean_per_sm = (double)total / sm_count;
  if (heaviest < 16) return 1;
  return ((double)heaviest > 0.75 * mean_per_sm || ctas < sm_count) ? 2 : 1;
}

// (head, batch) pairs per scheduling group (TcCta::setup). Under causal masking a group should hold about
// two waves of CTAs: enough light tiles to fill the tail its heavy tiles leave, while the CTAs running
// at any time still stream the K/V (or Q/dO) tiles of only a few heads, which keeps them in L2. Measured
// on causal B2 Hq32 Hkv8 S8192 D128 (whole step): one pair per group 13.44 ms, 4 pairs 13.02, 8 pairs
// 13.10, 16 pairs 13.23, all 64 pairs 13.51; on causal B4 H16 S2048: 1.24 / - / 1.10 / 1.09 / 1.11 ms.
// Without causal masking every tile weighs the same and only locality counts (non-causal B8 H32 S4096
// D64: all pairs in one group 18.1 ms against 14.6-14.8 for groups of 1 to 16).
int choose_group(const Params& p, bool dkv, int ntiles, int sm_count) {
  const int pairs = (dkv ? p.Hkv : p.Hq) * p.B;
  const int G = dkv ? 1 : p.Hq / p.Hkv;  // query heads that share a kv head stay in one group
  int g = p.group;                       // > 0: forced through fb_problem.flags
  if (g <= 0) {
    if (!p.causal) {
      g = G;
    } else {
      const int target = (2 * sm_count + ntiles - 1) / ntiles;
      const int ngroups = pairs / target > 1 ? pairs / target : 1;
      g = (pairs + ngroups - 1) / ngroups;
      g = (g + G - 1) / G * G;
    }
  }
  return g < pairs ? (g > 0 ? g : 1) : pairs;
}

template <typename T, int KIND, int D, bool TANGENT, bool FIRST, bool DOD, bool HOOK = false>
int launch_one(const TmaMaps& maps, const Params& p_in, cudaStream_t stream) {
  using C = Cfg<KIND, D, TANGENT, FIRST, DOD>;
  auto kern = tc_kernel<T, KIND, D, TANGENT, FIRST, DOD, HOOK>;
  static bool attr_set[64] = {};  // guarded by g_launch_mutex
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64) {
    std::lock_guard<std::mutex> lock(g_launch_mutex);
    if (!attr_set[dev]) {
      if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::smemBytes) != cudaSuccess) return FB_ERR_CUDA;
      attr_set[dev] = true;
    }
  }
  Params p = p_in;
  p.tma_out = (p.debug & 8) ? 0 : 1;  // FLASHBACK_DEBUG bit 3: per-row stores everywhere (A/B switch)
  p.ntiles = KIND == KIND_DKV ? (p.Sk + BM - 1) / BM : (p.Sq + BM - 1) / BM;
  p.split = KIND == KIND_DKV ? choose_split(p, p.ntiles, device_sm_count(dev)) : 1;
  p.group = choose_group(p, KIND == KIND_DKV, p.ntiles, device_sm_count(dev));
  const long long ctas = (long long)p.ntiles * (KIND == KIND_DKV ? p.Hkv : p.Hq) * p.B * p.split;
  if (ctas <= 0 || ctas > 0x7fffffffll) return FB_ERR_TOO_LARGE;

  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3((unsigned)ctas, 1, 1);
  cfg.blockDim = dim3(kThreads, 1, 1);
  cfg.dynamicSmemBytes = C::smemBytes;
  cfg.stream = stream;
  cudaLaunchAttribute attrs[2];
  int na = 0;
  // Programmatic dependent launch: this grid's CTAs may be scheduled while the previous kernel in the
  // stream drains; they synchronise with it in setup() (the reference chains K2 to K1 the same way,
  // hvp_bwd_sm90.py:418,794).
  attrs[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[na].val.programmaticStreamSerializationAllowed = 1;
  ++na;
  if (p.split > 1) {
    attrs[na].id = cudaLaunchAttributeClusterDimension;
    attrs[na].val.clusterDim.x = (unsigned)p.split;
    attrs[na].val.clusterDim.y = 1;
    attrs[na].val.clusterDim.z = 1;
    ++na;
  }
  cfg.attrs = attrs;
  cfg.numAttrs = na;
  return cudaLaunchKernelEx(&cfg, kern, maps, p) == cudaSuccess ? 1 : FB_ERR_CUDA;
}

template <typename T, int D>
int fwd_dispatch(const TmaMaps& maps, const Params& p, cudaStream_t s) {
  const bool tangent = p.qd.ptr != nullptr;
  if (!tangent) return launch_one<T, KIND_FWD, D, false, true, false>(maps, p, s);
  if (p.lse_known) return launch_one<T, KIND_FWD, D, true, false, false>(maps, p, s);
  return launch_one<T, KIND_FWD, D, true, true, false>(maps, p, s);
}

template <typename T, int D>
int dq_dispatch(const TmaMaps& maps, const Params& p, cudaStream_t s) {
  const bool first = p.dq.ptr != nullptr, tangent = p.dqd.ptr != nullptr, dod = p.doutd.ptr != nullptr;
  if (!tangent) return launch_one<T, KIND_DQ, D, false, true, false>(maps, p, s);
  if (first) return dod ? launch_one<T, KIND_DQ, D, true, true, true>(maps, p, s) : launch_one<T, KIND_DQ, D, true, true, false>(maps, p, s);
  return dod ? launch_one<T, KIND_DQ, D, true, false, true>(maps, p, s) : launch_one<T, KIND_DQ, D, true, false, false>(maps, p, s);
}

template <typename T, int D>
int dkv_dispatch(const TmaMaps& maps, const Params& p, cudaStream_t s) {
  // dK and dV (and their tangents) are produced pairwise; at head_dim 128 the four accumulators of
  // the combined mode do not fit TMEM next to the S-like tiles, so it runs as two launches.
  const bool first = p.dk.ptr || p.dv.ptr, tangent = p.dkd.ptr || p.dvd.ptr, dod = p.doutd.ptr != nullptr;
  int n = 0, r;
  if constexpr (D == 64) {
    // head_dim 64: all four accumulators fit, one launch produces dK, dV and their tangents
    if (first && tangent)
      return dod ? launch_one<T, KIND_DKV, D, true, true, true>(maps, p, s) : launch_one<T, KIND_DKV, D, true, true, false>(maps, p, s);
  }
  if (first) {
    Params p1 = p;
    p1.dkd.ptr = nullptr; p1.dvd.ptr = nullptr;
    if ((r = launch_one<T, KIND_DKV, D, false, true, false>(maps, p1, s)) < 0) return r;
    n += r;
  }
  if (tangent) {
    Params p2 = p;
    p2.dk.ptr = nullptr; p2.dv.ptr = nullptr;
    r = dod ? launch_one<T, KIND_DKV, D, true, false, true>(maps, p2, s) : launch_one<T, KIND_DKV, D, true, false, false>(maps, p2, s);
    if (r < 0) return r;
    n += r;
  }
  return n;
}

template <typename T>
int bwd_typed(const Params& p, cudaStream_t s) {
  int n = 0, r;
  if (p.dq.ptr || p.dqd.ptr) {
    TmaMaps maps;
    if ((r = build_maps(maps, p, KIND_DQ))) return r;
    r = p.D == 64 ? dq_dispatch<T, 64>(maps, p, s) : dq_dispatch<T, 128>(maps, p, s);
    if (r < 0) return r;
    n += r;
  }
  if (p.dk.ptr || p.dv.ptr || p.dkd.ptr || p.dvd.ptr) {
    TmaMaps maps;
    if ((r = build_maps(maps, p, KIND_DKV))) return r;
    r = p.D == 64 ? dkv_dispatch<T, 64>(maps, p, s) : dkv_dispatch<T, 128>(maps, p, s);
    if (r < 0) return r;
    n += r;
  }
  return n;
}

}  // namespace

int read_profile(long long* out16) {
  if (!kProfile) return FB_ERR_MODE;  // the instrumentation is compiled in with -DFB_PROFILE only
  return cudaMemcpyFromSymbol(out16, g_prof, sizeof(long long) * (kProfile ? 16 : 1)) == cudaSuccess ? FB_OK : FB_ERR_CUDA;
}

#ifdef FB_PROFILE
// Profile builds only: copies the per-CTA timeline of the last launch (n_ctas x 8 times + n_ctas meta words).
extern "C" int fb_debug_trace(unsigned long long* times, unsigned long long* meta, int n_ctas) {
  if (n_ctas > kTraceCtas) n_ctas = kTraceCtas;
  if (cudaDeviceSynchronize() != cudaSuccess) return FB_ERR_CUDA;
  if (cudaMemcpyFromSymbol(times, g_trace, sizeof(unsigned long long) * 8 * n_ctas) != cudaSuccess) return FB_ERR_CUDA;
  if (cudaMemcpyFromSymbol(meta, g_trace_meta, sizeof(unsigned long long) * n_ctas) != cudaSuccess) return FB_ERR_CUDA;
  return FB_OK;
}
#endif

int launch_tc_fwd_wait_hook(const Params& p, cudaStream_t s) {
  TmaMaps maps;
  int r = build_maps(maps, p, KIND_FWD);
  if (r) return r;
  return launch_one<__nv_bfloat16, KIND_FWD, 64, false, true, false, true>(maps, p, s);
}

int launch_tc_fwd(const Params& p, cudaStream_t s) {
  TmaMaps maps;
  int r = build_maps(maps, p, KIND_FWD);
  if (r) return r;
  if (p.dtype == FB_BF16) return p.D == 64 ? fwd_dispatch<__nv_bfloat16, 64>(maps, p, s) : fwd_dispatch<__nv_bfloat16, 128>(maps, p, s);
  return p.D == 64 ? fwd_dispatch<__half, 64>(maps, p, s) : fwd_dispatch<__half, 128>(maps, p, s);
}

int launch_tc_bwd(const Params& p, cudaStream_t s) {
  if (p.dtype == FB_BF16) return bwd_typed<__nv_bfloat16>(p, s);
  return bwd_typed<__half>(p, s);
}

}  // namespace fb
