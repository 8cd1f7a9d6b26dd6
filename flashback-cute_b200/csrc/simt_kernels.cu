// CUDA-core (SIMT) kernels for the attention JVP-forward / HVP-backward path.
//
// These are the float32-I/O path (float32 inputs must agree with the eager float32 result to
// 1e-4 relative, which a single-pass bf16/tf32 tensor-core product cannot give) and the
// any-shape, any-dtype second implementation the tensor-core kernels are cross-checked
// against on the GPU. All arithmetic is float32 with expf/logf; every output element is
// produced by exactly one thread in a fixed summation order, so results are deterministic.
//
// Work decomposition mirrors the two reference kernels:
//   simt_fwd_kernel  — query-row owner, like K1 (jvp_fwd_sm90.py:307): O, LSE, O_dot, z1 and the
//                      row statistics dpsum / ddot.
//   simt_dq_kernel   — query-row owner: dQ and dQ_dot.
//   simt_dkv_kernel  — key-row owner, like K2 (hvp_bwd_sm90.py:421): dK, dV, dK_dot, dV_dot,
//                      looping over the G query heads that share a kv head.
// One warp owns a row; its 32 lanes each take one row of the streamed 32-row tile for the
// S-like dot products, then each lane owns head_dim/32 output columns for the accumulations.
#include "fb_params.h"
#include "../../include/flashback_b200.h"

namespace fb {

namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = 2;
constexpr int kOwn = kWarps * kRowsPerWarp;  // owner rows per CTA
constexpr int kTile = 32;                    // streamed rows per tile (one per lane)
constexpr int kThreads = kWarps * 32;

__device__ __forceinline__ float warp_sum(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
  return x;
}
__device__ __forceinline__ float warp_max(float x) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) x = fmaxf(x, __shfl_xor_sync(0xffffffffu, x, o));
  return x;
}

// dst[r][0..D) (leading dimension D+1) <- rows [row0, row0+n) of t for `head`; rows >= nvalid and
// absent tensors read as zero.
template <typename T, int D>
__device__ __forceinline__ void load_rows(float* dst, const SeqT& t, int head, int64_t row0, int nvalid, int n) {
  constexpr int LD = D + 1;
  const T* base = t.ptr ? reinterpret_cast<const T*>(t.ptr) + (int64_t)head * t.head_stride : nullptr;
  for (int idx = threadIdx.x; idx < n * D; idx += kThreads) {
    int r = idx / D, d = idx - r * D;
    float x = 0.f;
    if (base && r < nvalid) x = to_f<T>(base[(row0 + r) * t.row_stride + d]);
    dst[r * LD + d] = x;
  }
}

template <typename T, int D>
__device__ __forceinline__ void store_row(const SeqT& t, int head, int64_t row, int lane, const float (&acc)[D / 32], float mul) {
  if (!t.ptr) return;
  T* dst = reinterpret_cast<T*>(t.ptr) + (int64_t)head * t.head_stride + row * t.row_stride;
#pragma unroll
  for (int i = 0; i < D / 32; ++i) dst[lane + 32 * i] = from_f<T>(acc[i] * mul);
}

// ---------------------------------------------------------------------------------------------
// Forward / JVP forward
// ---------------------------------------------------------------------------------------------
template <typename T, int D, bool TANGENT>
__global__ void __launch_bounds__(kThreads) simt_fwd_kernel(Params p) {
  extern __shared__ float smem[];
  constexpr int LD = D + 1;
  constexpr int NC = D / 32;
  float* qs = smem;
  float* qds = qs + kOwn * LD;
  float* ks = qds + kOwn * LD;
  float* kds = ks + kTile * LD;
  float* vs = kds + kTile * LD;
  float* vds = vs + kTile * LD;

  const int b = blockIdx.z, h = blockIdx.y, hk = h / (p.Hq / p.Hkv);
  const SeqInfo si = seq_info(p, b);
  const int m0 = blockIdx.x * kOwn;
  if (m0 >= si.sq) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = min(kOwn, si.sq - m0);
  load_rows<T, D>(qs, p.q, h, si.q0 + m0, nq, kOwn);
  if (TANGENT) load_rows<T, D>(qds, p.qd, h, si.q0 + m0, nq, kOwn);
  int n_end = si.sk;
  if (p.causal) n_end = max(0, min(si.sk, m0 + kOwn + causal_off(p, si, m0 + kOwn - 1)));

  float lse[kRowsPerWarp];
  if (p.lse_known) {
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      int i = m0 + warp * kRowsPerWarp + r;
      lse[r] = i < si.sq ? p.lse[(int64_t)h * p.Tq + si.q0 + i] : -INFINITY;
    }
  } else {
    float m_run[kRowsPerWarp], l_run[kRowsPerWarp];
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) { m_run[r] = -INFINITY; l_run[r] = 0.f; }
    for (int n0 = 0; n0 < n_end; n0 += kTile) {
      __syncthreads();
      load_rows<T, D>(ks, p.k, hk, si.k0 + n0, min(kTile, si.sk - n0), kTile);
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const int lr = warp * kRowsPerWarp + r, i = m0 + lr, j = n0 + lane;
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(qs[lr * LD + d], ks[lane * LD + d], s);
        s *= p.scale;
        bool ok = i < si.sq && j < si.sk && (!p.causal || j <= i + pair_off(p, si, i, j));
        if (ok) {
          float mn = fmaxf(m_run[r], s);
          l_run[r] = l_run[r] * expf(m_run[r] - mn) + expf(s - mn);
          m_run[r] = mn;
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      float M = warp_max(m_run[r]);
      float l = (m_run[r] == -INFINITY) ? 0.f : l_run[r] * expf(m_run[r] - M);
      l = warp_sum(l);
      lse[r] = l > 0.f ? M + logf(l) : -INFINITY;
    }
  }

  float acc_o[kRowsPerWarp][NC], acc_d[kRowsPerWarp][NC], zp[kRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    zp[r] = 0.f;
#pragma unroll
    for (int c = 0; c < NC; ++c) { acc_o[r][c] = 0.f; acc_d[r][c] = 0.f; }
  }
  for (int n0 = 0; n0 < n_end; n0 += kTile) {
    const int nk = min(kTile, si.sk - n0);
    __syncthreads();
    load_rows<T, D>(ks, p.k, hk, si.k0 + n0, nk, kTile);
    load_rows<T, D>(vs, p.v, hk, si.k0 + n0, nk, kTile);
    if (TANGENT) {
      load_rows<T, D>(kds, p.kd, hk, si.k0 + n0, nk, kTile);
      load_rows<T, D>(vds, p.vd, hk, si.k0 + n0, nk, kTile);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int lr = warp * kRowsPerWarp + r, i = m0 + lr, j = n0 + lane;
      float s = 0.f, sd = 0.f;
      for (int d = 0; d < D; ++d) {
        float qv = qs[lr * LD + d], kv = ks[lane * LD + d];
        s = fmaf(qv, kv, s);
        if (TANGENT) { sd = fmaf(qds[lr * LD + d], kv, sd); sd = fmaf(qv, kds[lane * LD + d], sd); }
      }
      s *= p.scale; sd *= p.scale;
      bool ok = i < si.sq && j < si.sk && (!p.causal || j <= i + pair_off(p, si, i, j)) && lse[r] != -INFINITY;
      float pr = ok ? expf(s - lse[r]) : 0.f;
      float w = pr * sd;
      zp[r] += w;
      for (int jj = 0; jj < kTile; ++jj) {
        float pj = __shfl_sync(0xffffffffu, pr, jj);
        float wj = __shfl_sync(0xffffffffu, w, jj);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float vv = vs[jj * LD + lane + 32 * c];
          acc_o[r][c] = fmaf(pj, vv, acc_o[r][c]);
          if (TANGENT) { acc_d[r][c] = fmaf(wj, vv, acc_d[r][c]); acc_d[r][c] = fmaf(pj, vds[jj * LD + lane + 32 * c], acc_d[r][c]); }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int i = m0 + warp * kRowsPerWarp + r;
    if (i >= si.sq) continue;
    const int64_t row = si.q0 + i;
    const int64_t srow = (int64_t)h * p.Tq + row;
    float o[NC];
    if (p.lse_known) {
      const T* op = reinterpret_cast<const T*>(p.o.ptr) + (int64_t)h * p.o.head_stride + row * p.o.row_stride;
#pragma unroll
      for (int c = 0; c < NC; ++c) o[c] = to_f<T>(op[lane + 32 * c]);
    } else {
#pragma unroll
      for (int c = 0; c < NC; ++c) o[c] = acc_o[r][c];
      store_row<T, D>(p.o, h, row, lane, o, 1.f);
      if (lane == 0) p.lse[srow] = lse[r];
    }
    float od[NC];
    if (TANGENT) {
      float z = warp_sum(zp[r]);
#pragma unroll
      for (int c = 0; c < NC; ++c) od[c] = acc_d[r][c] - z * o[c];
      store_row<T, D>(p.od, h, row, lane, od, 1.f);
      if (lane == 0) p.z1[srow] = z;
    }
    if (p.dout.ptr) {
      const T* dop = reinterpret_cast<const T*>(p.dout.ptr) + (int64_t)h * p.dout.head_stride + row * p.dout.row_stride;
      const T* ddp = p.doutd.ptr ? reinterpret_cast<const T*>(p.doutd.ptr) + (int64_t)h * p.doutd.head_stride + row * p.doutd.row_stride : nullptr;
      float a = 0.f, bsum = 0.f;
#pragma unroll
      for (int c = 0; c < NC; ++c) {
        float g = to_f<T>(dop[lane + 32 * c]);
        a = fmaf(g, o[c], a);
        if (TANGENT) {
          bsum = fmaf(g, od[c], bsum);
          if (ddp) bsum = fmaf(to_f<T>(ddp[lane + 32 * c]), o[c], bsum);
        }
      }
      a = warp_sum(a);
      if (lane == 0) p.dpsum[srow] = a;
      if (TANGENT) {
        bsum = warp_sum(bsum);
        if (lane == 0) p.ddot[srow] = bsum;
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, query-row owner: dQ, dQ_dot
// ---------------------------------------------------------------------------------------------
template <typename T, int D, bool TANGENT>
__global__ void __launch_bounds__(kThreads) simt_dq_kernel(Params p) {
  extern __shared__ float smem[];
  constexpr int LD = D + 1;
  constexpr int NC = D / 32;
  float* qs = smem;
  float* qds = qs + kOwn * LD;
  float* dos = qds + kOwn * LD;
  float* dods = dos + kOwn * LD;
  float* ks = dods + kOwn * LD;
  float* kds = ks + kTile * LD;
  float* vs = kds + kTile * LD;
  float* vds = vs + kTile * LD;

  const int b = blockIdx.z, h = blockIdx.y, hk = h / (p.Hq / p.Hkv);
  const SeqInfo si = seq_info(p, b);
  const int m0 = blockIdx.x * kOwn;
  if (m0 >= si.sq) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nq = min(kOwn, si.sq - m0);
  load_rows<T, D>(qs, p.q, h, si.q0 + m0, nq, kOwn);
  load_rows<T, D>(dos, p.dout, h, si.q0 + m0, nq, kOwn);
  if (TANGENT) {
    load_rows<T, D>(qds, p.qd, h, si.q0 + m0, nq, kOwn);
    load_rows<T, D>(dods, p.doutd, h, si.q0 + m0, nq, kOwn);
  }
  int n_end = si.sk;
  if (p.causal) n_end = max(0, min(si.sk, m0 + kOwn + causal_off(p, si, m0 + kOwn - 1)));

  float lse[kRowsPerWarp], dps[kRowsPerWarp], z1[kRowsPerWarp], ddt[kRowsPerWarp];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    int i = m0 + warp * kRowsPerWarp + r;
    bool ok = i < si.sq;
    int64_t srow = (int64_t)h * p.Tq + si.q0 + i;
    lse[r] = ok ? p.lse[srow] : -INFINITY;
    dps[r] = ok ? p.dpsum[srow] : 0.f;
    z1[r] = (ok && TANGENT) ? p.z1[srow] : 0.f;
    ddt[r] = (ok && TANGENT) ? p.ddot[srow] : 0.f;
  }
  float acc[kRowsPerWarp][NC], accd[kRowsPerWarp][NC];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
    for (int c = 0; c < NC; ++c) { acc[r][c] = 0.f; accd[r][c] = 0.f; }

  for (int n0 = 0; n0 < n_end; n0 += kTile) {
    const int nk = min(kTile, si.sk - n0);
    __syncthreads();
    load_rows<T, D>(ks, p.k, hk, si.k0 + n0, nk, kTile);
    load_rows<T, D>(vs, p.v, hk, si.k0 + n0, nk, kTile);
    if (TANGENT) {
      load_rows<T, D>(kds, p.kd, hk, si.k0 + n0, nk, kTile);
      load_rows<T, D>(vds, p.vd, hk, si.k0 + n0, nk, kTile);
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kRowsPerWarp; ++r) {
      const int lr = warp * kRowsPerWarp + r, i = m0 + lr, j = n0 + lane;
      float s = 0.f, sd = 0.f, dp = 0.f, dpd = 0.f;
      for (int d = 0; d < D; ++d) {
        float qv = qs[lr * LD + d], kv = ks[lane * LD + d], gv = dos[lr * LD + d], vv = vs[lane * LD + d];
        s = fmaf(qv, kv, s);
        dp = fmaf(gv, vv, dp);
        if (TANGENT) {
          sd = fmaf(qds[lr * LD + d], kv, sd);
          sd = fmaf(qv, kds[lane * LD + d], sd);
          dpd = fmaf(gv, vds[lane * LD + d], dpd);
          dpd = fmaf(dods[lr * LD + d], vv, dpd);
        }
      }
      s *= p.scale; sd *= p.scale;
      bool ok = i < si.sq && j < si.sk && (!p.causal || j <= i + pair_off(p, si, i, j)) && lse[r] != -INFINITY;
      float pr = ok ? expf(s - lse[r]) : 0.f;
      float a = dp - dps[r];
      float ds = pr * a;
      float dsd = 0.f;
      if (TANGENT) dsd = pr * (sd - z1[r]) * a + pr * (dpd - ddt[r]);
      for (int jj = 0; jj < kTile; ++jj) {
        float dsj = __shfl_sync(0xffffffffu, ds, jj);
        float dsdj = __shfl_sync(0xffffffffu, dsd, jj);
#pragma unroll
        for (int c = 0; c < NC; ++c) {
          float kv = ks[jj * LD + lane + 32 * c];
          acc[r][c] = fmaf(dsj, kv, acc[r][c]);
          if (TANGENT) { accd[r][c] = fmaf(dsdj, kv, accd[r][c]); accd[r][c] = fmaf(dsj, kds[jj * LD + lane + 32 * c], accd[r][c]); }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int i = m0 + warp * kRowsPerWarp + r;
    if (i >= si.sq) continue;
    store_row<T, D>(p.dq, h, si.q0 + i, lane, acc[r], p.scale);
    if (TANGENT) store_row<T, D>(p.dqd, h, si.q0 + i, lane, accd[r], p.scale);
  }
}

// ---------------------------------------------------------------------------------------------
// Backward, key-row owner: dK, dV, dK_dot, dV_dot (sums over the G query heads of a kv head)
// ---------------------------------------------------------------------------------------------
template <typename T, int D, bool TANGENT>
__global__ void __launch_bounds__(kThreads) simt_dkv_kernel(Params p) {
  extern __shared__ float smem[];
  constexpr int LD = D + 1;
  constexpr int NC = D / 32;
  float* ks = smem;
  float* kds = ks + kOwn * LD;
  float* vs = kds + kOwn * LD;
  float* vds = vs + kOwn * LD;
  float* qs = vds + kOwn * LD;
  float* qds = qs + kTile * LD;
  float* dos = qds + kTile * LD;
  float* dods = dos + kTile * LD;
  float* st = dods + kTile * LD;  // [4][kTile]: lse, dpsum, z1, ddot

  const int b = blockIdx.z, hk = blockIdx.y, G = p.Hq / p.Hkv;
  const SeqInfo si = seq_info(p, b);
  const int n0 = blockIdx.x * kOwn;
  if (n0 >= si.sk) return;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int nk = min(kOwn, si.sk - n0);
  load_rows<T, D>(ks, p.k, hk, si.k0 + n0, nk, kOwn);
  load_rows<T, D>(vs, p.v, hk, si.k0 + n0, nk, kOwn);
  if (TANGENT) {
    load_rows<T, D>(kds, p.kd, hk, si.k0 + n0, nk, kOwn);
    load_rows<T, D>(vds, p.vd, hk, si.k0 + n0, nk, kOwn);
  }
  int m_start = 0;
  if (p.causal) m_start = first_query_of_key(p, si, n0) / kTile * kTile;

  float adk[kRowsPerWarp][NC], adv[kRowsPerWarp][NC], adkd[kRowsPerWarp][NC], advd[kRowsPerWarp][NC];
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r)
#pragma unroll
    for (int c = 0; c < NC; ++c) { adk[r][c] = adv[r][c] = adkd[r][c] = advd[r][c] = 0.f; }

  for (int g = 0; g < G; ++g) {
    const int h = hk * G + g;
    for (int m0 = m_start; m0 < si.sq; m0 += kTile) {
      const int nq = min(kTile, si.sq - m0);
      __syncthreads();
      load_rows<T, D>(qs, p.q, h, si.q0 + m0, nq, kTile);
      load_rows<T, D>(dos, p.dout, h, si.q0 + m0, nq, kTile);
      if (TANGENT) {
        load_rows<T, D>(qds, p.qd, h, si.q0 + m0, nq, kTile);
        load_rows<T, D>(dods, p.doutd, h, si.q0 + m0, nq, kTile);
      }
      if (threadIdx.x < kTile) {
        int i = m0 + threadIdx.x;
        bool ok = i < si.sq;
        int64_t srow = (int64_t)h * p.Tq + si.q0 + i;
        st[0 * kTile + threadIdx.x] = ok ? p.lse[srow] : -INFINITY;
        st[1 * kTile + threadIdx.x] = ok ? p.dpsum[srow] : 0.f;
        st[2 * kTile + threadIdx.x] = (ok && TANGENT) ? p.z1[srow] : 0.f;
        st[3 * kTile + threadIdx.x] = (ok && TANGENT) ? p.ddot[srow] : 0.f;
      }
      __syncthreads();
#pragma unroll
      for (int r = 0; r < kRowsPerWarp; ++r) {
        const int lr = warp * kRowsPerWarp + r, j = n0 + lr, i = m0 + lane;
        float s = 0.f, sd = 0.f, dp = 0.f, dpd = 0.f;
        for (int d = 0; d < D; ++d) {
          float qv = qs[lane * LD + d], kv = ks[lr * LD + d], gv = dos[lane * LD + d], vv = vs[lr * LD + d];
          s = fmaf(qv, kv, s);
          dp = fmaf(gv, vv, dp);
          if (TANGENT) {
            sd = fmaf(qds[lane * LD + d], kv, sd);
            sd = fmaf(qv, kds[lr * LD + d], sd);
            dpd = fmaf(gv, vds[lr * LD + d], dpd);
            dpd = fmaf(dods[lane * LD + d], vv, dpd);
          }
        }
        s *= p.scale; sd *= p.scale;
        const float lse = st[lane];
        bool ok = i < si.sq && j < si.sk && (!p.causal || j <= i + pair_off(p, si, i, j)) && lse != -INFINITY;
        float pr = ok ? expf(s - lse) : 0.f;
        float a = dp - st[kTile + lane];
        float ds = pr * a;
        float pd = 0.f, dsd = 0.f;
        if (TANGENT) { pd = pr * (sd - st[2 * kTile + lane]); dsd = pd * a + pr * (dpd - st[3 * kTile + lane]); }
        for (int ii = 0; ii < kTile; ++ii) {
          float pi = __shfl_sync(0xffffffffu, pr, ii);
          float dsi = __shfl_sync(0xffffffffu, ds, ii);
          float pdi = __shfl_sync(0xffffffffu, pd, ii);
          float dsdi = __shfl_sync(0xffffffffu, dsd, ii);
#pragma unroll
          for (int c = 0; c < NC; ++c) {
            float gv = dos[ii * LD + lane + 32 * c], qv = qs[ii * LD + lane + 32 * c];
            adv[r][c] = fmaf(pi, gv, adv[r][c]);
            adk[r][c] = fmaf(dsi, qv, adk[r][c]);
            if (TANGENT) {
              advd[r][c] = fmaf(pdi, gv, advd[r][c]);
              advd[r][c] = fmaf(pi, dods[ii * LD + lane + 32 * c], advd[r][c]);
              adkd[r][c] = fmaf(dsdi, qv, adkd[r][c]);
              adkd[r][c] = fmaf(dsi, qds[ii * LD + lane + 32 * c], adkd[r][c]);
            }
          }
        }
      }
    }
  }
#pragma unroll
  for (int r = 0; r < kRowsPerWarp; ++r) {
    const int j = n0 + warp * kRowsPerWarp + r;
    if (j >= si.sk) continue;
    store_row<T, D>(p.dk, hk, si.k0 + j, lane, adk[r], p.scale);
    store_row<T, D>(p.dv, hk, si.k0 + j, lane, adv[r], 1.f);
    if (TANGENT) {
      store_row<T, D>(p.dkd, hk, si.k0 + j, lane, adkd[r], p.scale);
      store_row<T, D>(p.dvd, hk, si.k0 + j, lane, advd[r], 1.f);
    }
  }
}

// ---------------------------------------------------------------------------------------------
// Row statistics: dpsum = rowsum(dO*O), ddot = rowsum(dO_dot*O + dO*O_dot). One warp per row.
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads) row_stats_kernel(Params p) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int64_t row = (int64_t)blockIdx.x * kWarps + warp;
  const int h = blockIdx.y;
  if (row >= p.Tq) return;
  auto rowp = [&](const SeqT& t) -> const T* {
    return t.ptr ? reinterpret_cast<const T*>(t.ptr) + (int64_t)h * t.head_stride + row * t.row_stride : nullptr;
  };
  const T *o = rowp(p.o), *g = rowp(p.dout), *od = rowp(p.od), *gd = rowp(p.doutd);
  float a = 0.f, bsum = 0.f;
  for (int d = lane; d < p.D; d += 32) {
    float ov = to_f<T>(o[d]), gv = to_f<T>(g[d]);
    a = fmaf(gv, ov, a);
    if (od) bsum = fmaf(gv, to_f<T>(od[d]), bsum);
    if (gd) bsum = fmaf(to_f<T>(gd[d]), ov, bsum);
  }
  a = warp_sum(a);
  bsum = warp_sum(bsum);
  if (lane == 0) {
    p.dpsum[(int64_t)h * p.Tq + row] = a;
    if (p.ddot) p.ddot[(int64_t)h * p.Tq + row] = bsum;
  }
}

template <typename K>
int set_smem(K kernel, size_t bytes) {
  cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  return e == cudaSuccess ? 0 : FB_ERR_CUDA;
}

template <typename T, int D, bool TANGENT>
int fwd_impl(const Params& p, cudaStream_t s) {
  size_t bytes = sizeof(float) * (size_t)(D + 1) * (2 * kOwn + 4 * kTile);
  auto kern = simt_fwd_kernel<T, D, TANGENT>;
  if (set_smem(kern, bytes)) return FB_ERR_CUDA;
  dim3 grid((p.Sq + kOwn - 1) / kOwn, p.Hq, p.B);
  kern<<<grid, kThreads, bytes, s>>>(p);
  return cudaGetLastError() == cudaSuccess ? 1 : FB_ERR_CUDA;
}

template <typename T, int D, bool TANGENT>
int bwd_impl(const Params& p, cudaStream_t s) {
  int n = 0;
  if (p.dq.ptr || p.dqd.ptr) {
    size_t bytes = sizeof(float) * (size_t)(D + 1) * (4 * kOwn + 4 * kTile);
    auto kern = simt_dq_kernel<T, D, TANGENT>;
    if (set_smem(kern, bytes)) return FB_ERR_CUDA;
    dim3 grid((p.Sq + kOwn - 1) / kOwn, p.Hq, p.B);
    kern<<<grid, kThreads, bytes, s>>>(p);
    if (cudaGetLastError() != cudaSuccess) return FB_ERR_CUDA;
    ++n;
  }
  if (p.dk.ptr || p.dv.ptr || p.dkd.ptr || p.dvd.ptr) {
    size_t bytes = sizeof(float) * ((size_t)(D + 1) * (4 * kOwn + 4 * kTile) + 4 * kTile);
    auto kern = simt_dkv_kernel<T, D, TANGENT>;
    if (set_smem(kern, bytes)) return FB_ERR_CUDA;
    dim3 grid((p.Sk + kOwn - 1) / kOwn, p.Hkv, p.B);
    kern<<<grid, kThreads, bytes, s>>>(p);
    if (cudaGetLastError() != cudaSuccess) return FB_ERR_CUDA;
    ++n;
  }
  return n;
}

template <typename T>
int fwd_dispatch(const Params& p, cudaStream_t s) {
  const bool t = p.qd.ptr != nullptr;
  if (p.D == 64) return t ? fwd_impl<T, 64, true>(p, s) : fwd_impl<T, 64, false>(p, s);
  return t ? fwd_impl<T, 128, true>(p, s) : fwd_impl<T, 128, false>(p, s);
}
template <typename T>
int bwd_dispatch(const Params& p, cudaStream_t s) {
  const bool t = p.qd.ptr != nullptr;
  if (p.D == 64) return t ? bwd_impl<T, 64, true>(p, s) : bwd_impl<T, 64, false>(p, s);
  return t ? bwd_impl<T, 128, true>(p, s) : bwd_impl<T, 128, false>(p, s);
}

}  // namespace

int launch_simt_fwd(const Params& p, cudaStream_t s) {
  switch (p.dtype) {
    case FB_BF16: return fwd_dispatch<__nv_bfloat16>(p, s);
    case FB_F16: return fwd_dispatch<__half>(p, s);
    case FB_F32: return fwd_dispatch<float>(p, s);
  }
  return FB_ERR_DTYPE;
}

int launch_simt_bwd(const Params& p, cudaStream_t s) {
  switch (p.dtype) {
    case FB_BF16: return bwd_dispatch<__nv_bfloat16>(p, s);
    case FB_F16: return bwd_dispatch<__half>(p, s);
    case FB_F32: return bwd_dispatch<float>(p, s);
  }
  return FB_ERR_DTYPE;
}

int launch_row_stats(const Params& p, cudaStream_t s) {
  dim3 grid((unsigned)((p.Tq + kWarps - 1) / kWarps), p.Hq);
  switch (p.dtype) {
    case FB_BF16: row_stats_kernel<__nv_bfloat16><<<grid, kThreads, 0, s>>>(p); break;
    case FB_F16: row_stats_kernel<__half><<<grid, kThreads, 0, s>>>(p); break;
    case FB_F32: row_stats_kernel<float><<<grid, kThreads, 0, s>>>(p); break;
    default: return FB_ERR_DTYPE;
  }
  return cudaGetLastError() == cudaSuccess ? 1 : FB_ERR_CUDA;
}

// out[i] = sum over the slots s with (i mod period) < valid[s] of slots[s * slot_stride + i]: adds up, in
// a fixed order, the float32 partial results that the GPUs of a sequence-sharded backward stored into
// this GPU's memory (fb_sum_slots). HBM-bound: reads each valid float once, writes count floats;
// grid-stride over 16-byte units.
namespace {
struct SlotCounts {
  int64_t valid4[8];  // valid 16-byte units per slot
};
__global__ void __launch_bounds__(256) sum_slots_kernel(const float4* __restrict__ slots, int n_slots, int64_t slot_stride4, int64_t count4,
                                                        int64_t period4, SlotCounts sc, float4* __restrict__ out) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < count4; i += (int64_t)gridDim.x * blockDim.x) {
    const int64_t in_block = i % period4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n_slots; ++s) {
      if (in_block < sc.valid4[s]) {
        const float4 v = slots[s * slot_stride4 + i];
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    out[i] = acc;
  }
}
}  // namespace

int launch_sum_slots(const float* slots, int n_slots, int64_t slot_stride, int64_t count, int64_t period, const int64_t* valid, float* out,
                     cudaStream_t stream) {
  const int64_t count4 = count / 4, period4 = period > 0 ? period / 4 : count4;
  SlotCounts sc;
  for (int s = 0; s < 8; ++s) sc.valid4[s] = s < n_slots ? (valid ? (valid[s] < period4 * 4 ? valid[s] : period4 * 4) / 4 : period4) : 0;
  int64_t blocks = (count4 + 255) / 256;
  const int64_t cap = 148 * 8;  // 8 CTAs of 256 threads per SM
  if (blocks > cap) blocks = cap;
  sum_slots_kernel<<<(unsigned)blocks, 256, 0, stream>>>(reinterpret_cast<const float4*>(slots), n_slots, slot_stride / 4, count4, period4, sc,
                                                         reinterpret_cast<float4*>(out));
  return cudaGetLastError() == cudaSuccess ? 1 : FB_ERR_CUDA;
}

}  // namespace fb
