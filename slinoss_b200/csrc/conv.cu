// Depthwise causal conv1d (widths 2..4) on channel-last activations for sm_100a.
//
// y[b,t,c] = bias[c] + sum_j w[c,j] * cat[b, t+j, c],  cat = [state (W-1), x]
// (slinoss/layers/mixer.py:420-454; cross-correlation as F.conv1d).  The input
// may be a column slice of a wider row-major matrix (row stride > channels),
// which is how the mixer hands over the value slice of its input projection, so
// no contiguous copy or transpose is ever made.
//
// One thread owns VEC adjacent channels and walks a tile of tokens with the last three
// inputs in registers: one vector load and one vector store per channel-vector-token, i.e.
// the algorithmic 4 bytes per channel-token forward and 6 backward for half types.
// The aligned kernels (*_staged_kernel) bring their rows from global to shared memory with
// per-thread cp.async rings (every thread copies exactly the slices it reads, so there is
// no barrier), test nothing per row in the interior of a tile, and the backward does its
// arithmetic on channel pairs (fma.rn.f32x2) and sizes its tiles so that the grid is a
// whole number of waves.  The plain kernels (*_kernel, one channel per thread) serve
// unaligned inputs.
#include <initializer_list>
#include <type_traits>
#include <mutex>

#include "common.cuh"

namespace slx {

constexpr int kConvThreads = 128;
constexpr int kConvAhead = 8;      // plain kernels: rows each thread requests ahead of its walk (backward: x and dy)
constexpr int kConvAheadFwd = 8;   // plain forward: x only
constexpr int kConvVec = 4;    // staged backward: channels per thread (8-byte slices of half types, 16-byte of fp32)

template <typename T, int VEC>
__device__ __forceinline__ void ldv(const T *p, float (&v)[VEC]) {
  if constexpr (VEC * sizeof(T) == 16) {
    uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = to_f(e[i]);
  } else if constexpr (VEC * sizeof(T) == 8) {
    uint2 raw = *reinterpret_cast<const uint2 *>(p);
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = to_f(e[i]);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) v[i] = to_f(p[i]);
  }
}
template <typename T, int VEC>
__device__ __forceinline__ void stv(T *p, const float (&v)[VEC]) {
  if constexpr (VEC * sizeof(T) == 16) {
    uint4 raw;
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) e[i] = from_f<T>(v[i]);
    *reinterpret_cast<uint4 *>(p) = raw;
  } else if constexpr (VEC * sizeof(T) == 8) {
    uint2 raw;
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < VEC; ++i) e[i] = from_f<T>(v[i]);
    *reinterpret_cast<uint2 *>(p) = raw;
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) p[i] = from_f<T>(v[i]);
  }
}

// One thread's slice of a row as it lies in memory (kept packed while it waits in registers)
template <typename T, int VEC>
struct alignas(VEC * sizeof(T) >= 16 ? 16 : 8) RowSlice {
  T v[VEC];
};
template <typename T, int VEC>
__device__ __forceinline__ void ld_raw(const T *p, RowSlice<T, VEC> &r) {
  if constexpr (VEC * sizeof(T) == 16) {
    *reinterpret_cast<uint4 *>(r.v) = *reinterpret_cast<const uint4 *>(p);
  } else if constexpr (VEC * sizeof(T) == 8) {
    *reinterpret_cast<uint2 *>(r.v) = *reinterpret_cast<const uint2 *>(p);
  } else {
#pragma unroll
    for (int i = 0; i < VEC; ++i) r.v[i] = p[i];
  }
}

struct ConvDims {
  int batch, T, C, W, silu;
  long long xs, xbs;  // row stride / batch stride of x (elements)
};

// x at token index tau (may be negative: reads the carried state, else zero)
template <typename T, int VEC>
__device__ __forceinline__ void load_cat(const T *x, const T *state, const ConvDims &d, int b, int tau, int c0,
                                         float (&v)[VEC]) {
  if (tau >= 0) {
    ldv<T, VEC>(x + (long long)b * d.xbs + (long long)tau * d.xs + c0, v);
  } else {
    int i = tau + (d.W - 1);
#pragma unroll
    for (int e = 0; e < VEC; ++e)
      v[e] = (state && i >= 0) ? to_f(state[((long long)b * d.C + c0 + e) * (d.W - 1) + i]) : 0.f;
  }
}

// taps right-aligned into a window of four: w4[k] multiplies x[t-3+k]
template <typename T, int VEC>
__device__ __forceinline__ void load_taps(const T *weight, const T *bias, const ConvDims &d, int c0,
                                          float (&w4)[4][VEC], float (&bv)[VEC]) {
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      int j = k - (4 - d.W);
      w4[k][e] = (j >= 0) ? to_f(weight[(long long)(c0 + e) * d.W + j]) : 0.f;
    }
    bv[e] = bias ? to_f(bias[c0 + e]) : 0.f;
  }
}

template <typename T, int VEC>
__global__ void __launch_bounds__(kConvThreads) cconv1d_fwd_kernel(const T *__restrict__ x,
                                                                   const T *__restrict__ weight,
                                                                   const T *__restrict__ bias,
                                                                   const T *__restrict__ state, T *__restrict__ y,
                                                                   T *__restrict__ next_state, ConvDims d, int tile) {
  const int c0 = (blockIdx.x * kConvThreads + threadIdx.x) * VEC;
  if (c0 >= d.C) return;
  const int b = blockIdx.z;
  const int t_lo = blockIdx.y * tile, t_hi = min(d.T, t_lo + tile);
  float w4[4][VEC], bv[VEC];
  load_taps<T, VEC>(weight, bias, d, c0, w4, bv);
  float x0[VEC], x1[VEC], x2[VEC], x3[VEC];
  load_cat<T, VEC>(x, state, d, b, t_lo - 3, c0, x0);
  load_cat<T, VEC>(x, state, d, b, t_lo - 2, c0, x1);
  load_cat<T, VEC>(x, state, d, b, t_lo - 1, c0, x2);
  // kConvAheadFwd rows are requested before any of them is used, so that each thread keeps
  // several independent loads in flight along its otherwise sequential walk
  for (int tb = t_lo; tb < t_hi; tb += kConvAheadFwd) {
    RowSlice<T, VEC> xr[kConvAheadFwd];
#pragma unroll
    for (int u = 0; u < kConvAheadFwd; ++u)
      if (tb + u < t_hi) ld_raw<T, VEC>(x + (long long)b * d.xbs + (long long)(tb + u) * d.xs + c0, xr[u]);
#pragma unroll
    for (int u = 0; u < kConvAheadFwd; ++u) {
      const int t = tb + u;
      if (t >= t_hi) break;
      float o[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        x3[e] = to_f(xr[u].v[e]);
        float acc = bv[e];
        acc = fmaf(w4[0][e], x0[e], acc);
        acc = fmaf(w4[1][e], x1[e], acc);
        acc = fmaf(w4[2][e], x2[e], acc);
        acc = fmaf(w4[3][e], x3[e], acc);
        if (d.silu) acc = acc / (1.f + expf(-acc));
        o[e] = acc;
        x0[e] = x1[e];
        x1[e] = x2[e];
        x2[e] = x3[e];
      }
      stv<T, VEC>(y + ((long long)b * d.T + t) * d.C + c0, o);
    }
  }
  if (next_state && t_hi == d.T) {
    for (int i = 0; i < d.W - 1; ++i) {
      float v[VEC];
      load_cat<T, VEC>(x, state, d, b, d.T - (d.W - 1) + i, c0, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        next_state[((long long)b * d.C + c0 + e) * (d.W - 1) + i] = from_f<T>(v[e]);
    }
  }
}

// dy with the SiLU derivative folded in (recomputes the pre-activation)
template <typename T, int VEC>
__device__ __forceinline__ void load_dyact(const T *dy, const ConvDims &d, int b, int t, int c0,
                                           const float (&w4)[4][VEC], const float (&bv)[VEC], const float (&xa)[VEC],
                                           const float (&xb)[VEC], const float (&xc)[VEC], const float (&xd)[VEC],
                                           float (&g)[VEC]) {
  if (t >= d.T) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) g[e] = 0.f;
    return;
  }
  ldv<T, VEC>(dy + ((long long)b * d.T + t) * d.C + c0, g);
  if (d.silu) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float pre = bv[e];
      pre = fmaf(w4[0][e], xa[e], pre);
      pre = fmaf(w4[1][e], xb[e], pre);
      pre = fmaf(w4[2][e], xc[e], pre);
      pre = fmaf(w4[3][e], xd[e], pre);
      float s = 1.f / (1.f + expf(-pre));
      g[e] *= s * (1.f + pre * (1.f - s));
    }
  }
}

// same with dy already loaded (raw): g = dy * act'(pre), zero past the end of the sequence
template <typename T, int VEC>
__device__ __forceinline__ void apply_dyact(const ConvDims &d, int t, const float (&w4)[4][VEC], const float (&bv)[VEC],
                                            const float (&xa)[VEC], const float (&xb)[VEC], const float (&xc)[VEC],
                                            const float (&xd)[VEC], const RowSlice<T, VEC> &raw, float (&g)[VEC]) {
  if (t >= d.T) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) g[e] = 0.f;
    return;
  }
#pragma unroll
  for (int e = 0; e < VEC; ++e) g[e] = to_f(raw.v[e]);
  if (d.silu) {
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float pre = bv[e];
      pre = fmaf(w4[0][e], xa[e], pre);
      pre = fmaf(w4[1][e], xb[e], pre);
      pre = fmaf(w4[2][e], xc[e], pre);
      pre = fmaf(w4[3][e], xd[e], pre);
      float s = 1.f / (1.f + expf(-pre));
      g[e] *= s * (1.f + pre * (1.f - s));
    }
  }
}

// Gradient of the carried state (cat index i < W-1  <->  x index tau = i-(W-1)), a kernel of its own so
// that it adds nothing to the register count of the walk: one thread per VEC channels of one batch row,
// dyact[0..2] recomputed from the first three tokens.
template <typename T, int VEC>
__global__ void __launch_bounds__(kConvThreads) cconv1d_bwd_dstate_kernel(
    const T *__restrict__ x, const T *__restrict__ weight, const T *__restrict__ bias, const T *__restrict__ state,
    const T *__restrict__ dy, const T *__restrict__ d_next, float *__restrict__ dstate, ConvDims d) {
  const int c0 = (blockIdx.x * kConvThreads + threadIdx.x) * VEC;
  if (c0 >= d.C) return;
  const int b = blockIdx.z;
  float w4[4][VEC], bv[VEC];
  load_taps<T, VEC>(weight, bias, d, c0, w4, bv);
  float xa[VEC], xb[VEC], xc[VEC], xd[VEC], ga[3][VEC];
  load_cat<T, VEC>(x, state, d, b, -3, c0, xa);
  load_cat<T, VEC>(x, state, d, b, -2, c0, xb);
  load_cat<T, VEC>(x, state, d, b, -1, c0, xc);
#pragma unroll
  for (int t = 0; t < 3; ++t) {
    if (t < d.T) ldv<T, VEC>(x + (long long)b * d.xbs + (long long)t * d.xs + c0, xd);
    load_dyact<T, VEC>(dy, d, b, t, c0, w4, bv, xa, xb, xc, xd, ga[t]);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      xa[e] = xb[e];
      xb[e] = xc[e];
      xc[e] = xd[e];
    }
  }
  for (int i = 0; i < d.W - 1; ++i) {
    const int tau = i - (d.W - 1);
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      float acc = 0.f;
#pragma unroll
      for (int k = 0; k < 4; ++k) {
#pragma unroll
        for (int s = 0; s < 3; ++s)
          if (s == tau + 3 - k) acc = fmaf(w4[k][e], ga[s][e], acc);
      }
      int in = i - d.T;  // next_state index that aliases this state slot when T < W-1
      if (d_next && in >= 0) acc += to_f(d_next[((long long)b * d.C + c0 + e) * (d.W - 1) + in]);
      dstate[((long long)b * d.C + c0 + e) * (d.W - 1) + i] = acc;
    }
  }
}

// Writes this tile's partial sums part[(b*n_tiles + tile)][C][5] = (dw4[0..3], dbias)
template <int VEC>
__device__ __forceinline__ void conv_bwd_partials(float *part, int C, int b, int c0, const float (&dw)[4][VEC],
                                                  const float (&db)[VEC]) {
  float *pp = part + (((long long)b * gridDim.y + blockIdx.y) * C + c0) * 5;
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
#pragma unroll
    for (int k = 0; k < 4; ++k) pp[e * 5 + k] = dw[k][e];
    pp[e * 5 + 4] = db[e];
  }
}

// part[(b*n_tiles + tile)][C][5] = (dw4[0..3], dbias) partial sums of this tile
template <typename T, int VEC>
__global__ void __launch_bounds__(kConvThreads) cconv1d_bwd_kernel(
    const T *__restrict__ x, const T *__restrict__ weight, const T *__restrict__ bias, const T *__restrict__ state,
    const T *__restrict__ dy, const T *__restrict__ d_next, T *__restrict__ dx, float *__restrict__ part, ConvDims d,
    int tile) {
  const int c0 = (blockIdx.x * kConvThreads + threadIdx.x) * VEC;
  if (c0 >= d.C) return;
  const int b = blockIdx.z;
  const int t_lo = blockIdx.y * tile, t_hi = min(d.T, t_lo + tile);
  float w4[4][VEC], bv[VEC];
  load_taps<T, VEC>(weight, bias, d, c0, w4, bv);
  float x0[VEC], x1[VEC], x2[VEC], x3[VEC];
  load_cat<T, VEC>(x, state, d, b, t_lo - 3, c0, x0);
  load_cat<T, VEC>(x, state, d, b, t_lo - 2, c0, x1);
  load_cat<T, VEC>(x, state, d, b, t_lo - 1, c0, x2);
  float g0[VEC], g1[VEC], g2[VEC], g3[VEC];  // dyact[t-3..t]
  float dw[4][VEC], db[VEC];
#pragma unroll
  for (int e = 0; e < VEC; ++e) {
    g0[e] = g1[e] = g2[e] = 0.f;
    db[e] = 0.f;
#pragma unroll
    for (int k = 0; k < 4; ++k) dw[k][e] = 0.f;
  }
  const int t_end = min(d.T + 3, t_hi + 3);
  for (int tb = t_lo; tb < t_end; tb += kConvAhead) {
    RowSlice<T, VEC> xr[kConvAhead], gr[kConvAhead];
#pragma unroll
    for (int u = 0; u < kConvAhead; ++u) {
      const int t = tb + u;
      if (t < t_end && t < d.T) {
        ld_raw<T, VEC>(x + (long long)b * d.xbs + (long long)t * d.xs + c0, xr[u]);
        ld_raw<T, VEC>(dy + ((long long)b * d.T + t) * d.C + c0, gr[u]);
      }
    }
#pragma unroll
    for (int u = 0; u < kConvAhead; ++u) {
    const int t = tb + u;
    if (t >= t_end) break;
    if (t < d.T) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) x3[e] = to_f(xr[u].v[e]);
    }
    apply_dyact<T, VEC>(d, t, w4, bv, x0, x1, x2, x3, gr[u], g3);
    if (t < t_hi) {
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        dw[0][e] = fmaf(g3[e], x0[e], dw[0][e]);
        dw[1][e] = fmaf(g3[e], x1[e], dw[1][e]);
        dw[2][e] = fmaf(g3[e], x2[e], dw[2][e]);
        dw[3][e] = fmaf(g3[e], x3[e], dw[3][e]);
        db[e] += g3[e];
      }
    }
    const int tau = t - 3;  // dx[tau] = sum_k w4[k] dyact[tau+3-k]
    if (tau >= t_lo && tau < t_hi) {
      float o[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) {
        float acc = w4[0][e] * g3[e];
        acc = fmaf(w4[1][e], g2[e], acc);
        acc = fmaf(w4[2][e], g1[e], acc);
        acc = fmaf(w4[3][e], g0[e], acc);
        o[e] = acc;
      }
      const int i = tau - d.T + (d.W - 1);  // position inside next_state, if any
      if (d_next && i >= 0) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] += to_f(d_next[((long long)b * d.C + c0 + e) * (d.W - 1) + i]);
      }
      stv<T, VEC>(dx + ((long long)b * d.T + tau) * d.C + c0, o);
    }
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      x0[e] = x1[e];
      x1[e] = x2[e];
      x2[e] = x3[e];
      g0[e] = g1[e];
      g1[e] = g2[e];
      g2[e] = g3[e];
    }
    }
  }
  conv_bwd_partials<VEC>(part, d.C, b, c0, dw, db);
}

// ---- staged variants: rows travel global -> shared by cp.async, several groups ahead of the walk ----
// Every thread copies exactly the slices it will read itself, so no barrier is needed: the copy groups
// are tracked per thread (commit_group / wait_group).  The ring holds kConvRing groups of G rows; while
// one group is consumed, kConvRing-1 groups are in flight, without holding registers for them.
constexpr int kConvRing = 4;
constexpr int kConvRingFwd = 6;  // forward (one tensor in the ring): 4 measured 3 % slower, 8 slower than 4

template <int BYTES>
__device__ __forceinline__ void cp_async_slice(void *smem_dst, const void *gsrc, bool valid) {
  static_assert(BYTES == 8 || BYTES == 16, "slice of 8 or 16 bytes");
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int n = valid ? BYTES : 0;  // 0 source bytes: the slice is filled with zeros
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(gsrc), "r"(n) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(dst), "l"(gsrc), "r"(n) : "memory");
}
template <int BYTES>
__device__ __forceinline__ void cp_async_slice_full(void *smem_dst, const void *gsrc) {
  static_assert(BYTES == 8 || BYTES == 16, "slice of 8 or 16 bytes");
  const unsigned dst = (unsigned)__cvta_generic_to_shared(smem_dst);
  if constexpr (BYTES == 16)
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gsrc) : "memory");
  else
    asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

template <typename T, int VEC>
constexpr int conv_group_rows() { return sizeof(RowSlice<T, VEC>) == 8 ? 8 : 4; }
template <typename T, int VEC, int RING = kConvRing>
constexpr size_t conv_ring_bytes(int tensors) {
  return (size_t)RING * conv_group_rows<T, VEC>() * tensors * kConvThreads * sizeof(RowSlice<T, VEC>);
}

template <typename T, int VEC, int RING>
__global__ void __launch_bounds__(kConvThreads) cconv1d_bwd_staged_kernel(
    const T *__restrict__ x, const T *__restrict__ weight, const T *__restrict__ bias, const T *__restrict__ state,
    const T *__restrict__ dy, const T *__restrict__ d_next, T *__restrict__ dx, float *__restrict__ part, ConvDims d,
    int tile) {
  using Slice = RowSlice<T, VEC>;
  constexpr int G = conv_group_rows<T, VEC>();
  extern __shared__ __align__(16) unsigned char conv_ring[];
  const int c0 = (blockIdx.x * kConvThreads + threadIdx.x) * VEC;
  if (c0 >= d.C) return;
  Slice *ring = reinterpret_cast<Slice *>(conv_ring) + threadIdx.x;  // [RING*G rows][x, dy][thread]
  const int b = blockIdx.z;
  const int t_lo = blockIdx.y * tile, t_hi = min(d.T, t_lo + tile);
  const int t_end = min(d.T + 3, t_hi + 3);
  const int n_grp = (t_end - t_lo + G - 1) / G;
  const T *xb = x + (long long)b * d.xbs + c0;
  const T *gb = dy + (long long)b * d.T * d.C + c0;
  // requests the rows of group grp (rows past the tile or the sequence are filled with zeros) and closes
  // the group; past the last group only the (empty) group is closed, which keeps the wait count uniform
  const int t_lim = min(t_end, d.T);  // rows at or past it are not read
#define SLX_CONV_ISSUE(grp_)                                                                                     \
  do {                                                                                                           \
    const int gi_ = (grp_);                                                                                      \
    if (gi_ < n_grp) {                                                                                           \
      Slice *s_ = ring + (size_t)(gi_ % RING) * G * 2 * kConvThreads;                                       \
      const int t0_ = t_lo + gi_ * G;                                                                            \
      const T *px_ = xb + (long long)t0_ * d.xs, *pg_ = gb + (long long)t0_ * d.C;                               \
      if (t0_ + G <= t_lim) {                                                                                    \
        _Pragma("unroll") for (int u_ = 0; u_ < G; ++u_) {                                                       \
          cp_async_slice_full<sizeof(Slice)>(s_ + (u_ * 2 + 0) * kConvThreads, px_ + (long long)u_ * d.xs);      \
          cp_async_slice_full<sizeof(Slice)>(s_ + (u_ * 2 + 1) * kConvThreads, pg_ + (long long)u_ * d.C);       \
        }                                                                                                        \
      } else {                                                                                                   \
        _Pragma("unroll") for (int u_ = 0; u_ < G; ++u_) {                                                       \
          const bool ok_ = t0_ + u_ < t_lim;                                                                     \
          cp_async_slice<sizeof(Slice)>(s_ + (u_ * 2 + 0) * kConvThreads, ok_ ? px_ + (long long)u_ * d.xs : x, ok_); \
          cp_async_slice<sizeof(Slice)>(s_ + (u_ * 2 + 1) * kConvThreads, ok_ ? pg_ + (long long)u_ * d.C : dy, ok_); \
        }                                                                                                        \
      }                                                                                                          \
    }                                                                                                            \
    cp_async_commit();                                                                                           \
  } while (0)
#pragma unroll
  for (int g = 0; g < RING - 1; ++g) SLX_CONV_ISSUE(g);

  // arithmetic on pairs of adjacent channels (fma.rn.f32x2: each half is the same IEEE fma as the scalar
  // kernel's, so the results are identical)
  constexpr int H = VEC / 2;
  float2 w4[4][H], bv[H], x0[H], x1[H], x2[H], x3[H];
  {
    float wf[4][VEC], bf[VEC], xa[VEC], xb2[VEC], xc[VEC];
    load_taps<T, VEC>(weight, bias, d, c0, wf, bf);
    load_cat<T, VEC>(x, state, d, b, t_lo - 3, c0, xa);
    load_cat<T, VEC>(x, state, d, b, t_lo - 2, c0, xb2);
    load_cat<T, VEC>(x, state, d, b, t_lo - 1, c0, xc);
#pragma unroll
    for (int h = 0; h < H; ++h) {
#pragma unroll
      for (int k = 0; k < 4; ++k) w4[k][h] = make_float2(wf[k][2 * h], wf[k][2 * h + 1]);
      bv[h] = make_float2(bf[2 * h], bf[2 * h + 1]);
      x0[h] = make_float2(xa[2 * h], xa[2 * h + 1]);
      x1[h] = make_float2(xb2[2 * h], xb2[2 * h + 1]);
      x2[h] = make_float2(xc[2 * h], xc[2 * h + 1]);
    }
  }
  float2 g0[H], g1[H], g2[H], g3[H];  // dyact[t-3..t]
  float2 dw[4][H], db[H];
  const float2 zero2 = make_float2(0.f, 0.f);
#pragma unroll
  for (int h = 0; h < H; ++h) {
    g0[h] = g1[h] = g2[h] = zero2;
    x3[h] = zero2;
    db[h] = zero2;
#pragma unroll
    for (int k = 0; k < 4; ++k) dw[k][h] = zero2;
  }
  // One row of the walk.  INNER rows (three or more rows into the tile and before its end) need none of the
  // edge tests: every row is inside the sequence, counts toward the sums, and its dx row lies in the tile
  // and ahead of the last W-1 tokens, the only ones next_state's gradient reaches.
  auto row_step = [&](auto inner_tag, const Slice *s, int u, int t) {
    constexpr bool INNER = decltype(inner_tag)::value;
    Slice xr, gr;
    ld_raw<T, VEC>(s[(u * 2 + 0) * kConvThreads].v, xr);
    ld_raw<T, VEC>(s[(u * 2 + 1) * kConvThreads].v, gr);
    if (INNER || t < d.T) {
#pragma unroll
      for (int h = 0; h < H; ++h) x3[h] = make_float2(to_f(xr.v[2 * h]), to_f(xr.v[2 * h + 1]));
    }
    // rows past the sequence arrive as zeros, so g3 = 0 there without a test
#pragma unroll
    for (int h = 0; h < H; ++h) g3[h] = make_float2(to_f(gr.v[2 * h]), to_f(gr.v[2 * h + 1]));
    if (d.silu) {
#pragma unroll
      for (int h = 0; h < H; ++h) {
        float2 pre = __ffma2_rn(w4[0][h], x0[h], bv[h]);
        pre = __ffma2_rn(w4[1][h], x1[h], pre);
        pre = __ffma2_rn(w4[2][h], x2[h], pre);
        pre = __ffma2_rn(w4[3][h], x3[h], pre);
        const float sx = 1.f / (1.f + expf(-pre.x)), sy = 1.f / (1.f + expf(-pre.y));
        g3[h].x *= sx * (1.f + pre.x * (1.f - sx));
        g3[h].y *= sy * (1.f + pre.y * (1.f - sy));
      }
    }
    if (INNER || t < t_hi) {
#pragma unroll
      for (int h = 0; h < H; ++h) {
        dw[0][h] = __ffma2_rn(g3[h], x0[h], dw[0][h]);
        dw[1][h] = __ffma2_rn(g3[h], x1[h], dw[1][h]);
        dw[2][h] = __ffma2_rn(g3[h], x2[h], dw[2][h]);
        dw[3][h] = __ffma2_rn(g3[h], x3[h], dw[3][h]);
        db[h] = __fadd2_rn(db[h], g3[h]);
      }
    }
    const int tau = t - 3;  // dx[tau] = sum_k w4[k] dyact[tau+3-k]
    if (INNER || (tau >= t_lo && tau < t_hi)) {
      float o[VEC];
#pragma unroll
      for (int h = 0; h < H; ++h) {
        float2 acc = __fmul2_rn(w4[0][h], g3[h]);
        acc = __ffma2_rn(w4[1][h], g2[h], acc);
        acc = __ffma2_rn(w4[2][h], g1[h], acc);
        acc = __ffma2_rn(w4[3][h], g0[h], acc);
        o[2 * h] = acc.x;
        o[2 * h + 1] = acc.y;
      }
      if (!INNER) {
        const int i = tau - d.T + (d.W - 1);  // position inside next_state, if any
        if (d_next && i >= 0) {
#pragma unroll
          for (int e = 0; e < VEC; ++e) o[e] += to_f(d_next[((long long)b * d.C + c0 + e) * (d.W - 1) + i]);
        }
      }
      stv<T, VEC>(dx + ((long long)b * d.T + tau) * d.C + c0, o);
    }
#pragma unroll
    for (int h = 0; h < H; ++h) {
      x0[h] = x1[h];
      x1[h] = x2[h];
      x2[h] = x3[h];
      g0[h] = g1[h];
      g1[h] = g2[h];
      g2[h] = g3[h];
    }
  };
  for (int grp = 0; grp < n_grp; ++grp) {
    // the slot of group grp+R-1 is the one read in the previous iteration
    SLX_CONV_ISSUE(grp + RING - 1);
    cp_async_wait<RING - 1>();
    const Slice *s = ring + (size_t)(grp % RING) * G * 2 * kConvThreads;
    const int tg = t_lo + grp * G;
    if (grp * G >= 3 && tg + G <= t_hi) {
#pragma unroll
      for (int u = 0; u < G; ++u) row_step(std::true_type(), s, u, tg + u);
    } else {
#pragma unroll
      for (int u = 0; u < G; ++u) {
        if (tg + u >= t_end) break;
        row_step(std::false_type(), s, u, tg + u);
      }
    }
  }
  float dwf[4][VEC], dbf[VEC];
#pragma unroll
  for (int h = 0; h < H; ++h) {
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      dwf[k][2 * h] = dw[k][h].x;
      dwf[k][2 * h + 1] = dw[k][h].y;
    }
    dbf[2 * h] = db[h].x;
    dbf[2 * h + 1] = db[h].y;
  }
  cp_async_wait<0>();
#undef SLX_CONV_ISSUE
  conv_bwd_partials<VEC>(part, d.C, b, c0, dwf, dbf);
}

template <typename T, int VEC, int RING>
__global__ void __launch_bounds__(kConvThreads) cconv1d_fwd_staged_kernel(const T *__restrict__ x,
                                                                          const T *__restrict__ weight,
                                                                          const T *__restrict__ bias,
                                                                          const T *__restrict__ state,
                                                                          T *__restrict__ y, T *__restrict__ next_state,
                                                                          ConvDims d, int tile) {
  using Slice = RowSlice<T, VEC>;
  constexpr int G = conv_group_rows<T, VEC>();
  extern __shared__ __align__(16) unsigned char conv_ring[];
  const int c0 = (blockIdx.x * kConvThreads + threadIdx.x) * VEC;
  if (c0 >= d.C) return;
  Slice *ring = reinterpret_cast<Slice *>(conv_ring) + threadIdx.x;  // [RING*G rows][thread]
  const int b = blockIdx.z;
  const int t_lo = blockIdx.y * tile, t_hi = min(d.T, t_lo + tile);
  const int n_grp = (t_hi - t_lo + G - 1) / G;
  const T *xb = x + (long long)b * d.xbs + c0;
#define SLX_CONV_ISSUE(grp_)                                                                                  \
  do {                                                                                                        \
    const int gi_ = (grp_);                                                                                   \
    if (gi_ < n_grp) {                                                                                        \
      Slice *s_ = ring + (size_t)(gi_ % RING) * G * kConvThreads;                                        \
      const int t0_ = t_lo + gi_ * G;                                                                         \
      const T *px_ = xb + (long long)t0_ * d.xs;                                                              \
      if (t0_ + G <= t_hi) {                                                                                  \
        _Pragma("unroll") for (int u_ = 0; u_ < G; ++u_)                                                      \
            cp_async_slice_full<sizeof(Slice)>(s_ + u_ * kConvThreads, px_ + (long long)u_ * d.xs);           \
      } else {                                                                                                \
        _Pragma("unroll") for (int u_ = 0; u_ < G; ++u_) {                                                    \
          const bool ok_ = t0_ + u_ < t_hi;                                                                   \
          cp_async_slice<sizeof(Slice)>(s_ + u_ * kConvThreads, ok_ ? px_ + (long long)u_ * d.xs : x, ok_);   \
        }                                                                                                     \
      }                                                                                                       \
    }                                                                                                         \
    cp_async_commit();                                                                                        \
  } while (0)
#pragma unroll
  for (int g = 0; g < RING - 1; ++g) SLX_CONV_ISSUE(g);

  float w4[4][VEC], bv[VEC];
  load_taps<T, VEC>(weight, bias, d, c0, w4, bv);
  float x0[VEC], x1[VEC], x2[VEC], x3[VEC];
  load_cat<T, VEC>(x, state, d, b, t_lo - 3, c0, x0);
  load_cat<T, VEC>(x, state, d, b, t_lo - 2, c0, x1);
  load_cat<T, VEC>(x, state, d, b, t_lo - 1, c0, x2);
  auto row_step = [&](const Slice *s, int u, T *yrow) {
    Slice xr;
    ld_raw<T, VEC>(s[u * kConvThreads].v, xr);
    float o[VEC];
#pragma unroll
    for (int e = 0; e < VEC; ++e) {
      x3[e] = to_f(xr.v[e]);
      float acc = bv[e];
      acc = fmaf(w4[0][e], x0[e], acc);
      acc = fmaf(w4[1][e], x1[e], acc);
      acc = fmaf(w4[2][e], x2[e], acc);
      acc = fmaf(w4[3][e], x3[e], acc);
      if (d.silu) acc = acc / (1.f + expf(-acc));
      o[e] = acc;
      x0[e] = x1[e];
      x1[e] = x2[e];
      x2[e] = x3[e];
    }
    stv<T, VEC>(yrow, o);
  };
  T *yb = y + ((long long)b * d.T + t_lo) * d.C + c0;
  for (int grp = 0; grp < n_grp; ++grp) {
    SLX_CONV_ISSUE(grp + RING - 1);  // into the slot read in the previous iteration
    cp_async_wait<RING - 1>();
    const Slice *s = ring + (size_t)(grp % RING) * G * kConvThreads;
    T *yg = yb + (long long)grp * G * d.C;
    if (t_lo + (grp + 1) * G <= t_hi) {  // whole group inside the tile: no per-row test
#pragma unroll
      for (int u = 0; u < G; ++u) row_step(s, u, yg + (long long)u * d.C);
    } else {
#pragma unroll
      for (int u = 0; u < G; ++u) {
        if (t_lo + grp * G + u >= t_hi) break;
        row_step(s, u, yg + (long long)u * d.C);
      }
    }
  }
  cp_async_wait<0>();
#undef SLX_CONV_ISSUE
  if (next_state && t_hi == d.T) {
    for (int i = 0; i < d.W - 1; ++i) {
      float v[VEC];
      load_cat<T, VEC>(x, state, d, b, d.T - (d.W - 1) + i, c0, v);
#pragma unroll
      for (int e = 0; e < VEC; ++e)
        next_state[((long long)b * d.C + c0 + e) * (d.W - 1) + i] = from_f<T>(v[e]);
    }
  }
}

// Sums the per-tile partials: a block owns 32 adjacent (channel, slot) entries, slots = (dw4[0..3], dbias);
// its eight rows of threads each sum a contiguous share of the parts (eight loads in flight), and row 0 adds
// the eight shares.  The order of every sum is fixed, so the result does not vary from run to run.
constexpr int kConvReduceRows = 8;
__global__ void __launch_bounds__(32 * kConvReduceRows) cconv1d_reduce_kernel(const float *__restrict__ part,
                                                                              float *__restrict__ dweight,
                                                                              float *__restrict__ dbias, int n_parts,
                                                                              int C, int W) {
  __shared__ float share[kConvReduceRows][32];
  const int e = blockIdx.x * 32 + threadIdx.x, row = threadIdx.y;
  const size_t stride = (size_t)C * 5;
  float acc = 0.f;
  if (e < C * 5) {
    const int per = (n_parts + kConvReduceRows - 1) / kConvReduceRows;
    int p = row * per;
    const int p_end = min(n_parts, p + per);
    for (; p + 8 <= p_end; p += 8) {
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = part[(size_t)(p + i) * stride + e];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += v[i];
    }
    for (; p < p_end; ++p) acc += part[(size_t)p * stride + e];
  }
  share[row][threadIdx.x] = acc;
  __syncthreads();
  if (row != 0 || e >= C * 5) return;
#pragma unroll
  for (int r = 1; r < kConvReduceRows; ++r) acc += share[r][threadIdx.x];
  const int c = e / 5, k = e % 5;
  if (k == 4) {
    if (dbias) dbias[c] = acc;
  } else {
    const int j = k - (4 - W);
    if (j >= 0) dweight[(long long)c * W + j] = acc;
  }
}

// One decode token: y[b,c] = act(bias[c] + sum_k w[c,k] * cat[k]),  cat = [state[b,c,0..W-2], x[b,c]];
// next_state[b,c,:] = cat[1:].  One thread per channel; state and next_state may be the same buffer
// (a thread reads its channel's W-1 values before it writes them).
template <typename T>
__global__ void __launch_bounds__(128) cconv1d_update_kernel(const T *__restrict__ x, long long x_stride,
                                                             const T *__restrict__ weight, const T *__restrict__ bias,
                                                             const T *state, T *__restrict__ y, T *next_state, int C,
                                                             int W, int silu) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  float cat[4];
  const long long so = ((long long)b * C + c) * (W - 1);
#pragma unroll
  for (int k = 0; k < 3; ++k) cat[k] = (k < W - 1 && state) ? to_f(state[so + k]) : 0.f;
  cat[W - 1] = to_f(x[(long long)b * x_stride + c]);
  float acc = bias ? to_f(bias[c]) : 0.f;
#pragma unroll
  for (int k = 0; k < 4; ++k)
    if (k < W) acc = fmaf(to_f(weight[(long long)c * W + k]), cat[k], acc);
  if (silu) acc = acc / (1.f + __expf(-acc));
  y[(long long)b * C + c] = from_f<T>(acc);
  if (next_state) {
#pragma unroll
    for (int k = 0; k < 3; ++k)
      if (k < W - 1) next_state[so + k] = from_f<T>(cat[k + 1]);
  }
}

static int check_conv(const slx_conv_shape *s, ConvDims *d) {
  SLX_REQUIRE(s != nullptr, SLX_E_NULL, "shape is NULL");
  SLX_REQUIRE(s->batch > 0 && s->T > 0 && s->channels > 0, SLX_E_SHAPE, "cconv1d: sizes must be positive");
  SLX_REQUIRE(s->width >= 2 && s->width <= 4, SLX_E_UNSUPPORTED, "cconv1d: width %d not in 2..4", s->width);
  SLX_REQUIRE(s->dtype >= SLX_F32 && s->dtype <= SLX_F16, SLX_E_DTYPE, "cconv1d: bad dtype %d", s->dtype);
  SLX_REQUIRE(s->x_stride >= s->channels, SLX_E_SHAPE, "cconv1d: x_stride smaller than channels");
  SLX_REQUIRE(s->batch <= 65535, SLX_E_UNSUPPORTED, "cconv1d: batch exceeds 65535");
  d->batch = s->batch; d->T = s->T; d->C = s->channels; d->W = s->width; d->silu = s->silu;
  d->xs = s->x_stride; d->xbs = s->x_batch_stride;
  return SLX_OK;
}

// Smallest tile of the token axis: the backward workspace is sized for it (one set of partial sums per tile).
constexpr int kConvTileFwd = 64, kConvTileBwd = 128;

static int conv_tile(int T, bool bwd) {
  int tile = bwd ? kConvTileBwd : kConvTileFwd;
  return tile < T ? tile : T;
}

// CTAs of `kernel` (kConvThreads threads, `smem` dynamic bytes) that the current device holds at once
template <typename K>
static long conv_slots(K kernel, size_t smem) {
  return resident_ctas(kernel, kConvThreads, smem);
}

// Tile of the token axis for a grid of base_ctas x ceil(T / tile) CTAs.  With the smallest tile the grid
// may come to a few waves plus a thin last one; then the tile is grown (up to 512 tokens) to the size at
// which the grid is k full waves, for the smallest such k.
static int conv_tile_balanced(int T, int min_tile, long base_ctas, long slots) {
  if (T <= min_tile) return T;
  const long n_min = (T + min_tile - 1) / min_tile;
  if (slots <= 0 || base_ctas * n_min <= slots) return min_tile;
  for (long k = 1; k <= 16; ++k) {
    const long nt = k * slots / base_ctas;
    if (nt < 1) continue;
    long tile = (T + nt - 1) / nt;
    tile = (tile + 7) / 8 * 8;
    if (tile < min_tile) return min_tile;
    if (tile <= 512) return (int)tile;
  }
  return min_tile;
}

template <typename T>
static bool conv_vec_ok(const slx_conv_shape *s, std::initializer_list<const void *> ptrs) {
  const int v = 16 / (int)sizeof(T);
  bool ok = (s->channels % v == 0) && (s->x_stride % v == 0) && (s->x_batch_stride % v == 0);
  for (const void *p : ptrs) ok = ok && (p == nullptr || (reinterpret_cast<uintptr_t>(p) & 15) == 0);
  return ok;
}

}  // namespace slx

using namespace slx;

#define SLX_CONV_T(dt, ...)                                          \
  switch (dt) {                                                      \
    case SLX_F32: { using T_ = float; __VA_ARGS__; } break;          \
    case SLX_BF16: { using T_ = __nv_bfloat16; __VA_ARGS__; } break; \
    default: { using T_ = __half; __VA_ARGS__; } break;              \
  }

extern "C" {

int slx_cconv1d_fwd(const slx_conv_shape *s, const void *x, const void *weight, const void *bias, const void *state,
                    void *y, void *next_state, void *stream) {
  ConvDims d;
  int rc = check_conv(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(x && weight && y, SLX_E_NULL, "cconv1d_fwd: NULL tensor");
  cudaStream_t st = as_stream(stream);
  SLX_CONV_T(s->dtype, {
    constexpr int VFULL = kConvVec;
    const T_ *xp = (const T_ *)x, *wp = (const T_ *)weight, *bp = (const T_ *)bias, *sp = (const T_ *)state;
    if (conv_vec_ok<T_>(s, {x, y})) {
      // 16-byte slices (8 channels of a half type): fewer instructions per channel than the backward's 8-byte ones
      constexpr int VW = 16 / (int)sizeof(T_);
      const int nblk = (d.C / VW + kConvThreads - 1) / kConvThreads;
      constexpr size_t ring = conv_ring_bytes<T_, VW, kConvRingFwd>(1);
      auto kern = cconv1d_fwd_staged_kernel<T_, VW, kConvRingFwd>;
      rc = ensure_dyn_smem(kern, ring);
      if (rc) return rc;
      const int tile = conv_tile(d.T, false);  // growing the tile to whole waves measured no faster here
      const int n_tiles = (d.T + tile - 1) / tile;
      kern<<<dim3(nblk, n_tiles, d.batch), kConvThreads, ring, st>>>(xp, wp, bp, sp, (T_ *)y, (T_ *)next_state, d,
                                                                     tile);
    } else {
      const int nblk = (d.C + kConvThreads - 1) / kConvThreads;
      const int tile = conv_tile(d.T, false);
      const int n_tiles = (d.T + tile - 1) / tile;
      cconv1d_fwd_kernel<T_, 1><<<dim3(nblk, n_tiles, d.batch), kConvThreads, 0, st>>>(xp, wp, bp, sp, (T_ *)y,
                                                                                     (T_ *)next_state, d, tile);
    }
  });
  return check_launch("cconv1d_fwd");
}

int slx_cconv1d_update(const slx_conv_shape *s, const void *x, const void *weight, const void *bias,
                       const void *state, void *y, void *next_state, void *stream) {
  ConvDims d;
  int rc = check_conv(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(s->T == 1, SLX_E_SHAPE, "cconv1d_update: one token per call (T must be 1, got %d)", s->T);
  SLX_REQUIRE(x && weight && y, SLX_E_NULL, "cconv1d_update: NULL tensor");
  cudaStream_t st = as_stream(stream);
  SLX_CONV_T(s->dtype, {
    cconv1d_update_kernel<T_><<<dim3((d.C + 127) / 128, d.batch), 128, 0, st>>>(
        (const T_ *)x, s->x_batch_stride, (const T_ *)weight, (const T_ *)bias, (const T_ *)state, (T_ *)y,
        (T_ *)next_state, d.C, d.W, d.silu);
  });
  return check_launch("cconv1d_update");
}

size_t slx_cconv1d_bwd_workspace_bytes(const slx_conv_shape *s) {
  ConvDims d;
  if (check_conv(s, &d)) return 0;
  const int tile = conv_tile(d.T, true);
  const int n_tiles = (d.T + tile - 1) / tile;
  return sizeof(float) * (size_t)d.batch * n_tiles * d.C * 5;
}

int slx_cconv1d_bwd(const slx_conv_shape *s, const void *x, const void *weight, const void *bias, const void *state,
                    const void *dy, const void *d_next_state, void *dx, float *dweight, float *dbias, float *dstate,
                    void *workspace, size_t workspace_bytes, void *stream) {
  ConvDims d;
  int rc = check_conv(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(x && weight && dy && dx && dweight, SLX_E_NULL, "cconv1d_bwd: NULL tensor");
  size_t need = slx_cconv1d_bwd_workspace_bytes(s);
  SLX_REQUIRE(workspace && workspace_bytes >= need, SLX_E_WORKSPACE, "cconv1d_bwd: workspace of %zu bytes needed",
              need);
  cudaStream_t st = as_stream(stream);
  float *part = static_cast<float *>(workspace);
  int n_tiles = 0;  // at most ceil(T / kConvTileBwd), which the workspace is sized for
  SLX_CONV_T(s->dtype, {
    constexpr int VFULL = kConvVec;
    const T_ *xp = (const T_ *)x, *wp = (const T_ *)weight, *bp = (const T_ *)bias, *sp = (const T_ *)state;
    const T_ *gp = (const T_ *)dy, *np = (const T_ *)d_next_state;
    if (conv_vec_ok<T_>(s, {x, dy, dx})) {
      const int nblk = (d.C / VFULL + kConvThreads - 1) / kConvThreads;
      constexpr size_t ring = conv_ring_bytes<T_, VFULL>(2);
      auto kern = cconv1d_bwd_staged_kernel<T_, VFULL, kConvRing>;
      rc = ensure_dyn_smem(kern, ring);
      if (rc) return rc;
      const int tile = conv_tile_balanced(d.T, kConvTileBwd, (long)nblk * d.batch, conv_slots(kern, ring));
      n_tiles = (d.T + tile - 1) / tile;
      kern<<<dim3(nblk, n_tiles, d.batch), kConvThreads, ring, st>>>(xp, wp, bp, sp, gp, np, (T_ *)dx, part, d, tile);
      if (dstate)
        cconv1d_bwd_dstate_kernel<T_, VFULL><<<dim3(nblk, 1, d.batch), kConvThreads, 0, st>>>(xp, wp, bp, sp, gp, np,
                                                                                            dstate, d);
    } else {
      const int nblk = (d.C + kConvThreads - 1) / kConvThreads;
      const int tile = conv_tile(d.T, true);
      n_tiles = (d.T + tile - 1) / tile;
      cconv1d_bwd_kernel<T_, 1><<<dim3(nblk, n_tiles, d.batch), kConvThreads, 0, st>>>(xp, wp, bp, sp, gp, np,
                                                                                     (T_ *)dx, part, d, tile);
      if (dstate)
        cconv1d_bwd_dstate_kernel<T_, 1><<<dim3(nblk, 1, d.batch), kConvThreads, 0, st>>>(xp, wp, bp, sp, gp, np,
                                                                                        dstate, d);
    }
  });
  rc = check_launch("cconv1d_bwd");
  if (rc) return rc;
  cconv1d_reduce_kernel<<<(d.C * 5 + 31) / 32, dim3(32, kConvReduceRows), 0, st>>>(part, dweight, dbias,
                                                                                   d.batch * n_tiles, d.C, d.W);
  return check_launch("cconv1d_reduce");
}

}  // extern "C"

// ---- backward without caller-provided scratch ------------------------------------------------
// Scratch for the weight/bias partial sums lives in the library image itself: kNoAllocFloats
// floats (4 MiB) per GPU that loads the library, held until the process exits.
namespace slx {
constexpr size_t kNoAllocFloats = 1u << 20;
static __device__ __align__(256) float g_conv_noalloc_scratch[kNoAllocFloats];

// In host code the array's name is only a stand-in for the symbol; the device address has to be
// asked for, once per device, with that device current.
static float *noalloc_scratch_for_current_device(int *status) {
  static std::mutex mu;
  static float *cache[64] = {};
  *status = SLX_OK;
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess || dev < 0 || dev >= 64) {
    *status = fail(e != cudaSuccess ? (int)e : SLX_E_UNSUPPORTED, "cconv1d_bwd_noalloc: cannot identify the device");
    return nullptr;
  }
  std::lock_guard<std::mutex> lock(mu);
  if (cache[dev] == nullptr) {
    void *p = nullptr;
    e = cudaGetSymbolAddress(&p, g_conv_noalloc_scratch);
    if (e != cudaSuccess || p == nullptr) {
      *status = fail((int)e, "cconv1d_bwd_noalloc: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
      return nullptr;
    }
    cache[dev] = static_cast<float *>(p);
  }
  return cache[dev];
}
}  // namespace slx

extern "C" int slx_cconv1d_bwd_noalloc(const slx_conv_shape *s, const void *x, const void *weight, const void *bias,
                                       const void *state, const void *dy, const void *d_next_state, void *dx,
                                       float *dweight, float *dbias, float *dstate, void *stream) {
  using namespace slx;
  const size_t need = slx_cconv1d_bwd_workspace_bytes(s);
  SLX_REQUIRE(need != 0, SLX_E_SHAPE, "cconv1d_bwd_noalloc: bad shape");
  SLX_REQUIRE(need <= kNoAllocFloats * sizeof(float), SLX_E_UNSUPPORTED,
              "cconv1d_bwd_noalloc: this shape needs %zu bytes of scratch, the built-in buffer holds %zu "
              "(batch * ceil(T/128) * channels * 5 floats must not exceed %zu); use slx_cconv1d_bwd with a "
              "caller-provided workspace",
              need, kNoAllocFloats * sizeof(float), kNoAllocFloats);
  int rc = SLX_OK;
  float *scratch = noalloc_scratch_for_current_device(&rc);
  if (rc) return rc;
  return slx_cconv1d_bwd(s, x, weight, bias, state, dy, d_next_state, dx, dweight, dbias, dstate, scratch,
                         kNoAllocFloats * sizeof(float), stream);
}
