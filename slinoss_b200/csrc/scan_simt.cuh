// fp32-exact chunk kernels of the v2x2ssd scan (CUDA-core FFMA path).
//
// One CTA of 256 threads per (chunk, batch*head).  All contractions are done
// with fp32 FMAs on shared-memory tiles, so that fp32 inputs reproduce the
// reference to ~1e-6; half inputs are widened on load.
//
// Math (per chunk, local token index t, s in [0,L)):
//   p_t   = prod_{tau<=t} m_tau = exp(lp_t) * phi_t            (stable split)
//   gamma_s = m_{s+1} k^c_s + k^p_{s+1}                         (merged taps)
//   h_t = p_t z0 + (p_t/p_0) k^p_0 x_{-1} + sum_{s<t} (p_t/p_{s+1}) gamma_s x_s
//         + k^c_t x_t ,    x_s = u_s (x) b_s ,   y_t = Re <c_t, h_t>
// which is the reference recurrence (slinoss/ops/v2x2ssd/reference.py:704-803)
// with the two taps of source token s folded into one coefficient.
// With Qbar_t = c_t conj(phi_t) and kappa_s = gamma_s b_s conj(phi_{s+1}) stored
// as interleaved (re,im) floats, Re(conj(c_t) (p_t/p_{s+1}) gamma_s b_s) is the
// plain real dot <Qbar_t, kappa_s> times exp(lp_t - lp_{s+1}).
#pragma once

#include "common.cuh"

namespace slx {

__device__ int g_scan_bad = 0;  // becomes 1 when a kernel met a transition of magnitude exactly 0

constexpr int kThreads = 256;
constexpr int kPMax = 64;
constexpr int kLdP = kPMax + 1;

struct ScanDims {
  int BH, T, P, N, D, L, NC;
};

template <typename T>
__device__ __forceinline__ float2 load_pair(const T *p);
template <>
__device__ __forceinline__ float2 load_pair<float>(const float *p) {
  return *reinterpret_cast<const float2 *>(p);
}
template <>
__device__ __forceinline__ float2 load_pair<__nv_bfloat16>(const __nv_bfloat16 *p) {
  return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162 *>(p));
}
template <>
__device__ __forceinline__ float2 load_pair<__half>(const __half *p) {
  return __half22float2(*reinterpret_cast<const __half2 *>(p));
}
template <typename T>
__device__ __forceinline__ void store_pair(T *p, float2 v);
template <>
__device__ __forceinline__ void store_pair<float>(float *p, float2 v) {
  *reinterpret_cast<float2 *>(p) = v;
}
template <>
__device__ __forceinline__ void store_pair<__nv_bfloat16>(__nv_bfloat16 *p, float2 v) {
  *reinterpret_cast<__nv_bfloat162 *>(p) = __float22bfloat162_rn(v);
}
template <>
__device__ __forceinline__ void store_pair<__half>(__half *p, float2 v) {
  *reinterpret_cast<__half2 *>(p) = __float22half2_rn(v);
}

// acc[i][j] += sum_k fa(i,k) * fb(j,k)
template <int TM, int TN, typename FA, typename FB>
__device__ __forceinline__ void mm_acc(float (&acc)[TM][TN], int kdim, FA fa, FB fb) {
#pragma unroll 4
  for (int k = 0; k < kdim; ++k) {
    float av[TM], bv[TN];
#pragma unroll
    for (int i = 0; i < TM; ++i) av[i] = fa(i, k);
#pragma unroll
    for (int j = 0; j < TN; ++j) bv[j] = fb(j, k);
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
  }
}

// sum a float2 over groups of NL consecutive lanes (NL power of two <= 32)
template <int NL>
__device__ __forceinline__ float2 group_sum(float2 v) {
#pragma unroll
  for (int off = NL / 2; off > 0; off >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
  }
  return v;
}

// Column-slab geometry: an (L x DS) tile of interleaved complex pairs spread
// over 256 threads; NPT threads across the DS/2 pairs, RG row groups.
template <int L, int DS>
struct SlabMap {
  static constexpr int NP = DS / 2;
  static constexpr int NPT = NP >= 16 ? 16 : NP;
  static constexpr int TNP = NP / NPT;
  static constexpr int RG = kThreads / NPT;
  static constexpr int TMS = (L + RG - 1) / RG;
};

template <int L>
struct ChunkCfg {
  static constexpr int TM = L / 16;
  static constexpr int DS_FWD = (L <= 64) ? 64 : 32;
  static constexpr int DS_BWD = (L <= 64) ? 64 : 16;
};

// ---------------------------------------------------------------------------
// out[p, :] = sum_t A[t, p] * (coef_t * x_t[:])  (+ rank-1 boundary term)
// MODE 0: chunk increment.  A = U, x = B, coef_s = sigma_{s+1} gamma_s (= the
//         weight of source token s in the chunk-final state); boundary
//         u_{-1} (x) sigma_0 k^p_0 b_{-1}; also writes m_chunk.
//         Replaces reference.py:937 (chunk_increment).
// MODE 1: dZ0.  A = dY, x = C, coef_t = conj(p_t).
template <typename T>
struct OuterArgs {
  const T *A;       // (BH,T,P)
  const T *X;       // (BH,T,D)
  const float *M;   // (BH,T,2)
  const float *K;   // (BH,T,2,2)  (mode 0)
  const float *Bprev, *Uprev;  // (BH,D), (BH,P) fp32, nullable (mode 0)
  float *out;       // (BH,NC,P,D)
  float *m_chunk;   // (BH,NC,2) (mode 0)
  ScanDims d;
};

template <int L>
constexpr size_t outer_smem_bytes() {
  return sizeof(float) * (size_t)(L * kLdP + L * 65 + L /*lp*/ + 2 * L * 4 /*ph,mraw,coef,spare*/ + kPMax + 64 + 8);
}

template <typename T, int L, int MODE>
__global__ void __launch_bounds__(kThreads) chunk_outer_kernel(OuterArgs<T> a) {
  constexpr int DS = 64, NP = DS / 2, LDS = DS + 1;
  extern __shared__ float sm[];
  float *As = sm;                 // L * kLdP
  float *Xs = As + L * kLdP;      // L * LDS
  float *lp = Xs + L * LDS;       // L
  float2 *ph = reinterpret_cast<float2 *>(lp + L + ((L * kLdP + L * LDS + L) & 1));
  float2 *mraw = ph + L;
  float2 *coef = mraw + L;
  float2 *spare = coef + L;
  float *um1 = reinterpret_cast<float *>(spare + L);  // kPMax
  float *bh1 = um1 + kPMax;                            // DS  (boundary row, already weighted)

  const ScanDims d = a.d;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int t0 = c * L;
  const int valid = min(L, d.T - t0);
  const size_t tok0 = (size_t)bh * d.T + t0;

  chunk_prefix_warp0(a.M + tok0 * 2, L, valid, lp, ph, mraw, &g_scan_bad);
  for (int idx = tid; idx < L * d.P; idx += kThreads) {
    int t = idx / d.P, p = idx - t * d.P;
    As[t * kLdP + p] = (t < valid) ? to_f(a.A[(tok0 + t) * d.P + p]) : 0.f;
  }
  if (MODE == 0) {
    for (int p = tid; p < d.P; p += kThreads) {
      float v = 0.f;
      if (t0 > 0) v = to_f(a.A[(tok0 - 1) * d.P + p]);
      else if (a.Uprev) v = a.Uprev[(size_t)bh * d.P + p];
      um1[p] = v;
    }
  }
  __syncthreads();
  // per-row coefficient
  float2 k0p = make_float2(0.f, 0.f);
  for (int t = tid; t < L; t += kThreads) {
    float2 cf;
    if (MODE == 0) {
      float2 kc = make_float2(0.f, 0.f), kpn = make_float2(0.f, 0.f);
      if (t < valid) kc = *reinterpret_cast<const float2 *>(a.K + (tok0 + t) * 4 + 2);
      if (t + 1 < valid) kpn = *reinterpret_cast<const float2 *>(a.K + (tok0 + t + 1) * 4);
      if (t + 1 < L) {
        float2 gam = cadd(cmul(mraw[t + 1], kc), kpn);
        float2 sig = cscale(cmulc(ph[L - 1], ph[t + 1]), expf(lp[L - 1] - lp[t + 1]));
        cf = cmul(sig, gam);
      } else {
        cf = kc;
      }
    } else {
      cf = cscale(cconj(ph[t]), expf(lp[t]));
    }
    coef[t] = cf;
  }
  if (MODE == 0 && tid == 0) {
    // chunk transition by direct product (reference.py:509-516 accumulates the
    // same product in its reverse scan)
    float2 acc = make_float2(1.f, 0.f);
    for (int t = 0; t < L; ++t) acc = cmul(acc, mraw[t]);
    *reinterpret_cast<float2 *>(a.m_chunk + ((size_t)bh * d.NC + c) * 2) = acc;
  }
  if (MODE == 0) {
    if (valid > 0) k0p = *reinterpret_cast<const float2 *>(a.K + tok0 * 4);
    // weight of the boundary source: (p_{L-1}/p_0) k^p_0
    k0p = cmul(cscale(cmulc(ph[L - 1], ph[0]), expf(lp[L - 1] - lp[0])), k0p);
  }
  __syncthreads();

  float *outc = a.out + ((size_t)bh * d.NC + c) * d.P * d.D;
  for (int d0 = 0; d0 < d.D; d0 += DS) {
    for (int idx = tid; idx < L * NP; idx += kThreads) {
      int row = idx / NP, n = idx - row * NP;
      int dd = d0 + 2 * n;
      float2 xv = make_float2(0.f, 0.f);
      if (row < valid && dd < d.D) xv = load_pair<T>(a.X + (tok0 + row) * d.D + dd);
      float2 v = cmul(coef[row], xv);
      Xs[row * LDS + 2 * n] = v.x;
      Xs[row * LDS + 2 * n + 1] = v.y;
    }
    if (MODE == 0) {
      for (int n = tid; n < NP; n += kThreads) {
        int dd = d0 + 2 * n;
        float2 bv = make_float2(0.f, 0.f);
        if (dd < d.D) {
          if (t0 > 0) bv = load_pair<T>(a.X + (tok0 - 1) * d.D + dd);
          else if (a.Bprev) bv = *reinterpret_cast<const float2 *>(a.Bprev + (size_t)bh * d.D + dd);
        }
        float2 v = cmul(k0p, bv);
        bh1[2 * n] = v.x;
        bh1[2 * n + 1] = v.y;
      }
    }
    __syncthreads();
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;
    mm_acc<4, 4>(acc, L,
                 [&](int i, int k) { return As[k * kLdP + ty + 16 * i]; },
                 [&](int j, int k) { return Xs[k * LDS + 2 * (tx + 16 * (j >> 1)) + (j & 1)]; });
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int p = ty + 16 * i;
      if (p >= d.P) continue;
#pragma unroll
      for (int jj = 0; jj < 2; ++jj) {
        int cc = 2 * (tx + 16 * jj);
        int dd = d0 + cc;
        if (dd >= d.D) continue;
        float2 v = make_float2(acc[i][2 * jj], acc[i][2 * jj + 1]);
        if (MODE == 0) {
          v.x = fmaf(um1[p], bh1[cc], v.x);
          v.y = fmaf(um1[p], bh1[cc + 1], v.y);
        }
        *reinterpret_cast<float2 *>(outc + (size_t)p * d.D + dd) = v;
      }
    }
    __syncthreads();
  }
}

// ---------------------------------------------------------------------------
// Forward chunk scan.  Replaces reference.py:1059 (chunk_scan).
template <typename T>
struct ScanFwdArgs {
  const T *U, *B, *C;
  const float *M, *K, *starts, *Bprev, *Uprev;
  T *Y;
  int *bad;  // unused (the kernels report through g_scan_bad)
  ScanDims d;
};

template <int L>
constexpr size_t scan_fwd_smem_bytes() {
  constexpr int DS = ChunkCfg<L>::DS_FWD;
  return sizeof(float) * (size_t)(L * kLdP + 2 * L * (DS + 1) + kPMax * (DS + 1) + L * (L + 1) + L +
                                  2 * L * 7 + kPMax + DS + 8);
}

template <typename T, int L>
__global__ void __launch_bounds__(kThreads) chunk_scan_fwd_kernel(ScanFwdArgs<T> a) {
  constexpr int TM = ChunkCfg<L>::TM;
  constexpr int DS = ChunkCfg<L>::DS_FWD, NP = DS / 2, LDS = DS + 1, LDL = L + 1;
  extern __shared__ float sm[];
  float *Us = sm;                   // L*kLdP
  float *Qs = Us + L * kLdP;        // L*LDS
  float *Ks = Qs + L * LDS;         // L*LDS
  float *Zs = Ks + L * LDS;         // kPMax*LDS
  float *Ss = Zs + kPMax * LDS;     // L*LDL
  float *lp = Ss + L * LDL;         // L
  size_t off = (size_t)L * kLdP + 2 * L * LDS + kPMax * LDS + L * LDL + L;
  float2 *ph = reinterpret_cast<float2 *>(lp + L + (off & 1));
  float2 *mraw = ph + L, *kc = mraw + L, *kp = kc + L, *gam = kp + L, *cb = gam + L, *cbm = cb + L;
  float *um1 = reinterpret_cast<float *>(cbm + L);  // kPMax
  float *bm1 = um1 + kPMax;                          // DS

  const ScanDims d = a.d;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int t0 = c * L;
  const int valid = min(L, d.T - t0);
  const size_t tok0 = (size_t)bh * d.T + t0;

  chunk_prefix_warp0(a.M + tok0 * 2, L, valid, lp, ph, mraw, &g_scan_bad);
  for (int t = tid; t < L; t += kThreads) {
    float2 vp = make_float2(0.f, 0.f), vc = vp;
    if (t < valid) {
      float4 k4 = *reinterpret_cast<const float4 *>(a.K + (tok0 + t) * 4);
      vp = make_float2(k4.x, k4.y);
      vc = make_float2(k4.z, k4.w);
    }
    kp[t] = vp;
    kc[t] = vc;
    cb[t] = make_float2(0.f, 0.f);
    cbm[t] = make_float2(0.f, 0.f);
  }
  for (int idx = tid; idx < L * d.P; idx += kThreads) {
    int t = idx / d.P, p = idx - t * d.P;
    Us[t * kLdP + p] = (t < valid) ? to_f(a.U[(tok0 + t) * d.P + p]) : 0.f;
  }
  for (int p = tid; p < kPMax; p += kThreads) {
    float v = 0.f;
    if (p < d.P) {
      if (t0 > 0) v = to_f(a.U[(tok0 - 1) * d.P + p]);
      else if (a.Uprev) v = a.Uprev[(size_t)bh * d.P + p];
    }
    um1[p] = v;
  }
  for (int idx = tid; idx < kPMax * LDS; idx += kThreads) Zs[idx] = 0.f;
  __syncthreads();
  for (int t = tid; t < L; t += kThreads)
    gam[t] = (t + 1 < L) ? cadd(cmul(mraw[t + 1], kc[t]), kp[t + 1]) : make_float2(0.f, 0.f);
  __syncthreads();

  float S[TM][TM], Yo[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i) {
#pragma unroll
    for (int j = 0; j < TM; ++j) S[i][j] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) Yo[i][j] = 0.f;
  }
  const float *z0 = a.starts + ((size_t)bh * d.NC + c) * d.P * d.D;

  for (int d0 = 0; d0 < d.D; d0 += DS) {
    for (int n = tid; n < NP; n += kThreads) {
      int dd = d0 + 2 * n;
      float2 bv = make_float2(0.f, 0.f);
      if (dd < d.D) {
        if (t0 > 0) bv = load_pair<T>(a.B + (tok0 - 1) * d.D + dd);
        else if (a.Bprev) bv = *reinterpret_cast<const float2 *>(a.Bprev + (size_t)bh * d.D + dd);
      }
      bm1[2 * n] = bv.x;
      bm1[2 * n + 1] = bv.y;
    }
    __syncthreads();
    for (int idx = tid; idx < L * NP; idx += kThreads) {
      int row = idx / NP, n = idx - row * NP;
      int dd = d0 + 2 * n;
      float2 cv = make_float2(0.f, 0.f), bv = cv;
      if (row < valid && dd < d.D) {
        cv = load_pair<T>(a.C + (tok0 + row) * d.D + dd);
        bv = load_pair<T>(a.B + (tok0 + row) * d.D + dd);
      }
      float2 q = cmulc(cv, ph[row]);
      Qs[row * LDS + 2 * n] = q.x;
      Qs[row * LDS + 2 * n + 1] = q.y;
      float2 kap = make_float2(0.f, 0.f);
      if (row + 1 < L) kap = cmulc(cmul(gam[row], bv), ph[row + 1]);
      Ks[row * LDS + 2 * n] = kap.x;
      Ks[row * LDS + 2 * n + 1] = kap.y;
      float2 d1 = group_sum<NP>(cmul(cconj(cv), bv));
      float2 d2 = group_sum<NP>(cmul(cconj(cv), make_float2(bm1[2 * n], bm1[2 * n + 1])));
      if (n == 0) {
        cb[row] = cadd(cb[row], d1);
        cbm[row] = cadd(cbm[row], d2);
      }
    }
    for (int idx = tid; idx < d.P * NP; idx += kThreads) {
      int p = idx / NP, n = idx - p * NP;
      int dd = d0 + 2 * n;
      float2 zv = make_float2(0.f, 0.f);
      if (dd < d.D) zv = *reinterpret_cast<const float2 *>(z0 + (size_t)p * d.D + dd);
      Zs[p * LDS + 2 * n] = zv.x;
      Zs[p * LDS + 2 * n + 1] = zv.y;
    }
    __syncthreads();
    mm_acc<TM, TM>(S, DS, [&](int i, int k) { return Qs[(ty + 16 * i) * LDS + k]; },
                   [&](int j, int k) { return Ks[(tx + 16 * j) * LDS + k]; });
    mm_acc<TM, 4>(Yo, DS, [&](int i, int k) { return Qs[(ty + 16 * i) * LDS + k]; },
                  [&](int j, int k) { return Zs[(tx + 16 * j) * LDS + k]; });
    __syncthreads();
  }

#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int t = ty + 16 * i;
#pragma unroll
    for (int j = 0; j < TM; ++j) {
      int s = tx + 16 * j;
      float v = 0.f;
      if (s < t) v = S[i][j] * expf(lp[t] - lp[s + 1]);
      else if (s == t) v = kc[t].x * cb[t].x - kc[t].y * cb[t].y;
      Ss[t * LDL + s] = v;
    }
  }
  __syncthreads();
  float Yd[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) Yd[i][j] = 0.f;
  mm_acc<TM, 4>(Yd, L, [&](int i, int k) { return Ss[(ty + 16 * i) * LDL + k]; },
                [&](int j, int k) { return Us[k * kLdP + tx + 16 * j]; });
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int t = ty + 16 * i;
    if (t >= valid) continue;
    float el = expf(lp[t]);
    // boundary source (token before the chunk): weight (p_t/p_0) k^p_0
    float2 w = cmul(cmul(cmulc(ph[t], ph[0]), kp[0]), cbm[t]);
    float sig = expf(lp[t] - lp[0]) * w.x;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int p = tx + 16 * j;
      if (p < d.P) {
        float y = fmaf(el, Yo[i][j], Yd[i][j]);
        y = fmaf(sig, um1[p], y);
        a.Y[(tok0 + t) * d.P + p] = from_f<T>(y);
      }
    }
  }
}

// ---------------------------------------------------------------------------
// Backward of one chunk, given d_inc[c] = dL/d(chunk-final state) and the
// chunk's start state.  Writes dU, dB, dC (activation dtype), dM, dK (fp32) for
// the chunk's tokens, and the gradient carried to the token before the chunk
// (carryB (BH,NC,D), carryU (BH,NC,P)), which a follow-up kernel adds to the
// previous chunk's last row (or returns as dB_prev/dU_prev for chunk 0).
//
// dM uses the identity (local prefix p_tau; all quantities per chunk)
//   conj(p_tau) dL/dp_tau = sum_n c_tau conj(dC_tau) - conj(k^c_tau) dk^c_tau
//                           - conj(k^p_tau) dk^p_tau + [tau = L-1] <z_end, d_inc>
//   dM_t = (sum_{tau >= t} conj(p_tau) dL/dp_tau) / conj(m_t)
// so no per-token state is ever materialised.
template <typename T>
struct ScanBwdArgs {
  const T *U, *B, *C, *dY;
  const float *M, *K, *starts, *d_inc, *zdot, *Bprev, *Uprev;
  T *dU, *dB, *dC;
  float *dM, *dK, *carryB, *carryU;
  ScanDims d;
};

template <int L>
constexpr size_t scan_bwd_smem_bytes() {
  constexpr int DS = ChunkCfg<L>::DS_BWD;
  return sizeof(float) * (size_t)(2 * L * kLdP + L * (L + 1) + 4 * L * (DS + 1) + 2 * kPMax * (DS + 1) +
                                  3 * L /*lp,gd,gm1*/ + 2 * L * 12 /*complex rows*/ + 2 * kPMax + 6 * DS + 16);
}

template <typename T, int L>
__global__ void __launch_bounds__(kThreads) chunk_scan_bwd_kernel(ScanBwdArgs<T> a) {
  constexpr int TM = ChunkCfg<L>::TM;
  constexpr int DS = ChunkCfg<L>::DS_BWD, LDS = DS + 1, LDL = L + 1;
  using SM = SlabMap<L, DS>;
  constexpr int NP = SM::NP, NPT = SM::NPT, TNP = SM::TNP, RG = SM::RG, TMS = SM::TMS;

  extern __shared__ float sm[];
  float *dYs = sm;                     // L*kLdP
  float *Us = dYs + L * kLdP;          // L*kLdP
  float *dSs = Us + L * kLdP;          // L*LDL   (dS', later S')
  float *Qs = dSs + L * LDL;           // L*LDS   Qbar
  float *Ks = Qs + L * LDS;            // L*LDS   kappa
  float *Bh = Ks + L * LDS;            // L*LDS   w_s b_s  (increment operand)
  float *Bs = Bh + L * LDS;            // L*LDS   raw b
  float *Zs = Bs + L * LDS;            // kPMax*LDS
  float *Ls = Zs + kPMax * LDS;        // kPMax*LDS  d_inc slab
  float *lp = Ls + kPMax * LDS;        // L
  float *gd = lp + L;                  // L   G[t,t]
  float *gm1 = gd + L;                 // L   dY_t . u_{-1}
  size_t off = (size_t)2 * L * kLdP + L * LDL + 4 * L * LDS + 2 * kPMax * LDS + 3 * L;
  float2 *ph = reinterpret_cast<float2 *>(gm1 + L + (off & 1));
  float2 *mraw = ph + L, *kc = mraw + L, *kp = kc + L, *gam = kp + L, *wco = gam + L, *sg1 = wco + L;
  float2 *bc = sg1 + L, *cbm = bc + L, *bX = cbm + L, *gA = bX + L, *gsum = gA + L;
  float *um1 = reinterpret_cast<float *>(gsum + L);  // kPMax
  float *duc = um1 + kPMax;                           // kPMax  dU carry accumulator
  float *bm1 = duc + kPMax;                           // DS raw b_{-1}
  float *km1 = bm1 + DS;                              // DS kappa_{-1}
  float *bh1 = km1 + DS;                              // DS w_{-1} b_{-1}
  float *ul1 = bh1 + DS;                              // DS (u_{-1} . d_inc)[n]
  float *xi1 = ul1 + DS;                              // DS Xi_{-1}
  float2 *misc = reinterpret_cast<float2 *>(xi1 + DS);  // [0] = bLam (last row), [1] = dk^p_0, [2]= w_{-1}

  const ScanDims d = a.d;
  const int tid = threadIdx.x, ty = tid >> 4, tx = tid & 15;
  const int rg = tid / NPT, pcl = tid % NPT;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int t0 = c * L;
  const int valid = min(L, d.T - t0);
  const size_t tok0 = (size_t)bh * d.T + t0;

  chunk_prefix_warp0(a.M + tok0 * 2, L, valid, lp, ph, mraw, &g_scan_bad);
  for (int t = tid; t < L; t += kThreads) {
    float2 vp = make_float2(0.f, 0.f), vc = vp;
    if (t < valid) {
      float4 k4 = *reinterpret_cast<const float4 *>(a.K + (tok0 + t) * 4);
      vp = make_float2(k4.x, k4.y);
      vc = make_float2(k4.z, k4.w);
    }
    kp[t] = vp;
    kc[t] = vc;
    bc[t] = cbm[t] = bX[t] = gA[t] = make_float2(0.f, 0.f);
  }
  for (int idx = tid; idx < L * d.P; idx += kThreads) {
    int t = idx / d.P, p = idx - t * d.P;
    bool ok = t < valid;
    Us[t * kLdP + p] = ok ? to_f(a.U[(tok0 + t) * d.P + p]) : 0.f;
    dYs[t * kLdP + p] = ok ? to_f(a.dY[(tok0 + t) * d.P + p]) : 0.f;
  }
  // columns p >= P of the tiles are read by the tile products: keep them zero
  if (d.P < kPMax) {
    for (int idx = tid; idx < L * (kPMax - d.P); idx += kThreads) {
      int t = idx / (kPMax - d.P), p = d.P + idx % (kPMax - d.P);
      Us[t * kLdP + p] = 0.f;
      dYs[t * kLdP + p] = 0.f;
    }
  }
  for (int p = tid; p < kPMax; p += kThreads) {
    float v = 0.f;
    if (p < d.P) {
      if (t0 > 0) v = to_f(a.U[(tok0 - 1) * d.P + p]);
      else if (a.Uprev) v = a.Uprev[(size_t)bh * d.P + p];
    }
    um1[p] = v;
    duc[p] = 0.f;
  }
  for (int idx = tid; idx < kPMax * LDS; idx += kThreads) {
    Zs[idx] = 0.f;
    Ls[idx] = 0.f;
  }
  if (tid < 3) misc[tid] = make_float2(0.f, 0.f);
  __syncthreads();
  for (int t = tid; t < L; t += kThreads) {
    float2 g = make_float2(0.f, 0.f), w, s1 = make_float2(0.f, 0.f);
    if (t + 1 < L) {
      g = cadd(cmul(mraw[t + 1], kc[t]), kp[t + 1]);
      s1 = cscale(cmulc(ph[L - 1], ph[t + 1]), expf(lp[L - 1] - lp[t + 1]));  // p_{L-1}/p_{t+1}
      w = cmul(s1, g);
    } else {
      w = kc[t];
    }
    gam[t] = g;
    sg1[t] = s1;
    wco[t] = w;
    // g_{-1}[t] = dY_t . u_{-1}
    float acc = 0.f;
    for (int p = 0; p < d.P; ++p) acc = fmaf(dYs[t * kLdP + p], um1[p], acc);
    gm1[t] = acc;
  }
  if (tid == 0) misc[2] = cmul(cscale(cmulc(ph[L - 1], ph[0]), expf(lp[L - 1] - lp[0])), kp[0]);
  __syncthreads();

  // ---- G = dY U^T, dS' = G * exp(lp_t - lp_{s+1}) on s < t ---------------------
  {
    float G[TM][TM];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
      for (int j = 0; j < TM; ++j) G[i][j] = 0.f;
    mm_acc<TM, TM>(G, d.P, [&](int i, int k) { return dYs[(ty + 16 * i) * kLdP + k]; },
                   [&](int j, int k) { return Us[(tx + 16 * j) * kLdP + k]; });
#pragma unroll
    for (int i = 0; i < TM; ++i) {
      int t = ty + 16 * i;
#pragma unroll
      for (int j = 0; j < TM; ++j) {
        int s = tx + 16 * j;
        dSs[t * LDL + s] = (s < t) ? G[i][j] * expf(lp[t] - lp[s + 1]) : 0.f;
        if (s == t) gd[t] = G[i][j];
      }
    }
  }
  __syncthreads();

  float S[TM][TM], dUa[TM][4];
#pragma unroll
  for (int i = 0; i < TM; ++i) {
#pragma unroll
    for (int j = 0; j < TM; ++j) S[i][j] = 0.f;
#pragma unroll
    for (int j = 0; j < 4; ++j) dUa[i][j] = 0.f;
  }
  const float *z0 = a.starts + ((size_t)bh * d.NC + c) * d.P * d.D;
  const float *lam = a.d_inc + ((size_t)bh * d.NC + c) * d.P * d.D;
  const float2 w_m1 = misc[2];

  for (int d0 = 0; d0 < d.D; d0 += DS) {
    // ---- stage the slab ---------------------------------------------------
    for (int n = tid; n < NP; n += kThreads) {
      int dd = d0 + 2 * n;
      float2 bv = make_float2(0.f, 0.f);
      if (dd < d.D) {
        if (t0 > 0) bv = load_pair<T>(a.B + (tok0 - 1) * d.D + dd);
        else if (a.Bprev) bv = *reinterpret_cast<const float2 *>(a.Bprev + (size_t)bh * d.D + dd);
      }
      bm1[2 * n] = bv.x;
      bm1[2 * n + 1] = bv.y;
      float2 k1 = cmulc(cmul(kp[0], bv), ph[0]);  // kappa_{-1} = k^p_0 b_{-1} conj(phi_0)
      km1[2 * n] = k1.x;
      km1[2 * n + 1] = k1.y;
      float2 b1 = cmul(w_m1, bv);
      bh1[2 * n] = b1.x;
      bh1[2 * n + 1] = b1.y;
    }
    for (int idx = tid; idx < d.P * NP; idx += kThreads) {
      int p = idx / NP, n = idx - p * NP;
      int dd = d0 + 2 * n;
      float2 zv = make_float2(0.f, 0.f), lv = zv;
      if (dd < d.D) {
        zv = *reinterpret_cast<const float2 *>(z0 + (size_t)p * d.D + dd);
        lv = *reinterpret_cast<const float2 *>(lam + (size_t)p * d.D + dd);
      }
      Zs[p * LDS + 2 * n] = zv.x;
      Zs[p * LDS + 2 * n + 1] = zv.y;
      Ls[p * LDS + 2 * n] = lv.x;
      Ls[p * LDS + 2 * n + 1] = lv.y;
    }
    __syncthreads();
    for (int idx = tid; idx < L * NP; idx += kThreads) {
      int row = idx / NP, n = idx - row * NP;
      int dd = d0 + 2 * n;
      float2 cv = make_float2(0.f, 0.f), bv = cv;
      if (row < valid && dd < d.D) {
        cv = load_pair<T>(a.C + (tok0 + row) * d.D + dd);
        bv = load_pair<T>(a.B + (tok0 + row) * d.D + dd);
      }
      float2 q = cmulc(cv, ph[row]);
      Qs[row * LDS + 2 * n] = q.x;
      Qs[row * LDS + 2 * n + 1] = q.y;
      float2 kap = make_float2(0.f, 0.f);
      if (row + 1 < L) kap = cmulc(cmul(gam[row], bv), ph[row + 1]);
      Ks[row * LDS + 2 * n] = kap.x;
      Ks[row * LDS + 2 * n + 1] = kap.y;
      float2 bhv = cmul(wco[row], bv);
      Bh[row * LDS + 2 * n] = bhv.x;
      Bh[row * LDS + 2 * n + 1] = bhv.y;
      Bs[row * LDS + 2 * n] = bv.x;
      Bs[row * LDS + 2 * n + 1] = bv.y;
      float2 d1 = group_sum<NP>(cmul(cconj(bv), cv));  // conj(b) c
      float2 d2 = group_sum<NP>(cmul(cconj(cv), make_float2(bm1[2 * n], bm1[2 * n + 1])));
      if (n == 0) {
        bc[row] = cadd(bc[row], d1);
        cbm[row] = cadd(cbm[row], d2);
      }
    }
    // (u_{-1} . d_inc)[col], carry of dU through the increment, per column / per p
    for (int col = tid; col < DS; col += kThreads) {
      float acc = 0.f;
      for (int p = 0; p < d.P; ++p) acc = fmaf(um1[p], Ls[p * LDS + col], acc);
      ul1[col] = acc;
    }
    for (int p = tid; p < d.P; p += kThreads) {
      float acc = 0.f;
      for (int col = 0; col < DS; ++col) acc = fmaf(bh1[col], Ls[p * LDS + col], acc);
      duc[p] += acc;
    }
    __syncthreads();

    // ---- forward scores and the increment path of dU -------------------------
    mm_acc<TM, TM>(S, DS, [&](int i, int k) { return Qs[(ty + 16 * i) * LDS + k]; },
                   [&](int j, int k) { return Ks[(tx + 16 * j) * LDS + k]; });
    mm_acc<TM, 4>(dUa, DS, [&](int i, int k) { return Bh[(ty + 16 * i) * LDS + k]; },
                  [&](int j, int k) { return Ls[(tx + 16 * j) * LDS + k]; });

    // ---- slab tiles: dq, X, U.Lambda ------------------------------------------
    float dq[TMS][2 * TNP], X[TMS][2 * TNP], UL[TMS][2 * TNP];
#pragma unroll
    for (int i = 0; i < TMS; ++i)
#pragma unroll
      for (int j = 0; j < 2 * TNP; ++j) dq[i][j] = X[i][j] = UL[i][j] = 0.f;
    auto colof = [&](int j) { return 2 * (pcl + NPT * (j >> 1)) + (j & 1); };
    mm_acc<TMS, 2 * TNP>(dq, L, [&](int i, int k) { return dSs[(rg + RG * i) * LDL + k]; },
                         [&](int j, int k) { return Ks[k * LDS + colof(j)]; });
    mm_acc<TMS, 2 * TNP>(X, L, [&](int i, int k) { return dSs[k * LDL + rg + RG * i]; },
                         [&](int j, int k) { return Qs[k * LDS + colof(j)]; });
    {
      float dz[TMS][2 * TNP];
#pragma unroll
      for (int i = 0; i < TMS; ++i)
#pragma unroll
        for (int j = 0; j < 2 * TNP; ++j) dz[i][j] = 0.f;
      mm_acc<TMS, 2 * TNP>(dz, d.P, [&](int i, int k) { return dYs[(rg + RG * i) * kLdP + k]; },
                           [&](int j, int k) { return Zs[k * LDS + colof(j)]; });
      mm_acc<TMS, 2 * TNP>(UL, d.P, [&](int i, int k) { return Us[(rg + RG * i) * kLdP + k]; },
                           [&](int j, int k) { return Ls[k * LDS + colof(j)]; });
#pragma unroll
      for (int i = 0; i < TMS; ++i) {
        int t = rg + RG * i;
        float el = expf(lp[t]), e0 = expf(lp[t] - lp[0]) * gm1[t];
#pragma unroll
        for (int j = 0; j < 2 * TNP; ++j) dq[i][j] += el * dz[i][j] + e0 * km1[colof(j)];
      }
    }
    // Xi_{-1}[col] = phi_0 sum_t exp(lp_t-lp_0) g_{-1}[t] Qbar_t[col] + conj(p_{L-1}/p_0)(u_{-1}.Lambda)
    // (column sums over the chunk; one thread per complex column)
    for (int n = tid; n < NP; n += kThreads) {
      float2 acc = make_float2(0.f, 0.f);
      for (int t = 0; t < L; ++t) {
        float w = expf(lp[t] - lp[0]) * gm1[t];
        acc.x = fmaf(w, Qs[t * LDS + 2 * n], acc.x);
        acc.y = fmaf(w, Qs[t * LDS + 2 * n + 1], acc.y);
      }
      float2 s0 = cscale(cmulc(ph[L - 1], ph[0]), expf(lp[L - 1] - lp[0]));  // p_{L-1}/p_0
      float2 xi = cadd(cmul(ph[0], acc), cmul(cconj(s0), make_float2(ul1[2 * n], ul1[2 * n + 1])));
      xi1[2 * n] = xi.x;
      xi1[2 * n + 1] = xi.y;
    }

    // ---- epilogue of the slab ---------------------------------------------------
#pragma unroll
    for (int i = 0; i < TMS; ++i) {
      int t = rg + RG * i;
      float2 pgA = make_float2(0.f, 0.f), pbX = pgA, pbL = pgA;
      if (t < L) {
        const float2 pht = ph[t];
        const float2 ph1 = (t + 1 < L) ? ph[t + 1] : make_float2(0.f, 0.f);
#pragma unroll
        for (int jj = 0; jj < TNP; ++jj) {
          int cc = 2 * (pcl + NPT * jj);
          int dd = d0 + cc;
          float2 bv = make_float2(Bs[t * LDS + cc], Bs[t * LDS + cc + 1]);
          float2 qb = make_float2(Qs[t * LDS + cc], Qs[t * LDS + cc + 1]);
          float2 cv = cmul(qb, pht);  // c_t = Qbar_t phi_t
          // dC_t = phi_t dq_t + k^c_t G[t,t] b_t
          float2 dcv = cadd(cmul(pht, make_float2(dq[i][2 * jj], dq[i][2 * jj + 1])),
                            cscale(cmul(kc[t], bv), gd[t]));
          pgA = cadd(pgA, cmulc(cv, dcv));
          // Xi_t = phi_{t+1} X_t + conj(p_{L-1}/p_{t+1}) (U.Lambda)_t      (t <= L-2)
          float2 ulv = make_float2(UL[i][2 * jj], UL[i][2 * jj + 1]);
          float2 xi = make_float2(0.f, 0.f);
          if (t + 1 < L)
            xi = cadd(cmul(ph1, make_float2(X[i][2 * jj], X[i][2 * jj + 1])), cmul(cconj(sg1[t]), ulv));
          float2 dbe = cscale(cv, gd[t]);
          if (t == L - 1) {
            dbe = cadd(dbe, ulv);
            pbL = cadd(pbL, cmul(cconj(bv), ulv));
          }
          float2 dbv = cadd(cmul(cconj(kc[t]), dbe), cmul(cconj(gam[t]), xi));
          pbX = cadd(pbX, cmul(cconj(bv), xi));
          if (t < valid && dd < d.D) {
            store_pair<T>(a.dC + (tok0 + t) * d.D + dd, dcv);
            store_pair<T>(a.dB + (tok0 + t) * d.D + dd, dbv);
          }
        }
      }
      pgA = group_sum<NPT>(pgA);
      pbX = group_sum<NPT>(pbX);
      pbL = group_sum<NPT>(pbL);
      if (pcl == 0 && t < L) {
        gA[t] = cadd(gA[t], pgA);
        bX[t] = cadd(bX[t], pbX);
        if (t == L - 1) misc[0] = cadd(misc[0], pbL);
      }
    }
    __syncthreads();
    // carry to the token before the chunk: dB_{-1} = conj(k^p_0) Xi_{-1}; dk^p_0 += conj(b_{-1}).Xi_{-1}
    {
      float *cB = a.carryB + ((size_t)bh * d.NC + c) * d.D;
      for (int n = tid; n < NP; n += kThreads) {
        int dd = d0 + 2 * n;
        if (dd < d.D) {
          float2 v = cmul(cconj(kp[0]), make_float2(xi1[2 * n], xi1[2 * n + 1]));
          *reinterpret_cast<float2 *>(cB + dd) = v;
        }
      }
      if (tid == 0) {
        float2 acc = misc[1];
        for (int n = 0; n < NP; ++n)
          acc = cadd(acc, cmul(cconj(make_float2(bm1[2 * n], bm1[2 * n + 1])), make_float2(xi1[2 * n], xi1[2 * n + 1])));
        misc[1] = acc;
      }
    }
    __syncthreads();
  }

  // ---- S' (forward scores) into shared memory; dU -----------------------------
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int t = ty + 16 * i;
#pragma unroll
    for (int j = 0; j < TM; ++j) {
      int s = tx + 16 * j;
      float v = 0.f;
      if (s < t) v = S[i][j] * expf(lp[t] - lp[s + 1]);
      else if (s == t) v = kc[t].x * bc[t].x + kc[t].y * bc[t].y;  // Re(k^c_t conj(bc_t))
      dSs[t * LDL + s] = v;
    }
  }
  __syncthreads();
  mm_acc<TM, 4>(dUa, L, [&](int i, int k) { return dSs[k * LDL + ty + 16 * i]; },
                [&](int j, int k) { return dYs[k * kLdP + tx + 16 * j]; });
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    int s = ty + 16 * i;
    if (s >= valid) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      int p = tx + 16 * j;
      if (p < d.P) a.dU[(tok0 + s) * d.P + p] = from_f<T>(dUa[i][j]);
    }
  }
  // dU carried to the token before the chunk: sum_t sigma_t dY_t + increment path
  for (int p = tid; p < d.P; p += kThreads) {
    float acc = duc[p];
    for (int t = 0; t < L; ++t) {
      float2 w = cmul(cmul(cmulc(ph[t], ph[0]), kp[0]), cbm[t]);
      acc = fmaf(expf(lp[t] - lp[0]) * w.x, dYs[t * kLdP + p], acc);
    }
    a.carryU[((size_t)bh * d.NC + c) * d.P + p] = acc;
  }
  // ---- dK and the per-token terms of dM ------------------------------------------
  for (int t = tid; t < L; t += kThreads) {
    float2 dkc = cscale(bc[t], gd[t]);
    if (t + 1 < L) dkc = cadd(dkc, cmul(cconj(mraw[t + 1]), bX[t]));
    else dkc = cadd(dkc, misc[0]);
    float2 dkp = (t == 0) ? misc[1] : bX[t - 1];
    if (t < valid) {
      *reinterpret_cast<float4 *>(a.dK + (tok0 + t) * 4) = make_float4(dkp.x, dkp.y, dkc.x, dkc.y);
    }
    float2 g = csub(gA[t], cadd(cmul(cconj(kc[t]), dkc), cmul(cconj(kp[t]), dkp)));
    if (t == L - 1) {
      const float *zd = a.zdot + ((size_t)bh * d.NC + c) * 2;
      g = cadd(g, make_float2(zd[0], zd[1]));
    }
    gsum[t] = g;
  }
  __syncthreads();
  if (tid == 0) {
    float2 acc = make_float2(0.f, 0.f);
    for (int t = L - 1; t >= 0; --t) {
      acc = cadd(acc, gsum[t]);
      gsum[t] = acc;
    }
  }
  __syncthreads();
  for (int t = tid; t < valid; t += kThreads) {
    // dM_t = cum_t / conj(m_t) = cum_t m_t / |m_t|^2
    float2 m = mraw[t];
    float inv = 1.f / (m.x * m.x + m.y * m.y);
    float2 v = cscale(cmul(gsum[t], m), inv);
    *reinterpret_cast<float2 *>(a.dM + (tok0 + t) * 2) = v;
  }
}

}  // namespace slx
