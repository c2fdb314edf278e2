// SLinOSSScanPrep forward/backward for sm_100a: bandwidth-bound, one lane group
// per (batch, head, token) row, 128-bit vector loads/stores, deterministic
// two-level reductions for the parameter gradients.
//
// Forward map (slinoss/layers/scanprep.py:351-357):
//   U  = value.view(b,T,H,P).permute(0,2,1,3)
//   B,C = interleave(rms_norm(bc) * scale)       (scanprep.py:297-336)
//   M,K = coefficient map of the 13-wide params row (scanprep.py:208-286,
//         ops/scanprep/reference.py:26-57)
#include <initializer_list>

#include "common.cuh"
#include "prep_coef.cuh"

namespace slx {

// VJP of coef_forward: dp[13] from (dM, dKprev, dKcurr)
__device__ __forceinline__ void coef_backward(const CoefCtx &c, const PrepHyper &h, float2 dm, float2 dkp, float2 dkc,
                                              float *dp) {
  const float d_dt = h.dt_max - h.dt_min, d_r = h.r_max - h.r_min;
  auto rdot = [](float2 a, float2 g) { return a.x * g.x + a.y * g.y; };
  float2 dkps = cscale(dkp, c.mix_kp), dkpl = cscale(dkp, 1.f - c.mix_kp);
  float dmix_kp = rdot(csub(c.kps, c.kpl), dkp);
  float2 dkcs = cscale(dkc, c.mix_kc), dkcl = cscale(dkc, 1.f - c.mix_kc);
  float dmix_kc = rdot(csub(c.kcs, c.kcl), dkc);
  float2 dk2 = cscale(csub(dkps, dkcs), c.dt);
  float2 dk1 = cscale(dkcs, c.dt);
  float ddt = rdot(c.k2, dkps) + rdot(csub(c.k1, c.k2), dkcs);
  float2 k1p, k2p;
  const float2 z = c.z;
  k1p = c.k2;  // d/dz (e^z-1)/z = kappa2, in both branches
  if (c.small) k2p = c.k2p;                                      // series (prep_coef.cuh)
  else k2p = cdiv(csub(c.rho, cscale(c.k2, 2.f)), z);            // d/dz (e^z(z-1)+1)/z^2 = (e^z - 2 kappa2)/z
  // dz = conj(k1') dk1 + conj(k2') dk2 + conj(rho) dM
  float2 dz = cadd(cadd(cmul(cconj(k1p), dk1), cmul(cconj(k2p), dk2)), cmul(cconj(c.rho), dm));
  float dr = dz.x / c.r;
  float dtheta = dz.y;
  float dth_d = (1.f - c.mix_th) * dtheta, dth_s = c.mix_th * dtheta;
  float dmix_th = (c.th_struct - c.th_direct) * dtheta;
  float dr_d = (1.f - c.mix_r) * dr, dr_s = c.mix_r * dr;
  float dmix_r = (c.r_struct - c.r_direct) * dr;
  float dgamma = dr_s * d_r * c.e_gdt * (-c.dt);
  ddt += dr_s * d_r * c.e_gdt * (-c.gamma);
  float domega = dth_s * c.dt;
  ddt += dth_s * c.omega;
  auto dsig = [](float s) { return s * (1.f - s); };
  dp[0] = ddt * d_dt * dsig(c.dt_u);
  dp[1] = dgamma * c.sig_p1;
  dp[2] = domega;
  dp[3] = dr_d * d_r * dsig(c.r_dir_u);
  dp[4] = dth_d * h.theta_bound * (1.f - c.th_t * c.th_t);
  dp[5] = dmix_r * dsig(c.mix_r);
  dp[6] = dmix_th * dsig(c.mix_th);
  dp[7] = dmix_kp * dsig(c.mix_kp);
  dp[8] = dmix_kc * dsig(c.mix_kc);
  dp[9] = h.k_max * (1.f - c.tk[0] * c.tk[0]) * dkpl.x;
  dp[10] = h.k_max * (1.f - c.tk[1] * c.tk[1]) * dkpl.y;
  dp[11] = h.k_max * (1.f - c.tk[2] * c.tk[2]) * dkcl.x;
  dp[12] = h.k_max * (1.f - c.tk[3] * c.tk[3]) * dkcl.y;
}

// ---- vector access ------------------------------------------------------------
template <typename T, int VEC>
__device__ __forceinline__ void load_vec(const T *p, float (&v)[VEC]) {
  if constexpr (VEC * sizeof(T) == 32 && sizeof(T) == 4) {
    const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  } else if constexpr (VEC * sizeof(T) == 16) {
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
__device__ __forceinline__ void store_vec(T *p, const float (&v)[VEC]) {
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

// ---- the 13-value parameter row of one (batch, head, token) ---------------------------------
// Half types: the row is 26 bytes at an arbitrary 2-byte offset.  `wide` loads the two or three
// aligned 16-byte vectors that cover it and picks the 13 values out by the (per-thread) offset;
// the caller passes wide = true only when every such vector lies inside the tensor (base and row
// stride multiples of 16 bytes, row width a multiple of 16 bytes).  Stores pair the values into
// 4-byte words wherever the address allows: 7 stores instead of 13.
template <typename T, int O>
__device__ __forceinline__ void pick13(const uint32_t (&w)[12], float (&p)[13]) {
#pragma unroll
  for (int i = 0; i < 13; ++i) {
    const uint32_t word = w[(O + i) >> 1];
    const unsigned short hbits = ((O + i) & 1) ? (unsigned short)(word >> 16) : (unsigned short)(word & 0xffffu);
    T v;
    *reinterpret_cast<unsigned short *>(&v) = hbits;
    p[i] = to_f(v);
  }
}
template <typename T>
__device__ __forceinline__ void load_row13(const T *pr, bool wide, float (&p)[13]) {
  if constexpr (sizeof(T) == 2) {
    if (wide) {
      const uintptr_t a = reinterpret_cast<uintptr_t>(pr);
      const uint4 *base = reinterpret_cast<const uint4 *>(a & ~uintptr_t(15));
      const int o = (int)((a & 15) >> 1);
      const uint4 v0 = base[0], v1 = base[1];
      uint4 v2 = make_uint4(0, 0, 0, 0);
      if (o > 3) v2 = base[2];  // elements o .. o+12 reach past the second vector
      const uint32_t w[12] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w, v2.x, v2.y, v2.z, v2.w};
      switch (o) {
        case 0: pick13<T, 0>(w, p); break;
        case 1: pick13<T, 1>(w, p); break;
        case 2: pick13<T, 2>(w, p); break;
        case 3: pick13<T, 3>(w, p); break;
        case 4: pick13<T, 4>(w, p); break;
        case 5: pick13<T, 5>(w, p); break;
        case 6: pick13<T, 6>(w, p); break;
        default: pick13<T, 7>(w, p); break;
      }
      return;
    }
  }
#pragma unroll
  for (int i = 0; i < 13; ++i) p[i] = to_f(pr[i]);
}
template <typename T>
__device__ __forceinline__ void store_row13(T *pr, const float (&v)[13]) {
  if constexpr (sizeof(T) == 2) {
    auto pair = [&](int i) {
      T lo = from_f<T>(v[i]), hi = from_f<T>(v[i + 1]);
      const uint32_t word = (uint32_t)(*reinterpret_cast<unsigned short *>(&lo)) |
                            ((uint32_t)(*reinterpret_cast<unsigned short *>(&hi)) << 16);
      *reinterpret_cast<uint32_t *>(pr + i) = word;
    };
    if ((reinterpret_cast<uintptr_t>(pr) & 3) == 0) {
#pragma unroll
      for (int i = 0; i < 12; i += 2) pair(i);
      pr[12] = from_f<T>(v[12]);
    } else {
      pr[0] = from_f<T>(v[0]);
#pragma unroll
      for (int i = 1; i < 13; i += 2) pair(i);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 13; ++i) pr[i] = from_f<T>(v[i]);
  }
}

template <int G>
__device__ __forceinline__ float group_sum_f(float v) {
#pragma unroll
  for (int off = G / 2; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
  return v;
}

struct PrepDims {
  int batch, T, H, P, N;
  int normalize;
  long long vs, ps, bs;  // row strides (elements)
  int wide_params;        // the covering 16-byte vectors of every params row lie inside the tensor
};

// Rows are ordered (b, h, t) so that a CTA's consecutive rows write contiguous
// output.  A group of G lanes handles one row; lane q of the group owns the
// state lanes n in [VEC*(q + G*k), VEC*(q + G*k) + VEC).
template <typename T, int VEC, int G>
__global__ void __launch_bounds__(256) scanprep_fwd_kernel(const T *__restrict__ value, const T *__restrict__ params,
                                                           const T *__restrict__ bc, const float *__restrict__ bias,
                                                           const float *__restrict__ scale, T *__restrict__ U,
                                                           float *__restrict__ M, float *__restrict__ K,
                                                           T *__restrict__ Bo, T *__restrict__ Co, PrepDims d,
                                                           PrepHyper hp) {
  // A CTA pass covers 256 consecutive rows.  Phase 1: one row per THREAD for the
  // coefficient map (its ~500 scalar instructions then cost one issue slot per 32 rows
  // instead of one per row).  Phase 2: one row per lane group for the wide copies.
  constexpr int GPB = 256 / G;   // lane groups per CTA
  constexpr int RPG = 256 / GPB; // rows each group walks through per pass (= G)
  const int q = threadIdx.x % G;
  const int grp = threadIdx.x / G;
  const long long n_rows = (long long)d.batch * d.H * d.T;
  const int D = 2 * d.N;
  for (long long row0 = (long long)blockIdx.x * 256; row0 < n_rows; row0 += (long long)gridDim.x * 256) {
    {
      const long long row = row0 + threadIdx.x;
      if (row < n_rows) {
        const int t = (int)(row % d.T);
        const int h = (int)((row / d.T) % d.H);
        const int b = (int)(row / ((long long)d.T * d.H));
        float p[13];
        const T *pr = params + ((long long)b * d.T + t) * d.ps + (long long)h * 13;
        load_row13<T>(pr, d.wide_params != 0, p);
#pragma unroll
        for (int i = 0; i < 13; ++i) p[i] += bias[h * 13 + i];
        CoefOut o = coef_forward(p, hp, nullptr);
        *reinterpret_cast<float2 *>(M + row * 2) = o.rho;
        *reinterpret_cast<float4 *>(K + row * 4) = make_float4(o.kp.x, o.kp.y, o.kc.x, o.kc.y);
      }
    }
    // (b, h, t) of the group's first row by division once per pass, then by increment
    const long long grow0 = row0 + (long long)grp * RPG;
    int gt, gh, gb;
    {
      const long long r = grow0 < n_rows ? grow0 : 0;
      gt = (int)(r % d.T);
      gh = (int)((r / d.T) % d.H);
      gb = (int)(r / ((long long)d.T * d.H));
    }
    constexpr bool kPacked = (VEC > 1) && (VEC * sizeof(T) == 16);
    const bool one_sweep = d.N <= G * VEC;
    // raw 16-byte slices of the next row (value + four bc planes), requested one row ahead
    uint4 nx[5];
    auto fetch_row = [&](long long row, int b, int h, int t) {
      if constexpr (kPacked) {
#pragma unroll
        for (int j = 0; j < 5; ++j) nx[j] = make_uint4(0, 0, 0, 0);
        if (row < n_rows) {
          const long long in_row = (long long)b * d.T + t;
          const int n0 = q * VEC;
          if (n0 < d.P) nx[4] = *reinterpret_cast<const uint4 *>(value + in_row * d.vs + (long long)h * d.P + n0);
          if (n0 < d.N) {
            const T *bcr = bc + in_row * d.bs + (long long)h * 4 * d.N;
#pragma unroll
            for (int j = 0; j < 4; ++j) nx[j] = *reinterpret_cast<const uint4 *>(bcr + j * d.N + n0);
          }
        }
      }
    };
    const bool packed_path = kPacked && one_sweep && d.P <= G * VEC;
    if (packed_path) fetch_row(grow0, gb, gh, gt);
    for (int k = 0; k < RPG; ++k) {
      const long long row = grow0 + k;
      const bool live = row < n_rows;
      const long long rr = live ? row : 0;
      const int t = live ? gt : 0, h = live ? gh : 0, b = live ? gb : 0;
      // advance (b, h, t) to the next row
      if (++gt == d.T) {
        gt = 0;
        if (++gh == d.H) {
          gh = 0;
          ++gb;
        }
      }
      const long long in_row = (long long)b * d.T + t;
      if constexpr (kPacked) {
        if (packed_path) {
          uint4 cur[5];
#pragma unroll
          for (int j = 0; j < 5; ++j) cur[j] = nx[j];
          if (k + 1 < RPG) fetch_row(row + 1, gb, gh, gt);
          const int n0 = q * VEC;
          if (live && n0 < d.P) *reinterpret_cast<uint4 *>(U + rr * d.P + n0) = cur[4];
          const bool mine = live && n0 < d.N;
          float y[4][VEC];
          float ss[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const T *e = reinterpret_cast<const T *>(&cur[j]);
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              y[j][i] = to_f(e[i]);
              a = fmaf(y[j][i], y[j][i], a);
            }
            ss[j] = a;
          }
          if (d.normalize) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              ss[j] = rsqrtf(group_sum_f<G>(ss[j]) / (float)d.N + 1e-5f);
              if (mine) {
                float sc[VEC];
                load_vec<float, VEC>(scale + ((long long)h * 4 + j) * d.N + n0, sc);
#pragma unroll
                for (int i = 0; i < VEC; ++i) y[j][i] = (y[j][i] * ss[j]) * sc[i];
              }
            }
          }
          if (mine) {
            float ob[2][VEC], oc[2][VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              int o = 2 * i;
              ob[o / VEC][o % VEC] = y[0][i];
              ob[(o + 1) / VEC][(o + 1) % VEC] = y[1][i];
              oc[o / VEC][o % VEC] = y[2][i];
              oc[(o + 1) / VEC][(o + 1) % VEC] = y[3][i];
            }
            store_vec<T, VEC>(Bo + rr * D + 2 * n0, ob[0]);
            store_vec<T, VEC>(Bo + rr * D + 2 * n0 + VEC, ob[1]);
            store_vec<T, VEC>(Co + rr * D + 2 * n0, oc[0]);
            store_vec<T, VEC>(Co + rr * D + 2 * n0 + VEC, oc[1]);
          }
          continue;
        }
      }
      // ---- U: copy P values ----
      if (live) {
        const T *src = value + in_row * d.vs + (long long)h * d.P;
        T *dst = U + rr * d.P;
        for (int p0 = q * VEC; p0 < d.P; p0 += G * VEC) {
          float v[VEC];
          load_vec<T, VEC>(src + p0, v);
          store_vec<T, VEC>(dst + p0, v);
        }
      }
      // ---- B, C ----
      const T *bcr = bc + in_row * d.bs + (long long)h * 4 * d.N;
      if (one_sweep) {
        // one sweep: every lane keeps its four row slices in registers
        const int n0 = q * VEC;
        const bool mine = live && n0 < d.N;
        float y[4][VEC];
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          if (mine) load_vec<T, VEC>(bcr + j * d.N + n0, y[j]);
          else {
#pragma unroll
            for (int i = 0; i < VEC; ++i) y[j][i] = 0.f;
          }
#pragma unroll
          for (int i = 0; i < VEC; ++i) ss[j] = fmaf(y[j][i], y[j][i], ss[j]);
        }
        if (d.normalize) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            ss[j] = rsqrtf(group_sum_f<G>(ss[j]) / (float)d.N + 1e-5f);
            if (mine) {
              float sc[VEC];
              load_vec<float, VEC>(scale + ((long long)h * 4 + j) * d.N + n0, sc);
#pragma unroll
              for (int i = 0; i < VEC; ++i) y[j][i] = (y[j][i] * ss[j]) * sc[i];
            }
          }
        }
        if (mine) {
          float ob[2][VEC], oc[2][VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            int o = 2 * i;
            ob[o / VEC][o % VEC] = y[0][i];
            ob[(o + 1) / VEC][(o + 1) % VEC] = y[1][i];
            oc[o / VEC][o % VEC] = y[2][i];
            oc[(o + 1) / VEC][(o + 1) % VEC] = y[3][i];
          }
          store_vec<T, VEC>(Bo + rr * D + 2 * n0, ob[0]);
          store_vec<T, VEC>(Bo + rr * D + 2 * n0 + VEC, ob[1]);
          store_vec<T, VEC>(Co + rr * D + 2 * n0, oc[0]);
          store_vec<T, VEC>(Co + rr * D + 2 * n0 + VEC, oc[1]);
        }
      } else {
        float ss[4] = {0.f, 0.f, 0.f, 0.f};
        if (d.normalize) {
          if (live) {
            for (int n0 = q * VEC; n0 < d.N; n0 += G * VEC) {
#pragma unroll
              for (int j = 0; j < 4; ++j) {
                float v[VEC];
                load_vec<T, VEC>(bcr + j * d.N + n0, v);
#pragma unroll
                for (int i = 0; i < VEC; ++i) ss[j] = fmaf(v[i], v[i], ss[j]);
              }
            }
          }
#pragma unroll
          for (int j = 0; j < 4; ++j) ss[j] = rsqrtf(group_sum_f<G>(ss[j]) / (float)d.N + 1e-5f);
        }
        if (live) {
          for (int n0 = q * VEC; n0 < d.N; n0 += G * VEC) {
            float y[4][VEC];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
              load_vec<T, VEC>(bcr + j * d.N + n0, y[j]);
              if (d.normalize) {
                const float *sc = scale + ((long long)h * 4 + j) * d.N + n0;
#pragma unroll
                for (int i = 0; i < VEC; ++i) y[j][i] = (y[j][i] * ss[j]) * sc[i];
              }
            }
            float ob[2][VEC], oc[2][VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i) {
              int o = 2 * i;
              ob[o / VEC][o % VEC] = y[0][i];
              ob[(o + 1) / VEC][(o + 1) % VEC] = y[1][i];
              oc[o / VEC][o % VEC] = y[2][i];
              oc[(o + 1) / VEC][(o + 1) % VEC] = y[3][i];
            }
            store_vec<T, VEC>(Bo + rr * D + 2 * n0, ob[0]);
            store_vec<T, VEC>(Bo + rr * D + 2 * n0 + VEC, ob[1]);
            store_vec<T, VEC>(Co + rr * D + 2 * n0, oc[0]);
            store_vec<T, VEC>(Co + rr * D + 2 * n0 + VEC, oc[1]);
          }
        }
      }
    }
  }
}

template <typename T>
__device__ __forceinline__ void scanprep_bwd_coef_tile(const T *__restrict__ params, const float *__restrict__ bias,
                                                       const float *__restrict__ dM, const float *__restrict__ dK,
                                                       T *__restrict__ d_params, float *__restrict__ part,
                                                       const PrepDims &d, const PrepHyper &hp, int rows_per_tile,
                                                       int tile, int n_tiles);

// Backward.  grid = (2 * tiles over T, batch*H).  CTAs with blockIdx.x < n_tiles stream the wide
// rows; the others run the coefficient-map VJP of the same tiles (scanprep_bwd_coef_tile): its long
// scalar chains fill issue slots that the streaming CTAs leave idle while they wait on memory.
// Every CTA works on one head, so the
// per-head parameter gradients reduce inside the CTA first (registers ->
// shared memory in a fixed order) and then across CTAs in a second kernel.
// Partial layout: part[(bh * n_tiles + tile)][4*N + 13].
template <typename T, int VEC, int G, int KMAX>
__global__ void __launch_bounds__(256, KMAX == 1 ? 2 : 1) scanprep_bwd_kernel(const T *__restrict__ params, const T *__restrict__ bc,
                                                           const float *__restrict__ bias,
                                                           const float *__restrict__ scale, const T *__restrict__ dU,
                                                           const float *__restrict__ dM, const float *__restrict__ dK,
                                                           const T *__restrict__ dB, const T *__restrict__ dC,
                                                           T *__restrict__ d_value, T *__restrict__ d_params,
                                                           T *__restrict__ d_bc, float *__restrict__ part, PrepDims d,
                                                           PrepHyper hp, int rows_per_tile, int n_tiles) {
  if ((int)blockIdx.x >= n_tiles) {
    scanprep_bwd_coef_tile<T>(params, bias, dM, dK, d_params, part, d, hp, rows_per_tile, (int)blockIdx.x - n_tiles,
                              n_tiles);
    return;
  }
  constexpr int GPB = 256 / G;  // KMAX sweeps of VEC*G state lanes cover N
  extern __shared__ float red[];  // GPB * (4N + 13)
  const int q = threadIdx.x % G, grp = threadIdx.x / G;
  const int bh = blockIdx.y, b = bh / d.H, h = bh % d.H;
  const int D = 2 * d.N;
  const int W = 4 * d.N + 13;
  const int t_lo = blockIdx.x * rows_per_tile;
  const int t_hi = min(d.T, t_lo + rows_per_tile);

  float dsc[KMAX][4][VEC];
#pragma unroll
  for (int k = 0; k < KMAX; ++k)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int i = 0; i < VEC; ++i) dsc[k][j][i] = 0.f;
  // Single-sweep path (one 16-byte vector per lane covers N): the row's raw bc and dB/dC stay
  // packed in registers (8 x 16 bytes) and are expanded twice, once for the row sums and once
  // for the output, instead of holding expanded fp32 copies; the head's scale sits in shared memory.
  constexpr bool kPacked = (KMAX == 1) && (VEC > 1) && (VEC * sizeof(T) == 16);
  float *sscale = red + (size_t)GPB * W;
  if (kPacked && d.normalize) {
    for (int e = threadIdx.x; e < 4 * d.N; e += 256) sscale[e] = scale[(long long)h * 4 * d.N + e];
    __syncthreads();
  }
  if constexpr (kPacked) {
    const int n0 = q * VEC;
    const bool lane_on = n0 < d.N;
    for (int tb = t_lo; tb < t_hi; tb += GPB) {
      const int t = tb + grp;
      const bool live = (t < t_hi);
      const int tt = live ? t : t_lo;
      const long long in_row = (long long)b * d.T + tt;
      const long long orow = ((long long)bh) * d.T + tt;
      const T *bcr = bc + in_row * d.bs + (long long)h * 4 * d.N;
      T *dbcr = d_bc + in_row * ((long long)d.H * 4 * d.N) + (long long)h * 4 * d.N;
      uint4 xr[4], gr[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) xr[j] = gr[j] = make_uint4(0, 0, 0, 0);
      if (live && lane_on) {
#pragma unroll
        for (int j = 0; j < 4; ++j) xr[j] = *reinterpret_cast<const uint4 *>(bcr + j * d.N + n0);
        gr[0] = *reinterpret_cast<const uint4 *>(dB + orow * D + 2 * n0);
        gr[1] = *reinterpret_cast<const uint4 *>(dB + orow * D + 2 * n0 + VEC);
        gr[2] = *reinterpret_cast<const uint4 *>(dC + orow * D + 2 * n0);
        gr[3] = *reinterpret_cast<const uint4 *>(dC + orow * D + 2 * n0 + VEC);
      }
      if (live) {
        const T *src = dU + orow * d.P;
        T *dst = d_value + in_row * ((long long)d.H * d.P) + (long long)h * d.P;
        for (int p0 = q * VEC; p0 < d.P; p0 += G * VEC)
          *reinterpret_cast<uint4 *>(dst + p0) = *reinterpret_cast<const uint4 *>(src + p0);
      }
      auto elem = [](const uint4 &raw, int i) { return to_f(reinterpret_cast<const T *>(&raw)[i]); };
      // dy of (plane j, lane i): de-interleave (re, im) pairs of dB (j < 2) or dC
      auto dy_of = [&](int j, int i) {
        const int o = 2 * i + (j & 1);
        return elem(gr[(j < 2 ? 0 : 2) + o / VEC], o % VEC);
      };
      if (d.normalize) {
        float ss[4], gx[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = 0.f;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float v = elem(xr[j], i);
            a = fmaf(v, v, a);
          }
          ss[j] = rsqrtf(group_sum_f<G>(a) / (float)d.N + 1e-5f);
        }
        // keep the packed words opaque between the passes: expanding them again costs a few
        // shifts, holding 64 expanded values across the group sums costs the occupancy
#define SLX_OPAQUE4(u) asm volatile("" : "+r"((u).x), "+r"((u).y), "+r"((u).z), "+r"((u).w))
#pragma unroll
        for (int j = 0; j < 4; ++j) SLX_OPAQUE4(xr[j]);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float a = 0.f;
          const float4 s0 = *reinterpret_cast<const float4 *>(sscale + j * d.N + (lane_on ? n0 : 0));
          const float4 s1 = *reinterpret_cast<const float4 *>(sscale + j * d.N + (lane_on ? n0 : 0) + 4);
          const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float xv = elem(xr[j], i) * ss[j];
            const float dy = dy_of(j, i);
            dsc[0][j][i] = fmaf(dy, xv, dsc[0][j][i]);
            a = fmaf(dy * sc[i], xv, a);
          }
          gx[j] = group_sum_f<G>(a) / (float)d.N;
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          SLX_OPAQUE4(xr[j]);
          SLX_OPAQUE4(gr[j]);
        }
#undef SLX_OPAQUE4
        if (live && lane_on) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const float4 s0 = *reinterpret_cast<const float4 *>(sscale + j * d.N + n0);
            const float4 s1 = *reinterpret_cast<const float4 *>(sscale + j * d.N + n0 + 4);
            const float sc[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
            float o[VEC];
#pragma unroll
            for (int i = 0; i < VEC; ++i)
              o[i] = ss[j] * (dy_of(j, i) * sc[i] - elem(xr[j], i) * ss[j] * gx[j]);
            store_vec<T, VEC>(dbcr + j * d.N + n0, o);
          }
        }
      } else if (live && lane_on) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float o[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i) o[i] = dy_of(j, i);
          store_vec<T, VEC>(dbcr + j * d.N + n0, o);
        }
      }
    }
  } else
  for (int tb = t_lo; tb < t_hi; tb += GPB) {
    const int t = tb + grp;
    const bool live = t < t_hi;
    const int tt = live ? t : t_lo;
    const long long in_row = (long long)b * d.T + tt;
    const long long orow = ((long long)bh) * d.T + tt;
    if (live) {
      const T *src = dU + orow * d.P;
      T *dst = d_value + in_row * ((long long)d.H * d.P) + (long long)h * d.P;
      for (int p0 = q * VEC; p0 < d.P; p0 += G * VEC) {
        float v[VEC];
        load_vec<T, VEC>(src + p0, v);
        store_vec<T, VEC>(dst + p0, v);
      }
    }
    const T *bcr = bc + in_row * d.bs + (long long)h * 4 * d.N;
    T *dbcr = d_bc + in_row * ((long long)d.H * 4 * d.N) + (long long)h * 4 * d.N;
    float ss[4] = {0.f, 0.f, 0.f, 0.f}, gx[4] = {0.f, 0.f, 0.f, 0.f};
    if (d.normalize) {
      if (live) {
        int k = 0;
        for (int n0 = q * VEC; n0 < d.N; n0 += G * VEC, ++k) {
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            float v[VEC];
            load_vec<T, VEC>(bcr + j * d.N + n0, v);
#pragma unroll
            for (int i = 0; i < VEC; ++i) ss[j] = fmaf(v[i], v[i], ss[j]);
          }
        }
      }
#pragma unroll
      for (int j = 0; j < 4; ++j) ss[j] = rsqrtf(group_sum_f<G>(ss[j]) / (float)d.N + 1e-5f);
    }
    // second sweep: dy (de-interleaved), dscale, sum g*xhat
    float xh[KMAX][4][VEC], gg[KMAX][4][VEC];
    {
      int k = 0;
      for (int n0 = q * VEC; n0 < d.N && k < KMAX; n0 += G * VEC, ++k) {
        float ib[2][VEC], ic[2][VEC];
        if (live) {
          load_vec<T, VEC>(dB + orow * D + 2 * n0, ib[0]);
          load_vec<T, VEC>(dB + orow * D + 2 * n0 + VEC, ib[1]);
          load_vec<T, VEC>(dC + orow * D + 2 * n0, ic[0]);
          load_vec<T, VEC>(dC + orow * D + 2 * n0 + VEC, ic[1]);
        }
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float x[VEC];
          if (live) load_vec<T, VEC>(bcr + j * d.N + n0, x);
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            int o = 2 * i + (j & 1);
            float dy = 0.f;
            if (live) dy = (j < 2) ? ib[o / VEC][o % VEC] : ic[o / VEC][o % VEC];
            if (d.normalize) {
              float xv = live ? x[i] * ss[j] : 0.f;
              float g = dy * scale[((long long)h * 4 + j) * d.N + n0 + i];
              xh[k][j][i] = xv;
              gg[k][j][i] = g;
              dsc[k][j][i] = fmaf(dy, xv, dsc[k][j][i]);
              gx[j] = fmaf(g, xv, gx[j]);
            } else {
              gg[k][j][i] = dy;
            }
          }
        }
      }
    }
    if (d.normalize) {
#pragma unroll
      for (int j = 0; j < 4; ++j) gx[j] = group_sum_f<G>(gx[j]) / (float)d.N;
    }
    if (live) {
      int k = 0;
      for (int n0 = q * VEC; n0 < d.N && k < KMAX; n0 += G * VEC, ++k) {
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          float o[VEC];
#pragma unroll
          for (int i = 0; i < VEC; ++i)
            o[i] = d.normalize ? ss[j] * (gg[k][j][i] - xh[k][j][i] * gx[j]) : gg[k][j][i];
          store_vec<T, VEC>(dbcr + j * d.N + n0, o);
        }
      }
    }
  }
  // ---- CTA-level reduction in a fixed order ----
  {
    float *mine = red + (size_t)grp * W;
    if (d.normalize) {
      int k = 0;
      for (int n0 = q * VEC; n0 < d.N && k < KMAX; n0 += G * VEC, ++k)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
          for (int i = 0; i < VEC; ++i) mine[j * d.N + n0 + i] = dsc[k][j][i];
    }
  }
  __syncthreads();
  float *outp = part + ((size_t)bh * n_tiles + blockIdx.x) * W;
  for (int e = threadIdx.x; e < W; e += 256) {
    if (!d.normalize && e < 4 * d.N) {
      outp[e] = 0.f;
      continue;
    }
    if (e >= 4 * d.N) continue;  // the 13 bias slots belong to the coefficient CTAs
    float acc = 0.f;
    for (int g = 0; g < GPB; ++g) acc += red[(size_t)g * W + e];
    outp[e] = acc;
  }
}

// Coefficient-map VJP of the backward: one row per thread (rows_per_tile == blockDim.x),
// d_params rows and the per-tile partial sums of the 13 bias gradients
// (part[(bh * n_tiles + tile)][4N .. 4N+13)).  Little traffic, long scalar chains: run by CTAs of
// their own inside the backward launch.
template <typename T>
__device__ __forceinline__ void scanprep_bwd_coef_tile(const T *__restrict__ params, const float *__restrict__ bias,
                                                       const float *__restrict__ dM, const float *__restrict__ dK,
                                                       T *__restrict__ d_params, float *__restrict__ part,
                                                       const PrepDims &d, const PrepHyper &hp, int rows_per_tile,
                                                       int tile, int n_tiles) {
  const int bh = blockIdx.y, b = bh / d.H, h = bh % d.H;
  const int W = 4 * d.N + 13;
  const int t_lo = tile * rows_per_tile;
  const int t_hi = min(d.T, t_lo + rows_per_tile);
  __shared__ float sbias[8][13];
  {
    float dbias[13];
#pragma unroll
    for (int i = 0; i < 13; ++i) dbias[i] = 0.f;
    for (int t = t_lo + (int)threadIdx.x; t < t_hi; t += 256) {
      const long long in_row = (long long)b * d.T + t;
      const long long orow = ((long long)bh) * d.T + t;
      float p[13], dp[13];
      const T *pr = params + in_row * d.ps + (long long)h * 13;
      load_row13<T>(pr, d.wide_params != 0, p);
#pragma unroll
      for (int i = 0; i < 13; ++i) p[i] += bias[h * 13 + i];
      CoefCtx ctx;
      coef_forward(p, hp, &ctx);
      float2 dm = *reinterpret_cast<const float2 *>(dM + orow * 2);
      float4 dk = *reinterpret_cast<const float4 *>(dK + orow * 4);
      coef_backward(ctx, hp, dm, make_float2(dk.x, dk.y), make_float2(dk.z, dk.w), dp);
      store_row13<T>(d_params + in_row * ((long long)d.H * 13) + (long long)h * 13, dp);
#pragma unroll
      for (int i = 0; i < 13; ++i) dbias[i] += dp[i];
    }
#pragma unroll
    for (int i = 0; i < 13; ++i) {
      float v = dbias[i];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
      if ((threadIdx.x & 31) == 0) sbias[threadIdx.x >> 5][i] = v;
    }
  }

  __syncthreads();
  if (threadIdx.x < 13) {
    float acc = 0.f;
    for (int w = 0; w < 8; ++w) acc += sbias[w][threadIdx.x];
    part[((size_t)bh * n_tiles + tile) * W + 4 * d.N + threadIdx.x] = acc;
  }
}

// d_scale[h][e], d_bias[h][i] = sum over batch and tiles of the partials, fixed order
__global__ void scanprep_reduce_kernel(const float *__restrict__ part, float *__restrict__ d_bias,
                                       float *__restrict__ d_scale, int batch, int H, int n_tiles, int N) {
  const int W = 4 * N + 13;
  const int h = blockIdx.y;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= W) return;
  float acc = 0.f;
  for (int b = 0; b < batch; ++b) {
    const float *pb = part + ((size_t)(b * H + h) * n_tiles) * W + e;
    int tile = 0;
    for (; tile + 8 <= n_tiles; tile += 8) {  // eight loads in flight, summed in the fixed order
      float v[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = pb[(size_t)(tile + i) * W];
#pragma unroll
      for (int i = 0; i < 8; ++i) acc += v[i];
    }
    for (; tile < n_tiles; ++tile) acc += pb[(size_t)tile * W];
  }
  if (e < 4 * N) {
    if (d_scale) d_scale[(size_t)h * 4 * N + e] = acc;
  } else {
    d_bias[h * 13 + (e - 4 * N)] = acc;
  }
}

static PrepHyper make_hyper(const slx_prep_shape *s) {
  PrepHyper h;
  h.dt_min = s->dt_min; h.dt_max = s->dt_max; h.r_min = s->r_min; h.r_max = s->r_max;
  h.theta_bound = s->theta_bound; h.k_max = s->k_max;
  float e = s->eps > 1e-12f ? s->eps : 1e-12f;
  float thr = sqrtf(e);
  if (thr < 1e-4f) thr = 1e-4f;
  h.z_thr2 = thr * thr;
  return h;
}

static int check_prep(const slx_prep_shape *s, PrepDims *d) {
  SLX_REQUIRE(s != nullptr, SLX_E_NULL, "shape is NULL");
  SLX_REQUIRE(s->batch > 0 && s->T > 0 && s->heads > 0 && s->P > 0 && s->N > 0, SLX_E_SHAPE,
              "scanprep: sizes must be positive");
  SLX_REQUIRE(s->dtype >= SLX_F32 && s->dtype <= SLX_F16, SLX_E_DTYPE, "scanprep: bad dtype %d", s->dtype);
  SLX_REQUIRE(s->value_stride >= (int64_t)s->heads * s->P && s->params_stride >= (int64_t)s->heads * 13 &&
                  s->bc_stride >= (int64_t)s->heads * 4 * s->N,
              SLX_E_SHAPE, "scanprep: row stride smaller than the row width");
  SLX_REQUIRE((long long)s->batch * s->heads <= 65535, SLX_E_UNSUPPORTED, "scanprep: batch*heads exceeds 65535");
  d->batch = s->batch; d->T = s->T; d->H = s->heads; d->P = s->P; d->N = s->N;
  d->normalize = s->normalize_bc;
  d->vs = s->value_stride; d->ps = s->params_stride; d->bs = s->bc_stride;
  d->wide_params = 0;
  return SLX_OK;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// every aligned 16-byte vector that covers a 13-value params row of a half type lies inside its
// own (16-byte aligned, 16-byte multiple) row of the tensor
static int params_rows_wide(const slx_prep_shape *s, const void *params) {
  return s->dtype != SLX_F32 && aligned16(params) && (s->params_stride * 2) % 16 == 0 &&
         ((long long)s->heads * 13 * 2) % 16 == 0;
}

// vector width (elements) usable for this problem: 16-byte vectors when every row start and row
// width is 16-byte aligned, 8-byte vectors when they are 8-byte aligned (a projection whose row
// is a multiple of 4 but not of 8 half values, e.g. 4764 = 2*768 + 12*13 + 4*12*64), else scalar
template <typename T>
static int pick_vec(const slx_prep_shape *s, std::initializer_list<const void *> ptrs) {
  for (int bytes = 16; bytes >= 8; bytes /= 2) {
    const int v = bytes / (int)sizeof(T);
    bool ok = (s->N % v == 0) && (s->P % v == 0) && (s->value_stride % v == 0) && (s->bc_stride % v == 0);
    for (const void *p : ptrs) ok = ok && (p == nullptr || (reinterpret_cast<uintptr_t>(p) % bytes) == 0);
    if (ok) return v;
  }
  return 1;
}

// lane-group width: 16 lanes x 16-byte vectors cover N = 128 half values in one
// sweep; the scalar mapping uses a full warp per row
template <int VEC>
constexpr int prep_group() { return VEC == 1 ? 32 : 16; }

template <typename T, int VEC>
static int launch_prep_fwd(const slx_prep_shape *s, const PrepDims &d, const void *value, const void *params,
                           const void *bc, const float *bias, const float *scale, void *U, float *M, float *K,
                           void *B, void *C, cudaStream_t st) {
  PrepHyper hp = make_hyper(s);
  constexpr int G = prep_group<VEC>();
  long long n_rows = (long long)d.batch * d.H * d.T;
  long long blocks = (n_rows + 255) / 256;
  if (blocks > 148LL * 32) blocks = 148LL * 32;
  scanprep_fwd_kernel<T, VEC, G><<<(unsigned)blocks, 256, 0, st>>>(
      (const T *)value, (const T *)params, (const T *)bc, bias, scale, (T *)U, M, K, (T *)B, (T *)C, d, hp);
  return check_launch("scanprep_fwd");
}

struct PrepBwdPlan {
  int G, kmax, rows_per_tile, n_tiles;
  size_t smem, ws_bytes;
};

static PrepBwdPlan prep_bwd_plan(const slx_prep_shape *s, int VEC) {
  PrepBwdPlan p;
  p.G = VEC == 1 ? 32 : 16;
  p.kmax = (s->N + VEC * p.G - 1) / (VEC * p.G);
  p.rows_per_tile = 256;
  p.n_tiles = (s->T + p.rows_per_tile - 1) / p.rows_per_tile;
  int W = 4 * s->N + 13;
  p.smem = sizeof(float) * ((size_t)(256 / p.G) * W + 4 * (size_t)s->N);  // group partials + the head's scale
  p.ws_bytes = sizeof(float) * (size_t)s->batch * s->heads * p.n_tiles * W;
  return p;
}

template <typename T, int VEC>
static int launch_prep_bwd(const slx_prep_shape *s, const PrepDims &d, const void *params, const void *bc,
                           const float *bias, const float *scale, const void *dU, const float *dM, const float *dK,
                           const void *dB, const void *dC, void *d_value, void *d_params, void *d_bc, float *d_bias,
                           float *d_scale, float *part, cudaStream_t st) {
  PrepHyper hp = make_hyper(s);
  PrepBwdPlan pl = prep_bwd_plan(s, VEC);
  SLX_REQUIRE(pl.kmax <= 4, SLX_E_UNSUPPORTED, "scanprep_bwd: N=%d too large for the lane mapping", d.N);
  SLX_REQUIRE(pl.smem <= 200 * 1024, SLX_E_UNSUPPORTED, "scanprep_bwd: N=%d needs too much shared memory", d.N);
  constexpr int G = prep_group<VEC>();
#define SLX_PREP_BWD(KM)                                                                                      \
  {                                                                                                           \
    auto kern = scanprep_bwd_kernel<T, VEC, G, KM>;                                                           \
    int rc_smem = ensure_dyn_smem(kern, pl.smem);                                                             \
    if (rc_smem) return rc_smem;                                                                              \
    kern<<<dim3(2 * pl.n_tiles, d.batch * d.H), 256, pl.smem, st>>>(                                          \
        (const T *)params, (const T *)bc, bias, scale, (const T *)dU, dM, dK, (const T *)dB, (const T *)dC,   \
        (T *)d_value, (T *)d_params, (T *)d_bc, part, d, hp, pl.rows_per_tile, pl.n_tiles);                   \
  }
  if (pl.kmax <= 1) SLX_PREP_BWD(1)
  else if (pl.kmax == 2) SLX_PREP_BWD(2)
  else SLX_PREP_BWD(4)
#undef SLX_PREP_BWD
  int rc = check_launch("scanprep_bwd");
  if (rc) return rc;
  int W = 4 * d.N + 13;
  scanprep_reduce_kernel<<<dim3((W + 127) / 128, d.H), 128, 0, st>>>(part, d_bias, d_scale, d.batch, d.H, pl.n_tiles,
                                                                      d.N);
  return check_launch("scanprep_reduce");
}

}  // namespace slx

using namespace slx;

#define SLX_PREP_T(dt, ...)                                          \
  switch (dt) {                                                      \
    case SLX_F32: { using T_ = float; __VA_ARGS__; } break;          \
    case SLX_BF16: { using T_ = __nv_bfloat16; __VA_ARGS__; } break; \
    default: { using T_ = __half; __VA_ARGS__; } break;              \
  }

extern "C" {

int slx_scanprep_fwd(const slx_prep_shape *s, const void *value, const void *params, const void *bc,
                     const float *bias, const float *scale, void *U, float *M, float *K, void *B, void *C,
                     void *stream) {
  PrepDims d;
  int rc = check_prep(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(value && params && bc && bias && U && M && K && B && C, SLX_E_NULL, "scanprep_fwd: NULL tensor");
  SLX_REQUIRE(!s->normalize_bc || scale, SLX_E_NULL, "scanprep_fwd: scale is NULL with normalize_bc set");
  d.wide_params = params_rows_wide(s, params);
  cudaStream_t st = as_stream(stream);
  SLX_PREP_T(s->dtype, {
    int vec = pick_vec<T_>(s, {value, bc, U, B, C});
    constexpr int VFULL = 16 / (int)sizeof(T_);
    if (vec == VFULL) rc = launch_prep_fwd<T_, VFULL>(s, d, value, params, bc, bias, scale, U, M, K, B, C, st);
    else if (vec == VFULL / 2)
      rc = launch_prep_fwd<T_, VFULL / 2>(s, d, value, params, bc, bias, scale, U, M, K, B, C, st);
    else rc = launch_prep_fwd<T_, 1>(s, d, value, params, bc, bias, scale, U, M, K, B, C, st);
  });
  return rc;
}

size_t slx_scanprep_bwd_workspace_bytes(const slx_prep_shape *s) {
  PrepDims d;
  if (check_prep(s, &d)) return 0;
  // the scalar mapping needs the most tiles-independent space; both use the same tile count
  return prep_bwd_plan(s, 1).ws_bytes;
}

int slx_scanprep_bwd(const slx_prep_shape *s, const void *params, const void *bc, const float *bias,
                     const float *scale, const void *dU, const float *dM, const float *dK, const void *dB,
                     const void *dC, void *d_value, void *d_params, void *d_bc, float *d_bias, float *d_scale,
                     void *workspace, size_t workspace_bytes, void *stream) {
  PrepDims d;
  int rc = check_prep(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(params && bc && bias && dU && dM && dK && dB && dC && d_value && d_params && d_bc && d_bias, SLX_E_NULL,
              "scanprep_bwd: NULL tensor");
  SLX_REQUIRE(!s->normalize_bc || (scale && d_scale), SLX_E_NULL, "scanprep_bwd: scale/d_scale NULL");
  d.wide_params = params_rows_wide(s, params);
  size_t need = slx_scanprep_bwd_workspace_bytes(s);
  SLX_REQUIRE(workspace && workspace_bytes >= need, SLX_E_WORKSPACE, "scanprep_bwd: workspace of %zu bytes needed",
              need);
  cudaStream_t st = as_stream(stream);
  float *part = static_cast<float *>(workspace);
  SLX_PREP_T(s->dtype, {
    int vec = pick_vec<T_>(s, {bc, dU, dB, dC, d_value, d_bc});
    constexpr int VFULL = 16 / (int)sizeof(T_);
    if (vec == VFULL)
      rc = launch_prep_bwd<T_, VFULL>(s, d, params, bc, bias, scale, dU, dM, dK, dB, dC, d_value, d_params, d_bc,
                                      d_bias, d_scale, part, st);
    else if (vec == VFULL / 2)
      rc = launch_prep_bwd<T_, VFULL / 2>(s, d, params, bc, bias, scale, dU, dM, dK, dB, dC, d_value, d_params, d_bc,
                                          d_bias, d_scale, part, st);
    else
      rc = launch_prep_bwd<T_, 1>(s, d, params, bc, bias, scale, dU, dM, dK, dB, dC, d_value, d_params, d_bc, d_bias,
                                  d_scale, part, st);
  });
  return rc;
}

}  // extern "C"
