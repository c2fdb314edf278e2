// Coefficient map of SLinOSSScanPrep: the 13-wide parameter row of one (batch, head, token)
// -> transition rho = r e^{i theta} and the two first-order-hold taps
// (slinoss/layers/scanprep.py:208-286, slinoss/ops/scanprep/reference.py:26-57).
// Shared by the scan-prep kernels and the one-token decode step.
#pragma once

#include "common.cuh"

namespace slx {

struct PrepHyper {
  float dt_min, dt_max, r_min, r_max, theta_bound, k_max, z_thr2;
};

struct CoefOut {
  float2 rho, kp, kc;
};

// intermediates kept for the backward
struct CoefCtx {
  float dt_u, dt, gamma, omega, e_gdt, r_struct, th_struct, r_dir_u, r_direct, th_t, th_direct;
  float mix_r, mix_th, mix_kp, mix_kc, tk[4], r, sig_p1;
  float2 rho, z, k1, k2, k2p, kps, kcs, kpl, kcl;  // k2p = d kappa2 / dz where the series branch ran
  bool small;
};

__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + expf(-x)); }
__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(expf(x)); }
// torch.lerp: a + w (b-a) for w < 0.5, b - (b-a)(1-w) otherwise
__device__ __forceinline__ float lerpf_(float a, float b, float w) {
  float d = b - a;
  return w < 0.5f ? fmaf(w, d, a) : b - d * (1.f - w);
}
__device__ __forceinline__ float2 cdiv(float2 a, float2 b) {
  float inv = 1.f / (b.x * b.x + b.y * b.y);
  return make_float2((a.x * b.x + a.y * b.y) * inv, (a.y * b.x - a.x * b.y) * inv);
}

// FOH tap factors as power series (complex Horner, 11 terms: exact to fp32 for |z| <= 1/2):
//   kappa1 = (e^z - 1)/z           = sum_k z^k / (k+1)!
//   kappa2 = (e^z (z-1) + 1)/z^2   = sum_k (k+1) z^k / (k+2)!
//   d kappa2/dz                    = sum_k (k+1)(k+2) z^k / (k+3)!        (d kappa1/dz = kappa2)
// The closed forms cancel in fp32 (relative error ~6e-8 / |z|^2 for kappa2: 6e-4 at |z| = 0.01, which is where
// the reference's own fp32 evaluation is that far from its float64 value); the series do not, so they are used
// for every |z|^2 < 1/4 and the closed forms only beyond, where the cancellation is harmless.
__device__ __forceinline__ void kappa_series(float2 z, float2 &k1, float2 &k2, float2 &k2p) {
  constexpr int NT = 11;
  float c1[NT], c2[NT], c3[NT];
  float f = 1.f;  // (k+1)!
#pragma unroll
  for (int k = 0; k < NT; ++k) {
    f *= (float)(k + 1);
    c1[k] = 1.f / f;
    c2[k] = (float)(k + 1) / (f * (float)(k + 2));
    c3[k] = (float)(k + 1) * (float)(k + 2) / (f * (float)(k + 2) * (float)(k + 3));
  }
  float2 a1 = make_float2(c1[NT - 1], 0.f), a2 = make_float2(c2[NT - 1], 0.f), a3 = make_float2(c3[NT - 1], 0.f);
#pragma unroll
  for (int k = NT - 2; k >= 0; --k) {
    a1 = cmul(a1, z);
    a1.x += c1[k];
    a2 = cmul(a2, z);
    a2.x += c2[k];
    a3 = cmul(a3, z);
    a3.x += c3[k];
  }
  k1 = a1;
  k2 = a2;
  k2p = a3;
}

__device__ __forceinline__ CoefOut coef_forward(const float *p, const PrepHyper &h, CoefCtx *ctx) {
  const float kPi = 3.14159265358979323846f;
  const float d_dt = h.dt_max - h.dt_min, d_r = h.r_max - h.r_min;
  float dt_u = sigmoidf_(p[0]);
  float dt = fmaf(d_dt, dt_u, h.dt_min);
  float gamma = softplusf_(p[1]);
  float omega = p[2];
  float e_gdt = expf(-gamma * dt);
  float r_struct = fmaf(d_r, e_gdt, h.r_min);
  float th_struct = omega * dt;
  float r_dir_u = sigmoidf_(p[3]);
  float r_direct = fmaf(d_r, r_dir_u, h.r_min);
  float th_t = tanhf(p[4]);
  float th_direct = h.theta_bound * th_t;
  float mix_r = sigmoidf_(p[5]), mix_th = sigmoidf_(p[6]);
  float mix_kp = sigmoidf_(p[7]), mix_kc = sigmoidf_(p[8]);
  float tk0 = tanhf(p[9]), tk1 = tanhf(p[10]), tk2 = tanhf(p[11]), tk3 = tanhf(p[12]);
  float2 kpl = make_float2(h.k_max * tk0, h.k_max * tk1);
  float2 kcl = make_float2(h.k_max * tk2, h.k_max * tk3);
  float r = lerpf_(r_direct, r_struct, mix_r);
  float th_raw = lerpf_(th_direct, th_struct, mix_th);
  // principal angle in [-pi, pi): remainder(theta + pi, 2 pi) - pi
  float rem = fmodf(th_raw + kPi, 2.f * kPi);
  if (rem < 0.f) rem += 2.f * kPi;
  float theta = rem - kPi;
  float log_r = logf(r);
  float sn, cs;
  sincosf(theta, &sn, &cs);
  float2 rho = make_float2(r * cs, r * sn);
  float2 z = make_float2(log_r, theta);
  // (the reference switches to a 3rd-order series below |z|^2 = z_thr2, layers/scanprep.py:255-268; the longer
  // series used here agrees with it there to fp32 and stays exact up to the wider bound)
  bool small = (log_r * log_r + theta * theta) < fmaxf(h.z_thr2, 0.25f);
  float2 k1, k2, k2p = make_float2(0.f, 0.f);
  if (small) {
    kappa_series(z, k1, k2, k2p);
  } else {
    k1 = cdiv(make_float2(rho.x - 1.f, rho.y), z);
    float2 num = cmul(rho, make_float2(z.x - 1.f, z.y));
    num.x += 1.f;
    k2 = cdiv(num, cmul(z, z));
  }
  float2 kps = cscale(k2, dt);
  float2 kcs = csub(cscale(k1, dt), kps);
  CoefOut o;
  o.rho = rho;
  o.kp = make_float2(lerpf_(kpl.x, kps.x, mix_kp), lerpf_(kpl.y, kps.y, mix_kp));
  o.kc = make_float2(lerpf_(kcl.x, kcs.x, mix_kc), lerpf_(kcl.y, kcs.y, mix_kc));
  if (ctx) {
    ctx->dt_u = dt_u; ctx->dt = dt; ctx->gamma = gamma; ctx->omega = omega; ctx->e_gdt = e_gdt;
    ctx->r_struct = r_struct; ctx->th_struct = th_struct; ctx->r_dir_u = r_dir_u; ctx->r_direct = r_direct;
    ctx->th_t = th_t; ctx->th_direct = th_direct; ctx->mix_r = mix_r; ctx->mix_th = mix_th;
    ctx->mix_kp = mix_kp; ctx->mix_kc = mix_kc; ctx->tk[0] = tk0; ctx->tk[1] = tk1; ctx->tk[2] = tk2;
    ctx->tk[3] = tk3; ctx->r = r; ctx->sig_p1 = sigmoidf_(p[1]); ctx->rho = rho; ctx->z = z; ctx->k1 = k1;
    ctx->k2 = k2; ctx->k2p = k2p; ctx->kps = kps; ctx->kcs = kcs; ctx->kpl = kpl; ctx->kcl = kcl; ctx->small = small;
  }
  return o;
}

}  // namespace slx
