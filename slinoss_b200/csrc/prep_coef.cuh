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
  float2 rho, z, k1, k2, kps, kcs, kpl, kcl;
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
  bool small = (log_r * log_r + theta * theta) < h.z_thr2;
  float2 k1, k2;
  if (small) {
    float2 z2 = cmul(z, z), z3 = cmul(z2, z);
    k1 = make_float2(1.f + 0.5f * z.x + z2.x / 6.f + z3.x / 24.f, 0.5f * z.y + z2.y / 6.f + z3.y / 24.f);
    k2 = make_float2(0.5f + z.x / 3.f + z2.x / 8.f + z3.x / 30.f, z.y / 3.f + z2.y / 8.f + z3.y / 30.f);
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
    ctx->k2 = k2; ctx->kps = kps; ctx->kcs = kcs; ctx->kpl = kpl; ctx->kcl = kcl; ctx->small = small;
  }
  return o;
}

}  // namespace slx
