// One-token mixer decode step for sm_100a: scan prep of the token, one step of the
// recurrence on the carried state, skip and gate, in one kernel.
//
// Mirrors SLinOSSMixer._decode_step_reference (slinoss/layers/mixer.py:714-748) and the
// contract of mixer_decode_step_cute (slinoss/ops/v2x2ssd/cute/decode.py:117-149) without
// its shape restrictions (that kernel takes P = 64, N = 64, batch in {1,2,4,8,16} only):
//   (rho, k^p, k^c) = coefficient map(params + bias)              (prep_coef.cuh)
//   b, c            = interleave(rms_norm(bc) * scale), rounded to the activation dtype
//   z'[p][n]        = rho z[p][n] + k^p u_prev[p] b_prev[n] + k^c u[p] b[n]
//   y[p]            = sum_n Re(conj(c[n]) z'[p][n])
//   out[p]          = (y[p] + skip[p] u[p]) * silu(gate[p])
// One CTA per (batch, head).  The fp32 state (P x 2N) is the only large operand: every warp
// streams whole rows with 16-byte accesses (a row is contiguous), four rows in flight, and
// reduces its own y[p] by shuffles, so there is no cross-warp reduction and no atomics.
// The step is bound by HBM: 2 * P * 2N * 4 bytes per (batch, head).
#include "common.cuh"
#include "prep_coef.cuh"

namespace slx {

struct DecodeDims {
  int batch, H, P, N, normalize;
};

constexpr int kDecodeThreads = 256;
constexpr int kDecodeRowsAhead = 4;

template <typename T>
__global__ void __launch_bounds__(kDecodeThreads) decode_step_kernel(
    const T *__restrict__ value, const T *__restrict__ params, const T *__restrict__ bc, const T *__restrict__ gate,
    const T *__restrict__ skip, const float *__restrict__ bias, const float *__restrict__ scale, const float *state_in,
    const T *b_prev, const T *u_prev, T *__restrict__ out, float *state_out, T *b_last, T *u_last, DecodeDims d,
    PrepHyper hp) {
  extern __shared__ float sm[];
  const int D = 2 * d.N;
  float *sb = sm;            // [D]  b (interleaved complex), already rounded to T
  float *sc = sb + D;        // [D]  c
  float *skb = sc + D;       // [D]  k^c b
  float *skbp = skb + D;     // [D]  k^p b_prev
  float *su = skbp + D;      // [P]  u
  float *sup = su + d.P;     // [P]  u_prev
  float *sy = sup + d.P;     // [P]  y
  float *scoef = sy + d.P;   // [6]  rho, k^p, k^c
  float *srstd = scoef + 8;  // [4]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int bh = blockIdx.x, h = bh % d.H;

  if (tid == 0) {
    float p[13];
#pragma unroll
    for (int i = 0; i < 13; ++i) p[i] = to_f(params[(size_t)bh * 13 + i]) + bias[h * 13 + i];
    const CoefOut o = coef_forward(p, hp, nullptr);
    scoef[0] = o.rho.x; scoef[1] = o.rho.y; scoef[2] = o.kp.x; scoef[3] = o.kp.y; scoef[4] = o.kc.x; scoef[5] = o.kc.y;
  }
  // rms-norm statistics: warp j < 4 owns plane j of bc
  const T *bcr = bc + (size_t)bh * 4 * d.N;
  if (warp < 4) {
    float ss = 0.f;
    for (int n = lane; n < d.N; n += 32) {
      const float v = to_f(bcr[warp * d.N + n]);
      ss = fmaf(v, v, ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if (lane == 0) srstd[warp] = d.normalize ? rsqrtf(ss / (float)d.N + 1e-5f) : 1.f;
  }
  for (int p = tid; p < d.P; p += kDecodeThreads) {
    su[p] = to_f(value[(size_t)bh * d.P + p]);
    sup[p] = u_prev ? to_f(u_prev[(size_t)bh * d.P + p]) : 0.f;
  }
  __syncthreads();
  const float2 kp = make_float2(scoef[2], scoef[3]), kc = make_float2(scoef[4], scoef[5]);
  for (int n = tid; n < d.N; n += kDecodeThreads) {
    float y[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      float v = to_f(bcr[j * d.N + n]);
      if (d.normalize) v = (v * srstd[j]) * scale[((size_t)h * 4 + j) * d.N + n];
      y[j] = to_f(from_f<T>(v));  // the reference casts the normalised rows back before the scan
    }
    const float2 b = make_float2(y[0], y[1]);
    float2 bp = make_float2(0.f, 0.f);
    if (b_prev) bp = make_float2(to_f(b_prev[(size_t)bh * D + 2 * n]), to_f(b_prev[(size_t)bh * D + 2 * n + 1]));
    const float2 kb = cmul(kc, b), kbp = cmul(kp, bp);
    sb[2 * n] = b.x; sb[2 * n + 1] = b.y;
    sc[2 * n] = y[2]; sc[2 * n + 1] = y[3];
    skb[2 * n] = kb.x; skb[2 * n + 1] = kb.y;
    skbp[2 * n] = kbp.x; skbp[2 * n + 1] = kbp.y;
  }
  __syncthreads();

  // ---- stream the state: warp w owns rows w, w+8, ...; a lane owns the float4 items q = lane + 32 i
  const float2 m = make_float2(scoef[0], scoef[1]);
  const int n_items = D / 4;
  const float *zin = state_in ? state_in + (size_t)bh * d.P * D : nullptr;
  float *zout = state_out + (size_t)bh * d.P * D;
  constexpr int NW = kDecodeThreads / 32;
  for (int p0 = warp; p0 < d.P; p0 += NW * kDecodeRowsAhead) {
    float acc[kDecodeRowsAhead];
#pragma unroll
    for (int r = 0; r < kDecodeRowsAhead; ++r) acc[r] = 0.f;
    for (int q0 = lane; q0 < n_items; q0 += 32) {
      float4 z[kDecodeRowsAhead];
#pragma unroll
      for (int r = 0; r < kDecodeRowsAhead; ++r) {
        const int p = p0 + r * NW;
        z[r] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (p < d.P && zin) z[r] = *reinterpret_cast<const float4 *>(zin + (size_t)p * D + 4 * q0);
      }
      const float4 vkb = *reinterpret_cast<const float4 *>(skb + 4 * q0);
      const float4 vkbp = *reinterpret_cast<const float4 *>(skbp + 4 * q0);
      const float4 vc = *reinterpret_cast<const float4 *>(sc + 4 * q0);
#pragma unroll
      for (int r = 0; r < kDecodeRowsAhead; ++r) {
        const int p = p0 + r * NW;
        if (p < d.P) {
          const float u = su[p], up = sup[p];
          float4 o;
          o.x = fmaf(m.x, z[r].x, fmaf(-m.y, z[r].y, fmaf(up, vkbp.x, u * vkb.x)));
          o.y = fmaf(m.x, z[r].y, fmaf(m.y, z[r].x, fmaf(up, vkbp.y, u * vkb.y)));
          o.z = fmaf(m.x, z[r].z, fmaf(-m.y, z[r].w, fmaf(up, vkbp.z, u * vkb.z)));
          o.w = fmaf(m.x, z[r].w, fmaf(m.y, z[r].z, fmaf(up, vkbp.w, u * vkb.w)));
          *reinterpret_cast<float4 *>(zout + (size_t)p * D + 4 * q0) = o;
          acc[r] += fmaf(vc.x, o.x, fmaf(vc.y, o.y, fmaf(vc.z, o.z, vc.w * o.w)));
        }
      }
    }
#pragma unroll
    for (int r = 0; r < kDecodeRowsAhead; ++r) {
      float a = acc[r];
#pragma unroll
      for (int off = 16; off > 0; off >>= 1) a += __shfl_xor_sync(0xffffffffu, a, off);
      const int p = p0 + r * NW;
      if (lane == 0 && p < d.P) sy[p] = a;
    }
  }
  __syncthreads();
  for (int p = tid; p < d.P; p += kDecodeThreads) {
    const float g = to_f(gate[(size_t)bh * d.P + p]);
    const float y = sy[p] + to_f(skip[h * d.P + p]) * su[p];
    out[(size_t)bh * d.P + p] = from_f<T>(y * (g / (1.f + expf(-g))));
    if (u_last) u_last[(size_t)bh * d.P + p] = from_f<T>(su[p]);
  }
  if (b_last)
    for (int i = tid; i < D; i += kDecodeThreads) b_last[(size_t)bh * D + i] = from_f<T>(sb[i]);
}

}  // namespace slx

using namespace slx;

extern "C" int slx_decode_step(const slx_decode_shape *s, const void *value, const void *params, const void *bc,
                               const void *gate, const void *skip, const float *bias, const float *scale,
                               const float *state_in, const void *b_prev, const void *u_prev, void *out,
                               float *state_out, void *b_last, void *u_last, void *stream) {
  SLX_REQUIRE(s != nullptr, SLX_E_NULL, "decode_step: shape is NULL");
  SLX_REQUIRE(s->batch > 0 && s->heads > 0 && s->P > 0 && s->N > 0, SLX_E_SHAPE, "decode_step: sizes must be positive");
  SLX_REQUIRE(s->N % 2 == 0, SLX_E_UNSUPPORTED, "decode_step: N=%d must be even (16-byte state accesses)", s->N);
  SLX_REQUIRE(s->dtype == SLX_F32 || s->dtype == SLX_BF16 || s->dtype == SLX_F16, SLX_E_DTYPE,
              "decode_step: unknown dtype code %d", s->dtype);
  SLX_REQUIRE(value && params && bc && gate && skip && bias && out && state_out, SLX_E_NULL,
              "decode_step: NULL tensor");
  SLX_REQUIRE(!s->normalize_bc || scale, SLX_E_NULL, "decode_step: scale is NULL with normalize_bc set");
  SLX_REQUIRE((b_prev == nullptr) == (u_prev == nullptr), SLX_E_NULL,
              "decode_step: b_prev and u_prev go together");
  SLX_REQUIRE((reinterpret_cast<uintptr_t>(state_out) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(state_in) & 15) == 0,
              SLX_E_UNSUPPORTED, "decode_step: state pointers must be 16-byte aligned");
  DecodeDims d{s->batch, s->heads, s->P, s->N, s->normalize_bc};
  PrepHyper hp;
  hp.dt_min = s->dt_min; hp.dt_max = s->dt_max; hp.r_min = s->r_min; hp.r_max = s->r_max;
  hp.theta_bound = s->theta_bound; hp.k_max = s->k_max;
  {
    float e = s->eps > 1e-12f ? s->eps : 1e-12f;
    float thr = sqrtf(e);
    if (thr < 1e-4f) thr = 1e-4f;
    hp.z_thr2 = thr * thr;
  }
  const size_t smem = sizeof(float) * ((size_t)8 * s->N + 3 * (size_t)s->P + 16);
  SLX_REQUIRE(smem <= 48 * 1024, SLX_E_UNSUPPORTED, "decode_step: N=%d, P=%d need %zu bytes of shared memory",
              s->N, s->P, smem);
  const long long ctas = (long long)s->batch * s->heads;
  SLX_REQUIRE(ctas <= 2147483647LL, SLX_E_UNSUPPORTED, "decode_step: batch*heads too large");
  cudaStream_t st = as_stream(stream);
#define SLX_DECODE(TT)                                                                                            \
  decode_step_kernel<TT><<<(unsigned)ctas, kDecodeThreads, smem, st>>>(                                           \
      (const TT *)value, (const TT *)params, (const TT *)bc, (const TT *)gate, (const TT *)skip, bias, scale,     \
      state_in, (const TT *)b_prev, (const TT *)u_prev, (TT *)out, state_out, (TT *)b_last, (TT *)u_last, d, hp)
  if (s->dtype == SLX_F32) SLX_DECODE(float);
  else if (s->dtype == SLX_BF16) SLX_DECODE(__nv_bfloat16);
  else SLX_DECODE(__half);
#undef SLX_DECODE
  return check_launch("decode_step");
}
