// Mixer glue around the scan in one pass each way: skip connection, (b,H,T,P) -> (b,T,H*P)
// re-layout and SiLU gate,
//     out[b,t,h*P+p] = (y[b,h,t,p] + skip[h*P+p] * u[b,h,t,p]) * silu(gate[b,t,h*P+p])
// (slinoss/layers/mixer.py:585-599 _apply_gate_skip, which runs five elementwise passes and a
// transposing copy), and its backward.  HBM-bound: 8 bytes per element forward (read y, u, gate,
// write out), 14 backward for half types.
//
// One thread owns 8 adjacent channels of one head (16 bytes of a half type) and walks a tile of
// tokens; consecutive threads cover a (head, channel) row, so every access is a 128-byte segment.
// The backward accumulates d_skip per thread over its tile; a second kernel sums the per-tile
// partials in a fixed order (no atomics: results are bitwise repeatable).
#include <initializer_list>

#include "common.cuh"

namespace slx {

constexpr int kGlueTile = 32;  // tokens per CTA

struct GlueDims {
  int batch, T, H, P;
  long long gate_stride;  // elements between tokens of gate (it may be a column slice of a wider row)
  long long gate_batch_stride;
};

template <typename T>
__device__ __forceinline__ void ld8(const T *p, float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    const uint4 raw = *reinterpret_cast<const uint4 *>(p);
    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = to_f(e[i]);
  } else {
    const float4 a = reinterpret_cast<const float4 *>(p)[0], b = reinterpret_cast<const float4 *>(p)[1];
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
  }
}
template <typename T>
__device__ __forceinline__ void st8(T *p, const float (&v)[8]) {
  if constexpr (sizeof(T) == 2) {
    uint4 raw;
    T *e = reinterpret_cast<T *>(&raw);
#pragma unroll
    for (int i = 0; i < 8; ++i) e[i] = from_f<T>(v[i]);
    *reinterpret_cast<uint4 *>(p) = raw;
  } else {
    reinterpret_cast<float4 *>(p)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4 *>(p)[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// thread index -> (head, first channel); C8 = H*P/8 threads carry data
template <typename T>
__global__ void __launch_bounds__(256) gate_skip_fwd_kernel(const T *__restrict__ y, const T *__restrict__ u,
                                                            const T *__restrict__ gate, const float *__restrict__ skip,
                                                            T *__restrict__ out, GlueDims d) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int C8 = d.H * d.P / 8;
  if (v >= C8) return;
  const int ch = 8 * v, h = ch / d.P, p = ch % d.P;
  const int b = blockIdx.z, t0 = blockIdx.y * kGlueTile;
  const int t1 = min(t0 + kGlueTile, d.T);
  float sk[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) sk[i] = skip[ch + i];
  const size_t yrow = (((size_t)b * d.H + h) * d.T) * d.P + p;
  for (int t = t0; t < t1; ++t) {
    float yv[8], uv[8], gv[8], o[8];
    ld8<T>(y + yrow + (size_t)t * d.P, yv);
    ld8<T>(u + yrow + (size_t)t * d.P, uv);
    ld8<T>(gate + (size_t)b * d.gate_batch_stride + (size_t)t * d.gate_stride + ch, gv);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      // the reference rounds y + skip*u, silu(gate) and the product to the activation dtype one after the other
      const float s = to_f(from_f<T>(fmaf(to_f(from_f<T>(sk[i])) , uv[i], 0.f)));
      const float a = to_f(from_f<T>(yv[i] + s));
      const float sg = to_f(from_f<T>(gv[i] / (1.f + __expf(-gv[i]))));
      o[i] = a * sg;
    }
    st8<T>(out + ((size_t)b * d.T + t) * d.H * d.P + ch, o);
  }
}

// d_out (b,T,H*P) -> dy, du (b,H,T,P), d_gate (b,T,H*P) contiguous, per-tile partials of d_skip
template <typename T>
__global__ void __launch_bounds__(256) gate_skip_bwd_kernel(const T *__restrict__ y, const T *__restrict__ u,
                                                            const T *__restrict__ gate, const float *__restrict__ skip,
                                                            const T *__restrict__ d_out, T *__restrict__ dy,
                                                            T *__restrict__ du, T *__restrict__ d_gate,
                                                            float *__restrict__ part, GlueDims d) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int C8 = d.H * d.P / 8;
  if (v >= C8) return;
  const int ch = 8 * v, h = ch / d.P, p = ch % d.P;
  const int b = blockIdx.z, t0 = blockIdx.y * kGlueTile;
  const int t1 = min(t0 + kGlueTile, d.T);
  float sk[8], acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    sk[i] = to_f(from_f<T>(skip[ch + i]));
    acc[i] = 0.f;
  }
  const size_t yrow = (((size_t)b * d.H + h) * d.T) * d.P + p;
  for (int t = t0; t < t1; ++t) {
    float yv[8], uv[8], gv[8], go[8], o1[8], o2[8], o3[8];
    ld8<T>(y + yrow + (size_t)t * d.P, yv);
    ld8<T>(u + yrow + (size_t)t * d.P, uv);
    ld8<T>(gate + (size_t)b * d.gate_batch_stride + (size_t)t * d.gate_stride + ch, gv);
    ld8<T>(d_out + ((size_t)b * d.T + t) * d.H * d.P + ch, go);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float sig = 1.f / (1.f + __expf(-gv[i]));
      const float sg = to_f(from_f<T>(gv[i] * sig));
      const float a = to_f(from_f<T>(yv[i] + to_f(from_f<T>(sk[i] * uv[i]))));
      const float g = go[i] * sg;                       // gradient of y + skip*u
      o1[i] = g;
      o2[i] = g * sk[i];
      o3[i] = go[i] * a * sig * (1.f + gv[i] * (1.f - sig));  // d silu(g)/dg = sig (1 + g (1 - sig))
      acc[i] = fmaf(g, uv[i], acc[i]);
    }
    st8<T>(dy + yrow + (size_t)t * d.P, o1);
    st8<T>(du + yrow + (size_t)t * d.P, o2);
    st8<T>(d_gate + ((size_t)b * d.T + t) * d.H * d.P + ch, o3);
  }
  float *pp = part + ((size_t)b * gridDim.y + blockIdx.y) * d.H * d.P + ch;
  reinterpret_cast<float4 *>(pp)[0] = make_float4(acc[0], acc[1], acc[2], acc[3]);
  reinterpret_cast<float4 *>(pp)[1] = make_float4(acc[4], acc[5], acc[6], acc[7]);
}

// d_skip[c] = sum over the partial rows, in a fixed order: 32 channels x 16 row groups per CTA, every
// thread adds the rows of its group (i = g, g + 16, ...), then the 16 group sums are added in order.
__global__ void __launch_bounds__(512) gate_skip_reduce_kernel(const float *__restrict__ part, float *__restrict__ d_skip,
                                                               int n_part, int C) {
  __shared__ float red[16][33];
  const int cx = threadIdx.x & 31, g = threadIdx.x >> 5;
  const int c = blockIdx.x * 32 + cx;
  float acc = 0.f;
  if (c < C)
    for (int i = g; i < n_part; i += 16) acc += part[(size_t)i * C + c];
  red[g][cx] = acc;
  __syncthreads();
  if (g == 0 && c < C) {
    float tot = 0.f;
#pragma unroll
    for (int k = 0; k < 16; ++k) tot += red[k][cx];
    d_skip[c] = tot;
  }
}

static int check_glue(const slx_glue_shape *s, GlueDims *d) {
  SLX_REQUIRE(s != nullptr, SLX_E_NULL, "shape is NULL");
  SLX_REQUIRE(s->batch > 0 && s->T > 0 && s->heads > 0 && s->P > 0, SLX_E_SHAPE, "gate_skip: sizes must be positive");
  SLX_REQUIRE(s->P % 8 == 0, SLX_E_UNSUPPORTED, "gate_skip: head dim %d must be a multiple of 8", s->P);
  SLX_REQUIRE(s->dtype >= SLX_F32 && s->dtype <= SLX_F16, SLX_E_DTYPE, "gate_skip: bad dtype %d", s->dtype);
  SLX_REQUIRE(s->batch <= 65535, SLX_E_UNSUPPORTED, "gate_skip: batch exceeds 65535");
  SLX_REQUIRE(s->gate_stride >= (int64_t)s->heads * s->P && s->gate_stride % 8 == 0 && s->gate_batch_stride % 8 == 0,
              SLX_E_UNSUPPORTED, "gate_skip: gate strides must be multiples of 8 elements and cover a row");
  d->batch = s->batch; d->T = s->T; d->H = s->heads; d->P = s->P;
  d->gate_stride = s->gate_stride; d->gate_batch_stride = s->gate_batch_stride;
  return SLX_OK;
}

static bool glue_aligned(std::initializer_list<const void *> ptrs) {
  for (const void *p : ptrs)
    if (p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
  return true;
}

}  // namespace slx

using namespace slx;

#define SLX_GLUE_T(dt, ...)                                          \
  switch (dt) {                                                      \
    case SLX_F32: { using T_ = float; __VA_ARGS__; } break;          \
    case SLX_BF16: { using T_ = __nv_bfloat16; __VA_ARGS__; } break; \
    default: { using T_ = __half; __VA_ARGS__; } break;              \
  }

extern "C" {

int slx_gate_skip_fwd(const slx_glue_shape *s, const void *y, const void *u, const void *gate, const float *skip,
                      void *out, void *stream) {
  GlueDims d;
  int rc = check_glue(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(y && u && gate && skip && out, SLX_E_NULL, "gate_skip_fwd: NULL tensor");
  SLX_REQUIRE(glue_aligned({y, u, gate, skip, out}), SLX_E_UNSUPPORTED, "gate_skip_fwd: pointers must be 16-byte aligned");
  const int C8 = d.H * d.P / 8;
  const int threads = C8 >= 256 ? 256 : ((C8 + 31) / 32) * 32;
  const dim3 grid((C8 + threads - 1) / threads, (d.T + kGlueTile - 1) / kGlueTile, d.batch);
  SLX_GLUE_T(s->dtype, {
    gate_skip_fwd_kernel<T_><<<grid, threads, 0, as_stream(stream)>>>((const T_ *)y, (const T_ *)u, (const T_ *)gate, skip,
                                                                 (T_ *)out, d);
  });
  return check_launch("gate_skip_fwd");
}

size_t slx_gate_skip_bwd_workspace_bytes(const slx_glue_shape *s) {
  GlueDims d;
  if (check_glue(s, &d)) return 0;
  return sizeof(float) * (size_t)d.batch * ((d.T + kGlueTile - 1) / kGlueTile) * d.H * d.P;
}

int slx_gate_skip_bwd(const slx_glue_shape *s, const void *y, const void *u, const void *gate, const float *skip,
                      const void *d_out, void *dy, void *du, void *d_gate, float *d_skip, void *workspace,
                      size_t workspace_bytes, void *stream) {
  GlueDims d;
  int rc = check_glue(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(y && u && gate && skip && d_out && dy && du && d_gate && d_skip, SLX_E_NULL, "gate_skip_bwd: NULL tensor");
  SLX_REQUIRE(glue_aligned({y, u, gate, skip, d_out, dy, du, d_gate, d_skip, workspace}), SLX_E_UNSUPPORTED,
              "gate_skip_bwd: pointers must be 16-byte aligned");
  const size_t need = slx_gate_skip_bwd_workspace_bytes(s);
  SLX_REQUIRE(workspace && workspace_bytes >= need, SLX_E_WORKSPACE, "gate_skip_bwd: workspace of %zu bytes needed",
              need);
  const int C8 = d.H * d.P / 8;
  const int n_tiles = (d.T + kGlueTile - 1) / kGlueTile;
  const int threads = C8 >= 256 ? 256 : ((C8 + 31) / 32) * 32;
  const dim3 grid((C8 + threads - 1) / threads, n_tiles, d.batch);
  float *part = static_cast<float *>(workspace);
  SLX_GLUE_T(s->dtype, {
    gate_skip_bwd_kernel<T_><<<grid, threads, 0, as_stream(stream)>>>((const T_ *)y, (const T_ *)u, (const T_ *)gate, skip,
                                                                 (const T_ *)d_out, (T_ *)dy, (T_ *)du, (T_ *)d_gate,
                                                                 part, d);
  });
  rc = check_launch("gate_skip_bwd");
  if (rc) return rc;
  const int C = d.H * d.P;
  gate_skip_reduce_kernel<<<(C + 31) / 32, 512, 0, as_stream(stream)>>>(part, d_skip, d.batch * n_tiles, C);
  return check_launch("gate_skip_reduce");
}

}  // extern "C"
