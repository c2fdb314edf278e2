// Bandwidth-bound cross-chunk kernels: forward/backward state passing, the
// chunk-level dot products that feed dM, and the boundary-carry fix-up.
#pragma once

#include "common.cuh"

namespace slx {

template <int VEC>
struct VecT;
template <>
struct VecT<2> {
  using type = float2;
};
template <>
struct VecT<4> {
  using type = float4;
};
// eight floats (four complex lanes): the unit of the passes whose stored tensors are all half
// precision, so that every access is still 16 bytes wide
struct alignas(16) Float8 {
  float4 a, b;
};
template <>
struct VecT<8> {
  using type = Float8;
};

__device__ __forceinline__ float2 axpy_c(float2 m, float2 z, float2 v) {  // m*z + v
  return make_float2(fmaf(m.x, z.x, fmaf(-m.y, z.y, v.x)), fmaf(m.x, z.y, fmaf(m.y, z.x, v.y)));
}
__device__ __forceinline__ float4 axpy_c(float2 m, float4 z, float4 v) {
  float2 a = axpy_c(m, make_float2(z.x, z.y), make_float2(v.x, v.y));
  float2 b = axpy_c(m, make_float2(z.z, z.w), make_float2(v.z, v.w));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ Float8 axpy_c(float2 m, Float8 z, Float8 v) {
  Float8 r;
  r.a = axpy_c(m, z.a, v.a);
  r.b = axpy_c(m, z.b, v.b);
  return r;
}
// chunk-start states are stored as ST (float, or the activation dtype on the tensor-core path:
// those kernels round Z0 to it anyway); the recurrence itself stays in fp32 registers
template <typename ST, int VEC>
struct alignas(sizeof(ST) * VEC) PackedVec {
  ST v[VEC];
};
template <typename ST>
__device__ __forceinline__ void st_store(ST *p, float2 v) {
  PackedVec<ST, 2> q;
  q.v[0] = from_f<ST>(v.x);
  q.v[1] = from_f<ST>(v.y);
  *reinterpret_cast<PackedVec<ST, 2> *>(p) = q;
}
template <typename ST>
__device__ __forceinline__ void st_store(ST *p, float4 v) {
  PackedVec<ST, 4> q;
  q.v[0] = from_f<ST>(v.x);
  q.v[1] = from_f<ST>(v.y);
  q.v[2] = from_f<ST>(v.z);
  q.v[3] = from_f<ST>(v.w);
  *reinterpret_cast<PackedVec<ST, 4> *>(p) = q;
}
template <typename ST>
__device__ __forceinline__ void st_load(const ST *p, float2 &v) {
  const PackedVec<ST, 2> q = *reinterpret_cast<const PackedVec<ST, 2> *>(p);
  v = make_float2(to_f(q.v[0]), to_f(q.v[1]));
}
template <typename ST>
__device__ __forceinline__ void st_load(const ST *p, float4 &v) {
  const PackedVec<ST, 4> q = *reinterpret_cast<const PackedVec<ST, 4> *>(p);
  v = make_float4(to_f(q.v[0]), to_f(q.v[1]), to_f(q.v[2]), to_f(q.v[3]));
}
template <typename ST>
__device__ __forceinline__ void st_store(ST *p, Float8 v) {
  PackedVec<ST, 8> q;
  q.v[0] = from_f<ST>(v.a.x);
  q.v[1] = from_f<ST>(v.a.y);
  q.v[2] = from_f<ST>(v.a.z);
  q.v[3] = from_f<ST>(v.a.w);
  q.v[4] = from_f<ST>(v.b.x);
  q.v[5] = from_f<ST>(v.b.y);
  q.v[6] = from_f<ST>(v.b.z);
  q.v[7] = from_f<ST>(v.b.w);
  *reinterpret_cast<PackedVec<ST, 8> *>(p) = q;
}
template <typename ST>
__device__ __forceinline__ void st_load(const ST *p, Float8 &v) {
  const PackedVec<ST, 8> q = *reinterpret_cast<const PackedVec<ST, 8> *>(p);
  v.a = make_float4(to_f(q.v[0]), to_f(q.v[1]), to_f(q.v[2]), to_f(q.v[3]));
  v.b = make_float4(to_f(q.v[4]), to_f(q.v[5]), to_f(q.v[6]), to_f(q.v[7]));
}
__device__ __forceinline__ Float8 vzero(Float8) {
  Float8 r;
  r.a = r.b = make_float4(0.f, 0.f, 0.f, 0.f);
  return r;
}
__device__ __forceinline__ float2 vzero(float2) { return make_float2(0.f, 0.f); }
__device__ __forceinline__ float4 vzero(float4) { return make_float4(0.f, 0.f, 0.f, 0.f); }
// sum over the complex lanes of conj(a) * b
__device__ __forceinline__ float2 cdot(float2 a, float2 b) { return cmul(cconj(a), b); }
__device__ __forceinline__ float2 cdot(float4 a, float4 b) {
  return cadd(cmul(make_float2(a.x, -a.y), make_float2(b.x, b.y)), cmul(make_float2(a.z, -a.w), make_float2(b.z, b.w)));
}
__device__ __forceinline__ float2 cdot(Float8 a, Float8 b) { return cadd(cdot(a.a, b.a), cdot(a.b, b.b)); }

// starts[c] = z; z = m_chunk[c] * z + inc[c]     (reference.py:439-457)
// One thread owns VEC/2 complex state lanes for the whole sequence of chunks;
// consecutive threads own consecutive lanes, so every access is a full-width
// coalesced 8/16-byte vector.  `starts` may alias `inc`: each chunk's increment
// is read before its slot is overwritten.  `starts` may be NULL: only the final state is wanted
// (the affine offset of a segment in the context-parallel chain), and the pass writes nothing else.
// The increments are stored as IT (float, or the activation dtype where the tensor-core chunk
// kernel wrote them so); the recurrence is fp32 either way.
template <int VEC, typename ST, typename IT>
__global__ void __launch_bounds__(256) state_passing_fwd_kernel(const IT *inc, const float *__restrict__ m_chunk,
                                                                const float *__restrict__ init, ST *starts,
                                                                float *__restrict__ final_state, int NC,
                                                                int n_vec /* P*D/VEC */) {
  using V = typename VecT<VEC>::type;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int bh = blockIdx.y;
  if (i >= n_vec) return;
  const size_t per = (size_t)n_vec;
  const IT *incv = inc + ((size_t)bh * NC * per + i) * VEC;  // + c * per * VEC per chunk
  ST *stv = starts ? starts + ((size_t)bh * NC * per + i) * VEC : nullptr;  // + c * per * VEC per chunk
  const size_t cs = per * VEC;
  const float2 *mc = reinterpret_cast<const float2 *>(m_chunk) + (size_t)bh * NC;
  V z = init ? reinterpret_cast<const V *>(init)[(size_t)bh * per + i] : vzero(V());
  int c = 0;
  for (; c + 4 <= NC; c += 4) {
    V v0, v1, v2, v3;
    st_load<IT>(incv + (size_t)(c + 0) * cs, v0);
    st_load<IT>(incv + (size_t)(c + 1) * cs, v1);
    st_load<IT>(incv + (size_t)(c + 2) * cs, v2);
    st_load<IT>(incv + (size_t)(c + 3) * cs, v3);
    float2 m0 = mc[c], m1 = mc[c + 1], m2 = mc[c + 2], m3 = mc[c + 3];
    if (stv) st_store<ST>(stv + (size_t)(c + 0) * cs, z);
    z = axpy_c(m0, z, v0);
    if (stv) st_store<ST>(stv + (size_t)(c + 1) * cs, z);
    z = axpy_c(m1, z, v1);
    if (stv) st_store<ST>(stv + (size_t)(c + 2) * cs, z);
    z = axpy_c(m2, z, v2);
    if (stv) st_store<ST>(stv + (size_t)(c + 3) * cs, z);
    z = axpy_c(m3, z, v3);
  }
  for (; c < NC; ++c) {
    V v;
    st_load<IT>(incv + (size_t)c * cs, v);
    float2 m = mc[c];
    if (stv) st_store<ST>(stv + (size_t)c * cs, z);
    z = axpy_c(m, z, v);
  }
  reinterpret_cast<V *>(final_state)[(size_t)bh * per + i] = z;
}

// Reverse pass: g = d_final; for c = NC-1..0:
//   zdot_partial[c][warp] = sum over the warp's lanes of conj(end_state_c) * g   (end_state_c = starts[c+1] or final)
//   d_inc[c] = g;  g = dZ0[c] + conj(m_chunk[c]) * g
// d_initial = g.  d_inc is stored as ST like the chunk-start states (the per-chunk backward rounds
// it to the activation dtype for its products anyway); with ST = float it may alias dZ0.  With zdot_partials == NULL the dot products (and the reads
// of starts / final_state) are skipped, with d_inc == NULL nothing but d_initial is written: that
// is the reduce-only pass that gives a segment's d_initial for a zero d_final.
template <int VEC, typename ST, typename IT>
__global__ void __launch_bounds__(256) state_passing_bwd_kernel(const IT *dZ0, const float *__restrict__ m_chunk,
                                                                const ST *__restrict__ starts,
                                                                const float *__restrict__ final_state,
                                                                const float *__restrict__ d_final, ST *d_inc,
                                                                float *__restrict__ d_initial,
                                                                float *__restrict__ zdot_partials, int NC, int n_vec) {
  using V = typename VecT<VEC>::type;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  const int bh = blockIdx.y;
  const bool live = i < n_vec;
  const int iv = live ? i : 0;
  const size_t per = (size_t)n_vec;
  const IT *dzv = dZ0 + ((size_t)bh * NC * per + iv) * VEC;  // + c * per * VEC per chunk, stored as IT
  ST *div = d_inc ? d_inc + ((size_t)bh * NC * per + iv) * VEC : nullptr;  // + c * per * VEC per chunk
  const size_t ds = per * VEC;
  if (zdot_partials == nullptr) {  // reduce-only / no dot products: a plain reverse recurrence
    const float2 *mc0 = reinterpret_cast<const float2 *>(m_chunk) + (size_t)bh * NC;
    V g0 = (d_final && live) ? reinterpret_cast<const V *>(d_final)[(size_t)bh * per + iv] : vzero(V());
    int c = NC - 1;
    for (; c >= 3; c -= 4) {  // four loads in flight
      V d0, d1, d2, d3;
      st_load<IT>(dzv + (size_t)(c - 0) * ds, d0);
      st_load<IT>(dzv + (size_t)(c - 1) * ds, d1);
      st_load<IT>(dzv + (size_t)(c - 2) * ds, d2);
      st_load<IT>(dzv + (size_t)(c - 3) * ds, d3);
      const float2 m0 = mc0[c], m1 = mc0[c - 1], m2 = mc0[c - 2], m3 = mc0[c - 3];
      if (div && live) st_store<ST>(div + (size_t)(c - 0) * ds, g0);
      g0 = axpy_c(cconj(m0), g0, d0);
      if (div && live) st_store<ST>(div + (size_t)(c - 1) * ds, g0);
      g0 = axpy_c(cconj(m1), g0, d1);
      if (div && live) st_store<ST>(div + (size_t)(c - 2) * ds, g0);
      g0 = axpy_c(cconj(m2), g0, d2);
      if (div && live) st_store<ST>(div + (size_t)(c - 3) * ds, g0);
      g0 = axpy_c(cconj(m3), g0, d3);
    }
    for (; c >= 0; --c) {
      V dz;
      st_load<IT>(dzv + (size_t)c * ds, dz);
      if (div && live) st_store<ST>(div + (size_t)c * ds, g0);
      g0 = axpy_c(cconj(mc0[c]), g0, dz);
    }
    if (d_initial && live) reinterpret_cast<V *>(d_initial)[(size_t)bh * per + iv] = g0;
    return;
  }
  // With the dot products: every warp writes its own partial of every chunk (no barrier in the
  // loop, so the loads of four chunks are in flight together); zdot_reduce_kernel adds the
  // gridDim.x * warps partials of a chunk in a fixed order.
  const ST *stv = starts + ((size_t)bh * NC * per + iv) * VEC;
  const size_t cs = per * VEC;
  const float2 *mc = reinterpret_cast<const float2 *>(m_chunk) + (size_t)bh * NC;
  V g = (d_final && live) ? reinterpret_cast<const V *>(d_final)[(size_t)bh * per + iv] : vzero(V());
  V endst = reinterpret_cast<const V *>(final_state)[(size_t)bh * per + iv];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = blockDim.x >> 5;
  const size_t nparts = (size_t)gridDim.x * nwarp;
  float2 *pout = reinterpret_cast<float2 *>(zdot_partials) + (size_t)bh * NC * nparts + blockIdx.x * nwarp + warp;
  auto step = [&](int c, const V &dz, const V &st, float2 m) {
    float2 part = live ? cdot(endst, g) : make_float2(0.f, 0.f);
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) {
      part.x += __shfl_xor_sync(0xffffffffu, part.x, off);
      part.y += __shfl_xor_sync(0xffffffffu, part.y, off);
    }
    if (lane == 0) pout[(size_t)c * nparts] = part;
    if (live && div) st_store<ST>(div + (size_t)c * ds, g);
    g = axpy_c(cconj(m), g, dz);
    endst = st;  // start of chunk c = end state of chunk c-1
  };
  int c = NC - 1;
  for (; c >= 3; c -= 4) {
    V d0, d1, d2, d3, s0, s1, s2, s3;
    st_load<IT>(dzv + (size_t)(c - 0) * ds, d0);
    st_load<ST>(stv + (size_t)(c - 0) * cs, s0);
    st_load<IT>(dzv + (size_t)(c - 1) * ds, d1);
    st_load<ST>(stv + (size_t)(c - 1) * cs, s1);
    st_load<IT>(dzv + (size_t)(c - 2) * ds, d2);
    st_load<ST>(stv + (size_t)(c - 2) * cs, s2);
    st_load<IT>(dzv + (size_t)(c - 3) * ds, d3);
    st_load<ST>(stv + (size_t)(c - 3) * cs, s3);
    const float2 m0 = mc[c], m1 = mc[c - 1], m2 = mc[c - 2], m3 = mc[c - 3];
    step(c, d0, s0, m0);
    step(c - 1, d1, s1, m1);
    step(c - 2, d2, s2, m2);
    step(c - 3, d3, s3, m3);
  }
  for (; c >= 0; --c) {
    V dz, st;
    st_load<IT>(dzv + (size_t)c * ds, dz);
    st_load<ST>(stv + (size_t)c * cs, st);
    step(c, dz, st, mc[c]);
  }
  if (d_initial && live) reinterpret_cast<V *>(d_initial)[(size_t)bh * per + iv] = g;
}

__global__ void zdot_reduce_kernel(const float *__restrict__ partials, float *__restrict__ zdot, int n_rows, int nblk) {
  int r = blockIdx.x * blockDim.x + threadIdx.x;
  if (r >= n_rows) return;
  const float2 *p = reinterpret_cast<const float2 *>(partials) + (size_t)r * nblk;
  float2 acc = make_float2(0.f, 0.f);
  for (int b = 0; b < nblk; ++b) acc = cadd(acc, p[b]);
  reinterpret_cast<float2 *>(zdot)[r] = acc;
}

// Adds the gradient a chunk sends to the token before it (prev-tap terms of its
// first token) to the last row of the previous chunk; chunk 0's carry is the
// gradient of the streaming inputs (B_prev, U_prev).
template <typename T>
__global__ void carry_fixup_kernel(const float *__restrict__ carryB, const float *__restrict__ carryU, T *dB, T *dU,
                                   float *dB_prev, float *dU_prev, int T_len, int P, int D, int L, int NC) {
  const int c = blockIdx.x, bh = blockIdx.y;
  const float *cb = carryB + ((size_t)bh * NC + c) * D;
  const float *cu = carryU + ((size_t)bh * NC + c) * P;
  if (c == 0) {
    if (dB_prev)
      for (int i = threadIdx.x; i < D; i += blockDim.x) dB_prev[(size_t)bh * D + i] = cb[i];
    if (dU_prev)
      for (int i = threadIdx.x; i < P; i += blockDim.x) dU_prev[(size_t)bh * P + i] = cu[i];
    return;
  }
  const size_t row = (size_t)bh * T_len + (size_t)c * L - 1;
  for (int i = threadIdx.x; i < D; i += blockDim.x) dB[row * D + i] = from_f<T>(to_f(dB[row * D + i]) + cb[i]);
  for (int i = threadIdx.x; i < P; i += blockDim.x) dU[row * P + i] = from_f<T>(to_f(dU[row * P + i]) + cu[i]);
}

}  // namespace slx
