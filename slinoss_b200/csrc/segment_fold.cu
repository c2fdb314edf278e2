// Composition of segment-level affine maps of the scan state, used when one sequence is split
// over several devices (context-parallel mode): every device contributes its segment's
// transition m_j (one complex number per batch*head) and offset f_j (one state), all devices
// gather the pairs, and each one folds the pairs of the segments in front of it (forward) or
// behind it (backward) into the state that enters its own segment:
//     z <- f_first;  then for every following pair  z <- m_j * z + f_j
// (conjugated transitions for the backward chain).  One thread per two complex state entries,
// 16-byte accesses; the loop over segments is the only dependent chain.
#include "common.cuh"

namespace slx {

__global__ void __launch_bounds__(256) segment_fold_kernel(const float *__restrict__ offsets, const float *__restrict__ m,
                                                           long long slice_stride, long long m_stride, int count,
                                                           int conj, float *__restrict__ out, int nvec) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int bh = blockIdx.y;
  if (v >= nvec) return;
  const size_t e = ((size_t)bh * nvec + v) * 4;
  float4 z = *reinterpret_cast<const float4 *>(offsets + e);
  for (int j = 1; j < count; ++j) {
    const float4 f = *reinterpret_cast<const float4 *>(offsets + (long long)j * slice_stride + (long long)e);
    float2 mm = *reinterpret_cast<const float2 *>(m + (long long)j * m_stride + 2 * (long long)bh);
    if (conj) mm.y = -mm.y;
    const float2 a = cmul(mm, make_float2(z.x, z.y)), b = cmul(mm, make_float2(z.z, z.w));
    z = make_float4(a.x + f.x, a.y + f.y, b.x + f.z, b.y + f.w);
  }
  *reinterpret_cast<float4 *>(out + e) = z;
}

// out = m (*) z + f for one segment (the offset a device contributes when it already knows the
// state entering it: the first device of the forward chain, the last one of the backward chain)
__global__ void __launch_bounds__(256) segment_axpy_kernel(const float *__restrict__ m, const float *__restrict__ z,
                                                           const float *__restrict__ f, int conj,
                                                           float *__restrict__ out, int nvec) {
  const int v = blockIdx.x * blockDim.x + threadIdx.x;
  const int bh = blockIdx.y;
  if (v >= nvec) return;
  const size_t e = ((size_t)bh * nvec + v) * 4;
  float2 mm = *reinterpret_cast<const float2 *>(m + 2 * (size_t)bh);
  if (conj) mm.y = -mm.y;
  const float4 zz = *reinterpret_cast<const float4 *>(z + e);
  const float4 ff = *reinterpret_cast<const float4 *>(f + e);
  const float2 a = cmul(mm, make_float2(zz.x, zz.y)), b = cmul(mm, make_float2(zz.z, zz.w));
  *reinterpret_cast<float4 *>(out + e) = make_float4(a.x + ff.x, a.y + ff.y, b.x + ff.z, b.y + ff.w);
}

// m_seg[bh] = prod_c m_chunk[bh][c]  (one thread per batch*head; NC is small next to the scan)
__global__ void __launch_bounds__(128) segment_transition_kernel(const float *__restrict__ m_chunk, int NC, int BH,
                                                                 float *__restrict__ m_seg) {
  const int bh = blockIdx.x * blockDim.x + threadIdx.x;
  if (bh >= BH) return;
  float2 acc = make_float2(1.f, 0.f);
  const float2 *row = reinterpret_cast<const float2 *>(m_chunk) + (size_t)bh * NC;
  for (int c = 0; c < NC; ++c) acc = cmul(row[c], acc);
  reinterpret_cast<float2 *>(m_seg)[bh] = acc;
}

}  // namespace slx

using namespace slx;

extern "C" {

int slx_segment_fold(int32_t BH, int32_t P, int32_t N, int32_t count, const float *offsets, int64_t slice_stride,
                     const float *m, int64_t m_stride, int32_t conj, float *out, void *stream) {
  SLX_REQUIRE(BH > 0 && P > 0 && N > 0 && count > 0, SLX_E_SHAPE, "segment_fold: sizes must be positive");
  SLX_REQUIRE(BH <= 65535, SLX_E_UNSUPPORTED, "batch_heads=%d exceeds 65535", BH);
  SLX_REQUIRE(offsets && out && (count == 1 || m), SLX_E_NULL, "segment_fold: NULL tensor");
  SLX_REQUIRE((P * 2 * N) % 4 == 0, SLX_E_UNSUPPORTED, "segment_fold: P*2N must be a multiple of 4");
  SLX_REQUIRE(((reinterpret_cast<uintptr_t>(offsets) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                  (slice_stride % 4) == 0 && (reinterpret_cast<uintptr_t>(m) & 7) == 0 && (m_stride % 2) == 0,
              SLX_E_UNSUPPORTED, "segment_fold: states must be 16-byte aligned, transitions 8-byte aligned");
  const int nvec = P * 2 * N / 4;
  segment_fold_kernel<<<dim3((nvec + 255) / 256, BH), 256, 0, as_stream(stream)>>>(offsets, m, slice_stride, m_stride,
                                                                                   count, conj, out, nvec);
  return check_launch("segment_fold");
}

int slx_segment_axpy(int32_t BH, int32_t P, int32_t N, const float *m, const float *z, const float *f, int32_t conj,
                     float *out, void *stream) {
  SLX_REQUIRE(BH > 0 && P > 0 && N > 0, SLX_E_SHAPE, "segment_axpy: sizes must be positive");
  SLX_REQUIRE(BH <= 65535, SLX_E_UNSUPPORTED, "batch_heads=%d exceeds 65535", BH);
  SLX_REQUIRE(m && z && f && out, SLX_E_NULL, "segment_axpy: NULL tensor");
  SLX_REQUIRE((P * 2 * N) % 4 == 0, SLX_E_UNSUPPORTED, "segment_axpy: P*2N must be a multiple of 4");
  SLX_REQUIRE(((reinterpret_cast<uintptr_t>(z) | reinterpret_cast<uintptr_t>(f) | reinterpret_cast<uintptr_t>(out)) & 15) == 0 &&
                  (reinterpret_cast<uintptr_t>(m) & 7) == 0,
              SLX_E_UNSUPPORTED, "segment_axpy: states must be 16-byte aligned, transitions 8-byte aligned");
  const int nvec = P * 2 * N / 4;
  segment_axpy_kernel<<<dim3((nvec + 255) / 256, BH), 256, 0, as_stream(stream)>>>(m, z, f, conj, out, nvec);
  return check_launch("segment_axpy");
}

int slx_segment_transition(int32_t BH, int32_t NC, const float *m_chunk, float *m_seg, void *stream) {
  SLX_REQUIRE(BH > 0 && NC > 0, SLX_E_SHAPE, "segment_transition: sizes must be positive");
  SLX_REQUIRE(m_chunk && m_seg, SLX_E_NULL, "segment_transition: NULL tensor");
  SLX_REQUIRE(((reinterpret_cast<uintptr_t>(m_chunk) | reinterpret_cast<uintptr_t>(m_seg)) & 7) == 0, SLX_E_UNSUPPORTED,
              "segment_transition: pointers must be 8-byte aligned");
  segment_transition_kernel<<<(BH + 127) / 128, 128, 0, as_stream(stream)>>>(m_chunk, NC, BH, m_seg);
  return check_launch("segment_transition");
}

}  // extern "C"
