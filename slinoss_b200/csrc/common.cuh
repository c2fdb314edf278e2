// Shared device/host helpers for the sm_100a scan kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <map>
#include <mutex>
#include <utility>

#include "../../include/slinoss_b200.h"

namespace slx {

// ---- host-side status plumbing --------------------------------------------
// one thread-local message buffer per shared library that includes this header
inline thread_local char g_err[512] = "";

inline void set_error(const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}
inline int fail(int code, const char *fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}
inline int check_launch(const char *what) {  // cudaGetLastError -> status
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) {
    set_error("%s: %s", what, cudaGetErrorString(e));
    return (int)e;
  }
  return SLX_OK;
}

#define SLX_REQUIRE(cond, code, ...)            \
  do {                                          \
    if (!(cond)) return ::slx::fail(code, __VA_ARGS__); \
  } while (0)

inline cudaStream_t as_stream(void *s) { return reinterpret_cast<cudaStream_t>(s); }

// Per-kernel set-up that the driver keeps per device is done once per (kernel, device) and
// remembered, so that a launch costs no driver call beyond the launch itself.
struct KernelSetup {
  size_t smem = 0;   // largest dynamic shared-memory size granted so far
  long slots = -1;   // CTAs the device holds at once (occupancy query), -1 = not asked yet
};
inline std::mutex &kernel_setup_mutex() {
  static std::mutex mu;
  return mu;
}
inline std::map<std::pair<const void *, int>, KernelSetup> &kernel_setup_table() {
  static std::map<std::pair<const void *, int>, KernelSetup> table;
  return table;
}
// cudaFuncAttributeMaxDynamicSharedMemorySize >= bytes for `kernel` on the current device.
template <typename K>
inline int ensure_dyn_smem(K kernel, size_t bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail((int)e, "cudaGetDevice: %s", cudaGetErrorString(e));
  std::lock_guard<std::mutex> lock(kernel_setup_mutex());
  KernelSetup &ks = kernel_setup_table()[{reinterpret_cast<const void *>(kernel), dev}];
  if (ks.smem >= bytes) return SLX_OK;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e != cudaSuccess) return fail((int)e, "cudaFuncSetAttribute(%zu bytes): %s", bytes, cudaGetErrorString(e));
  ks.smem = bytes;
  return SLX_OK;
}
// CTAs of `kernel` (threads per CTA, dynamic bytes) the current device holds at once; 0 if unknown.
template <typename K>
inline long resident_ctas(K kernel, int threads, size_t smem) {
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  std::lock_guard<std::mutex> lock(kernel_setup_mutex());
  KernelSetup &ks = kernel_setup_table()[{reinterpret_cast<const void *>(kernel), dev}];
  if (ks.slots >= 0) return ks.slots;
  int sms = 0, per_sm = 0;
  if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
      cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, threads, smem) != cudaSuccess) {
    cudaGetLastError();
    return 0;
  }
  ks.slots = (long)sms * per_sm;
  return ks.slots;
}

// ---- element access in the activation dtype ---------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }

// ---- complex numbers as float2 ------------------------------------------------
__device__ __forceinline__ float2 cmul(float2 a, float2 b) {
  return make_float2(a.x * b.x - a.y * b.y, a.x * b.y + a.y * b.x);
}
__device__ __forceinline__ float2 cmulc(float2 a, float2 b) {  // a * conj(b)
  return make_float2(a.x * b.x + a.y * b.y, a.y * b.x - a.x * b.y);
}
__device__ __forceinline__ float2 cconj(float2 a) { return make_float2(a.x, -a.y); }
__device__ __forceinline__ float2 cadd(float2 a, float2 b) { return make_float2(a.x + b.x, a.y + b.y); }
__device__ __forceinline__ float2 csub(float2 a, float2 b) { return make_float2(a.x - b.x, a.y - b.y); }
__device__ __forceinline__ float2 cscale(float2 a, float s) { return make_float2(a.x * s, a.y * s); }

// Per-chunk transition prefix in the stable split form of the reference
// (slinoss/ops/v2x2ssd/reference.py:466-491): lp[t] = sum_{tau<=t} log|m_tau|,
// ph[t] = normalised prod_{tau<=t} m_tau/|m_tau|.  Tokens >= valid act as m = 1.
// Executed by warp 0 of the CTA; results land in shared memory (lp, ph of
// length L) and the caller synchronises.  An exactly-zero |m| has no log-magnitude / phase
// split (the reference raises, reference.py:480-485): it sets *bad_flag and poisons the chunk
// with NaN, which the state pass carries into everything downstream.
template <bool FAST = false>
__device__ __forceinline__ void chunk_prefix_warp(int run_warp, const float *__restrict__ Mchunk, int L, int valid,
                                                  float *lp, float2 *ph, float2 *mraw, int *bad_flag) {
  const int lane = threadIdx.x & 31;
  if ((int)(threadIdx.x >> 5) != run_warp) return;
  const int per = (L + 31) / 32;
  const int t0 = lane * per;
  float lsum = 0.f;
  float2 psum = make_float2(1.f, 0.f);
  for (int i = 0; i < per; ++i) {
    int t = t0 + i;
    if (t < L) {
      float2 m = make_float2(1.f, 0.f);
      if (t < valid) m = *reinterpret_cast<const float2 *>(Mchunk + 2 * (size_t)t);
      float mag, inv, lg;
      if (FAST) {  // half-input kernels: fast intrinsics are far inside their error budget
        float m2 = fmaf(m.x, m.x, m.y * m.y);
        if (m2 == 0.f) {
          if (bad_flag) atomicExch(bad_flag, 1);
          m2 = 1.f;
          m = make_float2(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));  // poison: see header
        }
        inv = rsqrtf(m2);
        lg = 0.5f * __logf(m2);
      } else {
        mag = hypotf(m.x, m.y);
        if (mag == 0.f) {
          if (bad_flag) atomicExch(bad_flag, 1);
          mag = 1.f;
          m = make_float2(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
        }
        inv = 1.f / mag;
        lg = logf(mag);
      }
      mraw[t] = m;
      lsum += lg;
      psum = cmul(psum, make_float2(m.x * inv, m.y * inv));
      lp[t] = lsum;
      ph[t] = psum;
    }
  }
  // exclusive scan of the per-lane totals
  float lincl = lsum;
  float2 pincl = psum;
  for (int off = 1; off < 32; off <<= 1) {
    float lo = __shfl_up_sync(0xffffffffu, lincl, off);
    float px = __shfl_up_sync(0xffffffffu, pincl.x, off);
    float py = __shfl_up_sync(0xffffffffu, pincl.y, off);
    if (lane >= off) {
      lincl += lo;
      pincl = cmul(pincl, make_float2(px, py));
    }
  }
  float lex = __shfl_up_sync(0xffffffffu, lincl, 1);
  float pex_x = __shfl_up_sync(0xffffffffu, pincl.x, 1);
  float pex_y = __shfl_up_sync(0xffffffffu, pincl.y, 1);
  if (lane == 0) {
    lex = 0.f;
    pex_x = 1.f;
    pex_y = 0.f;
  }
  for (int i = 0; i < per; ++i) {
    int t = t0 + i;
    if (t < L) {
      float2 p = cmul(ph[t], make_float2(pex_x, pex_y));
      float inv = rsqrtf(p.x * p.x + p.y * p.y);
      ph[t] = make_float2(p.x * inv, p.y * inv);
      lp[t] += lex;
    }
  }
}

// The same prefix for chunks of 128 tokens with the four multipliers of every lane already in
// registers (tokens 4*lane .. 4*lane+3; 1 past the end of the sequence): lets a kernel request
// them before its bulk copies and run the prefix when they have arrived.  Called by one warp.
__device__ __forceinline__ void chunk_prefix_load4(const float *__restrict__ Mchunk, int valid, float2 (&m)[4]) {
  const int lane = threadIdx.x & 31;
  const int t0 = 4 * lane;
  if (t0 + 3 < valid && (reinterpret_cast<uintptr_t>(Mchunk) & 15) == 0) {
    const float4 a = *reinterpret_cast<const float4 *>(Mchunk + 2 * (size_t)t0);
    const float4 b = *reinterpret_cast<const float4 *>(Mchunk + 2 * (size_t)t0 + 4);
    m[0] = make_float2(a.x, a.y);
    m[1] = make_float2(a.z, a.w);
    m[2] = make_float2(b.x, b.y);
    m[3] = make_float2(b.z, b.w);
  } else {
#pragma unroll
    for (int i = 0; i < 4; ++i)
      m[i] = (t0 + i < valid) ? *reinterpret_cast<const float2 *>(Mchunk + 2 * (size_t)(t0 + i)) : make_float2(1.f, 0.f);
  }
}
__device__ __forceinline__ void chunk_prefix_fast128(const float2 (&min)[4], float *lp, float2 *ph, float2 *mraw,
                                                     int *bad_flag) {
  const int lane = threadIdx.x & 31;
  const int t0 = 4 * lane;
  float lsum = 0.f;
  float2 psum = make_float2(1.f, 0.f);
  float lloc[4];
  float2 ploc[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 m = min[i];
    float m2 = fmaf(m.x, m.x, m.y * m.y);
    if (m2 == 0.f) {
      if (bad_flag) atomicExch(bad_flag, 1);
      m2 = 1.f;
      m = make_float2(__int_as_float(0x7fc00000), __int_as_float(0x7fc00000));
    }
    const float inv = rsqrtf(m2);
    mraw[t0 + i] = m;
    lsum += 0.5f * __logf(m2);
    psum = cmul(psum, make_float2(m.x * inv, m.y * inv));
    lloc[i] = lsum;
    ploc[i] = psum;
  }
  float lincl = lsum;
  float2 pincl = psum;
#pragma unroll
  for (int off = 1; off < 32; off <<= 1) {
    const float lo = __shfl_up_sync(0xffffffffu, lincl, off);
    const float px = __shfl_up_sync(0xffffffffu, pincl.x, off);
    const float py = __shfl_up_sync(0xffffffffu, pincl.y, off);
    if (lane >= off) {
      lincl += lo;
      pincl = cmul(pincl, make_float2(px, py));
    }
  }
  float lex = __shfl_up_sync(0xffffffffu, lincl, 1);
  float pex_x = __shfl_up_sync(0xffffffffu, pincl.x, 1);
  float pex_y = __shfl_up_sync(0xffffffffu, pincl.y, 1);
  if (lane == 0) {
    lex = 0.f;
    pex_x = 1.f;
    pex_y = 0.f;
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 p = cmul(ploc[i], make_float2(pex_x, pex_y));
    const float inv = rsqrtf(p.x * p.x + p.y * p.y);
    ph[t0 + i] = make_float2(p.x * inv, p.y * inv);
    lp[t0 + i] = lloc[i] + lex;
  }
}

__device__ __forceinline__ void chunk_prefix_warp0(const float *__restrict__ Mchunk, int L, int valid, float *lp,
                                                   float2 *ph, float2 *mraw, int *bad_flag) {
  chunk_prefix_warp<false>(0, Mchunk, L, valid, lp, ph, mraw, bad_flag);
}

}  // namespace slx
