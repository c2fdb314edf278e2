// C-ABI entry points of the scan (argument checks + launches; no allocation,
// no synchronisation).
#include <cstdarg>
#include <cstdio>
#include <type_traits>

#include <atomic>
#include <initializer_list>
#include <mutex>

#include "scan_simt.cuh"
#include "scan_tc.cuh"
#include "scan_tc_bwd.cuh"
#include "scan_ws_bwd.cuh"
#include "state_passing.cuh"

namespace slx {

// shapes the tcgen05 kernels cover
static bool tc_capable(const slx_scan_shape *s) {
  return (s->dtype == SLX_BF16 || s->dtype == SLX_F16) && s->chunk == 128 && s->P == 64 && s->N % 32 == 0 &&
         s->N >= 32 && s->N <= 128;
}

static int check_shape(const slx_scan_shape *s, ScanDims *d) {
  SLX_REQUIRE(s != nullptr, SLX_E_NULL, "shape is NULL");
  SLX_REQUIRE(s->batch_heads > 0 && s->T > 0 && s->P > 0 && s->N > 0 && s->chunk > 0, SLX_E_SHAPE,
              "batch_heads, T, P, N and chunk must be positive (got %d %d %d %d %d)", s->batch_heads, s->T, s->P,
              s->N, s->chunk);
  SLX_REQUIRE(s->P <= kPMax, SLX_E_UNSUPPORTED, "P=%d exceeds the supported maximum %d", s->P, kPMax);
  SLX_REQUIRE(s->chunk == 16 || s->chunk == 32 || s->chunk == 64 || s->chunk == 128, SLX_E_UNSUPPORTED,
              "chunk=%d: supported chunk lengths are 16, 32, 64, 128", s->chunk);
  SLX_REQUIRE(s->dtype == SLX_F32 || s->dtype == SLX_BF16 || s->dtype == SLX_F16, SLX_E_DTYPE, "bad dtype %d",
              s->dtype);
  SLX_REQUIRE(s->batch_heads <= 65535, SLX_E_UNSUPPORTED, "batch_heads=%d exceeds 65535", s->batch_heads);
  SLX_REQUIRE(s->starts_dtype == SLX_F32 || s->starts_dtype == s->dtype, SLX_E_DTYPE,
              "starts_dtype %d must be fp32 or the activation dtype %d", s->starts_dtype, s->dtype);
  SLX_REQUIRE(s->starts_dtype == SLX_F32 || tc_capable(s), SLX_E_UNSUPPORTED,
              "half-precision chunk_starts select the tensor-core kernels, which need half inputs, chunk 128, "
              "P 64 and 2N in {64,128,192,256} (got chunk %d P %d N %d)", s->chunk, s->P, s->N);
  d->BH = s->batch_heads;
  d->T = s->T;
  d->P = s->P;
  d->N = s->N;
  d->D = 2 * s->N;
  d->L = s->chunk;
  d->NC = (s->T + s->chunk - 1) / s->chunk;
  return SLX_OK;
}

template <typename K>
static int set_smem(K kernel, size_t bytes) {
  return ensure_dyn_smem(kernel, bytes);
}

#define SLX_DISPATCH_L(Lval, ...)            \
  switch (Lval) {                            \
    case 16: { constexpr int L_ = 16; __VA_ARGS__; } break;   \
    case 32: { constexpr int L_ = 32; __VA_ARGS__; } break;   \
    case 64: { constexpr int L_ = 64; __VA_ARGS__; } break;   \
    default: { constexpr int L_ = 128; __VA_ARGS__; } break;  \
  }

#define SLX_DISPATCH_T(dt, ...)                                   \
  switch (dt) {                                                   \
    case SLX_F32: { using T_ = float; __VA_ARGS__; } break;       \
    case SLX_BF16: { using T_ = __nv_bfloat16; __VA_ARGS__; } break; \
    default: { using T_ = __half; __VA_ARGS__; } break;           \
  }

// ---- stage launchers ----------------------------------------------------------
template <typename T, int L, int MODE>
static int launch_outer(const ScanDims &d, const void *A, const void *X, const float *M, const float *K,
                        const float *Bprev, const float *Uprev, float *out, float *m_chunk, cudaStream_t st) {
  OuterArgs<T> a{(const T *)A, (const T *)X, M, K, Bprev, Uprev, out, m_chunk, d};
  auto kern = chunk_outer_kernel<T, L, MODE>;
  size_t smem = outer_smem_bytes<L>();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3(d.NC, d.BH), kThreads, smem, st>>>(a);
  return check_launch(MODE == 0 ? "chunk_increment_fwd" : "chunk_scan_bwd_dz0");
}

template <typename T, int L>
static int launch_scan_fwd(const ScanDims &d, const void *U, const float *M, const float *K, const void *B,
                           const void *C, const float *starts, const float *Bprev, const float *Uprev, void *Y,
                           cudaStream_t st) {
  ScanFwdArgs<T> a{(const T *)U, (const T *)B, (const T *)C, M, K, starts, Bprev, Uprev, (T *)Y, nullptr, d};
  auto kern = chunk_scan_fwd_kernel<T, L>;
  size_t smem = scan_fwd_smem_bytes<L>();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3(d.NC, d.BH), kThreads, smem, st>>>(a);
  return check_launch("chunk_scan_fwd");
}

template <typename T, int L>
static int launch_scan_bwd(const ScanDims &d, const ScanBwdArgs<T> &a, cudaStream_t st) {
  auto kern = chunk_scan_bwd_kernel<T, L>;
  size_t smem = scan_bwd_smem_bytes<L>();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3(d.NC, d.BH), kThreads, smem, st>>>(a);
  return check_launch("chunk_scan_bwd");
}

// ---- tensor-core path selection ----------------------------------------------------
static int g_use_tc = 1;  // 0: fp32-exact CUDA-core kernels for every dtype; 1: per-chunk tcgen05 kernels; 2: persistent ones

// every kernel of this file reads and writes its tensors with 8- and 16-byte accesses
static bool all_aligned16(std::initializer_list<const void *> ptrs) {
  for (const void *p : ptrs)
    if (p != nullptr && (reinterpret_cast<uintptr_t>(p) & 15) != 0) return false;
  return true;
}
#define SLX_REQUIRE_ALIGNED(what, ...) \
  SLX_REQUIRE(all_aligned16({__VA_ARGS__}), SLX_E_UNSUPPORTED, what ": tensor pointers must be 16-byte aligned")

// The kernel family follows from the shape alone: half-precision chunk_starts (s->starts_dtype)
// mean the tensor-core kernels, fp32 chunk_starts the exact CUDA-core kernels.  check_shape has
// verified that the combination exists.
static bool use_tc(const slx_scan_shape *s) { return s->starts_dtype != SLX_F32; }

// Tensor map of a (BH, T, width) half tensor for boxes of [rows][64 columns], 128-byte swizzle.
template <typename T>
static int make_tile_map(CUtensorMap *map, const void *base, int BH, int T_, int width, int box_rows, const char *what) {
  const cuuint64_t dims[3] = {(cuuint64_t)width, (cuuint64_t)T_, (cuuint64_t)BH};
  const cuuint64_t strides[2] = {(cuuint64_t)width * sizeof(T), (cuuint64_t)T_ * width * sizeof(T)};
  const cuuint32_t box[3] = {64u, (cuuint32_t)box_rows, 1u};
  const cuuint32_t estr[3] = {1u, 1u, 1u};
  const CUtensorMapDataType dt =
      std::is_same<T, __half>::value ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
  // the driver entry point is looked up at run time so that the library loads on machines without a driver
  typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                               const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
  static std::atomic<EncodeFn> encode_fn{nullptr};
  EncodeFn encode = encode_fn.load(std::memory_order_acquire);
  if (encode == nullptr) {
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || fn == nullptr)
      return fail(SLX_E_UNSUPPORTED, "%s: cuTensorMapEncodeTiled is not available from this driver", what);
    encode = reinterpret_cast<EncodeFn>(fn);
    encode_fn.store(encode, std::memory_order_release);
  }
  CUresult r = encode(map, dt, 3, const_cast<void *>(base), dims, strides, box, estr,
                                      CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                      CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) return fail(SLX_E_UNSUPPORTED, "%s: tensor map could not be encoded (CUresult %d)", what, (int)r);
  return SLX_OK;
}

// dtype of the chunk-start states between the stages: the activation dtype on the tensor-core
// path (those kernels round Z0 to it anyway; half the bytes of fp32), fp32 otherwise

template <typename T>
static int launch_scan_fwd_tc(const ScanDims &d, const void *U, const float *M, const float *K, const void *B,
                              const void *C, const float *starts, const float *Bprev, const float *Uprev, void *Y,
                              cudaStream_t st) {
  ScanFwdArgs<T> a{(const T *)U, (const T *)B, (const T *)C, M, K, starts, Bprev, Uprev, (T *)Y, nullptr, d};
  auto kern = chunk_scan_fwd_tc_kernel<T>;
  size_t smem = scan_fwd_tc_smem_bytes();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3(d.NC, d.BH), kTcThreads, smem, st>>>(a);
  return check_launch("chunk_scan_fwd_tc");
}

// CTAs of the persistent kernels: one per SM unless a smaller number was asked for
// (slx_set_persistent_ctas; the tests use it to walk the multi-chunk loop on small inputs)
static std::atomic<int> g_max_ctas{0};

static int sm_count() {
  static std::atomic<int> cached[64];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

static int persistent_grid(int total) {
  int g = sm_count();
  const int cap = g_max_ctas.load(std::memory_order_relaxed);
  if (cap > 0 && cap < g) g = cap;
  return total < g ? total : g;
}

// Forward chunk scan, persistent warp-specialised kernel (scan_ws_fwd.cuh)
template <typename T>
static int launch_scan_fwd_ws(const ScanDims &d, const void *U, const float *M, const float *K, const void *B,
                              const void *C, const void *starts, const float *Bprev, const float *Uprev, void *Y,
                              cudaStream_t st) {
  ScanFwdArgs<T> a{(const T *)U, (const T *)B, (const T *)C, M, K, (const float *)starts, Bprev, Uprev, (T *)Y, nullptr, d};
  auto kern = chunk_scan_fwd_ws_kernel<T>;
  const size_t smem = scan_ws_fwd_smem_bytes();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  WsFwdMaps maps;
  if ((rc = make_tile_map<T>(&maps.C, C, d.BH, d.T, d.D, 128, "chunk_scan_fwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.B, B, d.BH, d.T, d.D, 128, "chunk_scan_fwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.Z, starts, d.BH * d.NC, d.P, d.D, 64, "chunk_scan_fwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.U, U, d.BH, d.T, d.P, 128, "chunk_scan_fwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.Y, Y, d.BH, d.T, d.P, 128, "chunk_scan_fwd"))) return rc;
  const int grid = persistent_grid(d.BH * d.NC);
  kern<<<grid, kWsThreads, smem, st>>>(a, maps);
  return check_launch("chunk_scan_fwd_ws");
}

template <typename T, int MODE, typename OT>
static int launch_outer_tc_t(const ScanDims &d, const void *A, const void *X, const float *M, const float *K,
                             const float *Bprev, const float *Uprev, void *out, float *m_chunk, cudaStream_t st) {
  OuterArgs<T> a{(const T *)A, (const T *)X, M, K, Bprev, Uprev, (float *)out, m_chunk, d};
  auto kern = chunk_outer_tc_kernel<T, MODE, OT>;
  size_t smem = outer_tc_smem_bytes();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  kern<<<dim3(d.NC, d.BH), kTcThreads, smem, st>>>(a);
  return check_launch(MODE == 0 ? "chunk_increment_fwd_tc" : "chunk_scan_bwd_dz0_tc");
}
// `out` holds fp32 values, or (half_out) values of the activation dtype T
template <typename T, int MODE>
static int launch_outer_tc(const ScanDims &d, const void *A, const void *X, const float *M, const float *K,
                           const float *Bprev, const float *Uprev, void *out, bool half_out, float *m_chunk,
                           cudaStream_t st) {
  if (half_out) return launch_outer_tc_t<T, MODE, T>(d, A, X, M, K, Bprev, Uprev, out, m_chunk, st);
  return launch_outer_tc_t<T, MODE, float>(d, A, X, M, K, Bprev, Uprev, out, m_chunk, st);
}

template <typename T>
static int launch_scan_bwd_tc(const ScanDims &d, const ScanBwdArgs<T> &a, cudaStream_t st) {
  auto kern = chunk_scan_bwd_tc_kernel<T>;
  size_t smem = scan_bwd_tc_smem_bytes();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  ScanBwdMaps maps;
  rc = make_tile_map<T>(&maps.C, a.C, d.BH, d.T, d.D, 128, "chunk_scan_bwd");
  if (rc) return rc;
  rc = make_tile_map<T>(&maps.B, a.B, d.BH, d.T, d.D, 128, "chunk_scan_bwd");
  if (rc) return rc;
  if ((rc = make_tile_map<T>(&maps.dC, a.dC, d.BH, d.T, d.D, 128, "chunk_scan_bwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.dB, a.dB, d.BH, d.T, d.D, 128, "chunk_scan_bwd"))) return rc;
  kern<<<dim3(d.NC, d.BH), kTcBwdThreads, smem, st>>>(a, maps);
  return check_launch("chunk_scan_bwd_tc");
}

// Per-chunk backward, persistent warp-specialised kernel (scan_ws_bwd.cuh)
template <typename T>
static int launch_scan_bwd_ws(const ScanDims &d, const ScanBwdArgs<T> &a, cudaStream_t st) {
  auto kern = chunk_scan_bwd_ws_kernel<T>;
  const size_t smem = scan_ws_bwd_smem_bytes();
  int rc = set_smem(kern, smem);
  if (rc) return rc;
  WsBwdMaps maps;
  if ((rc = make_tile_map<T>(&maps.C, a.C, d.BH, d.T, d.D, 128, "chunk_scan_bwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.B, a.B, d.BH, d.T, d.D, 128, "chunk_scan_bwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.Z, a.starts, d.BH * d.NC, d.P, d.D, 64, "chunk_scan_bwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.Lm, a.d_inc, d.BH * d.NC, d.P, d.D, 64, "chunk_scan_bwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.U, a.U, d.BH, d.T, d.P, 128, "chunk_scan_bwd"))) return rc;
  if ((rc = make_tile_map<T>(&maps.dY, a.dY, d.BH, d.T, d.P, 128, "chunk_scan_bwd"))) return rc;
  const int grid = persistent_grid(d.BH * d.NC);
  kern<<<grid, kWsThreads, smem, st>>>(a, maps);
  return check_launch("chunk_scan_bwd_ws");
}

template <typename ST, typename IT>
static int launch_state_fwd_t(int BH, int NC, int P, int N, const IT *inc, const float *m_chunk, const float *init,
                              ST *starts, float *final_state, cudaStream_t st) {
  const int elems = P * 2 * N;
  // (eight values per thread, as the reverse pass uses for all-half storage, measured 0.100 against 0.095 ms here)
  if (elems % 4 == 0) {
    int nv = elems / 4;
    state_passing_fwd_kernel<4, ST, IT><<<dim3((nv + 255) / 256, BH), 256, 0, st>>>(inc, m_chunk, init, starts,
                                                                                  final_state, NC, nv);
  } else {
    int nv = elems / 2;
    state_passing_fwd_kernel<2, ST, IT><<<dim3((nv + 255) / 256, BH), 256, 0, st>>>(inc, m_chunk, init, starts,
                                                                                  final_state, NC, nv);
  }
  return check_launch("state_passing_fwd");
}
// inc_dtype is fp32 or starts_dtype (checked by the callers)
static int launch_state_fwd(int BH, int NC, int P, int N, const void *inc, int inc_dtype, const float *m_chunk,
                            const float *init, void *starts, int starts_dtype, float *final_state, cudaStream_t st) {
  const bool half_inc = inc_dtype != SLX_F32;
  if (starts_dtype == SLX_BF16) {
    using H = __nv_bfloat16;
    if (half_inc) return launch_state_fwd_t<H, H>(BH, NC, P, N, (const H *)inc, m_chunk, init, (H *)starts, final_state, st);
    return launch_state_fwd_t<H, float>(BH, NC, P, N, (const float *)inc, m_chunk, init, (H *)starts, final_state, st);
  }
  if (starts_dtype == SLX_F16) {
    using H = __half;
    if (half_inc) return launch_state_fwd_t<H, H>(BH, NC, P, N, (const H *)inc, m_chunk, init, (H *)starts, final_state, st);
    return launch_state_fwd_t<H, float>(BH, NC, P, N, (const float *)inc, m_chunk, init, (H *)starts, final_state, st);
  }
  return launch_state_fwd_t<float, float>(BH, NC, P, N, (const float *)inc, m_chunk, init, (float *)starts, final_state,
                                          st);
}

static int state_bwd_vec(int P, int N, bool all_half) {
  const int elems = P * 2 * N;
  return (all_half && elems % 8 == 0) ? 8 : (elems % 4 == 0) ? 4 : 2;
}
// partial sums per chunk of the reverse pass (one per warp): upper bound over the vector widths,
// which the workspace is sized with
static int state_bwd_parts(int P, int N) {
  const int elems = P * 2 * N;
  int nv = (elems % 4 == 0) ? elems / 4 : elems / 2;
  return (nv + 255) / 256 * 8;
}

template <typename ST, typename IT>
static int launch_state_bwd_t(int BH, int NC, int P, int N, const IT *dZ0, const float *m_chunk, const ST *starts,
                              const float *final_state, const float *d_final, ST *d_inc, float *d_initial,
                              float *zdot, float *partials, cudaStream_t st) {
  const int elems = P * 2 * N;
  const int vec = state_bwd_vec(P, N, sizeof(ST) == 2 && sizeof(IT) == 2);
  const int nblk = (elems / vec + 255) / 256;
  if (vec == 8) {
    if constexpr (sizeof(ST) == 2 && sizeof(IT) == 2)
      state_passing_bwd_kernel<8, ST, IT><<<dim3(nblk, BH), 256, 0, st>>>(dZ0, m_chunk, starts, final_state, d_final,
                                                                         d_inc, d_initial, partials, NC, elems / 8);
  } else if (vec == 4) {
    state_passing_bwd_kernel<4, ST, IT><<<dim3(nblk, BH), 256, 0, st>>>(dZ0, m_chunk, starts, final_state, d_final,
                                                                       d_inc, d_initial, partials, NC, elems / 4);
  } else {
    state_passing_bwd_kernel<2, ST, IT><<<dim3(nblk, BH), 256, 0, st>>>(dZ0, m_chunk, starts, final_state, d_final,
                                                                       d_inc, d_initial, partials, NC, elems / 2);
  }
  int rc = check_launch("state_passing_bwd");
  if (rc || partials == nullptr) return rc;
  int rows = BH * NC;
  zdot_reduce_kernel<<<(rows + 255) / 256, 256, 0, st>>>(partials, zdot, rows, nblk * 8);
  return check_launch("zdot_reduce");
}
// dz0_dtype is fp32 or starts_dtype (checked by the callers)
static int launch_state_bwd(int BH, int NC, int P, int N, const void *dZ0, int dz0_dtype, const float *m_chunk,
                            const void *starts, int starts_dtype, const float *final_state, const float *d_final,
                            void *d_inc, float *d_initial, float *zdot, float *partials, cudaStream_t st) {
  const bool half_dz = dz0_dtype != SLX_F32;
  if (starts_dtype == SLX_BF16) {
    using H = __nv_bfloat16;
    if (half_dz)
      return launch_state_bwd_t<H, H>(BH, NC, P, N, (const H *)dZ0, m_chunk, (const H *)starts, final_state, d_final,
                                      (H *)d_inc, d_initial, zdot, partials, st);
    return launch_state_bwd_t<H, float>(BH, NC, P, N, (const float *)dZ0, m_chunk, (const H *)starts, final_state,
                                        d_final, (H *)d_inc, d_initial, zdot, partials, st);
  }
  if (starts_dtype == SLX_F16) {
    using H = __half;
    if (half_dz)
      return launch_state_bwd_t<H, H>(BH, NC, P, N, (const H *)dZ0, m_chunk, (const H *)starts, final_state, d_final,
                                      (H *)d_inc, d_initial, zdot, partials, st);
    return launch_state_bwd_t<H, float>(BH, NC, P, N, (const float *)dZ0, m_chunk, (const H *)starts, final_state,
                                        d_final, (H *)d_inc, d_initial, zdot, partials, st);
  }
  return launch_state_bwd_t<float, float>(BH, NC, P, N, (const float *)dZ0, m_chunk, (const float *)starts, final_state,
                                          d_final, (float *)d_inc, d_initial, zdot, partials, st);
}

// workspace layout of the backward (256-byte aligned sections; dZ0 and d_inc as starts_dtype, the rest fp32)
struct BwdWs {
  size_t d_inc, dz0, zdot, partials, carryB, carryU, total;  // dz0 == d_inc where the reverse pass runs in place
};
static size_t align256(size_t x) { return (x + 255) & ~(size_t)255; }
static BwdWs bwd_ws(const ScanDims &d, int starts_dtype) {
  BwdWs w;
  size_t off = 0;
  const size_t n_state = (size_t)d.BH * d.NC * d.P * d.D;
  w.dz0 = off;
  if (starts_dtype == SLX_F32) {
    off += align256(sizeof(float) * n_state);
    w.d_inc = w.dz0;  // fp32 d_inc overwrites dZ0 chunk by chunk
  } else {  // dZ0 and d_inc both in the activation dtype, side by side
    off += align256(2 * n_state);
    w.d_inc = off;
    off += align256(2 * n_state);
  }
  w.zdot = off;
  off += align256(sizeof(float) * (size_t)d.BH * d.NC * 2);
  w.partials = off;
  off += align256(sizeof(float) * (size_t)d.BH * d.NC * 2 * state_bwd_parts(d.P, d.N));
  w.carryB = off;
  off += align256(sizeof(float) * (size_t)d.BH * d.NC * d.D);
  w.carryU = off;
  off += align256(sizeof(float) * (size_t)d.BH * d.NC * d.P);
  w.total = off;
  return w;
}

// Read-and-clear of a device status word as ONE atomic exchange on the device (a flag raised by a
// kernel that is still running is either returned by this read or kept for the next one, never
// lost).  The exchanged value travels through a second device word; the host mutex keeps two
// host threads from interleaving their kernel + copy pairs.  Runs on the legacy default stream
// of the current device and synchronises.
__device__ int g_status_mailbox = 0;
__global__ void status_exchange_kernel(int which) {
  g_status_mailbox = atomicExch(which == 0 ? &g_tc_status : &g_scan_bad, 0);
}
static std::mutex g_status_mutex;
static int exchange_status(int which, int *host_out, const char *what) {
  std::lock_guard<std::mutex> lock(g_status_mutex);
  status_exchange_kernel<<<1, 1>>>(which);
  cudaError_t e = cudaGetLastError();
  if (e == cudaSuccess) e = cudaMemcpyFromSymbol(host_out, g_status_mailbox, sizeof(int));
  if (e != cudaSuccess) return fail((int)e, "%s: %s", what, cudaGetErrorString(e));
  return SLX_OK;
}

}  // namespace slx

using namespace slx;

extern "C" {

int slx_abi_version(void) { return SLX_ABI_VERSION; }

int slx_set_tensor_path(int enable) {
  int old = g_use_tc;
  g_use_tc = enable < 0 ? 0 : (enable > 2 ? 2 : enable);
  return old;
}

#ifdef SLX_DIAG
int slx_read_phase_clock(long long *host_out64) {
  SLX_REQUIRE(host_out64 != nullptr, SLX_E_NULL, "read_phase_clock: NULL pointer");
  cudaError_t e = cudaMemcpyFromSymbol(host_out64, g_phase_clock, sizeof(long long) * 128);
  if (e != cudaSuccess) return fail((int)e, "read_phase_clock: %s", cudaGetErrorString(e));
  return SLX_OK;
}
#endif

int slx_set_persistent_ctas(int max_ctas) {
  return g_max_ctas.exchange(max_ctas > 0 ? max_ctas : 0, std::memory_order_relaxed);
}

int slx_read_tc_status(int *host_out) {
  SLX_REQUIRE(host_out != nullptr, SLX_E_NULL, "read_tc_status: NULL pointer");
  return exchange_status(0, host_out, "read_tc_status");
}
int slx_scan_starts_dtype(const slx_scan_shape *s) {
  if (s == nullptr) return SLX_F32;
  return (g_use_tc && tc_capable(s)) ? s->dtype : (int)SLX_F32;
}

int slx_read_scan_status(int *host_out) {
  SLX_REQUIRE(host_out != nullptr, SLX_E_NULL, "read_scan_status: NULL pointer");
  return exchange_status(1, host_out, "read_scan_status");
}
const char *slx_last_error_string(void) { return g_err; }

int slx_chunk_increment_fwd(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                            const float *B_prev, const float *U_prev, void *inc, int32_t inc_dtype, float *m_chunk,
                            void *stream) {
  ScanDims d;
  int rc = check_shape(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(U && M && K && B && inc && m_chunk, SLX_E_NULL, "chunk_increment_fwd: NULL tensor");
  SLX_REQUIRE(inc_dtype == SLX_F32 || (use_tc(s) && inc_dtype == s->dtype), SLX_E_DTYPE,
              "chunk_increment_fwd: inc_dtype %d must be fp32, or the activation dtype on the tensor-core path",
              inc_dtype);
  SLX_REQUIRE_ALIGNED("chunk_increment_fwd", U, M, K, B, B_prev, U_prev, inc, m_chunk);
  SLX_REQUIRE((B_prev == nullptr) == (U_prev == nullptr), SLX_E_NULL, "B_prev and U_prev must be passed together");
  if (use_tc(s)) {
    if (s->dtype == SLX_BF16)
      return launch_outer_tc<__nv_bfloat16, 0>(d, U, B, M, K, B_prev, U_prev, inc, inc_dtype != SLX_F32, m_chunk,
                                               as_stream(stream));
    return launch_outer_tc<__half, 0>(d, U, B, M, K, B_prev, U_prev, inc, inc_dtype != SLX_F32, m_chunk,
                                      as_stream(stream));
  }
  SLX_DISPATCH_T(s->dtype, SLX_DISPATCH_L(d.L, rc = (launch_outer<T_, L_, 0>(d, U, B, M, K, B_prev, U_prev, (float *)inc,
                                                                              m_chunk, as_stream(stream)))));
  return rc;
}

int slx_state_passing_fwd(int32_t BH, int32_t NC, int32_t P, int32_t N, const void *inc, int32_t inc_dtype,
                          const float *m_chunk, const float *initial_states, void *chunk_starts, int32_t starts_dtype,
                          float *final_state, void *stream) {
  SLX_REQUIRE(BH > 0 && NC > 0 && P > 0 && N > 0, SLX_E_SHAPE, "state_passing_fwd: sizes must be positive");
  SLX_REQUIRE(BH <= 65535, SLX_E_UNSUPPORTED, "batch_heads=%d exceeds 65535", BH);
  SLX_REQUIRE(inc && m_chunk && final_state, SLX_E_NULL, "state_passing_fwd: NULL tensor");
  SLX_REQUIRE_ALIGNED("state_passing_fwd", inc, initial_states, chunk_starts, final_state);
  SLX_REQUIRE(starts_dtype == SLX_F32 || starts_dtype == SLX_BF16 || starts_dtype == SLX_F16, SLX_E_DTYPE,
              "state_passing_fwd: bad starts_dtype %d", starts_dtype);
  SLX_REQUIRE(starts_dtype == SLX_F32 || chunk_starts != (void *)inc, SLX_E_UNSUPPORTED,
              "state_passing_fwd: the in-place pass needs fp32 chunk_starts");
  SLX_REQUIRE(inc_dtype == SLX_F32 || inc_dtype == SLX_BF16 || inc_dtype == SLX_F16, SLX_E_DTYPE,
              "state_passing_fwd: bad inc_dtype %d", inc_dtype);
  if (chunk_starts == nullptr && inc_dtype != SLX_F32) starts_dtype = inc_dtype;  // nothing is stored as starts_dtype
  SLX_REQUIRE(inc_dtype == SLX_F32 || inc_dtype == starts_dtype, SLX_E_DTYPE,
              "state_passing_fwd: inc_dtype %d must be fp32 or starts_dtype %d", inc_dtype, starts_dtype);
  return launch_state_fwd(BH, NC, P, N, inc, inc_dtype, m_chunk, initial_states, chunk_starts, starts_dtype,
                          final_state, as_stream(stream));
}

int slx_chunk_scan_fwd(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                       const void *C, const void *chunk_starts, const float *B_prev, const float *U_prev, void *Y,
                       void *stream) {
  ScanDims d;
  int rc = check_shape(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(U && M && K && B && C && chunk_starts && Y, SLX_E_NULL, "chunk_scan_fwd: NULL tensor");
  SLX_REQUIRE_ALIGNED("chunk_scan_fwd", U, M, K, B, C, chunk_starts, B_prev, U_prev, Y);
  SLX_REQUIRE((B_prev == nullptr) == (U_prev == nullptr), SLX_E_NULL, "B_prev and U_prev must be passed together");
  if (use_tc(s) && g_use_tc == 2) {
    if (s->dtype == SLX_BF16)
      return launch_scan_fwd_ws<__nv_bfloat16>(d, U, M, K, B, C, chunk_starts, B_prev, U_prev, Y, as_stream(stream));
    return launch_scan_fwd_ws<__half>(d, U, M, K, B, C, chunk_starts, B_prev, U_prev, Y, as_stream(stream));
  }
  if (use_tc(s)) {
    if (s->dtype == SLX_BF16)
      return launch_scan_fwd_tc<__nv_bfloat16>(d, U, M, K, B, C, (const float *)chunk_starts, B_prev, U_prev, Y,
                                               as_stream(stream));
    return launch_scan_fwd_tc<__half>(d, U, M, K, B, C, (const float *)chunk_starts, B_prev, U_prev, Y,
                                      as_stream(stream));
  }
  SLX_DISPATCH_T(s->dtype, SLX_DISPATCH_L(d.L, rc = (launch_scan_fwd<T_, L_>(d, U, M, K, B, C, (const float *)chunk_starts, B_prev,
                                                                             U_prev, Y, as_stream(stream)))));
  return rc;
}

int slx_v2x2ssd_fwd(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                    const void *C, const float *initial_states, const float *B_prev, const float *U_prev, void *Y,
                    float *final_state, void *chunk_starts, float *m_chunk, void *increments, void *stream) {
  ScanDims d0;
  {
    int rc0 = check_shape(s, &d0);
    if (rc0) return rc0;
  }
  const int sdt = s->starts_dtype;
  SLX_REQUIRE(increments != nullptr || sdt == SLX_F32, SLX_E_NULL,
              "v2x2ssd_fwd: this shape keeps chunk_starts in the activation dtype and needs the increments buffer");
  void *inc = increments ? increments : chunk_starts;  // increments are stored as starts_dtype, like the states
  int rc = slx_chunk_increment_fwd(s, U, M, K, B, B_prev, U_prev, inc, sdt, m_chunk, stream);
  if (rc) return rc;
  SLX_REQUIRE(final_state != nullptr, SLX_E_NULL, "v2x2ssd_fwd: final_state is NULL");
  const int NC = (s->T + s->chunk - 1) / s->chunk;
  rc = slx_state_passing_fwd(s->batch_heads, NC, s->P, s->N, inc, sdt, m_chunk, initial_states, chunk_starts, sdt,
                             final_state, stream);
  if (rc) return rc;
  return slx_chunk_scan_fwd(s, U, M, K, B, C, chunk_starts, B_prev, U_prev, Y, stream);
}

size_t slx_state_passing_bwd_partials_bytes(int32_t BH, int32_t NC, int32_t P, int32_t N) {
  if (BH <= 0 || NC <= 0 || P <= 0 || N <= 0) return 0;
  return sizeof(float) * (size_t)BH * NC * 2 * state_bwd_parts(P, N);
}

size_t slx_v2x2ssd_bwd_workspace_bytes(const slx_scan_shape *s) {
  ScanDims d;
  if (check_shape(s, &d)) return 0;
  return bwd_ws(d, s->starts_dtype).total;
}

int slx_chunk_scan_bwd_dz0(const slx_scan_shape *s, const float *M, const void *C, const void *dY, void *dZ0,
                           int32_t dz0_dtype, void *stream) {
  ScanDims d;
  int rc = check_shape(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(M && C && dY && dZ0, SLX_E_NULL, "chunk_scan_bwd_dz0: NULL tensor");
  SLX_REQUIRE(dz0_dtype == SLX_F32 || (use_tc(s) && dz0_dtype == s->dtype), SLX_E_DTYPE,
              "chunk_scan_bwd_dz0: dz0_dtype %d must be fp32, or the activation dtype on the tensor-core path",
              dz0_dtype);
  SLX_REQUIRE_ALIGNED("chunk_scan_bwd_dz0", M, C, dY, dZ0);
  if (use_tc(s)) {
    if (s->dtype == SLX_BF16)
      return launch_outer_tc<__nv_bfloat16, 1>(d, dY, C, M, nullptr, nullptr, nullptr, dZ0, dz0_dtype != SLX_F32,
                                               nullptr, as_stream(stream));
    return launch_outer_tc<__half, 1>(d, dY, C, M, nullptr, nullptr, nullptr, dZ0, dz0_dtype != SLX_F32, nullptr,
                                      as_stream(stream));
  }
  SLX_DISPATCH_T(s->dtype, SLX_DISPATCH_L(d.L, rc = (launch_outer<T_, L_, 1>(d, dY, C, M, nullptr, nullptr, nullptr,
                                                                              (float *)dZ0, nullptr, as_stream(stream)))));
  return rc;
}

int slx_state_passing_bwd(int32_t BH, int32_t NC, int32_t P, int32_t N, const void *dZ0, int32_t dz0_dtype,
                          const float *m_chunk,
                          const void *chunk_starts, int32_t starts_dtype, const float *final_state,
                          const float *d_final, void *d_inc,
                          float *d_initial, float *zdot, float *zdot_partials, void *stream) {
  SLX_REQUIRE(BH > 0 && NC > 0 && P > 0 && N > 0, SLX_E_SHAPE, "state_passing_bwd: sizes must be positive");
  SLX_REQUIRE(BH <= 65535, SLX_E_UNSUPPORTED, "batch_heads=%d exceeds 65535", BH);
  SLX_REQUIRE(dZ0 && m_chunk, SLX_E_NULL, "state_passing_bwd: NULL tensor");
  SLX_REQUIRE_ALIGNED("state_passing_bwd", dZ0, chunk_starts, final_state, d_final, d_inc, d_initial);
  SLX_REQUIRE((zdot == nullptr) == (zdot_partials == nullptr), SLX_E_NULL,
              "state_passing_bwd: zdot and zdot_partials go together");
  SLX_REQUIRE(zdot == nullptr || (chunk_starts && final_state), SLX_E_NULL,
              "state_passing_bwd: zdot needs chunk_starts and final_state");
  SLX_REQUIRE(d_inc || d_initial, SLX_E_NULL, "state_passing_bwd: neither d_inc nor d_initial asked for");
  SLX_REQUIRE(starts_dtype == SLX_F32 || d_inc != (const void *)dZ0, SLX_E_UNSUPPORTED,
              "state_passing_bwd: the in-place pass needs fp32 d_inc");
  SLX_REQUIRE(starts_dtype == SLX_F32 || starts_dtype == SLX_BF16 || starts_dtype == SLX_F16, SLX_E_DTYPE,
              "state_passing_bwd: bad starts_dtype %d", starts_dtype);
  SLX_REQUIRE(dz0_dtype == SLX_F32 || dz0_dtype == SLX_BF16 || dz0_dtype == SLX_F16, SLX_E_DTYPE,
              "state_passing_bwd: bad dz0_dtype %d", dz0_dtype);
  // with neither d_inc nor the dot products asked for, nothing is read or stored as starts_dtype
  if (d_inc == nullptr && zdot == nullptr && dz0_dtype != SLX_F32) starts_dtype = dz0_dtype;
  SLX_REQUIRE(dz0_dtype == SLX_F32 || dz0_dtype == starts_dtype, SLX_E_DTYPE,
              "state_passing_bwd: dz0_dtype %d must be fp32 or starts_dtype %d", dz0_dtype, starts_dtype);
  return launch_state_bwd(BH, NC, P, N, dZ0, dz0_dtype, m_chunk, chunk_starts, starts_dtype, final_state, d_final,
                          d_inc, d_initial, zdot, zdot_partials, as_stream(stream));
}

int slx_chunk_scan_bwd(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                       const void *C, const float *B_prev, const float *U_prev, const void *chunk_starts,
                       const void *d_inc, const float *zdot, const void *dY, void *dU, float *dM, float *dK,
                       void *dB, void *dC, float *carryB, float *carryU, void *stream) {
  ScanDims d;
  int rc = check_shape(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(U && M && K && B && C && chunk_starts && d_inc && zdot && dY && dU && dM && dK && dB && dC && carryB &&
                  carryU,
              SLX_E_NULL, "chunk_scan_bwd: NULL tensor");
  SLX_REQUIRE_ALIGNED("chunk_scan_bwd", U, M, K, B, C, B_prev, U_prev, chunk_starts, d_inc, dY, dU, dM, dK, dB, dC,
                      carryB, carryU);
  SLX_REQUIRE((B_prev == nullptr) == (U_prev == nullptr), SLX_E_NULL, "B_prev and U_prev must be passed together");
  const bool tc = use_tc(s);
  SLX_DISPATCH_T(s->dtype, {
    ScanBwdArgs<T_> a{(const T_ *)U, (const T_ *)B, (const T_ *)C, (const T_ *)dY, M, K, (const float *)chunk_starts,
                      (const float *)d_inc, zdot,
                      B_prev, U_prev, (T_ *)dU, (T_ *)dB, (T_ *)dC, dM, dK, carryB, carryU, d};
    if constexpr (!std::is_same<T_, float>::value) {
      if (tc && g_use_tc == 2) return launch_scan_bwd_ws<T_>(d, a, as_stream(stream));
      if (tc) return launch_scan_bwd_tc<T_>(d, a, as_stream(stream));
    }
    SLX_DISPATCH_L(d.L, rc = (launch_scan_bwd<T_, L_>(d, a, as_stream(stream))));
  });
  return rc;
}

static int v2x2ssd_bwd_impl(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                            const void *C, const float *B_prev, const float *U_prev, const void *chunk_starts,
                            const float *m_chunk, const float *final_state, const void *dY, const float *d_final,
                            void *dU, float *dM, float *dK, void *dB, void *dC, float *d_initial, float *dB_prev,
                            float *dU_prev, void *workspace, size_t workspace_bytes, void *stream, bool dz0_ready) {
  ScanDims d;
  int rc = check_shape(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(U && M && K && B && C && chunk_starts && m_chunk && final_state && dY && dU && dM && dK && dB && dC,
              SLX_E_NULL, "v2x2ssd_bwd: NULL tensor");
  SLX_REQUIRE_ALIGNED("v2x2ssd_bwd", final_state, d_final, d_initial, dB_prev, dU_prev);
  SLX_REQUIRE((B_prev == nullptr) == (U_prev == nullptr), SLX_E_NULL, "B_prev and U_prev must be passed together");
  const BwdWs w = bwd_ws(d, s->starts_dtype);
  SLX_REQUIRE(workspace != nullptr && workspace_bytes >= w.total, SLX_E_WORKSPACE,
              "v2x2ssd_bwd: workspace of %zu bytes needed, %zu given", w.total, workspace_bytes);
  SLX_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, SLX_E_WORKSPACE,
              "v2x2ssd_bwd: workspace must be 256-byte aligned");
  char *base = static_cast<char *>(workspace);
  void *d_inc = base + w.d_inc;
  void *dz0 = base + w.dz0;  // stored as starts_dtype
  float *zdot = reinterpret_cast<float *>(base + w.zdot);
  float *partials = reinterpret_cast<float *>(base + w.partials);
  float *carryB = reinterpret_cast<float *>(base + w.carryB);
  float *carryU = reinterpret_cast<float *>(base + w.carryU);
  cudaStream_t st = as_stream(stream);

  if (!dz0_ready) {
    rc = slx_chunk_scan_bwd_dz0(s, M, C, dY, dz0, s->starts_dtype, stream);
    if (rc) return rc;
  }
  rc = launch_state_bwd(d.BH, d.NC, d.P, d.N, dz0, s->starts_dtype, m_chunk, chunk_starts, s->starts_dtype,
                        final_state, d_final, d_inc, d_initial, zdot, partials, st);
  if (rc) return rc;
  rc = slx_chunk_scan_bwd(s, U, M, K, B, C, B_prev, U_prev, chunk_starts, d_inc, zdot, dY, dU, dM, dK, dB, dC, carryB,
                          carryU, stream);
  if (rc) return rc;
  SLX_DISPATCH_T(s->dtype, {
    carry_fixup_kernel<T_><<<dim3(d.NC, d.BH), 128, 0, st>>>(carryB, carryU, (T_ *)dB, (T_ *)dU, dB_prev, dU_prev,
                                                              d.T, d.P, d.D, d.L, d.NC);
    rc = check_launch("carry_fixup");
  });
  return rc;
}

int slx_v2x2ssd_bwd(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                    const void *C, const float *B_prev, const float *U_prev, const void *chunk_starts,
                    const float *m_chunk, const float *final_state, const void *dY, const float *d_final, void *dU,
                    float *dM, float *dK, void *dB, void *dC, float *d_initial, float *dB_prev, float *dU_prev,
                    void *workspace, size_t workspace_bytes, void *stream) {
  return v2x2ssd_bwd_impl(s, U, M, K, B, C, B_prev, U_prev, chunk_starts, m_chunk, final_state, dY, d_final, dU, dM,
                          dK, dB, dC, d_initial, dB_prev, dU_prev, workspace, workspace_bytes, stream, false);
}

int slx_v2x2ssd_bwd_begin(const slx_scan_shape *s, const float *M, const void *C, const float *m_chunk,
                          const void *dY, float *d_initial_zero_final, void *workspace, size_t workspace_bytes,
                          void *stream) {
  ScanDims d;
  int rc = check_shape(s, &d);
  if (rc) return rc;
  SLX_REQUIRE(M && C && m_chunk && dY && d_initial_zero_final, SLX_E_NULL, "v2x2ssd_bwd_begin: NULL tensor");
  const BwdWs w = bwd_ws(d, s->starts_dtype);
  SLX_REQUIRE(workspace != nullptr && workspace_bytes >= w.total, SLX_E_WORKSPACE,
              "v2x2ssd_bwd_begin: workspace of %zu bytes needed, %zu given", w.total, workspace_bytes);
  SLX_REQUIRE((reinterpret_cast<uintptr_t>(workspace) & 255) == 0, SLX_E_WORKSPACE,
              "v2x2ssd_bwd_begin: workspace must be 256-byte aligned");
  void *dz0 = static_cast<char *>(workspace) + w.dz0;
  rc = slx_chunk_scan_bwd_dz0(s, M, C, dY, dz0, s->starts_dtype, stream);
  if (rc) return rc;
  return launch_state_bwd(d.BH, d.NC, d.P, d.N, dz0, s->starts_dtype, m_chunk, nullptr, s->starts_dtype, nullptr,
                          nullptr, nullptr, d_initial_zero_final, nullptr, nullptr, as_stream(stream));
}

int slx_v2x2ssd_bwd_finish(const slx_scan_shape *s, const void *U, const float *M, const float *K, const void *B,
                           const void *C, const float *B_prev, const float *U_prev, const void *chunk_starts,
                           const float *m_chunk, const float *final_state, const void *dY, const float *d_final,
                           void *dU, float *dM, float *dK, void *dB, void *dC, float *d_initial, float *dB_prev,
                           float *dU_prev, void *workspace, size_t workspace_bytes, void *stream) {
  return v2x2ssd_bwd_impl(s, U, M, K, B, C, B_prev, U_prev, chunk_starts, m_chunk, final_state, dY, d_final, dU, dM,
                          dK, dB, dC, d_initial, dB_prev, dU_prev, workspace, workspace_bytes, stream, true);
}

}  // extern "C"
