// Self-test of the tcgen05 tile engine (umma.cuh): small single-CTA products in
// every operand arrangement the scan kernels use, checked by the tests against a
// plain matrix product.  Diagnostic entry point; not on any hot path.
#include "../common.cuh"
#include "../umma.cuh"

namespace slx {

// copy a row-major [rows][64] bf16 block (leading dimension ld elements) into a swizzled tile
__device__ __forceinline__ void load_tile_swz(unsigned char *tile, const __nv_bfloat16 *src, int ld, int rows) {
  for (int idx = threadIdx.x; idx < rows * 8; idx += blockDim.x) {
    int r = idx >> 3, j = idx & 7;
    uint4 v = *reinterpret_cast<const uint4 *>(src + (size_t)r * ld + j * 8);
    *reinterpret_cast<uint4 *>(tile + umma::swz_off(r, j)) = v;
  }
}

// mode 0: C[128x128] = A[128x64] * B[128x64]^T          (A, B K-major)
// mode 1: C[128x64]  = A[128x128] * B[128x64]           (A K-major in two blocks, B MN-major)
// mode 2: C[128x64]  = A[128x128]^T * B[128x64]         (A MN-major in two blocks, B MN-major)
// mode 3: C[128x64]  = A[128x64] * B[64x64]^T           (A, B K-major, N = 64)
__global__ void __launch_bounds__(128) umma_selftest_kernel(int mode, const __nv_bfloat16 *A, const __nv_bfloat16 *B,
                                                            float *C, int *status) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base = reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *tA = base;              // up to two [128][64] tiles (32 KB)
  unsigned char *tB = base + 32768;      // up to [128][64] (16 KB)
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_slot;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
  if (threadIdx.x == 0) {
    umma::mbar_init(umma::smem_u32(&mbar), 1);
    umma::fence_mbar_init();
  }
  if (mode == 0 || mode == 3) {
    load_tile_swz(tA, A, 64, 128);
    load_tile_swz(tB, B, 64, mode == 0 ? 128 : 64);
  } else {
    load_tile_swz(tA, A, 128, 128);
    load_tile_swz(tA + 16384, A + 64, 128, 128);
    load_tile_swz(tB, B, 64, 128);
  }
  umma::fence_smem_to_async();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const int N = (mode == 0) ? 128 : 64;
  if (threadIdx.x == 0) {
    const uint32_t sa = umma::smem_u32(tA), sb = umma::smem_u32(tB);
    if (mode == 0 || mode == 3) {
      const uint32_t idesc = umma::make_idesc(128, N, false, false, 1);
      for (int kk = 0; kk < 4; ++kk)
        umma::mma_ss(tmem, umma::desc_kmajor(sa, kk), umma::desc_kmajor(sb, kk), idesc, kk > 0);
    } else if (mode == 1) {
      const uint32_t idesc = umma::make_idesc(128, 64, false, true, 1);
      for (int kk = 0; kk < 8; ++kk)
        umma::mma_ss(tmem, umma::desc_kmajor(sa + 16384u * (kk >> 2), kk & 3), umma::desc_mnmajor(sb, kk, 0), idesc,
                     kk > 0);
    } else {
      const uint32_t idesc = umma::make_idesc(128, 64, true, true, 1);
      for (int kk = 0; kk < 8; ++kk)
        umma::mma_ss(tmem, umma::desc_mnmajor(sa, kk, 16384u), umma::desc_mnmajor(sb, kk, 0), idesc, kk > 0);
    }
    umma::commit(umma::smem_u32(&mbar));
  }
  bool ok = umma::mbar_wait(umma::smem_u32(&mbar), 0);
  umma::fence_after_sync();
  if (!ok && lane == 0) atomicExch(status, 1);
  if (ok) {
    const int row = 32 * warp + lane;
    for (int c0 = 0; c0 < N; c0 += 32) {
      float v[32];
      umma::tmem_ld32(umma::tmem_addr(tmem, 32 * warp, c0), v);
#pragma unroll
      for (int i = 0; i < 32; ++i) C[(size_t)row * N + c0 + i] = v[i];
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 0) umma::tmem_dealloc(tmem, 128);
}

}  // namespace slx

extern "C" int slx_umma_selftest(int mode, const void *A, const void *B, float *C, int *status, void *stream) {
  using namespace slx;
  SLX_REQUIRE(mode >= 0 && mode <= 3, SLX_E_SHAPE, "umma_selftest: mode %d not in 0..3", mode);
  SLX_REQUIRE(A && B && C && status, SLX_E_NULL, "umma_selftest: NULL pointer");
  const size_t smem = 49152 + 1024;
  cudaError_t e = cudaFuncSetAttribute(umma_selftest_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  if (e != cudaSuccess) return fail((int)e, "umma_selftest smem attribute: %s", cudaGetErrorString(e));
  umma_selftest_kernel<<<1, 128, smem, as_stream(stream)>>>(mode, (const __nv_bfloat16 *)A, (const __nv_bfloat16 *)B, C,
                                                           status);
  return check_launch("umma_selftest");
}

extern "C" const char *slx_selftest_last_error_string(void) { return slx::g_err; }
