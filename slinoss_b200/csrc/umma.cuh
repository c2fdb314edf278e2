// Blackwell (sm_100a) tensor-core tile primitives in inline PTX: tcgen05.mma
// with shared-memory operand descriptors, TMEM allocation and loads, mbarrier
// completion with bounded waits.
//
// Shared-memory operand tiles are always [R rows][64 halfs] with 128-byte rows,
// stored with the 128-byte swizzle (16-byte chunk index XOR row%8) at a
// 1024-byte aligned base.  Such a tile is, without any data movement,
//   * a K-major operand   (rows = M/N index, the 64 columns = 4 K-steps of 16), or
//   * an MN-major operand (rows = K index, the 64 columns = 64 M/N indices).
// Wider matrices are split into 64-column blocks, each one such tile.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

namespace slx {
namespace umma {

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
  return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- descriptors ------------------------------------------------------------
// 64-bit shared-memory matrix descriptor, SWIZZLE_128B, sm_100 version field.
__device__ __forceinline__ uint64_t make_desc(uint32_t saddr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((saddr & 0x3FFFFu) >> 4);
  d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3FFFu) << 16;
  d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3FFFu) << 32;
  d |= static_cast<uint64_t>(1) << 46;  // descriptor version (Blackwell)
  d |= static_cast<uint64_t>(2) << 61;  // SWIZZLE_128B
  return d;
}
// K-major view of a [R][64] tile: K-step kk (16 halfs = 32 bytes) of the block.
__device__ __forceinline__ uint64_t desc_kmajor(uint32_t tile_saddr, int kk) {
  return make_desc(tile_saddr + 32u * kk, 16u, 1024u);
}
// MN-major view: K-step kk = rows [16kk, 16kk+16); MN blocks of 64 are
// block_stride_bytes apart (irrelevant when the MN extent is 64).
__device__ __forceinline__ uint64_t desc_mnmajor(uint32_t tile_saddr, int kk, uint32_t block_stride_bytes) {
  return make_desc(tile_saddr + 2048u * kk, block_stride_bytes, 1024u);
}

// Descriptor of the same tile view advanced by `bytes` (a multiple of 16): only the
// 14-bit start-address field changes, so this is one 64-bit add.
__device__ __forceinline__ uint64_t desc_advance(uint64_t desc, uint32_t bytes) { return desc + (bytes >> 4); }
constexpr uint32_t kStepK = 32;     // K-major: next K-step of 16 halfs inside a 64-column tile
constexpr uint32_t kStepMN = 2048;  // MN-major: next K-step = 16 rows of 128 bytes

// 32-bit instruction descriptor for kind::f16 with fp32 accumulation.
// fmt: 0 = fp16 operands, 1 = bf16 operands.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, bool a_mn_major, bool b_mn_major, int fmt) {
  return (1u << 4) | (static_cast<uint32_t>(fmt) << 7) | (static_cast<uint32_t>(fmt) << 10) |
         ((a_mn_major ? 1u : 0u) << 15) | ((b_mn_major ? 1u : 0u) << 16) |
         (static_cast<uint32_t>(N >> 3) << 17) | (static_cast<uint32_t>(M >> 4) << 24);
}

template <typename T>
struct HalfFmt;
template <>
struct HalfFmt<__half> {
  static constexpr int value = 0;
};
template <>
struct HalfFmt<__nv_bfloat16> {
  static constexpr int value = 1;
};

// ---- issue / completion -------------------------------------------------------
// D[tmem] (+)= A * B, issued by ONE thread.
__device__ __forceinline__ void mma_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc,
                                       uint32_t accumulate) {
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "setp.ne.b32 p, %4, 0;\n\t"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t"
      "}\n" ::"r"(tmem_d),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
      : "memory");
}
// Arrive on an mbarrier once every MMA issued so far by this thread has completed.
__device__ __forceinline__ void commit(uint32_t mbar_saddr) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(mbar_saddr)
               : "memory");
}
__device__ __forceinline__ void fence_before_sync() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_after_sync() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
// make generic-proxy shared-memory writes visible to the tensor-core (async) proxy
__device__ __forceinline__ void fence_smem_to_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

__device__ __forceinline__ void mbar_init(uint32_t mbar_saddr, uint32_t count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(mbar_saddr), "r"(count) : "memory");
}
__device__ __forceinline__ void fence_mbar_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }

// ---- TMA (bulk tensor copies into swizzled shared-memory tiles) -----------------------------
// The 128-byte swizzle of a tiled copy is the layout swz_off() describes, so a [rows][64 half]
// box lands ready to be a tcgen05 operand.  Rows outside the tensor are filled with zeros.
// The x coordinate times the element size must be a multiple of 16 bytes.
__device__ __forceinline__ void mbar_expect_tx(uint32_t mbar_saddr, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(mbar_saddr), "r"(bytes) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst_saddr, const void *tensor_map, int x, int y, int z,
                                            uint32_t mbar_saddr) {
  asm volatile(
      "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
      ::"r"(dst_saddr), "l"(reinterpret_cast<uint64_t>(tensor_map)), "r"(x), "r"(y), "r"(z), "r"(mbar_saddr)
      : "memory");
}
__device__ __forceinline__ void tma_prefetch_map(const void *tensor_map) {
  asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(tensor_map)) : "memory");
}

// ---- pieces of the warp-specialised (producer / issuer / worker) kernels ---------------------------
__device__ __forceinline__ void mbar_arrive(uint32_t mbar_saddr) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(mbar_saddr) : "memory");
}
// Bulk tensor store of a swizzled shared-memory tile (rows outside the tensor are not written).
// Never give it a negative coordinate.
__device__ __forceinline__ void tma_store_3d(const void *tensor_map, int x, int y, int z, uint32_t src_saddr) {
  asm volatile("cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%1, %2, %3}], [%4];" ::"l"(
                   reinterpret_cast<uint64_t>(tensor_map)),
               "r"(x), "r"(y), "r"(z), "r"(src_saddr)
               : "memory");
}
__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// the issuing thread's earlier bulk stores have finished READING shared memory
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }

// Wait on an mbarrier phase inside a kernel whose warps play different roles.  What was measured on B200
// (clock stamps per phase, same kernels, only the wait changed):
//   * every thread of 16 warps parked in the blocking try_wait on one barrier: each synchronisation cost
//     about 2.5 K cycles (the parked threads are released one after the other);
//   * a spin on the non-blocking test_wait, or try_wait with a 100 ns suspend hint (which returns at once
//     and so spins as well): the pollers take shared-memory atomics and issue slots from the warps that are
//     still working; every phase ran two to five times slower;
//   * ONE lane per warp parked in the blocking try_wait, the other lanes held at the warp's convergence
//     barrier: what is used here.
// Gives up after `limit` clocks (about 0.2 s by default), and at once when another role has already given
// up: *abort_flag (shared memory) is set by the first wait that runs out and read by all others, so that a
// fault in one role ends the whole CTA within one timeout instead of one per wait.
__device__ __forceinline__ bool mbar_test(uint32_t mbar_saddr, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n\t"
      ".reg .pred p;\n\t"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
      "selp.b32 %0, 1, 0, p;\n\t"
      "}\n"
      : "=r"(done)
      : "r"(mbar_saddr), "r"(parity)
      : "memory");
  return done != 0;
}
// one thread waits (producer / issuer lanes)
__device__ __forceinline__ bool mbar_wait_abortable(uint32_t mbar_saddr, uint32_t parity, volatile int *abort_flag,
                                                    long long limit = 400000000LL) {
  long long t0 = 0;
  if (*abort_flag) return false;
  for (int spin = 0;; ++spin) {
    if (mbar_test(mbar_saddr, parity)) return true;
    __nanosleep(40);  // keep the poll off the shared-memory pipe that the working warps need
    if ((spin & 15) == 15) {
      if (*abort_flag) return false;
      if (t0 == 0) t0 = clock64();
      else if (clock64() - t0 > limit) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}
// a whole (converged) warp waits: lane 0 polls, the result is broadcast, and every lane then observes the
// completed phase itself with one test (which is what makes the data written by the asynchronous proxy
// visible to it)
__device__ __forceinline__ bool mbar_wait_warp(uint32_t mbar_saddr, uint32_t parity, volatile int *abort_flag) {
  int ok = 1;
  if ((threadIdx.x & 31) == 0) ok = mbar_wait_abortable(mbar_saddr, parity, abort_flag) ? 1 : 0;
  ok = __shfl_sync(0xffffffffu, ok, 0);
  if (ok) (void)mbar_test(mbar_saddr, parity);
  return ok != 0;
}

// i * v on a packed pair (re, im) of halfs: (re, im) -> (-im, re).  One byte permute and one xor;
// works for bf16 and fp16 alike (sign in the top bit).
__device__ __forceinline__ uint32_t jword(uint32_t w) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %1, 0x1032;" : "=r"(r) : "r"(w));
  return r ^ 0x00008000u;
}
__device__ __forceinline__ uint4 jchunk(uint4 v) { return make_uint4(jword(v.x), jword(v.y), jword(v.z), jword(v.w)); }

// Bounded wait: gives up after about a second of SM clock and reports failure
// instead of spinning forever (each try_wait poll blocks for a short
// hardware-defined time by itself).
__device__ __forceinline__ bool mbar_wait(uint32_t mbar_saddr, uint32_t parity) {
  const long long t0 = clock64();
  for (;;) {
    uint32_t done;
    asm volatile(
        "{\n\t"
        ".reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t"
        "}\n"
        : "=r"(done)
        : "r"(mbar_saddr), "r"(parity)
        : "memory");
    if (done) return true;
    if (clock64() - t0 > 2000000000LL) return false;
  }
}

// ---- tensor memory ----------------------------------------------------------------
// One full warp allocates `ncols` (power of two >= 32) columns; the base address
// is written to *slot (shared memory).
__device__ __forceinline__ void tmem_alloc(uint32_t *slot, uint32_t ncols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(ncols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, uint32_t ncols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(ncols) : "memory");
}

// Each thread of the warp reads 32 consecutive fp32 columns of its own lane
// (lane = 32*(warp%4) + laneid must be encoded in taddr bits 31..16 by the caller).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float (&v)[32]) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
      "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
}
// 16-column variant of tmem_ld32
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}
// Split form: several loads are issued back to back and waited for once.  The wait takes the
// destination registers as read-write operands so that no use of them can be scheduled above it;
// the first wait covers every outstanding load, the following ones return at once.
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t (&r)[16]) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];\n"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld16_wait(uint32_t (&r)[16]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7]),
                 "+r"(r[8]), "+r"(r[9]), "+r"(r[10]), "+r"(r[11]), "+r"(r[12]), "+r"(r[13]), "+r"(r[14]), "+r"(r[15])
               :
               : "memory");
}
// 8-column variants
__device__ __forceinline__ void tmem_ld8_issue(uint32_t taddr, uint32_t (&r)[8]) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}
__device__ __forceinline__ void tmem_ld8_wait(uint32_t (&r)[8]) {
  asm volatile("tcgen05.wait::ld.sync.aligned;"
               : "+r"(r[0]), "+r"(r[1]), "+r"(r[2]), "+r"(r[3]), "+r"(r[4]), "+r"(r[5]), "+r"(r[6]), "+r"(r[7])
               :
               : "memory");
}
__device__ __forceinline__ uint32_t tmem_addr(uint32_t base, int lane, int col) {
  return base + (static_cast<uint32_t>(lane) << 16) + static_cast<uint32_t>(col);
}

// ---- swizzled shared-memory tile access -----------------------------------------------
// byte offset of 16-byte chunk j (0..7) of row r inside a [R][64] swizzled tile
__device__ __forceinline__ uint32_t swz_off(int r, int j) {
  return static_cast<uint32_t>(r) * 128u + (static_cast<uint32_t>(j ^ (r & 7)) << 4);
}

__device__ __forceinline__ uint32_t pack2(float lo, float hi, __nv_bfloat16) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi, __half) {
  __half2 v = __floats2half2_rn(lo, hi);
  return *reinterpret_cast<uint32_t *>(&v);
}
__device__ __forceinline__ float2 unpack2(uint32_t w, __nv_bfloat16) {
  return __bfloat1622float2(*reinterpret_cast<__nv_bfloat162 *>(&w));
}
__device__ __forceinline__ float2 unpack2(uint32_t w, __half) {
  return __half22float2(*reinterpret_cast<__half2 *>(&w));
}

}  // namespace umma
}  // namespace slx
