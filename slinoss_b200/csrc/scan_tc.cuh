// Tensor-core (tcgen05 / TMEM) chunk kernels of the v2x2ssd scan for half
// inputs with fp32 state: chunk length 128, head dim 64, state width D = 2N a
// multiple of 64 up to 256.  One CTA per (chunk, batch*head).
//
// Same merged-tap formulation as scan_simt.cuh.  Operands are rotated/weighted on
// CUDA cores (fp32), rounded to the activation dtype and written into swizzled
// [rows][64] shared-memory tiles that tcgen05.mma consumes in place; all
// accumulators live in tensor memory and are read back once per tile.
#pragma once

#include <cuda.h>

#include "scan_simt.cuh"
#include "umma.cuh"

namespace slx {

// tensor maps of the raw C and B operands: (D, T, BH), boxes of 64 columns x 128 tokens, 128-byte swizzle
struct alignas(64) ScanTileMaps {
  CUtensorMap C, B;
};

__device__ int g_tc_status = 0;  // becomes non-zero when a bounded wait ran out
// Phase-clock stamps (clock64() of the CTA in the middle of the grid, i.e. of a steady-state wave, at the
// phase boundaries) exist only in builds with
// -DSLX_DIAG; the shipped library carries none.
#ifdef SLX_DIAG
__device__ long long g_phase_clock[128];
#define SLX_DIAG_STAMP(i) SLX_DIAG_STAMP_T(i, 0)
#define SLX_DIAG_STAMP_T(i, t) do { if (blockIdx.x == gridDim.x / 2 && blockIdx.y == gridDim.y / 2 && threadIdx.x == (t)) g_phase_clock[i] = clock64(); } while (0)
#else
#define SLX_DIAG_STAMP(i) do { } while (0)
#define SLX_DIAG_STAMP_T(i, t) do { } while (0)
#endif

constexpr int kTcL = 128;
constexpr int kTcP = 64;
constexpr int kTcThreads = 256;

// coef * (4 packed complex values) -> 4 packed complex values in T.
// fp32 rotation, one rounding to T: used wherever the gradient identities rely on
// consistently rounded operands (the packed variant above costs ~1e-2 on dM)
template <typename T>
__device__ __forceinline__ uint4 rotate_chunk(uint4 raw, float2 coef) {
  const uint32_t *w = reinterpret_cast<const uint32_t *>(&raw);
  uint4 out;
  uint32_t *o = reinterpret_cast<uint32_t *>(&out);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 v = umma::unpack2(w[i], T());
    float2 r = cmul(coef, v);
    o[i] = umma::pack2(r.x, r.y, T());
  }
  return out;
}
// acc += sum_i conj(a_i) * b_i over the 4 packed complex values of two chunks
template <typename T>
__device__ __forceinline__ void cdot_chunk(uint4 a, uint4 b, float2 &acc) {
  const uint32_t *wa = reinterpret_cast<const uint32_t *>(&a);
  const uint32_t *wb = reinterpret_cast<const uint32_t *>(&b);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = umma::unpack2(wa[i], T()), y = umma::unpack2(wb[i], T());
    acc.x = fmaf(x.x, y.x, fmaf(x.y, y.y, acc.x));
    acc.y = fmaf(x.x, y.y, fmaf(-x.y, y.x, acc.y));
  }
}
__device__ __forceinline__ float2 octet_sum(float2 v) {  // sum over the 8 lanes that share a tile row
#pragma unroll
  for (int off = 4; off > 0; off >>= 1) {
    v.x += __shfl_xor_sync(0xffffffffu, v.x, off);
    v.y += __shfl_xor_sync(0xffffffffu, v.y, off);
  }
  return v;
}
template <typename T>
__device__ __forceinline__ uint4 pack8(const float *v) {
  uint4 out;
  out.x = umma::pack2(v[0], v[1], T());
  out.y = umma::pack2(v[2], v[3], T());
  out.z = umma::pack2(v[4], v[5], T());
  out.w = umma::pack2(v[6], v[7], T());
  return out;
}

// Decay, causal mask and diagonal of one 32-column block of a score tile:
//   v[i] <- v[i] exp(lp_row - lp_{s+1})  for s = c0 + i < row,   diag  for s == row,   0 above.
// FAST factors the exponential as exp(lp_row - lp_{c0+1}) * e2[s] with the per-chunk table
//   e2[s] = exp(lp_{b+1} - lp_{s+1}),  b = 32 (s / 32),
// one exponential per thread instead of one per element.  The table cannot overflow while
// every per-token log-magnitude lies in [-1.9, 0.5] (31 * 1.9 < 88); chunks outside that
// range take the per-element path (decay_table_ok is evaluated once per chunk).
__device__ __forceinline__ bool decay_step_out_of_range(const float *lp, int t) {
  const float lg = lp[t] - (t > 0 ? lp[t - 1] : 0.f);
  return lg < -1.9f || lg > 0.5f;
}
__device__ __forceinline__ float decay_table_entry(const float *lp, int s, int L) {
  return (s + 1 < L) ? __expf(lp[32 * (s >> 5) + 1] - lp[s + 1]) : 0.f;
}
template <bool FAST>
__device__ __forceinline__ void decay_mask32(float (&v)[32], int c0, int row, float lp_row, const float *lp,
                                             const float *e2, float diag) {
  const float rf = FAST ? __expf(lp_row - lp[c0 + 1]) : 0.f;
#pragma unroll
  for (int i = 0; i < 32; ++i) {
    const int s = c0 + i;
    const float f = FAST ? rf * e2[s] : __expf(lp_row - lp[min(s + 1, kTcL - 1)]);
    v[i] = (s < row) ? v[i] * f : (s == row ? diag : 0.f);
  }
}

constexpr size_t scan_fwd_tc_smem_bytes() { return 1024 + 88 * 1024 + 12 * 1024; }

// Forward chunk scan (replaces reference.py:1059 chunk_scan) on tensor cores.
//   S  = Qbar kappa^T          (128 x 128, K = D)       tcgen05, fp32 in TMEM
//   Yo = Qbar Z0^T             (128 x 64,  K = D)       (one product with S: N = 192)
//   Yd = S' U                  (128 x 64,  K = 128),  S' = masked/decayed S (+ diagonal)
//   Y  = Yd + exp(lp_t) Yo;  the token in front of the chunk takes source slot 127 of S' / U, token 127's own
//        diagonal term is added by hand
template <typename T>
__global__ void __launch_bounds__(kTcThreads, 2) chunk_scan_fwd_tc_kernel(ScanFwdArgs<T> a) {
  constexpr int L = kTcL, P = kTcP;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *tQ = base;               // [128][64]  Qbar slab   (also the Y staging tile)
  unsigned char *tK = base + 16384;       // [128][64]  kappa slab
  unsigned char *tS = base;               // 2 x [128][64]  S' (over the Qbar and kappa tiles, idle by then)
  unsigned char *tZ = base + 32768;       // [64][64]   Z0 slab, right behind kappa: [kappa ; Z0] is ONE 192-row B operand
  unsigned char *tU = base + 40960;       // [128][64]  U
  unsigned char *sC = base + 57344;       // raw C slab, filled by cp.async one slab ahead
  unsigned char *sB = base + 73728;       // raw B slab
  float *lp = reinterpret_cast<float *>(base + 90112);  // 128
  float2 *ph = reinterpret_cast<float2 *>(lp + L);      // 128 each from here
  float2 *mraw = ph + L, *kc = mraw + L, *kp = kc + L, *gk = kp + L, *cbv = gk + L;
  float2 *bm1 = cbv + L;                                 // 128 (b_{-1}, all of D)
  float *um1 = reinterpret_cast<float *>(bm1 + 128);     // 64
  float *e2 = um1 + 64;                                  // 128: decay table (decay_mask32)
  unsigned char *u127 = reinterpret_cast<unsigned char *>(e2 + L);  // 128 bytes: token 127's own u row
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_slot;

  const ScanDims d = a.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int t0 = c * L;
  const int valid = min(L, d.T - t0);
  const size_t tok0 = (size_t)bh * d.T + t0;
  const int NB = d.D / 64;
  const uint32_t mbar_s = umma::smem_u32(&mbar);
  const int j = tid & 7, r0 = tid >> 3;  // staging: 16-byte chunk j of rows r0 + 32 i
  // on this path the chunk-start states are stored in the activation dtype (api: slx_scan_starts_dtype)
  const T *z0 = reinterpret_cast<const T *>(a.starts) + ((size_t)bh * d.NC + c) * P * d.D;
  auto prefetch_cb = [&](int sl) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + 32 * i;
      const int rr = r < valid ? r : 0;
      const uint32_t nbytes = r < valid ? 16u : 0u;
      const size_t g = (tok0 + rr) * d.D + sl * 64 + 8 * j;
      const uint32_t off = umma::swz_off(r, j);
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(sC + off)), "l"(a.C + g),
                   "r"(nbytes)
                   : "memory");
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(sB + off)), "l"(a.B + g),
                   "r"(nbytes)
                   : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  uint4 zr[2];
  auto prefetch_z = [&](int sl) {
#pragma unroll
    for (int k2 = 0; k2 < 2; ++k2) {
      const int q = tid + kTcThreads * k2;
      zr[k2] = *reinterpret_cast<const uint4 *>(z0 + (size_t)(q >> 3) * d.D + sl * 64 + 8 * (q & 7));
    }
  };
  float2 mreg[4];  // the prefix warp's multipliers, requested ahead of the bulk copies
  if ((tid >> 5) == 2) chunk_prefix_load4(a.M + tok0 * 2, valid, mreg);
  // U tile straight into its operand tile (no transform needed), same commit group as slab 0
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 32 * i;
    const int rr = r < valid ? r : 0;
    const uint32_t nbytes = r < valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(tU + umma::swz_off(r, j))),
                 "l"(a.U + (tok0 + rr) * P + 8 * j), "r"(nbytes)
                 : "memory");
  }
  prefetch_cb(0);
  prefetch_z(0);

#define SLX_FSTAMP(i) SLX_DIAG_STAMP(64 + (i))
  SLX_FSTAMP(0);
  if (warp == 0) umma::tmem_alloc(&tmem_slot, 256);
  if (tid == 32) {
    umma::mbar_init(mbar_s, 1);
    umma::fence_mbar_init();
  }
  if (warp == 2) chunk_prefix_fast128(mreg, lp, ph, mraw, &g_scan_bad);
  if (tid >= 128) {
    int t = tid - 128;
    float2 vp = make_float2(0.f, 0.f), vc = vp;
    if (t < valid) {
      float4 k4 = *reinterpret_cast<const float4 *>(a.K + (tok0 + t) * 4);
      vp = make_float2(k4.x, k4.y);
      vc = make_float2(k4.z, k4.w);
    }
    kp[t] = vp;
    kc[t] = vc;
  } else if (tid >= 64) {
    int p = tid - 64;
    float v = 0.f;
    if (t0 > 0) v = to_f(a.U[(tok0 - 1) * P + p]);
    else if (a.Uprev) v = a.Uprev[(size_t)bh * P + p];
    um1[p] = v;
  }
  if (tid < d.N) {
    float2 bv = make_float2(0.f, 0.f);
    if (t0 > 0) bv = load_pair<T>(a.B + (tok0 - 1) * d.D + 2 * tid);
    else if (a.Bprev) bv = *reinterpret_cast<const float2 *>(a.Bprev + (size_t)bh * d.D + 2 * tid);
    bm1[tid] = bv;
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (tid < L) {
    int t = tid;
    // gamma_t conj(phi_{t+1}); slot 127 (no query follows the last token, so its column is free) carries the
    // token in front of the chunk: kappa[127] = k^p_0 conj(phi_0) b_{-1}
    float2 g = cmulc(kp[0], ph[0]);
    if (t + 1 < L) g = cmulc(cadd(cmul(mraw[t + 1], kc[t]), kp[t + 1]), ph[t + 1]);
    gk[t] = g;
    e2[t] = decay_table_entry(lp, t, L);
  }
  const bool fast_decay = !__syncthreads_or(tid < L && decay_step_out_of_range(lp, tid));

  const uint32_t sQ = umma::smem_u32(tQ), sK = umma::smem_u32(tK), sU = umma::smem_u32(tU), sS = umma::smem_u32(tS);
  constexpr int fmt = umma::HalfFmt<T>::value;
  float2 acc_cb[4];
#pragma unroll
  for (int i = 0; i < 4; ++i) acc_cb[i] = make_float2(0.f, 0.f);
  uint32_t phase = 0;
  bool ok = true;

  SLX_FSTAMP(1);
  for (int sl = 0; sl < NB; ++sl) {
    SLX_FSTAMP(8 + 4 * sl);
    // this slab's raw C, B arrived through cp.async (issued one slab ahead)
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (sl > 0) {
      ok = umma::mbar_wait(mbar_s, phase) && ok;  // previous slab's products are done: tiles are free
      phase ^= 1;
    } else if (r0 == 31) {
      // source slot 127 of S' is the token in front of the chunk: its row of the U tile (which this thread
      // copied in) becomes u_{-1}; token 127's own diagonal term is added by hand in the epilogue
      float tmp[8];
#pragma unroll
      for (int e = 0; e < 8; ++e) tmp[e] = um1[8 * j + e];
      uint4 *cell = reinterpret_cast<uint4 *>(tU + umma::swz_off(L - 1, j));
      *reinterpret_cast<uint4 *>(u127 + 16 * j) = *cell;  // kept for the epilogue
      *cell = pack8<T>(tmp);
    }
    uint4 cr[4], br[4];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint32_t off = umma::swz_off(r0 + 32 * i, j);
      cr[i] = *reinterpret_cast<const uint4 *>(sC + off);
      br[i] = *reinterpret_cast<const uint4 *>(sB + off);
    }
    SLX_FSTAMP(9 + 4 * sl);
    // b_{-1} chunk of this slab: only the threads that stage row 127 (the boundary slot) need it
    uint4 bm = make_uint4(0, 0, 0, 0);
    if (r0 == 31) {
      float tmp[8];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float2 v = bm1[sl * 32 + 4 * j + e];
        tmp[2 * e] = v.x;
        tmp[2 * e + 1] = v.y;
      }
      bm = pack8<T>(tmp);
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      int r = r0 + 32 * i;
      *reinterpret_cast<uint4 *>(tQ + umma::swz_off(r, j)) = rotate_chunk<T>(cr[i], cconj(ph[r]));
      *reinterpret_cast<uint4 *>(tK + umma::swz_off(r, j)) = rotate_chunk<T>(r == L - 1 ? bm : br[i], gk[r]);
      cdot_chunk<T>(cr[i], br[i], acc_cb[i]);
    }
#pragma unroll
    for (int k = 0; k < 2; ++k) {
      int q = tid + kTcThreads * k;
      int p = q >> 3, jj = q & 7;
      *reinterpret_cast<uint4 *>(tZ + umma::swz_off(p, jj)) = zr[k];
    }
    // Every thread has consumed its own raw slots (it alone wrote and read them) and its Z0
    // registers: request the next slab now, a whole staging phase ahead of its use.
    if (sl + 1 < NB) {
      prefetch_cb(sl + 1);
      prefetch_z(sl + 1);
    }
    umma::fence_smem_to_async();
    SLX_FSTAMP(10 + 4 * sl);
    __syncthreads();
    SLX_FSTAMP(11 + 4 * sl);
    if (tid == 0) {
      umma::fence_after_sync();
      // [S | Yo] = Qbar [kappa ; Z0]^T as one product of N = 192 per K-step: Qbar is fetched once for both, and at
      // this width the fetches fit under the product's own time (two products of N = 128 and N = 64 do not)
      const uint32_t id_so = umma::make_idesc(128, 192, false, false, fmt);
#pragma unroll
      for (int kk = 0; kk < 4; ++kk)
        umma::mma_ss(tmem + 0, umma::desc_kmajor(sQ, kk), umma::desc_kmajor(sK, kk), id_so, (sl | kk) != 0);
      umma::commit(mbar_s);
    }
  }
  SLX_FSTAMP(2);
  // per-row dots: cb_t = <c_t, b_t>
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 s1 = octet_sum(acc_cb[i]);
    if (j == 0) cbv[r0 + 32 * i] = s1;
  }
  ok = umma::mbar_wait(mbar_s, phase) && ok;
  phase ^= 1;
  umma::fence_after_sync();
  __syncthreads();

  SLX_FSTAMP(3);
  // ---- S -> S' (decay, causal mask, diagonal) -> bf16 A operand ----------------------
  const int q4 = warp & 3, h = warp >> 2;
  const int t = 32 * q4 + lane;
  const float lpt = lp[t];
  {
    const float dg = kc[t].x * cbv[t].x - kc[t].y * cbv[t].y;  // Re(k^c_t <c_t,b_t>)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int c0 = 64 * h + 32 * half;
      float v[32];
      const bool last = c0 == 96;  // the block that holds column 127, the boundary slot
      if (c0 <= 32 * q4 + 31 || last) {
        umma::tmem_ld32(umma::tmem_addr(tmem, 32 * q4, c0), v);
        const float s127 = v[31];
        if (c0 <= 32 * q4 + 31) {
          if (fast_decay) decay_mask32<true>(v, c0, t, lpt, lp, e2, dg);
          else decay_mask32<false>(v, c0, t, lpt, lp, e2, dg);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) v[i] = 0.f;
        }
        // column 127: <Qbar_t, k^p_0 conj(phi_0) b_{-1}> exp(lp_t - lp_0), the term of the token in front of the
        // chunk, for every row (row 127 loses its diagonal entry here: added in the epilogue)
        if (last) v[31] = s127 * __expf(lpt - lp[0]);
      } else {
#pragma unroll
        for (int i = 0; i < 32; ++i) v[i] = 0.f;
      }
#pragma unroll
      for (int k = 0; k < 4; ++k)
        *reinterpret_cast<uint4 *>(tS + 16384 * h + umma::swz_off(t, 4 * half + k)) = pack8<T>(v + 8 * k);
    }
  }
  umma::fence_smem_to_async();
  umma::fence_before_sync();
  SLX_FSTAMP(4);
  __syncthreads();
  if (tid == 0) {
    umma::fence_after_sync();
    const uint32_t id_y = umma::make_idesc(128, 64, false, true, fmt);
#pragma unroll
    for (int kk = 0; kk < 8; ++kk)
      umma::mma_ss(tmem + 192, umma::desc_kmajor(sS + 16384u * (kk >> 2), kk & 3), umma::desc_mnmajor(sU, kk, 0), id_y,
                   kk != 0);
    umma::commit(mbar_s);
  }
  ok = umma::mbar_wait(mbar_s, phase) && ok;
  phase ^= 1;
  umma::fence_after_sync();

  SLX_FSTAMP(5);
  // ---- Y = Yd + exp(lp_t) Yo (+ the diagonal term of token 127) -> staging tile -> global -------------
  {
    float yo[32], yd[32];
    umma::tmem_ld32(umma::tmem_addr(tmem, 32 * q4, 128 + 32 * h), yo);
    umma::tmem_ld32(umma::tmem_addr(tmem, 32 * q4, 192 + 32 * h), yd);
    const float el = __expf(lpt);
#pragma unroll
    for (int i = 0; i < 32; ++i) yd[i] = fmaf(el, yo[i], yd[i]);
    if (t == L - 1) {  // token 127's diagonal term (zero for a row past the end of the sequence: c, b, u are zero)
      const float dg = kc[t].x * cbv[t].x - kc[t].y * cbv[t].y;  // Re(k^c_t <c_t,b_t>)
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        const uint4 ul = *reinterpret_cast<const uint4 *>(u127 + 64 * h + 16 * k);
        const uint32_t *w = reinterpret_cast<const uint32_t *>(&ul);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 uv = umma::unpack2(w[e], T());
          yd[8 * k + 2 * e] = fmaf(dg, uv.x, yd[8 * k + 2 * e]);
          yd[8 * k + 2 * e + 1] = fmaf(dg, uv.y, yd[8 * k + 2 * e + 1]);
        }
      }
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) *reinterpret_cast<uint4 *>(tQ + umma::swz_off(t, 4 * h + k)) = pack8<T>(yd + 8 * k);
  }
  umma::fence_before_sync();
  __syncthreads();
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    int r = r0 + 32 * i;
    if (r < valid)
      *reinterpret_cast<uint4 *>(a.Y + (tok0 + r) * P + 8 * j) = *reinterpret_cast<const uint4 *>(tQ + umma::swz_off(r, j));
  }
  SLX_FSTAMP(6);
  if (__syncthreads_or(!ok)) {
    // a bounded wait ran out: the rows just written came from unfinished products; overwrite them with NaN
    // so that the failure shows in the data as well as in the status word
    const T nanv = from_f<T>(__int_as_float(0x7fc00000));
    for (int e = tid; e < valid * P; e += kTcThreads) a.Y[tok0 * P + e] = nanv;
    if (tid == 0) atomicExch(&g_tc_status, 1);
  }
  if (warp == 0) umma::tmem_dealloc(tmem, 256);
#undef SLX_FSTAMP
}

// ---------------------------------------------------------------------------
// out[p, d] = sum_t A[t, p] * (coef_t x_t)[d]  (+ boundary), computed transposed
// on tensor cores: out^T (d x p) = Xop^T (d x t) * A (t x p), M = 128 state
// columns per product, N = 64, K = 128 tokens.  MODE as chunk_outer_kernel:
// 0 = chunk increment (A = U, x = B, writes m_chunk), 1 = dZ0 (A = dY, x = C).
// OT is the storage type of `out` (float, or T: the consumer is the fp32 state pass,
// whose own output is rounded to T for the chunk kernels' operands anyway).
constexpr size_t outer_tc_smem_bytes() { return 1024 + 80 * 1024 + 8 * 1024; }

template <typename T, int MODE, typename OT>
__global__ void __launch_bounds__(kTcThreads, 2) chunk_outer_tc_kernel(OuterArgs<T> a) {
  constexpr int L = kTcL, P = kTcP;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *tA = base;            // [128][64]   U or dY
  unsigned char *tX = base + 16384;    // 4 x [128][64] weighted B or C, one tile per 64 state columns
  float *lp = reinterpret_cast<float *>(base + 81920);
  float2 *ph = reinterpret_cast<float2 *>(lp + L);
  float2 *mraw = ph + L, *coef = mraw + L;
  float2 *bh1 = coef + L;                               // 128: weighted b_{-1}
  float *um1 = reinterpret_cast<float *>(bh1 + 128);    // 64
  __shared__ uint64_t mbar;
  __shared__ uint32_t tmem_slot;

  const ScanDims d = a.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int t0 = c * L;
  const int valid = min(L, d.T - t0);
  const size_t tok0 = (size_t)bh * d.T + t0;
  const int NB = d.D / 64, NG = (NB + 1) / 2;
  const uint32_t mbar_s = umma::smem_u32(&mbar);

  if (warp == 0) umma::tmem_alloc(&tmem_slot, 128);
  if (tid == 32) {
    umma::mbar_init(mbar_s, 1);
    umma::fence_mbar_init();
  }
  // Every operand byte of the chunk is requested before any arithmetic: the A tile lands in
  // place, the X slabs land raw in their operand tiles and are weighted in place by the
  // thread that requested them once the chunk's coefficients exist.
  const int j = tid & 7, r0 = tid >> 3;
  float2 mreg[4];  // the prefix warp's multipliers, requested first
  if (warp == 2) chunk_prefix_load4(a.M + tok0 * 2, valid, mreg);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = r0 + 32 * i;
    const int rr = r < valid ? r : 0;
    const uint32_t nbytes = r < valid ? 16u : 0u;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(tA + umma::swz_off(r, j))),
                 "l"(a.A + (tok0 + rr) * P + 8 * j), "r"(nbytes)
                 : "memory");
    for (int sl = 0; sl < NB; ++sl)
      asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(
                       umma::smem_u32(tX + 16384 * sl + umma::swz_off(r, j))),
                   "l"(a.X + (tok0 + rr) * d.D + sl * 64 + 8 * j), "r"(nbytes)
                   : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  // scalar inputs of the coefficient phase, requested before the prefix so that they are in
  // registers by the time it ends
  float2 kcv = make_float2(0.f, 0.f), kpn = kcv, bv = kcv;
  if (MODE == 0) {
    if (tid < L) {
      if (tid < valid) kcv = *reinterpret_cast<const float2 *>(a.K + (tok0 + tid) * 4 + 2);
      if (tid + 1 < valid) kpn = *reinterpret_cast<const float2 *>(a.K + (tok0 + tid + 1) * 4);
    } else if (tid - L < d.N) {
      const int n = tid - L;
      if (valid > 0) kpn = *reinterpret_cast<const float2 *>(a.K + tok0 * 4);
      if (t0 > 0) bv = load_pair<T>(a.X + (tok0 - 1) * d.D + 2 * n);
      else if (a.Bprev) bv = *reinterpret_cast<const float2 *>(a.Bprev + (size_t)bh * d.D + 2 * n);
    }
  }
  if (warp == 2) chunk_prefix_fast128(mreg, lp, ph, mraw, &g_scan_bad);
  if (MODE == 0 && warp == 2) {
    // chunk transition = product of the raw multipliers: four per lane, then a butterfly
    float2 acc = cmul(cmul(mraw[4 * lane], mraw[4 * lane + 1]), cmul(mraw[4 * lane + 2], mraw[4 * lane + 3]));
#pragma unroll
    for (int off = 1; off < 32; off <<= 1) {
      const float ox = __shfl_xor_sync(0xffffffffu, acc.x, off), oy = __shfl_xor_sync(0xffffffffu, acc.y, off);
      acc = cmul(acc, make_float2(ox, oy));
    }
    if (lane == 0) *reinterpret_cast<float2 *>(a.m_chunk + ((size_t)bh * d.NC + c) * 2) = acc;
  }
  if (MODE == 0 && tid >= 192) {
    int p = tid - 192;
    float v = 0.f;
    if (t0 > 0) v = to_f(a.A[(tok0 - 1) * P + p]);
    else if (a.Uprev) v = a.Uprev[(size_t)bh * P + p];
    um1[p] = v;
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  if (tid < L) {
    const int t = tid;
    float2 cf;
    if (MODE == 0) {
      if (t + 1 < L) {
        float2 gam = cadd(cmul(mraw[t + 1], kcv), kpn);
        cf = cmul(cscale(cmulc(ph[L - 1], ph[t + 1]), __expf(lp[L - 1] - lp[t + 1])), gam);
      } else {
        cf = kcv;
      }
    } else {
      cf = cscale(cconj(ph[t]), __expf(lp[t]));
    }
    coef[t] = cf;
  } else if (MODE == 0 && tid - L < d.N) {
    const int n = tid - L;
    const float2 k0p = cmul(cscale(cmulc(ph[L - 1], ph[0]), __expf(lp[L - 1] - lp[0])), kpn);
    bh1[n] = cmul(k0p, bv);
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");
  __syncthreads();
  for (int sl = 0; sl < NB; ++sl) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int r = r0 + 32 * i;
      uint4 *slot = reinterpret_cast<uint4 *>(tX + 16384 * sl + umma::swz_off(r, j));
      *slot = rotate_chunk<T>(*slot, coef[r]);
    }
  }
  umma::fence_smem_to_async();
  __syncthreads();
  if (tid == 0) {
    umma::fence_after_sync();
    const uint32_t id = umma::make_idesc(128, 64, true, true, umma::HalfFmt<T>::value);
    const uint32_t sA = umma::smem_u32(tA), sX = umma::smem_u32(tX);
    for (int g = 0; g < NG; ++g)
#pragma unroll
      for (int kk = 0; kk < 8; ++kk)
        umma::mma_ss(tmem + 64 * g, umma::desc_mnmajor(sX + 32768u * g, kk, 16384u), umma::desc_mnmajor(sA, kk, 0), id,
                     kk != 0);
    umma::commit(mbar_s);
  }
  const bool ok = umma::mbar_wait(mbar_s, 0);
  umma::fence_after_sync();
  const int q4 = warp & 3;
  OT *outc = reinterpret_cast<OT *>(a.out) + ((size_t)bh * d.NC + c) * P * d.D;
  for (int g = warp >> 2; g < NG; g += 2) {
    const int dd = 128 * g + 32 * q4 + lane;
    float v0[32], v1[32];
    umma::tmem_ld32(umma::tmem_addr(tmem, 32 * q4, 64 * g), v0);
    umma::tmem_ld32(umma::tmem_addr(tmem, 32 * q4, 64 * g + 32), v1);
    if (dd < d.D) {
      float bw = 0.f;
      if (MODE == 0) bw = (dd & 1) ? bh1[dd >> 1].y : bh1[dd >> 1].x;
      // (for half output, trading values between neighbouring lanes to store 4-byte pairs was
      // measured slower than these 2-byte stores: 0.227 against 0.203 ms at 8192 chunks)
#pragma unroll
      for (int p = 0; p < 32; ++p) {
        outc[(size_t)p * d.D + dd] = from_f<OT>((MODE == 0) ? fmaf(um1[p], bw, v0[p]) : v0[p]);
        outc[(size_t)(p + 32) * d.D + dd] = from_f<OT>((MODE == 0) ? fmaf(um1[p + 32], bw, v1[p]) : v1[p]);
      }
    }
  }
  umma::fence_before_sync();
  if (__syncthreads_or(!ok)) {  // a bounded wait ran out: NaN instead of values from an unfinished product
    const float nanf_ = __int_as_float(0x7fc00000);
    for (int e = tid; e < P * d.D; e += kTcThreads) outc[e] = from_f<OT>(nanf_);
    if (tid == 0) atomicExch(&g_tc_status, 1);
  }
  if (warp == 0) umma::tmem_dealloc(tmem, 128);
}

}  // namespace slx
