// Forward chunk scan (replaces reference.py:1059 chunk_scan) for half inputs with fp32 state,
// chunk 128, P 64, D = 2N in {64,128,192,256}: persistent, warp-specialised tcgen05 kernel.
//
// Formulation.  With the complex Gram matrix of the RAW operands
//     G[t][j] = sum_n conj(c_t[n]) b_j[n],        H[t][p] = sum_n conj(c_t[n]) z0[p][n],
// every score is  S'[t][j] = Re(w[t][j] G[t][j])  with a per-(t,j) complex weight
//     w[t][j] = exp(lp_t - lp_{j+1}) phi_t conj(phi_{j+1}) gamma_j   (j < t),    w[t][t] = k^c_t,
// and the chunk-start term is  Re(p_t H[t][p]).  Re G / Im G are two real products over the
// interleaved (re,im) columns: C B^T and (JC) B^T, where J swaps each pair and flips one sign
// (one byte permute + xor per 32-bit word).  So the D-wide operands reach the tensor cores as
// the bulk copies delivered them, and all complex arithmetic happens on the 128 x 128 tile:
//     Re part  [G | H]  = C    [B ; Z0]^T        (M 128, N 192, K = D)
//     Im part  [G | H]  = (JC) [B ; Z0]^T
//     Yd = S' U                                    (M 128, N 64,  K 128)
//     Y  = Yd + exp(lp_t) (Re phi_t ReH - Im phi_t ImH)
// The source token in front of the chunk (b_{-1}, u_{-1}) takes row 127 of the B and U tiles:
// token 127 is a source for nothing but its own diagonal term, which one warp adds by hand
// (d = Re(k^c_127 <c_127, b_127>), Y_127 += d u_127).
//
// Roles (576 threads, one CTA per SM, chunks handed out round-robin):
//   warp 16  producer: bulk tensor copies of the C, B, Z0 slabs (ring of three stages) and of U
//   warp 17  issuer:   every tcgen05.mma, completion by tcgen05.commit on mbarriers
//   warps 0-15 workers: JC transform of each slab, the score tile, the output rows
// All waits are bounded and share one abort flag; a CTA that gave up fills its remaining output
// rows with NaN and raises the device status word.
#pragma once

#include "scan_tc.cuh"

namespace slx {

struct alignas(64) WsFwdMaps {
  CUtensorMap C, B, Z, U, Y;
};

// clock64() stamps of CTA 0 while it works on its third chunk (builds with -DSLX_DIAG only)
#ifdef SLX_DIAG
#define WS_STAMP(cond, i) do { if ((cond) && blockIdx.x == 0) g_phase_clock[i] = clock64(); } while (0)
#else
#define WS_STAMP(cond, i) do { } while (0)
#endif

constexpr int kWsWorkers = 512;
constexpr int kWsThreads = kWsWorkers + 64;
constexpr int kWsStageBytes = 40960;  // one ring stage of bulk copies: C 16K | B 16K + Z0 8K
constexpr int kWsStages = 3;
constexpr int kWsFwdScal = 13312;     // per-chunk scalars and the staged rows (12,544 bytes used)
constexpr size_t scan_ws_fwd_smem_bytes() {
  return 1024 + kWsStages * kWsStageBytes + 2 * 16384 /* JC, two buffers */ + 16384 + 32768 + kWsFwdScal;
}

template <typename T>
__global__ void __launch_bounds__(kWsThreads, 1) chunk_scan_fwd_ws_kernel(ScanFwdArgs<T> a,
                                                                          const __grid_constant__ WsFwdMaps maps) {
  constexpr int L = kTcL, P = kTcP;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *tJ = base + kWsStages * kWsStageBytes;  // 2 x [128][64] JC (buffer = slab parity)
  unsigned char *tU = tJ + 2 * 16384;                    // [128][64] U (row 127 <- u_{-1})
  unsigned char *tS = tU + 16384;                // 2 x [128][64] S'; block 0 doubles as the Y staging tile
  unsigned char *sc = tS + 32768;                // scalars (kWsFwdScal bytes)
  float *lp = reinterpret_cast<float *>(sc);                 // 128
  float2 *ph = reinterpret_cast<float2 *>(lp + L);           // 128
  float2 *mraw = ph + L;                                     // 128
  float2 *gk = mraw + L;                                     // 128: g_j = gamma_j conj(phi_{j+1}); [127] = k^p_0 conj(phi_0)
  float2 *gk2 = gk + L;                                      // 128: g_j * decay-table entry
  float *u127 = reinterpret_cast<float *>(gk2 + L);          // 64
  float *misc = u127 + 64;                                   // [0] d of token 127
  float2 *Mst = reinterpret_cast<float2 *>(misc + 64);       // 2 x 128 staged M rows
  float4 *Kst = reinterpret_cast<float4 *>(Mst + 2 * L);     // 2 x 128 staged K rows
  T *bpst = reinterpret_cast<T *>(Kst + 2 * L);              // 2 x 256 staged b_{-1}
  T *upst = bpst + 2 * 256;                                  // 2 x 64 staged u_{-1}
  static_assert(512 + 4 * 1024 + 256 + 256 + 2048 + 4096 + 2 * 256 * 2 + 2 * 64 * 2 <= kWsFwdScal, "scalar area too small");
  __shared__ uint64_t bars[14];  // full[3] empty[3] jready[2] accfull sready ydone ufull tmemfree wbar
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag, slow_flag;

  const ScanDims d = a.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NB = d.D / 64;
  const int total = d.NC * d.BH;
  const uint32_t bar0 = umma::smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  enum { FULL = 0, EMPTY = 3, JREADY = 6, ACCFULL = 8, SREADY = 9, YDONE = 10, UFULL = 11, TMEMFREE = 12, WBAR = 13 };
  constexpr int fmt = umma::HalfFmt<T>::value;

  if (tid == 0) {
    for (int i = 0; i < 14; ++i) {
      const bool worker_bar = (i == JREADY || i == JREADY + 1 || i == SREADY || i == TMEMFREE || i == WBAR);
      umma::mbar_init(BAR(i), worker_bar ? 16u : 1u);
    }
    umma::fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 17) umma::tmem_alloc(&tmem_slot, 512);
  if (tid == 512) {
    umma::tma_prefetch_map(&maps.C);
    umma::tma_prefetch_map(&maps.B);
    umma::tma_prefetch_map(&maps.Z);
    umma::tma_prefetch_map(&maps.U);
  }
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  volatile int *ab = &abort_flag;
  auto WAIT = [&](int i, uint32_t parity) { return umma::mbar_wait_abortable(BAR(i), parity, ab); };  // one thread
  auto WAITW = [&](int i, uint32_t parity) { return umma::mbar_wait_warp(BAR(i), parity, ab); };        // a whole warp

  if (warp == 16) {
    // ------------------------------------------------------------------ producer
    if (lane == 0) {
      uint32_t g = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++it) {
        const int c = w % d.NC, bh = w / d.NC, t0 = c * L;
        for (int sl = 0; sl < NB && ok; ++sl, ++g) {
          const int st = g % kWsStages;
          if (g >= kWsStages) ok = WAIT(EMPTY + st, ((g / kWsStages) - 1) & 1);
          if (!ok) break;
          unsigned char *sb = base + st * kWsStageBytes;
          WS_STAMP(it == 2, 48 + sl);
          umma::mbar_expect_tx(BAR(FULL + st), 16384u + 16384u + 8192u);
          umma::tma_load_3d(umma::smem_u32(sb), &maps.C, sl * 64, t0, bh, BAR(FULL + st));
          umma::tma_load_3d(umma::smem_u32(sb + 16384), &maps.B, sl * 64, t0, bh, BAR(FULL + st));
          umma::tma_load_3d(umma::smem_u32(sb + 32768), &maps.Z, sl * 64, 0, w, BAR(FULL + st));
        }
        if (ok && it >= 1) ok = WAIT(YDONE, (it - 1) & 1);  // the previous chunk's S' U product has read the U tile
        if (!ok) break;
        umma::mbar_expect_tx(BAR(UFULL), 16384u);
        umma::tma_load_3d(umma::smem_u32(tU), &maps.U, 0, t0, bh, BAR(UFULL));
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      constexpr uint32_t id_g = umma::make_idesc(128, 192, false, false, fmt);
      constexpr uint32_t id_y = umma::make_idesc(128, 64, false, true, fmt);
      const uint32_t sS = umma::smem_u32(tS), sU = umma::smem_u32(tU);
      uint32_t g = 0, it = 0;
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++it) {
        if (it >= 1) ok = WAIT(TMEMFREE, (it - 1) & 1);  // the workers have read the previous chunk's accumulators
        umma::fence_after_sync();
        for (int sl = 0; sl < NB && ok; ++sl, ++g) {
          const int st = g % kWsStages, jb = g & 1;
          ok = WAIT(FULL + st, (g / kWsStages) & 1) && WAIT(JREADY + jb, (g >> 1) & 1);
          if (!ok) break;
          umma::fence_after_sync();
          WS_STAMP(it == 2, 32 + sl);
          const uint32_t sb = umma::smem_u32(base + st * kWsStageBytes);
          const uint64_t dC = umma::desc_kmajor(sb, 0), dBZ = umma::desc_kmajor(sb + 16384, 0),
                         dJ = umma::desc_kmajor(umma::smem_u32(tJ + 16384 * jb), 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint64_t bz = umma::desc_advance(dBZ, umma::kStepK * kk);
            umma::mma_ss(tmem + 0, umma::desc_advance(dC, umma::kStepK * kk), bz, id_g, (sl | kk) != 0);
            umma::mma_ss(tmem + 192, umma::desc_advance(dJ, umma::kStepK * kk), bz, id_g, (sl | kk) != 0);
          }
          umma::commit(BAR(EMPTY + st));
        }
        if (!ok) break;
        umma::commit(BAR(ACCFULL));
        WS_STAMP(it == 2, 36);
        ok = WAIT(SREADY, it & 1) && WAIT(UFULL, it & 1);
        if (!ok) break;
        umma::fence_after_sync();
        WS_STAMP(it == 2, 37);
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma::mma_ss(tmem + 384, umma::desc_kmajor(sS + 16384u * (kk >> 2), kk & 3), umma::desc_mnmajor(sU, kk, 0),
                       id_y, kk != 0);
        umma::commit(BAR(YDONE));
      }
    }
  } else {
    // ------------------------------------------------------------------ workers
    const int q4 = warp & 3, cb = warp >> 2, row = 32 * q4 + lane;
    const int j = tid & 7, r0 = tid >> 3;  // slab transform: 16-byte chunk j of rows r0 and r0 + 64
    // scalars of a chunk are requested one chunk ahead (per-thread asynchronous copies)
    auto prefetch_scalars = [&](int w, int buf) {
      const int c = w % d.NC, bh = w / d.NC, t0 = c * L;
      const int valid = min(L, d.T - t0);
      const size_t tok0 = (size_t)bh * d.T + t0;
      if (tid < 128) {
        const int t = tid;
        const int tt = t < valid ? t : 0;
        asm volatile("cp.async.ca.shared.global [%0], [%1], 8, %2;" ::"r"(umma::smem_u32(Mst + buf * L + t)),
                     "l"(a.M + (tok0 + tt) * 2), "r"(t < valid ? 8u : 0u)
                     : "memory");
      } else if (tid < 256) {
        const int t = tid - 128;
        const int tt = t < valid ? t : 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(Kst + buf * L + t)),
                     "l"(a.K + (tok0 + tt) * 4), "r"(t < valid ? 16u : 0u)
                     : "memory");
      } else if (tid < 256 + 32) {
        const int q = tid - 256;  // 16-byte piece of b_{-1} (32 pieces cover D = 256)
        if (8 * q < d.D) {
          const bool have = t0 > 0;
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(bpst + buf * 256 + 8 * q)),
                       "l"(a.B + (have ? (tok0 - 1) * d.D + 8 * q : 0)), "r"(have ? 16u : 0u)
                       : "memory");
        }
      } else if (tid < 256 + 40) {
        const int q = tid - 288;
        const bool have = t0 > 0;
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(upst + buf * 64 + 8 * q)),
                     "l"(a.U + (have ? (tok0 - 1) * P + 8 * q : 0)), "r"(have ? 16u : 0u)
                     : "memory");
      }
      asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if ((int)blockIdx.x < total) prefetch_scalars(blockIdx.x, 0);

    uint32_t g = 0, it = 0;
    bool ok = true;
    // Barrier among the 16 worker warps: the hardware barrier (an mbarrier-based one keeps 16 pollers on the
    // shared-memory pipe and slowed the warp that computes the prefix several times over).  A hardware barrier
    // cannot be abandoned, so a worker never leaves a chunk half way: once a wait has failed every later wait
    // returns at once (abort flag), the warps run through the rest of the chunk together and stop at its end.
    auto WSYNC = [&]() { asm volatile("bar.sync 1, 512;" ::: "memory"); };
    int w = blockIdx.x;
    for (; w < total && ok; w += gridDim.x, ++it) {
      const int c = w % d.NC, bh = w / d.NC, t0 = c * L;
      const int valid = min(L, d.T - t0);
      const int buf = it & 1;
      const bool more = w + (int)gridDim.x < total;
      WS_STAMP(it == 2 && tid == 0, 0);
      if (more) prefetch_scalars(w + gridDim.x, buf ^ 1);
      if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
      else asm volatile("cp.async.wait_group 0;" ::: "memory");
      if (tid == 0) {
        umma::tma_store_wait_read();  // the previous chunk's Y store has read the staging tile
        slow_flag = 0;
      }
      WS_STAMP(it == 2 && tid == 0, 20);
      WSYNC();
      WS_STAMP(it == 2 && tid == 0, 21);
      // ---- per-token scalars ------------------------------------------------------------------
      const float2 *Mc = Mst + buf * L;
      const float4 *Kc = Kst + buf * L;
      if (warp == 2) {
        float2 mreg[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) mreg[i] = (4 * lane + i < valid) ? Mc[4 * lane + i] : make_float2(1.f, 0.f);
        WS_STAMP(it == 2 && lane == 0, 60);
        chunk_prefix_fast128(mreg, lp, ph, mraw, &g_scan_bad);
        WS_STAMP(it == 2 && lane == 0, 61);
      }
      if (t0 == 0 && tid >= 256 && tid < 256 + 40) {  // first chunk: the streaming inputs (fp32) stand in for token -1
        if (tid < 288) {
          const int q = tid - 256;
          if (8 * q < d.D) {
            float tmp[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) tmp[e] = a.Bprev ? a.Bprev[(size_t)bh * d.D + 8 * q + e] : 0.f;
            *reinterpret_cast<uint4 *>(bpst + buf * 256 + 8 * q) = pack8<T>(tmp);
          }
        } else {
          const int q = tid - 288;
          float tmp[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) tmp[e] = a.Uprev ? a.Uprev[(size_t)bh * P + 8 * q + e] : 0.f;
          *reinterpret_cast<uint4 *>(upst + buf * 64 + 8 * q) = pack8<T>(tmp);
        }
      }
      WS_STAMP(it == 2 && tid == 0, 22);
      WSYNC();
      WS_STAMP(it == 2 && tid == 0, 23);
      if (tid < L) {
        const int t = tid;
        float2 gv;
        if (t + 1 < L) {
          const float4 k0 = Kc[t], k1 = Kc[t + 1];
          const float2 gam = cadd(cmul(mraw[t + 1], make_float2(k0.z, k0.w)), make_float2(k1.x, k1.y));
          gv = cmulc(gam, ph[t + 1]);
        } else {
          const float4 k0 = Kc[0];
          gv = cmulc(make_float2(k0.x, k0.y), ph[0]);  // boundary slot: k^p_0 conj(phi_0)
        }
        gk[t] = gv;
        gk2[t] = cscale(gv, decay_table_entry(lp, t, L));
        if (decay_step_out_of_range(lp, t)) slow_flag = 1;
      }
      WS_STAMP(it == 2 && tid == 0, 24);
      WSYNC();
      const bool fast_decay = slow_flag == 0;
      const bool stamp = (it == 2 && tid == 0);
      WS_STAMP(stamp, 1);

      // ---- slabs: JC transform, boundary row ----------------------------------------------------
      float2 acc127 = make_float2(0.f, 0.f);
      for (int sl = 0; sl < NB; ++sl, ++g) {
        const int st = g % kWsStages, jb = g & 1;
        ok = WAITW(FULL + st, (g / kWsStages) & 1) && ok;
        // the JC buffer of this parity was last read by the products of the slab two back
        if (g >= 2) ok = WAITW(EMPTY + (g - 2) % kWsStages, ((g - 2) / kWsStages) & 1) && ok;
        WS_STAMP(stamp, 2 + 2 * sl);
        unsigned char *sb = base + st * kWsStageBytes;
#pragma unroll
        for (int i = 0; i < 2; ++i) {
          const uint32_t off = umma::swz_off(r0 + 64 * i, j);
          const uint4 cv = *reinterpret_cast<const uint4 *>(sb + off);
          *reinterpret_cast<uint4 *>(tJ + 16384 * jb + off) = umma::jchunk(cv);
          if (i == 1 && r0 == 63) {  // row 127: keep <c_127, b_127> for the diagonal, hand the row to b_{-1}
            uint4 *brow = reinterpret_cast<uint4 *>(sb + 16384 + off);
            cdot_chunk<T>(cv, *brow, acc127);
            *brow = *reinterpret_cast<const uint4 *>(bpst + buf * 256 + sl * 64 + 8 * j);
          }
        }
        umma::fence_smem_to_async();
        __syncwarp();
        if (lane == 0) umma::mbar_arrive(BAR(JREADY + jb));
        WS_STAMP(stamp, 3 + 2 * sl);
      }
      if (warp == 15) {
        const float2 s = octet_sum(acc127);
        if (lane == 31) {
          const float4 k = Kc[L - 1];
          misc[0] = k.z * s.x - k.w * s.y;  // Re(k^c_127 <c_127, b_127>)
        }
      }
      // ---- U tile: keep u_127, hand row 127 to u_{-1} --------------------------------------------
      ok = WAITW(UFULL, it & 1) && ok;
      if (r0 == 63) {
        uint4 *urow = reinterpret_cast<uint4 *>(tU + umma::swz_off(L - 1, j));
        const uint4 uv = *urow;
        const uint32_t *uw = reinterpret_cast<const uint32_t *>(&uv);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = umma::unpack2(uw[e], T());
          u127[8 * j + 2 * e] = f.x;
          u127[8 * j + 2 * e + 1] = f.y;
        }
        *urow = *reinterpret_cast<const uint4 *>(upst + buf * 64 + 8 * j);
      }
      // ---- S -> S' ----------------------------------------------------------------------------------
      WS_STAMP(stamp, 10);
      ok = WAITW(ACCFULL, it & 1) && ok;
      umma::fence_after_sync();
      WS_STAMP(stamp, 11);
      const float lpt = lp[row];
      const float2 pht = ph[row];
      {
        const float4 kr = Kc[row];
        const float2 kct = make_float2(kr.z, kr.w);
        const float rf = fast_decay ? __expf(lpt - lp[32 * cb + 1]) : 0.f;
#pragma unroll
        for (int half = 0; half < 2; ++half) {
          const int c0 = 32 * cb + 16 * half;
          const bool has_boundary = (cb == 3 && half == 1);
          float v[16];
          if (c0 <= 32 * q4 + 31 || has_boundary) {
            uint32_t re[16], im[16];
            umma::tmem_ld16_issue(umma::tmem_addr(tmem, 32 * q4, c0), re);
            umma::tmem_ld16_issue(umma::tmem_addr(tmem, 32 * q4, 192 + c0), im);
            umma::tmem_ld16_wait(re);
            umma::tmem_ld16_wait(im);
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int s = c0 + i;
              const float gr = __uint_as_float(re[i]), gi = __uint_as_float(im[i]);
              const float2 gg = fast_decay ? gk2[s] : gk[s];
              const float f = fast_decay ? rf : __expf(lpt - lp[min(s + 1, L - 1)]);
              const float nr = pht.x * gg.x - pht.y * gg.y, ni = pht.x * gg.y + pht.y * gg.x;
              const float val = f * (nr * gr - ni * gi);
              const float dg = kct.x * gr - kct.y * gi;
              v[i] = (s < row) ? val : (s == row ? dg : 0.f);
            }
            if (has_boundary) {
              const float2 gb = gk[L - 1];
              const float nr = pht.x * gb.x - pht.y * gb.y, ni = pht.x * gb.y + pht.y * gb.x;
              v[15] = __expf(lpt - lp[0]) * (nr * __uint_as_float(re[15]) - ni * __uint_as_float(im[15]));
            }
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i) v[i] = 0.f;
          }
#pragma unroll
          for (int k = 0; k < 2; ++k)
            *reinterpret_cast<uint4 *>(tS + 16384 * (cb >> 1) + umma::swz_off(row, 4 * (cb & 1) + 2 * half + k)) =
                pack8<T>(v + 8 * k);
        }
      }
      umma::fence_smem_to_async();
      umma::fence_before_sync();
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(BAR(SREADY));
      WS_STAMP(stamp, 12);
      // ---- Y = Yd + exp(lp_t) Re(phi_t H) (+ the diagonal of token 127) -> staging tile -> bulk store ---
      ok = WAITW(YDONE, it & 1) && ok;
      umma::fence_after_sync();
      WS_STAMP(stamp, 13);
      {
        uint32_t r_yd[16], r_re[16], r_im[16];
        umma::tmem_ld16_issue(umma::tmem_addr(tmem, 32 * q4, 384 + 16 * cb), r_yd);
        umma::tmem_ld16_issue(umma::tmem_addr(tmem, 32 * q4, 128 + 16 * cb), r_re);
        umma::tmem_ld16_issue(umma::tmem_addr(tmem, 32 * q4, 320 + 16 * cb), r_im);
        umma::tmem_ld16_wait(r_yd);
        umma::tmem_ld16_wait(r_re);
        umma::tmem_ld16_wait(r_im);
        umma::fence_before_sync();
        const float el = __expf(lpt);
        const float er = el * pht.x, ei = el * pht.y;
        const float d127 = (row == L - 1) ? misc[0] : 0.f;
        float y[16];
#pragma unroll
        for (int i = 0; i < 16; ++i) {
          y[i] = fmaf(er, __uint_as_float(r_re[i]), fmaf(-ei, __uint_as_float(r_im[i]), __uint_as_float(r_yd[i])));
          y[i] = fmaf(d127, u127[16 * cb + i], y[i]);
        }
#pragma unroll
        for (int k = 0; k < 2; ++k)
          *reinterpret_cast<uint4 *>(tS + umma::swz_off(row, 2 * cb + k)) = pack8<T>(y + 8 * k);
      }
      umma::fence_smem_to_async();
      __syncwarp();
      if (lane == 0) umma::mbar_arrive(BAR(TMEMFREE));
      WSYNC();
      if (tid == 0 && ok) {
        umma::tma_store_3d(&maps.Y, 0, t0, bh, umma::smem_u32(tS));
        umma::tma_store_commit();
      }
      WS_STAMP(stamp, 14);
      if (!ok) break;  // (w stays at the failed chunk: it is poisoned below with the ones after it)
    }
    if (tid == 0) umma::tma_store_wait_all();
    if (!ok || abort_flag) {
      // a wait ran out: poison every output row this CTA still owed (the host reads the status word)
      const T nanv = from_f<T>(__int_as_float(0x7fc00000));
      for (; w < total; w += gridDim.x) {
        const int c = w % d.NC, bh = w / d.NC, t0 = c * L;
        const int valid = min(L, d.T - t0);
        for (int e = tid; e < valid * P; e += kWsWorkers) a.Y[((size_t)bh * d.T + t0) * P + e] = nanv;
      }
      if (tid == 0) atomicExch(&g_tc_status, 1);
    }
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 17) umma::tmem_dealloc(tmem, 512);
}

}  // namespace slx
