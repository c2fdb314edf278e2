// Per-chunk backward of the v2x2ssd scan for half inputs with fp32 state, chunk 128, P 64,
// D = 2N in {64,128,192,256}: persistent, warp-specialised tcgen05 kernel.  Replaces the
// chunk_scan and chunk_increment backward kernels of cute/kernels/bwd/__init__.py:930-1042.
//
// Formulation (forward side in scan_ws_fwd.cuh).  Source slot j of a chunk is token j for
// j <= 126 and the token in front of the chunk for j = 127 (b~, u~ denote rows with that
// substitution); token 127 is a source only for its own diagonal term and is handled by hand.
// With the complex weight matrix w[t][j] (decay, phases, taps; row 127 of it also weights the
// chunk increment) and the raw complex Gram matrices
//     G[t][j] = <c_t, b~_j>,   H[t][p] = <c_t, z0_p>,   T[j][p] = sum_n b~_j[n] conj(Lambda_p[n]),
//     A[t][j] = dY_t . u~_j                               (Lambda = gradient of the chunk's end state)
// every gradient is a real matrix product with operands as the bulk copies delivered them, or
// a sum over the 128 x 128 / 128 x 64 tiles:
//     W  = A (.) w                                        (complex, stored as two half tiles)
//     dC = P1 + J P2,    P1 = ReW B~ + dYr Z0,   P2 = ImW B~ + dYi Z0      (dYr + i dYi = p_t dY_t)
//     dB~= Q1 - J Q2,    Q1 = ReW^T C + Ur Lambda, Q2 = ImW^T C + Ui Lambda (Ur + i Ui = w[127][j] u~_j)
//     dU~= S'^T dY + Re(w[127][j] T[j][p]),   S' = Re(w (.) G)
//     dK, dM from row sums of conj(W (.) G), column sums of decay conj(phi_t) A conj(G), and the
//     row-wise dots dY (.) conj(H), U~ (.) conj(T)           (J v = i v on interleaved pairs)
// Row 127 of dB~ / dU~ is what the chunk sends to the token in front of it (carryB, carryU).
// The operands pass through shared memory twice: pass 1 accumulates G, H, T over the state
// slabs, pass 2 produces dC and dB slab by slab (the second read comes from L2).
//
// Roles (576 threads, one CTA per SM): warp 16 producer (bulk tensor copies), warp 17 issuer
// (every tcgen05.mma), warps 0-15 workers.  All waits are bounded and share one abort flag.
#pragma once

#include "scan_ws_fwd.cuh"

namespace slx {

struct alignas(64) WsBwdMaps {
  CUtensorMap C, B, Z, Lm, U, dY;
};

constexpr int kBwX = 131072;                 // region X: pass-1 stages + transforms | W, dYr, dYi, Ur, Ui
constexpr int kBwY = 73728;                  // region Y: U, dY, S' | ring of three half-stages of pass 2
constexpr int kBwScal = 21504;
constexpr size_t scan_ws_bwd_smem_bytes() { return 1024 + kBwX + kBwY + kBwScal; }

template <typename T>
__global__ void __launch_bounds__(kWsThreads, 1) chunk_scan_bwd_ws_kernel(ScanBwdArgs<T> a,
                                                                          const __grid_constant__ WsBwdMaps maps) {
  constexpr int L = kTcL, P = kTcP;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *X = base, *Y = base + kBwX;
  // pass 1: stage s at X + 49152 s: C | B~ | Z0 | Lambda; two transform buffers JC | JLambda (the second one
  // borrows the S' tile, which nothing else touches before phase S)
  // phase S / pass 2
  unsigned char *tWr = X, *tWi = X + 32768, *tYr = X + 65536, *tYi = X + 81920, *tUr = X + 98304, *tUi = X + 114688;
  unsigned char *tU = Y, *tdY = Y + 16384, *tS = Y + 32768;
  unsigned char *sc = Y + kBwY;
  float *lp = reinterpret_cast<float *>(sc);                   // 128
  float *e2 = lp + L;                                          // 128
  float2 *ph = reinterpret_cast<float2 *>(e2 + L);             // 128
  float2 *mraw = ph + L;                                       // 128
  float2 *gk = mraw + L;                                       // 128: g_j; [127] = k^p_0 conj(phi_0)
  float2 *om = gk + L;                                         // 128: w[127][j]
  float2 *red0 = om + L;                                       // [4][128] row sums: conj(W G) + conj(p) dY conj(H)
  // the other two partial-sum arrays sit in the 8 KB of region Y that no tile of phase S covers (the tail of
  // ring slot 2 of pass 2: the producer fills that slot only after REDREAD)
  float2 *red1 = reinterpret_cast<float2 *>(Y + 65536);        // [4][128] column sums of decay conj(phi_t) A conj(G)
  float2 *red2 = red1 + 4 * L;                                 // [4][128] U~ conj(T)
  float2 *dgam = red0 + 4 * L;                                 // 128
  float2 *gsum = dgam + L;                                     // 128
  float2 *dkcs = gsum + L;                                     // 128: direct diagonal term of dk^c
  float2 *td = dkcs + L;                                       // 64: T of token 127
  float *db127 = reinterpret_cast<float *>(td + 64);           // 256: dB of token 127
  float *bdiff = db127 + 256;                                  // 256: b_{-1} - b_127
  float *b127f = bdiff + 256;                                  // 256
  float *u127f = b127f + 256;                                  // 64
  float *dy127f = u127f + 64;                                  // 64
  float *miscf = dy127f + 64;                                  // 16: [0,1] G^d  [2] a^d
  // staged by asynchronous copies one chunk ahead (issued once the current chunk has read them for the last time)
  float2 *Mst = reinterpret_cast<float2 *>(miscf + 16);        // 128 M rows
  float4 *Kst = reinterpret_cast<float4 *>(Mst + L);           // 128 K rows
  T *rowst = reinterpret_cast<T *>(Kst + L);                   // 3 x 256 + 3 x 64: b_{-1} b_127 c_127 u_{-1} u_127 dy_127
  static_assert(512 * 2 + 1024 * 4 + 4096 + 1024 * 3 + 512 + 1024 * 3 + 576 + 1024 + 2048 + (3 * 256 + 3 * 64) * 2 <= kBwScal,
                "scalar area too small");
  __shared__ uint64_t bars[27];
  __shared__ uint32_t tmem_slot;
  __shared__ int abort_flag, slow_flag;

  const ScanDims d = a.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int NB = d.D / 64;
  const int total = d.NC * d.BH;
  const uint32_t bar0 = umma::smem_u32(&bars[0]);
  auto BAR = [&](int i) { return bar0 + 8u * i; };
  enum {
    UDYFULL = 0, UPATCH = 1, ADONE = 2, AREAD = 3, P1FULL = 4, P1JREADY = 6, P1EMPTY = 7, ACC1FULL = 9, SREADY = 10,
    DUDONE = 11, WREADY = 12, DUREAD = 13, H2FULL = 14, H2EMPTY = 17, ACC2FULL = 20, ACC2FREE = 22, WBAR = 24,
    REDREAD = 25, P1JREADY2 = 26
  };
  constexpr int fmt = umma::HalfFmt<T>::value;

  if (tid == 0) {
    for (int i = 0; i < 27; ++i) {
      const bool wb = (i == UPATCH || i == AREAD || i == P1JREADY || i == SREADY || i == WREADY || i == DUREAD ||
                       i == ACC2FREE || i == ACC2FREE + 1 || i == WBAR || i == REDREAD || i == P1JREADY2);
      umma::mbar_init(BAR(i), wb ? 16u : 1u);
    }
    umma::fence_mbar_init();
    abort_flag = 0;
  }
  if (warp == 17) umma::tmem_alloc(&tmem_slot, 512);
  if (tid == 512) {
    umma::tma_prefetch_map(&maps.C);
    umma::tma_prefetch_map(&maps.B);
    umma::tma_prefetch_map(&maps.Z);
    umma::tma_prefetch_map(&maps.Lm);
    umma::tma_prefetch_map(&maps.U);
    umma::tma_prefetch_map(&maps.dY);
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
      uint32_t g1 = 0, q2 = 0, it = 0, use[2] = {0, 0};
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++it) {
        const int c = w % d.NC, bh = w / d.NC, t0 = c * L;
        // everything below lands in memory that the previous chunk's second pass reads: wait for its last products
        if (it >= 1) {
          const int lb = (NB - 1) & 1;
          ok = WAIT(ACC2FULL + lb, (use[lb] - 1) & 1);
          if (ok && NB >= 2) ok = WAIT(ACC2FULL + (lb ^ 1), (use[lb ^ 1] - 1) & 1);
          if (!ok) break;
        }
        WS_STAMP(it == 2, 48);
        umma::mbar_expect_tx(BAR(UDYFULL), 32768u);
        umma::tma_load_3d(umma::smem_u32(tU), &maps.U, 0, t0, bh, BAR(UDYFULL));
        umma::tma_load_3d(umma::smem_u32(tdY), &maps.dY, 0, t0, bh, BAR(UDYFULL));
        for (int sl = 0; sl < NB && ok; ++sl, ++g1) {
          const int st = g1 & 1;
          if (sl >= 2) ok = WAIT(P1EMPTY + st, ((g1 >> 1) - 1) & 1);  // (the first two stages of a chunk are free)
          if (!ok) break;
          unsigned char *sb = X + st * 49152;
          umma::mbar_expect_tx(BAR(P1FULL + st), 49152u);
          umma::tma_load_3d(umma::smem_u32(sb), &maps.C, sl * 64, t0, bh, BAR(P1FULL + st));
          umma::tma_load_3d(umma::smem_u32(sb + 16384), &maps.B, sl * 64, t0, bh, BAR(P1FULL + st));
          umma::tma_load_3d(umma::smem_u32(sb + 32768), &maps.Z, sl * 64, 0, w, BAR(P1FULL + st));
          umma::tma_load_3d(umma::smem_u32(sb + 40960), &maps.Lm, sl * 64, 0, w, BAR(P1FULL + st));
        }
        if (!ok) break;
        // second pass: its ring lies over the U, dY and S' tiles
        WS_STAMP(it == 2, 49);
        ok = WAIT(WREADY, it & 1) && WAIT(DUDONE, it & 1);
        if (!ok) break;
        WS_STAMP(it == 2, 50);
        for (int hs = 0; hs < 2 * NB && ok; ++hs, ++q2) {
          const int slot = q2 % 3, sl = hs >> 1;
          if (hs >= 3) ok = WAIT(H2EMPTY + slot, ((q2 / 3) - 1) & 1);  // (three free slots at the start of a chunk)
          if (ok && hs == 2) ok = WAIT(REDREAD, it & 1);  // the tail of the third slot held partial sums of phase S
          if (!ok) break;
          unsigned char *hb = Y + slot * 24576;
          umma::mbar_expect_tx(BAR(H2FULL + slot), 24576u);
          if ((hs & 1) == 0) {
            umma::tma_load_3d(umma::smem_u32(hb), &maps.B, sl * 64, t0, bh, BAR(H2FULL + slot));
            umma::tma_load_3d(umma::smem_u32(hb + 16384), &maps.Z, sl * 64, 0, w, BAR(H2FULL + slot));
          } else {
            umma::tma_load_3d(umma::smem_u32(hb), &maps.C, sl * 64, t0, bh, BAR(H2FULL + slot));
            umma::tma_load_3d(umma::smem_u32(hb + 16384), &maps.Lm, sl * 64, 0, w, BAR(H2FULL + slot));
          }
        }
        for (int sl = 0; sl < NB; ++sl) ++use[sl & 1];
      }
    }
  } else if (warp == 17) {
    // ------------------------------------------------------------------ issuer
    if (lane == 0) {
      constexpr uint32_t id_a = umma::make_idesc(128, 128, false, false, fmt);
      constexpr uint32_t id_g = umma::make_idesc(128, 192, false, false, fmt);
      constexpr uint32_t id_kk = umma::make_idesc(128, 64, false, false, fmt);
      constexpr uint32_t id_km = umma::make_idesc(128, 64, false, true, fmt);
      constexpr uint32_t id_mm = umma::make_idesc(128, 64, true, true, fmt);
      const uint32_t sU = umma::smem_u32(tU), sdY = umma::smem_u32(tdY), sS = umma::smem_u32(tS);
      const uint32_t sWr = umma::smem_u32(tWr), sWi = umma::smem_u32(tWi), sYr = umma::smem_u32(tYr),
                     sYi = umma::smem_u32(tYi), sUr = umma::smem_u32(tUr), sUi = umma::smem_u32(tUi);
      uint32_t g1 = 0, q2 = 0, it = 0, use[2] = {0, 0};
      bool ok = true;
      for (int w = blockIdx.x; w < total && ok; w += gridDim.x, ++it) {
        // tensor memory of the previous chunk's second pass has been read out
        for (int b = 0; b < 2 && ok; ++b)
          if (use[b] >= 1) ok = WAIT(ACC2FREE + b, (use[b] - 1) & 1);
        if (!ok) break;
        // ---- A = dY U~^T
        WS_STAMP(it == 2, 32);
        ok = WAIT(UDYFULL, it & 1) && WAIT(UPATCH, it & 1);
        if (!ok) break;
        umma::fence_after_sync();
        WS_STAMP(it == 2, 33);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma::mma_ss(tmem, umma::desc_kmajor(sdY, kk), umma::desc_kmajor(sU, kk), id_a, kk != 0);
        umma::commit(BAR(ADONE));
        ok = WAIT(AREAD, it & 1);
        if (!ok) break;
        umma::fence_after_sync();
        // ---- pass 1: [G | H] (re, im), T (re, im) over the state slabs
        for (int sl = 0; sl < NB && ok; ++sl, ++g1) {
          const int st = g1 & 1;
          ok = WAIT(P1FULL + st, (g1 >> 1) & 1) && WAIT(st ? P1JREADY2 : P1JREADY, (g1 >> 1) & 1);
          if (!ok) break;
          umma::fence_after_sync();
          WS_STAMP(it == 2, 34 + sl);
          const uint32_t sb = umma::smem_u32(X + st * 49152);
          const uint64_t dC = umma::desc_kmajor(sb, 0), dBZ = umma::desc_kmajor(sb + 16384, 0),
                         dLm = umma::desc_kmajor(sb + 40960, 0),
                         dJC = umma::desc_kmajor(umma::smem_u32(st ? tS : X + 98304), 0),
                         dJL = umma::desc_kmajor(umma::smem_u32(st ? tS + 16384 : X + 114688), 0);
#pragma unroll
          for (int kk = 0; kk < 4; ++kk) {
            const uint32_t adv = umma::kStepK * kk;
            const uint64_t bz = umma::desc_advance(dBZ, adv);
            umma::mma_ss(tmem + 0, umma::desc_advance(dC, adv), bz, id_g, (sl | kk) != 0);
            umma::mma_ss(tmem + 192, umma::desc_advance(dJC, adv), bz, id_g, (sl | kk) != 0);
            umma::mma_ss(tmem + 384, bz, umma::desc_advance(dLm, adv), id_kk, (sl | kk) != 0);
            umma::mma_ss(tmem + 448, bz, umma::desc_advance(dJL, adv), id_kk, (sl | kk) != 0);
          }
          umma::commit(BAR(P1EMPTY + st));
        }
        if (!ok) break;
        umma::commit(BAR(ACC1FULL));
        WS_STAMP(it == 2, 38);
        // ---- dU~ (score path) = S'^T dY
        ok = WAIT(SREADY, it & 1);
        if (!ok) break;
        umma::fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < 8; ++kk)
          umma::mma_ss(tmem + 448, umma::desc_mnmajor(sS, kk, 16384u), umma::desc_mnmajor(sdY, kk, 0), id_mm, kk != 0);
        umma::commit(BAR(DUDONE));
        // ---- pass 2: dC, dB~ slab by slab, accumulators double-buffered
        ok = WAIT(WREADY, it & 1);
        for (int sl = 0; sl < NB && ok; ++sl) {
          const int buf = sl & 1;
          const uint32_t acc = tmem + 256u * buf;
          if (sl == 1) ok = WAIT(DUREAD, it & 1);
          if (ok && sl >= 2) ok = WAIT(ACC2FREE + buf, (use[buf] - 1) & 1);
          if (!ok) break;
          umma::fence_after_sync();
          {
            const int slot = q2 % 3;
            WS_STAMP(it == 2, 40 + 2 * sl);
            ok = WAIT(H2FULL + slot, (q2 / 3) & 1);
            if (!ok) break;
            umma::fence_after_sync();
            WS_STAMP(it == 2, 41 + 2 * sl);
            const uint32_t hb = umma::smem_u32(Y + slot * 24576);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t bm = umma::desc_mnmajor(hb, kk, 0);
              umma::mma_ss(acc + 0, umma::desc_kmajor(sWr + 16384u * (kk >> 2), kk & 3), bm, id_km, kk != 0);
              umma::mma_ss(acc + 64, umma::desc_kmajor(sWi + 16384u * (kk >> 2), kk & 3), bm, id_km, kk != 0);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t zm = umma::desc_mnmajor(hb + 16384, kk, 0);
              umma::mma_ss(acc + 0, umma::desc_kmajor(sYr, kk), zm, id_km, 1);
              umma::mma_ss(acc + 64, umma::desc_kmajor(sYi, kk), zm, id_km, 1);
            }
            umma::commit(BAR(H2EMPTY + slot));
            ++q2;
          }
          {
            const int slot = q2 % 3;
            ok = WAIT(H2FULL + slot, (q2 / 3) & 1);
            if (!ok) break;
            umma::fence_after_sync();
            const uint32_t hb = umma::smem_u32(Y + slot * 24576);
#pragma unroll
            for (int kk = 0; kk < 8; ++kk) {
              const uint64_t cm = umma::desc_mnmajor(hb, kk, 0);
              umma::mma_ss(acc + 128, umma::desc_mnmajor(sWr, kk, 16384u), cm, id_mm, kk != 0);
              umma::mma_ss(acc + 192, umma::desc_mnmajor(sWi, kk, 16384u), cm, id_mm, kk != 0);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
              const uint64_t lm = umma::desc_mnmajor(hb + 16384, kk, 0);
              umma::mma_ss(acc + 128, umma::desc_kmajor(sUr, kk), lm, id_km, 1);
              umma::mma_ss(acc + 192, umma::desc_kmajor(sUi, kk), lm, id_km, 1);
            }
            umma::commit(BAR(H2EMPTY + slot));
            ++q2;
          }
          umma::commit(BAR(ACC2FULL + buf));
          ++use[buf];
        }
      }
    }
  } else {
#include "scan_ws_bwd_workers.inc"
  }
  umma::fence_before_sync();
  __syncthreads();
  if (warp == 17) umma::tmem_dealloc(tmem, 512);
}

}  // namespace slx
