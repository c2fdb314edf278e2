// Tensor-core per-chunk backward of the v2x2ssd scan (chunk 128, P 64, half
// inputs, fp32 state).  Same mathematics as chunk_scan_bwd_kernel in
// scan_simt.cuh; every contraction runs on tcgen05 with fp32 accumulators in
// tensor memory.  One CTA of 512 threads per (chunk, batch*head), one CTA per SM.
//
// Tensor-memory map (fp32 columns):
//   [  0,128)  G = dY U^T, then S = Qbar kappa^T (accumulated over state slabs)
//   [128,192)  dU, increment path:  Bhat Lambda^T
//   [192,256)  dq  (slab)   = dS' kappa + (e^lp dY) Z0
//   [256,320)  X   (slab)   = dS'^T Qbar
//   [320,384)  UL  (slab)   = U Lambda
//   [384,448)  dU, score path:      S'^T dY
//
// The source token in front of the chunk (b_{-1}, u_{-1}) borrows key slot 127,
// whose own merged-tap column is empty (no query follows the last token):
//   dS'[t][127] = exp(lp_t - lp_0) dY_t.u_{-1},   kappa[127] = k^p_0 b_{-1} conj(phi_0)
// so that row 127 of X is the column sum the carry gradient needs, the boundary
// term of dq comes out of the same product, column 127 of S is the boundary
// score and row 127 of S'^T dY is the dU carried to the previous token.
//
// Thread roles: for staging, thread = (16-byte chunk j = tid%8, rows tid/8 and
// tid/8+64); for tensor-memory epilogues, thread = (row 32*(warp%4)+lane,
// column quarter warp/4).  Global loads a phase needs are issued before the
// wait on the preceding products, so that their latency overlaps the tensor work.
#pragma once

#include "scan_tc.cuh"

namespace slx {

// tensor maps of the raw C and B operands (loads) and of dC, dB (stores): (D, T, BH), boxes of 64 columns x 128 tokens
struct alignas(64) ScanBwdMaps {
  CUtensorMap C, B, dC, dB;
};

constexpr int kTcBwdThreads = 512;
constexpr size_t scan_bwd_tc_smem_bytes() { return 1024 + 144 * 1024 + 28 * 1024 + 32 * 1024; }

template <typename T>
__global__ void __launch_bounds__(kTcBwdThreads, 1) chunk_scan_bwd_tc_kernel(ScanBwdArgs<T> a,
                                                                              const __grid_constant__ ScanBwdMaps maps) {
  constexpr int L = kTcL, P = kTcP;
  extern __shared__ unsigned char smem_raw[];
  unsigned char *base =
      reinterpret_cast<unsigned char *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  unsigned char *tdY = base;                // [t][p]
  unsigned char *tdYe = base + 16384;       // [t][p]  exp(lp_t) dY
  unsigned char *tU = base + 32768;         // [s][p]
  unsigned char *tdS = base + 49152;        // 2 x [t][64 s]   dS', later S'
  unsigned char *tQ = base + 81920;         // [t][d]  Qbar slab
  unsigned char *tK = base + 98304;         // [s][d]  kappa slab
  unsigned char *tBh = base + 114688;       // [s][d]  w_s b_s slab
  unsigned char *tZ = base + 131072;        // [p][d]  Z0 slab        (8 KB)
  unsigned char *tLm = base + 139264;       // [p][d]  Lambda slab    (8 KB)
  float *lp = reinterpret_cast<float *>(base + 147456);
  float *gd = lp + L;                        // G[t][t]
  float *gm1 = gd + L;                       // dY_t . u_{-1}
  float *um1 = gm1 + L;                      // 64
  float *duc = um1 + 64;                     // 64  increment path of the carried dU
  float2 *ph = reinterpret_cast<float2 *>(duc + 64);
  float2 *mraw = ph + L, *kc = mraw + L, *kp = kc + L, *gam = kp + L, *gk = gam + L, *wco = gk + L, *sg1 = wco + L;
  float2 *bc = sg1 + L, *bX = bc + L, *gA = bX + L, *gsum = gA + L;
  float2 *bm1 = gsum + L;                    // 128  b_{-1}
  float2 *ul1 = bm1 + 128;                   // 128  (u_{-1} . Lambda)[n]
  float2 *bh1 = ul1 + 128;                   // 128  w_{-1} b_{-1}
  float2 *misc = bh1 + 128;                  // [0] bLam(last row) [1] dk^p_0 [2] w_{-1} [3] p_{L-1}/p_0
  float *ulw = reinterpret_cast<float *>(misc + 4);  // [16][64] per-warp partials of u_{-1}.Lambda
  float *e2 = ulw + 16 * 64;                          // 128: decay table (decay_mask32)
  float *xb = e2 + L;                                 // 256: row 127 of X (boundary column sums), all slabs
  float *ulf = xb + 256;                              // 256: u_{-1} . Lambda, all slabs
  unsigned char *sC = base + 147456 + 28672;          // raw C slab (swizzled tile), filled by cp.async
  unsigned char *sB = sC + 16384;                     // raw B slab
  __shared__ uint64_t mbar;   // completion of the tensor products
  __shared__ uint64_t tbar;   // arrival of a raw (C, B) slab by TMA
  __shared__ uint32_t tmem_slot;

  const ScanDims d = a.d;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int c = blockIdx.x, bh = blockIdx.y;
  const int t0 = c * L;
  const int valid = min(L, d.T - t0);
  const size_t tok0 = (size_t)bh * d.T + t0;
  const int NB = d.D / 64;
  const uint32_t mbar_s = umma::smem_u32(&mbar), tbar_s = umma::smem_u32(&tbar);
  constexpr int fmt = umma::HalfFmt<T>::value;

#define SLX_STAMP(i) SLX_DIAG_STAMP(i)
  SLX_STAMP(0);
  const int j = tid & 7, r0 = tid >> 3;  // r0 in [0,64)
  // on this path the chunk-start states are stored in the activation dtype (api: slx_scan_starts_dtype)
  const T *z0 = reinterpret_cast<const T *>(a.starts) + ((size_t)bh * d.NC + c) * P * d.D;
  const T *lam = reinterpret_cast<const T *>(a.d_inc) + ((size_t)bh * d.NC + c) * P * d.D;  // same dtype as z0
  float2 mreg[4];  // the prefix warp's multipliers, requested ahead of the bulk copies
  if (warp == 2) chunk_prefix_load4(a.M + tok0 * 2, valid, mreg);
  // U and dY land in their operand tiles by asynchronous copy (rows past the chunk end are
  // zero-filled); the first raw (C, B) slab follows as a second group
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    const int r = r0 + 64 * i;
    const int rr = r < valid ? r : 0;
    const uint32_t nbytes = r < valid ? 16u : 0u;
    const uint32_t off = umma::swz_off(r, j);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(tU + off)),
                 "l"(a.U + (tok0 + rr) * P + 8 * j), "r"(nbytes)
                 : "memory");
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(umma::smem_u32(tdY + off)),
                 "l"(a.dY + (tok0 + rr) * P + 8 * j), "r"(nbytes)
                 : "memory");
  }
  asm volatile("cp.async.commit_group;" ::: "memory");
  // One raw (C, B) slab = two TMA boxes of [128 tokens][64 columns] into the swizzled staging tiles,
  // issued by one thread; tokens past the end of the sequence arrive as zeros.
  auto prefetch_cb = [&](int sl) {
    if (tid == 32) {
      umma::fence_smem_to_async();  // the tiles' earlier (generic) readers are behind a barrier
      umma::mbar_expect_tx(tbar_s, 2u * 16384u);
      umma::tma_load_3d(umma::smem_u32(sC), &maps.C, sl * 64, t0, bh, tbar_s);
      umma::tma_load_3d(umma::smem_u32(sB), &maps.B, sl * 64, t0, bh, tbar_s);
    }
  };
  if (tid == 32) {
    umma::mbar_init(mbar_s, 1);
    umma::mbar_init(tbar_s, 1);
    umma::fence_mbar_init();
    umma::tma_prefetch_map(&maps.C);
    umma::tma_prefetch_map(&maps.B);
    umma::tma_prefetch_map(&maps.dC);
    umma::tma_prefetch_map(&maps.dB);
  }
  prefetch_cb(0);
  uint32_t tphase = 0;
  // Z0 / Lambda slab: one 8-value (16-byte) item per thread, prefetched into registers
  const int zp = tid >> 3, zj = tid & 7;
  uint4 zr, lr;
  auto prefetch_zl = [&](int sl) {
    zr = *reinterpret_cast<const uint4 *>(z0 + (size_t)zp * d.D + sl * 64 + 8 * zj);
    lr = *reinterpret_cast<const uint4 *>(lam + (size_t)zp * d.D + sl * 64 + 8 * zj);
  };
  prefetch_zl(0);

  if (warp == 0) umma::tmem_alloc(&tmem_slot, 512);
  if (warp == 2) chunk_prefix_fast128(mreg, lp, ph, mraw, &g_scan_bad);
  if (tid >= 128 && tid < 256) {
    int t = tid - 128;
    float2 vp = make_float2(0.f, 0.f), vc = vp;
    if (t < valid) {
      float4 k4 = *reinterpret_cast<const float4 *>(a.K + (tok0 + t) * 4);
      vp = make_float2(k4.x, k4.y);
      vc = make_float2(k4.z, k4.w);
    }
    kp[t] = vp;
    kc[t] = vc;
  } else if (tid >= 256 && tid < 320) {
    int p = tid - 256;
    float v = 0.f;
    if (t0 > 0) v = to_f(a.U[(tok0 - 1) * P + p]);
    else if (a.Uprev) v = a.Uprev[(size_t)bh * P + p];
    um1[p] = v;
    duc[p] = 0.f;
  } else if (tid >= 320 && tid < 320 + d.N) {
    int n = tid - 320;
    float2 bv = make_float2(0.f, 0.f);
    if (t0 > 0) bv = load_pair<T>(a.B + (tok0 - 1) * d.D + 2 * n);
    else if (a.Bprev) bv = *reinterpret_cast<const float2 *>(a.Bprev + (size_t)bh * d.D + 2 * n);
    bm1[n] = bv;
  }
  asm volatile("cp.async.wait_group 0;" ::: "memory");  // U, dY tiles
  umma::fence_smem_to_async();
  umma::fence_before_sync();
  __syncthreads();
  umma::fence_after_sync();
  const uint32_t tmem = tmem_slot;
  const uint32_t sdY = umma::smem_u32(tdY), sdYe = umma::smem_u32(tdYe), sU = umma::smem_u32(tU),
                 sdS = umma::smem_u32(tdS), sQ = umma::smem_u32(tQ), sK = umma::smem_u32(tK),
                 sBh = umma::smem_u32(tBh), sZ = umma::smem_u32(tZ), sLm = umma::smem_u32(tLm);
  SLX_STAMP(1);
  // ---- G = dY U^T (runs while the per-token coefficients are computed) -----------------------
  if (tid == 0) {
    const uint32_t id = umma::make_idesc(128, 128, false, false, fmt);
#pragma unroll
    for (int kk = 0; kk < 4; ++kk)
      umma::mma_ss(tmem, umma::desc_kmajor(sdY, kk), umma::desc_kmajor(sU, kk), id, kk != 0);
    umma::commit(mbar_s);
  }
  // exp(lp_t) dY and g_{-1}[t] = dY_t . u_{-1}
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    int r = r0 + 64 * i;
    const uint4 dyr = *reinterpret_cast<const uint4 *>(tdY + umma::swz_off(r, j));
    const uint32_t *w = reinterpret_cast<const uint32_t *>(&dyr);
    const float el = __expf(lp[r]);
    float tmp[8], dot = 0.f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      float2 v = umma::unpack2(w[e], T());
      dot = fmaf(v.x, um1[8 * j + 2 * e], fmaf(v.y, um1[8 * j + 2 * e + 1], dot));
      tmp[2 * e] = el * v.x;
      tmp[2 * e + 1] = el * v.y;
    }
    *reinterpret_cast<uint4 *>(tdYe + umma::swz_off(r, j)) = pack8<T>(tmp);
#pragma unroll
    for (int off = 4; off > 0; off >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, off);
    if (j == 0) gm1[r] = dot;
  }
  if (tid < L) {
    const int t = tid;
    float2 g = make_float2(0.f, 0.f), w, s1 = g, gkv = g;
    if (t + 1 < L) {
      g = cadd(cmul(mraw[t + 1], kc[t]), kp[t + 1]);
      gkv = cmulc(g, ph[t + 1]);
      s1 = cscale(cmulc(ph[L - 1], ph[t + 1]), __expf(lp[L - 1] - lp[t + 1]));  // p_{L-1}/p_{t+1}
      w = cmul(s1, g);
    } else {
      w = kc[t];
      gkv = cmulc(kp[0], ph[0]);  // boundary slot: kappa[127] = k^p_0 b_{-1} conj(phi_0)
    }
    gam[t] = g;
    gk[t] = gkv;
    sg1[t] = s1;
    wco[t] = w;
    e2[t] = decay_table_entry(lp, t, L);
  } else if (tid >= 256 && tid < 256 + d.N) {
    const int n = tid - 256;
    const float2 s0 = cscale(cmulc(ph[L - 1], ph[0]), __expf(lp[L - 1] - lp[0]));  // p_{L-1}/p_0
    const float2 w1 = cmul(s0, kp[0]);
    bh1[n] = cmul(w1, bm1[n]);
    if (n == 0) {
      misc[0] = misc[1] = make_float2(0.f, 0.f);
      misc[2] = w1;
      misc[3] = s0;
    }
  }
  umma::fence_smem_to_async();
  const bool fast_decay = !__syncthreads_or(tid < L && decay_step_out_of_range(lp, tid));

  uint32_t phase = 0;
  bool ok = true;
  const int q4 = warp & 3, qc = warp >> 2;  // lane quarter of tensor memory, column quarter
  const int row = 32 * q4 + lane;
#include "scan_tc_bwd_body.inc"
#undef SLX_STAMP
}

}  // namespace slx
