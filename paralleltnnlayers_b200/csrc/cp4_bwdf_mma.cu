// CP4 conv2d backward-filter (3x3 filters) with warp-level tensor-core contractions (mma.sync, tf32 in three
// terms, fp32 accumulation: fp32-grade results).
//
// One CTA of 8 warps owns a TH x TW tile of one image and works on its halo tile ((TH+2) x (TW+2) pixels, the
// columns of every shared-memory plane; warp w owns a contiguous range of them).  Three streaming passes over
// the channels, each through a warp-private cp.async FIFO (16 channels per group):
//   pass 1 (X):   P[r, px]  = sum_c K1[c, r] X[c, px]                      M = pixels, K = channels, N = ranks
//   stencil A:    Z[r, px]  = sum_{y,x} KH[y,r] KW[x,r] P[r, px + (y-1, x-1)]   interior pixels; 0 on the halo ring
//   pass 2 (dU):  Q[r, px]  = sum_t K0[t, r] dU[t, px]                     same GEMM shape
//                 dK0[t, r] += sum_px dU[t, px] Z[r, px]                   M = channels, K = pixels, N = ranks
//   stencil B:    Qt[r, px] = sum_{y,x} KH[y,r] KW[x,r] Q[r, px - (y-1, x-1)]  interior pixels; 0 on the halo ring
//                 dKH[y, r] += Q[r, px] * sum_x KW[x,r] P[r, px + (y-1, x-1)],  dKW[x, r] likewise   (CUDA cores)
//   pass 3 (X):   dK1[c, r] += sum_px X[c, px] Qt[r, px]
// Both orientations of a channel group (pixels x channels for the contraction, channels x pixels for the
// reduction) are read as mma fragments from the same FIFO stage.  Pixels outside the image are zero-filled by
// the copies, which is the zero padding of the convolution.  Each CTA writes its partial gradients to
// workspace[cta][...]; a second kernel sums the partials in CTA order, so results are bitwise reproducible.
// Formulas: Cuda_kernels/cp4Conv2dBackwardFilter.cu:91-104,142-155,192-205,241-254.
// CORE = true is the three-factor CP conv (Kernels/cp_fused_nchw.cu, test/layers.py:265-283): the per-rank 3x3
// filter is a free [3,3,R] core instead of the outer product KH x KW, and its gradient has nine rows,
// dKC[y, x, r] = sum_px Q[r, px] * P[r, px + (y-1, x-1)].
#include <algorithm>
#include <cstdlib>

#include "common.cuh"
#include "mma_util.cuh"

namespace b200cp {

namespace {

using namespace mma;

constexpr int kNT = 256, kWarps = 8;
constexpr int kGC = 16;    // channels per cp.async group: two contraction k-steps, one reduction m-block
constexpr int kFifo = 2;   // cp.async groups per warp (one being consumed)

struct BGeom {
  int N, C, T, H, W, R, Rs, r0;
  int TH, TW, TWh, HPX, tilesH, tilesW;
  int MBW;     // 16-pixel blocks of the halo tile per warp
  int nparam;  // (T + C + 6) * R floats per partial (T + C + 9 with a free 3x3 core)
  int pp;      // row pitch of the P and Q planes (odd)
};

template <int RP>
struct BCfg {
  static constexpr int NB = RP / 8;
  static constexpr int MB2 = NB <= 2 ? 4 : NB == 4 ? 2 : 1;  // channel blocks whose gradient sums stay in registers
  static constexpr int CHA = MB2 * 16;                       // channels per accumulation chunk
  static constexpr int FIN = RP == 8 ? 24 : RP + 8;          // factor plane pitch (see the forward kernel)
};

template <int RP>
size_t bwdf_mma_smem_floats(const BGeom& g) {
  using K = BCfg<RP>;
  const int cols = kWarps * g.MBW * 16;
  const size_t fifo = (size_t)kFifo * kGC * (cols + 12);
  const size_t red = (size_t)kWarps * K::CHA * RP;
  const size_t planes = 2 * (size_t)RP * g.pp + (size_t)RP * (cols + 4);
  const size_t fac = 2 * (size_t)K::CHA * K::FIN;
  return std::max(fifo, red) + planes + fac + 9 * RP + kNT * 9;
}

// One pass over the channels of `src_n`.  CONTRACT: Out[r][px] = sum_ch F[ch][r] src[ch][px].
// REDUCE: part[ch][r] = sum_px src[ch][px] * Zh[r][px] (over this CTA's halo tile).
template <int RP, int MBW, bool CONTRACT, bool REDUCE>
__device__ __forceinline__ void stream_pass(const BGeom& g, const float* __restrict__ src_n, int nch,
                                            const float* __restrict__ Fg, float* Xf, float* Fh, float* Out,
                                            const float* Zh, float* __restrict__ part, const float* const (&gp)[(MBW + 1) / 2],
                                            const int (&gsz)[(MBW + 1) / 2], int tid) {
  using K = BCfg<RP>;
  constexpr int NB = K::NB, MB2 = K::MB2, CHA = K::CHA, FIN = K::FIN;
  constexpr int WCOLS = MBW * 16, COLS = kWarps * WCOLS, CPL = (MBW + 1) / 2;
  constexpr int XP = COLS + 12;   // 12 mod 32: the channel-major fragment loads are conflict-free, the
                                  // pixel-major ones two-way on a quarter of the lanes
  constexpr int ZP = COLS + 4;    // 4 mod 32
  constexpr int kFpl = CHA * FIN; // floats per factor plane
  const int lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const size_t HW = (size_t)g.H * g.W;
  const unsigned xw_s = (unsigned)__cvta_generic_to_shared(Xf + warp * WCOLS + lane);
  const float* xw = Xf + warp * WCOLS;

  float cacc[MBW][NB][4];
  if (CONTRACT) {
#pragma unroll
    for (int j = 0; j < MBW; ++j)
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) cacc[j][nb][0] = cacc[j][nb][1] = cacc[j][nb][2] = cacc[j][nb][3] = 0.f;
  }

  for (int c0 = 0; c0 < nch; c0 += CHA) {
    const int cc = min(CHA, nch - c0);
    const int ng = (cc + kGC - 1) / kGC;
    auto issue = [&](int grp) {
      if (grp < ng) {
        const unsigned dst = xw_s + (unsigned)((grp % kFifo) * kGC * XP * 4);
        const size_t coff = (size_t)(c0 + grp * kGC) * HW;
        if (grp * kGC + kGC <= cc) {
#pragma unroll
          for (int q = 0; q < CPL; ++q)
            if (CPL * 32 == WCOLS || lane + 32 * q < WCOLS) {
              const float* sp = gp[q] + coff;
#pragma unroll
              for (int jc = 0; jc < kGC; ++jc) {
                cp_async4_s(dst + (unsigned)((jc * XP + 32 * q) * 4), sp, gsz[q]);
                sp += HW;
              }
            }
        } else {
#pragma unroll
          for (int q = 0; q < CPL; ++q)
            if (CPL * 32 == WCOLS || lane + 32 * q < WCOLS) {
#pragma unroll
              for (int jc = 0; jc < kGC; ++jc) {
                const bool cin = grp * kGC + jc < cc;
                cp_async4_s(dst + (unsigned)((jc * XP + 32 * q) * 4), cin ? gp[q] + coff + (size_t)jc * HW : src_n,
                            cin ? gsz[q] : 0);
              }
            }
        }
      }
      cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kFifo - 1; ++s) issue(s);
    if (CONTRACT) {
      __syncthreads();  // every warp is done with the previous chunk's factor planes
      for (int i = tid; i < ng * kGC * RP; i += kNT) {
        const int c = i / RP, r = i % RP;
        const float v = (r < g.R && c < cc) ? __ldg(Fg + (size_t)(c0 + c) * g.Rs + g.r0 + r) : 0.f;
        const float hi = tf32_round(v);
        Fh[c * FIN + r] = hi;
        Fh[kFpl + c * FIN + r] = tf32_round(v - hi);
      }
      __syncthreads();
    }
    float racc[MB2][NB][4];
    if (REDUCE) {
#pragma unroll
      for (int m = 0; m < MB2; ++m)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) racc[m][nb][0] = racc[m][nb][1] = racc[m][nb][2] = racc[m][nb][3] = 0.f;
    }
#pragma unroll
    for (int grp = 0; grp < MB2; ++grp) {
      if (grp < ng) {
        issue(grp + kFifo - 1);
        cp_async_wait<kFifo - 1>();
        __syncwarp();
        const float* xs = xw + (grp % kFifo) * kGC * XP;
        if (CONTRACT) {
#pragma unroll
          for (int ks = 0; ks < 2; ++ks) {
            // B fragments: element (k = channel, n = rank)
            uint32_t bh[NB][2], bl[NB][2];
            const float* f = Fh + (grp * kGC + ks * 8 + tq) * FIN + gq;
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              bh[nb][0] = __float_as_uint(f[nb * 8]);
              bh[nb][1] = __float_as_uint(f[nb * 8 + 4 * FIN]);
              bl[nb][0] = __float_as_uint(f[nb * 8 + kFpl]);
              bl[nb][1] = __float_as_uint(f[nb * 8 + kFpl + 4 * FIN]);
            }
            // A fragments: element (m = pixel, k = channel)
            uint32_t ah[MBW][4], al[MBW][4];
            const float* xa = xs + (ks * 8 + tq) * XP + gq;
#pragma unroll
            for (int j = 0; j < MBW; ++j) {
              split_tf32(xa[j * 16], ah[j][0], al[j][0]);
              split_tf32(xa[j * 16 + 8], ah[j][1], al[j][1]);
              split_tf32(xa[j * 16 + 4 * XP], ah[j][2], al[j][2]);
              split_tf32(xa[j * 16 + 4 * XP + 8], ah[j][3], al[j][3]);
            }
#pragma unroll
            for (int j = 0; j < MBW; ++j)
#pragma unroll
              for (int nb = 0; nb < NB; ++nb) mma_tf32(cacc[j][nb], al[j], bh[nb]);
#pragma unroll
            for (int j = 0; j < MBW; ++j)
#pragma unroll
              for (int nb = 0; nb < NB; ++nb) mma_tf32(cacc[j][nb], ah[j], bl[nb]);
#pragma unroll
            for (int j = 0; j < MBW; ++j)
#pragma unroll
              for (int nb = 0; nb < NB; ++nb) mma_tf32(cacc[j][nb], ah[j], bh[nb]);
          }
        }
        if (REDUCE) {
          const float* zb = Zh + gq * ZP + warp * WCOLS + tq;
#pragma unroll
          for (int kp = 0; kp < 2 * MBW; ++kp) {
            // A fragment: element (m = channel, k = pixel);  B fragment: element (k = pixel, n = rank)
            uint32_t ah[4], al[4];
            const float* xa = xs + gq * XP + kp * 8 + tq;
            split_tf32(xa[0], ah[0], al[0]);
            split_tf32(xa[8 * XP], ah[1], al[1]);
            split_tf32(xa[4], ah[2], al[2]);
            split_tf32(xa[8 * XP + 4], ah[3], al[3]);
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
              uint32_t bh[2], bl[2];
              split_tf32(zb[nb * 8 * ZP + kp * 8], bh[0], bl[0]);
              split_tf32(zb[nb * 8 * ZP + kp * 8 + 4], bh[1], bl[1]);
              mma_tf32(racc[grp][nb], al, bh);
              mma_tf32(racc[grp][nb], ah, bl);
              mma_tf32(racc[grp][nb], ah, bh);
            }
          }
        }
        __syncwarp();  // every lane has read this FIFO stage: a later group may overwrite it
      }
    }
    cp_async_wait<0>();
    if (REDUCE) {
      // the warps' partial sums meet in shared memory (over the FIFO) and are added in warp order
      float* red = Xf;
      __syncthreads();
#pragma unroll
      for (int m = 0; m < MB2; ++m)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          float* d = red + ((size_t)warp * CHA + m * 16 + gq) * RP + nb * 8 + 2 * tq;
          d[0] = racc[m][nb][0];
          d[1] = racc[m][nb][1];
          d[8 * RP] = racc[m][nb][2];
          d[8 * RP + 1] = racc[m][nb][3];
        }
      __syncthreads();
      for (int i = tid; i < cc * RP; i += kNT) {
        const int r = i % RP;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) s += red[(size_t)w * CHA * RP + i];
        if (r < g.R) part[(size_t)(c0 + i / RP) * g.R + r] = s;
      }
      __syncthreads();
    }
  }
  if (CONTRACT) {
#pragma unroll
    for (int j = 0; j < MBW; ++j) {
      float* p = Out + (size_t)(2 * tq) * g.pp + warp * WCOLS + j * 16 + gq;
#pragma unroll
      for (int nb = 0; nb < NB; ++nb) {
        p[(nb * 8) * g.pp] = cacc[j][nb][0];
        p[(nb * 8 + 1) * g.pp] = cacc[j][nb][1];
        p[(nb * 8) * g.pp + 8] = cacc[j][nb][2];
        p[(nb * 8 + 1) * g.pp + 8] = cacc[j][nb][3];
      }
    }
  }
}

template <int RP, int MBW, bool CORE>
__global__ void __launch_bounds__(kNT, 2) cp4_bwdf_mma_kernel(const BGeom g, const float* __restrict__ X,
                                                             const float* __restrict__ dU,
                                                             const float* __restrict__ K0,
                                                             const float* __restrict__ K1,
                                                             const float* __restrict__ KH,
                                                             const float* __restrict__ KW,
                                                             const float* __restrict__ KC, float* __restrict__ ws) {
  using K = BCfg<RP>;
  constexpr int WCOLS = MBW * 16, COLS = kWarps * WCOLS, CPL = (MBW + 1) / 2;
  constexpr int XP = COLS + 12, ZP = COLS + 4;
  constexpr int kXR = kFifo * kGC * XP > kWarps * K::CHA * RP ? kFifo * kGC * XP : kWarps * K::CHA * RP;
  extern __shared__ __align__(16) float smem[];
  float* Xf = smem;                          // FIFO [kFifo][kGC][XP]; between passes: reduction scratch
  float* Ps = Xf + kXR;                      // [RP][pp]
  float* Qs = Ps + (size_t)RP * g.pp;        // [RP][pp]
  float* Zh = Qs + (size_t)RP * g.pp;        // [RP][ZP]  Z, later Qt; zero outside the tile's interior
  float* Fh = Zh + RP * ZP;                  // factor planes hi | lo of the current channel chunk
  constexpr int NG = CORE ? 9 : 6;           // rows of the spatial-factor gradient
  float* KHs = Fh + 2 * K::CHA * K::FIN;     // [3][RP] KH then [3][RP] KW, or the [9][RP] core
  float* redk = KHs + 9 * RP;                // [kNT][NG]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  int b = blockIdx.x;
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  const size_t HW = (size_t)g.H * g.W;
  const float* X_n = X + (size_t)n * g.C * HW;
  const float* dU_n = dU + (size_t)n * g.T * HW;
  float* part = ws + (size_t)blockIdx.x * g.nparam;

  for (int i = tid; i < NG * RP; i += kNT) {
    const int r = i % RP, row = i / RP;
    const float* src = CORE ? KC + (size_t)row * g.Rs : (row < 3 ? KH + (size_t)row * g.Rs : KW + (size_t)(row - 3) * g.Rs);
    KHs[i] = r < g.R ? __ldg(src + g.r0 + r) : 0.f;
  }
  for (int i = tid; i < RP * ZP / 4; i += kNT) reinterpret_cast<float4*>(Zh)[i] = make_float4(0.f, 0.f, 0.f, 0.f);
  // the slack columns of P and Q (read by the last strip of a row, never written) must be finite
  for (int i = tid; i < 2 * RP * (g.pp - COLS); i += kNT) {
    const int row = i / (g.pp - COLS), col = COLS + i % (g.pp - COLS);
    Ps[(size_t)row * g.pp + col] = 0.f;   // rows RP..2RP-1 are Q's
  }

  // this lane's halo pixels: column = halo pixel index, warp w owns [w*WCOLS, (w+1)*WCOLS)
  const float* gpx[CPL];
  const float* gpu[CPL];
  int gsz[CPL];
#pragma unroll
  for (int q = 0; q < CPL; ++q) {
    const int wc = lane + 32 * q;
    const int hp = warp * WCOLS + wc;
    const int hy = hp / g.TWh, hx = hp - hy * g.TWh;
    const int gy = h0 - 1 + hy, gx = w0 - 1 + hx;
    const bool ok = wc < WCOLS && hp < g.HPX && gy >= 0 && gy < g.H && gx >= 0 && gx < g.W;
    const int off = ok ? gy * g.W + gx : 0;
    gpx[q] = X_n + off;
    gpu[q] = dU_n + off;
    gsz[q] = ok ? 4 : 0;
  }

  // ---- pass 1: P ----
  stream_pass<RP, MBW, true, false>(g, X_n, g.C, K1, Xf, Fh, Ps, nullptr, nullptr, gpx, gsz, tid);
  __syncthreads();

  // ---- stencil A: Z on the interior pixels ----
  const int r = tid % RP;   // fixed per thread (kNT is a multiple of RP)
  float kh[3], kw[3], w9[9];   // separable factors, and the 3x3 filter of this thread's rank either way
#pragma unroll
  for (int t = 0; t < 3; ++t) { kh[t] = CORE ? 0.f : KHs[t * RP + r]; kw[t] = CORE ? 0.f : KHs[(3 + t) * RP + r]; }
#pragma unroll
  for (int t = 0; t < 9; ++t) w9[t] = CORE ? KHs[t * RP + r] : kh[t / 3] * kw[t % 3];
  constexpr int SW = 8;
  const int spr = (g.TW + SW - 1) / SW;
  const int items = g.TH * spr;
  for (int it = tid / RP; it < items; it += kNT / RP) {
    const int oy = it / spr, x0 = (it - oy * spr) * SW;
    float z[SW];
#pragma unroll
    for (int j = 0; j < SW; ++j) z[j] = 0.f;
    const float* p = Ps + (size_t)r * g.pp + oy * g.TWh + x0;
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
      float v[SW + 2];
#pragma unroll
      for (int j = 0; j < SW + 2; ++j) v[j] = p[j];
      p += g.TWh;
#pragma unroll
      for (int j = 0; j < SW; ++j) {
        z[j] = fmaf(w9[dy * 3 + 0], v[j], z[j]);
        z[j] = fmaf(w9[dy * 3 + 1], v[j + 1], z[j]);
        z[j] = fmaf(w9[dy * 3 + 2], v[j + 2], z[j]);
      }
    }
    float* zd = Zh + r * ZP + (oy + 1) * g.TWh + x0 + 1;
#pragma unroll
    for (int j = 0; j < SW; ++j)
      if (x0 + j < g.TW) zd[j] = z[j];
  }
  __syncthreads();

  // ---- pass 2: Q and dK0 ----
  stream_pass<RP, MBW, true, true>(g, dU_n, g.T, K0, Xf, Fh, Qs, Zh, part, gpu, gsz, tid);
  __syncthreads();

  // ---- stencil B: Qt on the interior pixels, dKH, dKW ----
  float dk[NG];   // separable: dKH[0..2], dKW[0..2];  free core: dKC[y*3 + x]
#pragma unroll
  for (int t = 0; t < NG; ++t) dk[t] = 0.f;
  for (int it = tid / RP; it < items; it += kNT / RP) {
    const int oy = it / spr, x0 = (it - oy * spr) * SW;
    float qt[SW], qc[SW];
#pragma unroll
    for (int j = 0; j < SW; ++j) qt[j] = 0.f;
    const float* p = Ps + (size_t)r * g.pp + oy * g.TWh + x0;
    const float* q = Qs + (size_t)r * g.pp + oy * g.TWh + x0;
    // the centre of the neighbourhood is the interior pixel; strips may run past the tile's last column
#pragma unroll
    for (int j = 0; j < SW; ++j) qc[j] = (x0 + j < g.TW) ? q[g.TWh + j + 1] : 0.f;
    float vc[3][SW];           // separable: vc[x][j] = sum_y KH[y] P[oy+y][x0+j+x]
    if (!CORE) {
#pragma unroll
      for (int j = 0; j < SW; ++j) vc[0][j] = vc[1][j] = vc[2][j] = 0.f;
    }
#pragma unroll
    for (int dy = 0; dy < 3; ++dy) {
      float v[SW + 2], u[SW + 2];
#pragma unroll
      for (int j = 0; j < SW + 2; ++j) { v[j] = p[j]; u[j] = q[j]; }
      p += g.TWh;
      q += g.TWh;
#pragma unroll
      for (int j = 0; j < SW; ++j) {
        // flipped taps: row dy of the neighbourhood carries filter row 2-dy, column dx carries filter column 2-dx
        qt[j] = fmaf(w9[(2 - dy) * 3 + 2], u[j], qt[j]);
        qt[j] = fmaf(w9[(2 - dy) * 3 + 1], u[j + 1], qt[j]);
        qt[j] = fmaf(w9[(2 - dy) * 3 + 0], u[j + 2], qt[j]);
        if (CORE) {
          dk[dy * 3 + 0] = fmaf(qc[j], v[j], dk[dy * 3 + 0]);
          dk[dy * 3 + 1] = fmaf(qc[j], v[j + 1], dk[dy * 3 + 1]);
          dk[dy * 3 + 2] = fmaf(qc[j], v[j + 2], dk[dy * 3 + 2]);
        } else {
          const float th_ = fmaf(kw[2], v[j + 2], fmaf(kw[1], v[j + 1], kw[0] * v[j]));   // sum_x KW[x] P[oy+dy][..+x]
          dk[dy] = fmaf(qc[j], th_, dk[dy]);
          vc[0][j] = fmaf(kh[dy], v[j], vc[0][j]);
          vc[1][j] = fmaf(kh[dy], v[j + 1], vc[1][j]);
          vc[2][j] = fmaf(kh[dy], v[j + 2], vc[2][j]);
        }
      }
    }
    if (!CORE) {
#pragma unroll
      for (int j = 0; j < SW; ++j)
#pragma unroll
        for (int t = 0; t < 3; ++t) dk[3 + t] = fmaf(qc[j], vc[t][j], dk[3 + t]);
    }
    float* zd = Zh + r * ZP + (oy + 1) * g.TWh + x0 + 1;
#pragma unroll
    for (int j = 0; j < SW; ++j)
      if (x0 + j < g.TW) zd[j] = qt[j];
  }
#pragma unroll
  for (int t = 0; t < NG; ++t) redk[tid * NG + t] = dk[t];
  __syncthreads();
  for (int i = tid; i < NG * RP; i += kNT) {
    // threads rr + RP*k hold the sums of rank rr: add them in k order
    const int rr = i % RP, t = i / RP;
    float s = 0.f;
    for (int k = 0; k < kNT / RP; ++k) s += redk[(rr + RP * k) * NG + t];
    if (rr < g.R) part[(size_t)(g.T + g.C + t) * g.R + rr] = s;
  }

  // ---- pass 3: dK1 ----
  stream_pass<RP, MBW, false, true>(g, X_n, g.C, nullptr, Xf, Fh, nullptr, Zh, part + (size_t)g.T * g.R, gpx, gsz, tid);
}

// =====================================================================================================
// Backward-filter from saved rank planes.  Inside one training step the forward kernel has already
// computed P = K1^T X and the backward-data kernel Q = K0^T dU; when they write these planes ([N][R][H][W],
// a quarter of the input at C = 4R) the factor gradients need no channel contraction any more:
//   load the P and Q halo tiles, one merged stencil phase (Z, Qt, dKH / dKW or dKC), then two reduce-only passes
//   dK0^T[r, t] = sum_px Z[r, px] dU[t, px],  dK1^T[r, c] = sum_px Qt[r, px] X[c, px]   over the tile's own pixels,
// with M = ranks (the Z fragments of a warp's pixels are split once and stay in registers), N = channels and
// K = pixels; both fragments come from ldmatrix because their K index is contiguous in shared memory.
// =====================================================================================================
struct SGeom {
  int N, C, T, H, W, R, Rs, r0;
  int TH, TW, TWh, HPX, OPX, tilesH, tilesW;
  int MBW;     // 16-pixel blocks of the output tile per warp
  int nparam;  // (T + C + 6 or 9) * R floats per partial
  int pp;      // row pitch of the P and Q halo planes (odd)
  int vec;     // 1: TW, W and the tile origins are multiples of 4 and the tensors 16-byte aligned: 16-byte copies
  int h0, w0;  // origin of the CTA's tile (filled in by the kernel)
  int S, t_slice, c_slice;  // channel slices per tile (gridDim.y) and channels per slice: small images with many
                            // channels have too few tiles to fill the GPU; the slices own disjoint rows of dK0 / dK1
};

template <int RP>
struct SCfg {
  static constexpr int RPZ = RP < 16 ? 16 : RP;              // rows of the Z planes: whole 16-rank mma blocks
  static constexpr int MR = RPZ / 16;
  static constexpr int MB2 = MR <= 1 ? 4 : MR == 2 ? 2 : 1;  // 16-channel groups whose sums stay in registers
  static constexpr int CHA = MB2 * 16;
};

template <int RP>
size_t bwdf_saved_smem_floats(const SGeom& g) {
  using K = SCfg<RP>;
  const int cols = kWarps * g.MBW * 16;
  const size_t fifo = (size_t)kFifo * kGC * (cols + 12);
  const size_t red = (size_t)kWarps * K::CHA * K::RPZ;
  return std::max(fifo, red) + 2 * (size_t)RP * g.pp + 2 * (size_t)K::RPZ * (cols + 4) + 9 * RP + kNT * 9;
}

// part[ch][r] = sum over this tile's pixels of src[ch][px] * Zs[r][px]
// ALLIN: the FIFO has a stage for every group of a chunk, so all of them are in flight before the first is used
template <int RP, int MBW, bool ALLIN>
__device__ __forceinline__ void reduce_pass(const SGeom& g, const float* __restrict__ src_n, int nch, float* Xf,
                                            const float* Zs, float* __restrict__ part,
                                            const float* const (&gp)[(MBW + 1) / 2], const int (&gsz)[(MBW + 1) / 2],
                                            int tid) {
  using K = SCfg<RP>;
  constexpr int RPZ = K::RPZ, MR = K::MR, MB2 = K::MB2, CHA = K::CHA;
  constexpr int WCOLS = MBW * 16, COLS = kWarps * WCOLS, CPL = (MBW + 1) / 2;
  constexpr int XP = COLS + 12, ZP = COLS + 4, KP = 2 * MBW;
  constexpr bool HOIST = KP * MR * 8 <= 32;
  const int lane = tid & 31, warp = tid >> 5, gq = lane >> 2, tq = lane & 3;
  const size_t HW = (size_t)g.H * g.W;
  const unsigned xw_s = (unsigned)__cvta_generic_to_shared(Xf + warp * WCOLS + lane);
  const float* xw = Xf + warp * WCOLS;
  // ldmatrix row addresses: A tiles (rows 0-7 | 8-15) x (pixels 0-3 | 4-7); B tiles (channels 0-7 | 8-15) likewise
  const float* za = Zs + ((lane & 7) + ((lane >> 3) & 1) * 8) * ZP + warp * WCOLS + (lane >> 4) * 4;
  const int xb = ((lane >> 4) * 8 + (lane & 7)) * XP + ((lane >> 3) & 1) * 4;
  // 16-byte copy role (g.vec): lane = (channel row within an instruction, 4-pixel chunk of the warp's columns)
  constexpr int VCH = WCOLS / 4;                        // chunks per warp
  constexpr int VCPI = (32 % VCH == 0) ? 32 / VCH : 1;  // channel rows per instruction (vec needs 32 % VCH == 0)
  const int vrow = lane / VCH, vchunk = lane % VCH;
  const float* vsrc = src_n;
  int vsz = 0;
  if (g.vec) {
    const int op = warp * WCOLS + vchunk * 4;
    const int oy = op / g.TW, ox = op - oy * g.TW;
    const int gy = g.h0 + oy, gx = g.w0 + ox;
    if (op < g.OPX && gy < g.H && gx < g.W) { vsrc = src_n + (size_t)gy * g.W + gx; vsz = 16; }
  }
  const unsigned vdst = (unsigned)__cvta_generic_to_shared(Xf + vrow * XP + warp * WCOLS + vchunk * 4);

  uint32_t zh[HOIST ? KP : 1][MR][4], zl[HOIST ? KP : 1][MR][4];
  auto load_z = [&](int kp, int mr, uint32_t (&h)[4], uint32_t (&l)[4]) {
    uint32_t v[4];
    ldmatrix_x4(v, za + mr * 16 * ZP + kp * 8);
#pragma unroll
    for (int e = 0; e < 4; ++e) split_tf32_bits(v[e], h[e], l[e]);
  };
  if (HOIST) {
#pragma unroll
    for (int kp = 0; kp < KP; ++kp)
#pragma unroll
      for (int mr = 0; mr < MR; ++mr) load_z(kp, mr, zh[kp][mr], zl[kp][mr]);
  }

  for (int c0 = 0; c0 < nch; c0 += CHA) {
    const int cc = min(CHA, nch - c0);
    const int ng = (cc + kGC - 1) / kGC;
    auto issue = [&](int grp) {
      if (grp < ng) {
        const size_t coff = (size_t)(c0 + grp * kGC) * HW;
        if (g.vec) {
          // 16-byte copies: a lane owns four consecutive pixels (never across a tile row: TW % 4 == 0) of
          // 32 / (4*MBW) channel rows per instruction
          const unsigned dst = vdst + (unsigned)((grp % (ALLIN ? MB2 : kFifo)) * kGC * XP * 4);
          if (grp * kGC + kGC <= cc) {      // all channels of the group exist: no per-copy selects
            const float* sp = vsrc + coff + (size_t)vrow * HW;
#pragma unroll
            for (int jc = 0; jc < kGC / VCPI; ++jc) {
              cp_async16_s(dst + (unsigned)(jc * VCPI * XP * 4), sp, vsz);
              sp += (size_t)VCPI * HW;
            }
          } else {
#pragma unroll
            for (int jc = 0; jc < kGC / VCPI; ++jc) {
              const int ch = jc * VCPI + vrow;
              const bool cin = grp * kGC + ch < cc;
              cp_async16_s(dst + (unsigned)(jc * VCPI * XP * 4), cin ? vsrc + coff + (size_t)ch * HW : src_n, cin ? vsz : 0);
            }
          }
        } else {
          const unsigned dst = xw_s + (unsigned)((grp % (ALLIN ? MB2 : kFifo)) * kGC * XP * 4);
          if (grp * kGC + kGC <= cc) {
#pragma unroll
            for (int q = 0; q < CPL; ++q)
              if (CPL * 32 == WCOLS || lane + 32 * q < WCOLS) {
                const float* sp = gp[q] + coff;
#pragma unroll
                for (int jc = 0; jc < kGC; ++jc) {
                  cp_async4_s(dst + (unsigned)((jc * XP + 32 * q) * 4), sp, gsz[q]);
                  sp += HW;
                }
              }
          } else {
#pragma unroll
            for (int q = 0; q < CPL; ++q)
              if (CPL * 32 == WCOLS || lane + 32 * q < WCOLS) {
#pragma unroll
                for (int jc = 0; jc < kGC; ++jc) {
                  const bool cin = grp * kGC + jc < cc;
                  cp_async4_s(dst + (unsigned)((jc * XP + 32 * q) * 4), cin ? gp[q] + coff + (size_t)jc * HW : src_n,
                              cin ? gsz[q] : 0);
                }
              }
          }
        }
      }
      cp_async_commit();
    };
    constexpr int NST = ALLIN ? MB2 : kFifo;
#pragma unroll
    for (int s = 0; s < (ALLIN ? MB2 : kFifo - 1); ++s) issue(s);
    float racc[MB2][MR][2][4];
#pragma unroll
    for (int m = 0; m < MB2; ++m)
#pragma unroll
      for (int mr = 0; mr < MR; ++mr)
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) racc[m][mr][nb][0] = racc[m][mr][nb][1] = racc[m][mr][nb][2] = racc[m][mr][nb][3] = 0.f;
#pragma unroll
    for (int grp = 0; grp < MB2; ++grp) {
      if (grp < ng) {
        if (ALLIN) {
          cp_async_wait_upto(MB2 - 1 - grp);
        } else {
          issue(grp + kFifo - 1);
          cp_async_wait<kFifo - 1>();
        }
        __syncwarp();
        const float* xs = xw + (grp % NST) * kGC * XP + xb;
#pragma unroll
        for (int kp = 0; kp < KP; ++kp) {
          uint32_t b[4], bh[4], bl[4];   // [channel block 0: pixels 0-3, 4-7 | channel block 1: pixels 0-3, 4-7]
          ldmatrix_x4(b, xs + kp * 8);
#pragma unroll
          for (int e = 0; e < 4; ++e) split_tf32_bits(b[e], bh[e], bl[e]);
#pragma unroll
          for (int mr = 0; mr < MR; ++mr) {
            uint32_t th[4], tl[4];
            if (!HOIST) load_z(kp, mr, th, tl);
            const uint32_t(&ah)[4] = HOIST ? zh[kp][mr] : th;
            const uint32_t(&al)[4] = HOIST ? zl[kp][mr] : tl;
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
              const uint32_t h2[2] = {bh[2 * nb], bh[2 * nb + 1]}, l2[2] = {bl[2 * nb], bl[2 * nb + 1]};
              mma_tf32(racc[grp][mr][nb], al, h2);
              mma_tf32(racc[grp][mr][nb], ah, l2);
              mma_tf32(racc[grp][mr][nb], ah, h2);
            }
          }
        }
        __syncwarp();  // every lane has read this FIFO stage: a later group may overwrite it
      }
    }
    cp_async_wait<0>();
    // the warps' partial sums meet in shared memory (over the FIFO) and are added in warp order
    float* red = Xf;
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MB2; ++m)
#pragma unroll
      for (int mr = 0; mr < MR; ++mr)
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
          float* d = red + ((size_t)warp * CHA + m * 16 + nb * 8 + 2 * tq) * RPZ + mr * 16 + gq;
          d[0] = racc[m][mr][nb][0];
          d[RPZ] = racc[m][mr][nb][1];
          d[8] = racc[m][mr][nb][2];
          d[RPZ + 8] = racc[m][mr][nb][3];
        }
    __syncthreads();
    for (int i = tid; i < cc * RPZ; i += kNT) {
      const int r = i % RPZ;
      float s = 0.f;
#pragma unroll
      for (int w = 0; w < kWarps; ++w) s += red[(size_t)w * CHA * RPZ + i];
      if (r < g.R) part[(size_t)(c0 + i / RPZ) * g.R + r] = s;
    }
    __syncthreads();
  }
}

// PART 0: everything.  PART 1: Z and dK0 only (needs the forward's plane P only).  PART 2: Qt, dK1 and the
// spatial-factor gradients.  The two halves write disjoint rows of the CTA's partial vector, so a step can run
// them side by side on two streams.
template <int RP, int MBW, bool CORE, int PART>
__global__ void __launch_bounds__(kNT, 2) cp4_bwdf_saved_kernel(const SGeom g_in, const float* __restrict__ X,
                                                               const float* __restrict__ dU,
                                                               const float* __restrict__ Pg,
                                                               const float* __restrict__ Qg,
                                                               const float* __restrict__ KH,
                                                               const float* __restrict__ KW,
                                                               const float* __restrict__ KC, float* __restrict__ ws) {
  using K = SCfg<RP>;
  constexpr int RPZ = K::RPZ;
  constexpr int WCOLS = MBW * 16, COLS = kWarps * WCOLS, CPL = (MBW + 1) / 2;
  constexpr int XP = COLS + 12, ZP = COLS + 4;
  constexpr int kXR = kFifo * kGC * XP > kWarps * K::CHA * RPZ ? kFifo * kGC * XP : kWarps * K::CHA * RPZ;
  constexpr int NG = CORE ? 9 : 6;
  constexpr bool DOZ = PART != 2, DOQ = PART != 1;
  SGeom g = g_in;
  extern __shared__ __align__(16) float smem[];
  float* Xf = smem;                          // FIFO stages 0, 1; at the end of a chunk: reduction scratch
  float* Ps = Xf + kXR;                      // [RP][pp]   halo tile of P   } dead after the stencil phase: further
  float* Qs = Ps + (size_t)RP * g.pp;        // [RP][pp]   halo tile of Q   } FIFO stages when they are large enough
  float* Zs = Qs + (size_t)RP * g.pp;        // [RPZ][ZP]  Z on the tile's pixels, zero elsewhere
  float* Qts = Zs + RPZ * ZP;                // [RPZ][ZP]  Qt
  float* KHs = Qts + RPZ * ZP;               // [3][RP] KH then [3][RP] KW, or the [9][RP] core
  float* redk = KHs + 9 * RP;                // [kNT][NG]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

  int b = blockIdx.x;
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  g.h0 = h0;
  g.w0 = w0;
  const size_t HW = (size_t)g.H * g.W;
  float* part = ws + (size_t)blockIdx.x * g.nparam;
  const int sl = blockIdx.y;   // channel slice: every slice repeats the stencil phase, slice 0 writes the spatial sums
  const int t_lo = min(g.T, sl * g.t_slice), t_hi = min(g.T, t_lo + g.t_slice);
  const int c_lo = min(g.C, sl * g.c_slice), c_hi = min(g.C, c_lo + g.c_slice);

  // halo tiles of P and Q: one column per thread, one 4-byte copy per rank plane; zero outside the image and in the
  // slack columns the last strip of a row reads
  {
    const float* Pn = Pg + ((size_t)n * g.Rs + g.r0) * HW;
    const float* Qn = Qg + ((size_t)n * g.Rs + g.r0) * HW;
    for (int hp = tid; hp < g.pp; hp += kNT) {
      const int hy = hp / g.TWh, hx = hp - hy * g.TWh;
      const int gy = h0 - 1 + hy, gx = w0 - 1 + hx;
      const bool ok = hp < g.HPX && gy >= 0 && gy < g.H && gx >= 0 && gx < g.W;
      const size_t off = ok ? (size_t)gy * g.W + gx : 0;
      const unsigned dp = (unsigned)__cvta_generic_to_shared(Ps + hp), dq = (unsigned)__cvta_generic_to_shared(Qs + hp);
      for (int r = 0; r < RP; ++r) {
        const int sz = ok && r < g.R ? 4 : 0;
        const size_t o = sz ? (size_t)r * HW + off : 0;
        cp_async4_s(dp + (unsigned)(r * g.pp * 4), Pn + o, sz);
        if (DOQ) cp_async4_s(dq + (unsigned)(r * g.pp * 4), Qn + o, sz);
      }
    }
    cp_async_commit();
  }
  for (int i = tid; i < NG * RP; i += kNT) {
    const int r = i % RP, row = i / RP;
    const float* src = CORE ? KC + (size_t)row * g.Rs : (row < 3 ? KH + (size_t)row * g.Rs : KW + (size_t)(row - 3) * g.Rs);
    KHs[i] = r < g.R ? __ldg(src + g.r0 + r) : 0.f;
  }
  for (int i = tid; i < 2 * RPZ * ZP / 4; i += kNT) reinterpret_cast<float4*>(Zs)[i] = make_float4(0.f, 0.f, 0.f, 0.f);

  // this lane's pixels of the tile: column = pixel index in the tile, warp w owns [w*WCOLS, (w+1)*WCOLS)
  const float* gpx[CPL];
  const float* gpu[CPL];
  int gsz[CPL];
#pragma unroll
  for (int q = 0; q < CPL; ++q) {
    const int wc = lane + 32 * q;
    const int op = warp * WCOLS + wc;
    const int oy = op / g.TW, ox = op - oy * g.TW;
    const int gy = h0 + oy, gx = w0 + ox;
    const bool ok = wc < WCOLS && op < g.OPX && gy < g.H && gx < g.W;
    const int off = ok ? gy * g.W + gx : 0;
    gpx[q] = X + ((size_t)n * g.C + c_lo) * HW + off;
    gpu[q] = dU + ((size_t)n * g.T + t_lo) * HW + off;
    gsz[q] = ok ? 4 : 0;
  }
  cp_async_wait<0>();
  __syncthreads();

  // ---- merged stencil phase: Z, Qt and the spatial-factor gradients ----
  {
    const int r = tid % RP;   // fixed per thread (kNT is a multiple of RP)
    float kh[3], kw[3], w9[9];
#pragma unroll
    for (int t = 0; t < 3; ++t) { kh[t] = CORE ? 0.f : KHs[t * RP + r]; kw[t] = CORE ? 0.f : KHs[(3 + t) * RP + r]; }
#pragma unroll
    for (int t = 0; t < 9; ++t) w9[t] = CORE ? KHs[t * RP + r] : kh[t / 3] * kw[t % 3];
    constexpr int SW = 8;
    const int spr = (g.TW + SW - 1) / SW;
    const int items = g.TH * spr;
    float dk[NG];
#pragma unroll
    for (int t = 0; t < NG; ++t) dk[t] = 0.f;
    for (int it = tid / RP; it < items; it += kNT / RP) {
      const int oy = it / spr, x0 = (it - oy * spr) * SW;
      float z[SW], qt[SW], qc[SW];
#pragma unroll
      for (int j = 0; j < SW; ++j) z[j] = qt[j] = 0.f;
      const float* p = Ps + (size_t)r * g.pp + oy * g.TWh + x0;
      const float* q = Qs + (size_t)r * g.pp + oy * g.TWh + x0;
#pragma unroll
      for (int j = 0; j < SW; ++j) qc[j] = (DOQ && x0 + j < g.TW) ? q[g.TWh + j + 1] : 0.f;
      float vc[3][SW];
      if (!CORE) {
#pragma unroll
        for (int j = 0; j < SW; ++j) vc[0][j] = vc[1][j] = vc[2][j] = 0.f;
      }
#pragma unroll
      for (int dy = 0; dy < 3; ++dy) {
        float v[SW + 2], u[SW + 2];
#pragma unroll
        for (int j = 0; j < SW + 2; ++j) { v[j] = p[j]; u[j] = DOQ ? q[j] : 0.f; }
        p += g.TWh;
        q += g.TWh;
#pragma unroll
        for (int j = 0; j < SW; ++j) {
          if (DOZ) {
            z[j] = fmaf(w9[dy * 3 + 0], v[j], z[j]);
            z[j] = fmaf(w9[dy * 3 + 1], v[j + 1], z[j]);
            z[j] = fmaf(w9[dy * 3 + 2], v[j + 2], z[j]);
          }
          if (DOQ) {
            qt[j] = fmaf(w9[(2 - dy) * 3 + 2], u[j], qt[j]);
            qt[j] = fmaf(w9[(2 - dy) * 3 + 1], u[j + 1], qt[j]);
            qt[j] = fmaf(w9[(2 - dy) * 3 + 0], u[j + 2], qt[j]);
            if (CORE) {
              dk[dy * 3 + 0] = fmaf(qc[j], v[j], dk[dy * 3 + 0]);
              dk[dy * 3 + 1] = fmaf(qc[j], v[j + 1], dk[dy * 3 + 1]);
              dk[dy * 3 + 2] = fmaf(qc[j], v[j + 2], dk[dy * 3 + 2]);
            } else {
              const float th_ = fmaf(kw[2], v[j + 2], fmaf(kw[1], v[j + 1], kw[0] * v[j]));
              dk[dy] = fmaf(qc[j], th_, dk[dy]);
              vc[0][j] = fmaf(kh[dy], v[j], vc[0][j]);
              vc[1][j] = fmaf(kh[dy], v[j + 1], vc[1][j]);
              vc[2][j] = fmaf(kh[dy], v[j + 2], vc[2][j]);
            }
          }
        }
      }
      if (!CORE && DOQ) {
#pragma unroll
        for (int j = 0; j < SW; ++j)
#pragma unroll
          for (int t = 0; t < 3; ++t) dk[3 + t] = fmaf(qc[j], vc[t][j], dk[3 + t]);
      }
      float* zd = Zs + r * ZP + oy * g.TW + x0;
      float* qd = Qts + r * ZP + oy * g.TW + x0;
#pragma unroll
      for (int j = 0; j < SW; ++j)
        if (x0 + j < g.TW) {
          if (DOZ) zd[j] = z[j];
          if (DOQ) qd[j] = qt[j];
        }
    }
    if (DOQ) {
#pragma unroll
      for (int t = 0; t < NG; ++t) redk[tid * NG + t] = dk[t];
    }
  }
  __syncthreads();
  if (DOQ && sl == 0) {
    for (int i = tid; i < NG * RP; i += kNT) {
      const int rr = i % RP, t = i / RP;
      float s = 0.f;
      for (int k = 0; k < kNT / RP; ++k) s += redk[(rr + RP * k) * NG + t];
      if (rr < g.R) part[(size_t)(g.T + g.C + t) * g.R + rr] = s;
    }
  }

  // every group of a 16*MB2-channel chunk gets its own FIFO stage when the dead P / Q tiles give the room
  // (the host sizes their pitch for it), else two stages rotate
  constexpr bool kAllIn = kXR == kFifo * kGC * XP;   // the first two stages are exactly the FIFO, the tiles follow
  const bool allin = kAllIn && (size_t)kFifo * kGC * XP + 2 * (size_t)RP * g.pp >= (size_t)K::MB2 * kGC * XP;
  __syncthreads();   // the stencil phase is over: P and Q may be overwritten
  const float* dUs = dU + ((size_t)n * g.T + t_lo) * HW;
  const float* Xs = X + ((size_t)n * g.C + c_lo) * HW;
  float* part0 = part + (size_t)t_lo * g.R;
  float* part1 = part + (size_t)(g.T + c_lo) * g.R;
  if (allin) {
    if (DOZ) reduce_pass<RP, MBW, true>(g, dUs, t_hi - t_lo, Xf, Zs, part0, gpu, gsz, tid);
    if (DOQ) reduce_pass<RP, MBW, true>(g, Xs, c_hi - c_lo, Xf, Qts, part1, gpx, gsz, tid);
  } else {
    if (DOZ) reduce_pass<RP, MBW, false>(g, dUs, t_hi - t_lo, Xf, Zs, part0, gpu, gsz, tid);
    if (DOQ) reduce_pass<RP, MBW, false>(g, Xs, c_hi - c_lo, Xf, Qts, part1, gpx, gsz, tid);
  }
}

template <int RP>
bool plan_saved(const Cp4BwdFilterArgs& a, const DeviceInfo& di, SGeom* out, size_t* smem_out) {
  SGeom best{};
  double best_cost = 1e300;
  size_t best_smem = 0;
  int fTH = 0, fTW = 0;
  if (const char* e = getenv("B200CP_MMA_TILE")) {  // "TH,TW": experiments
    if (sscanf(e, "%d,%d", &fTH, &fTW) != 2) fTH = fTW = 0;
  }
  for (int TW = 1; TW <= std::min(a.W, 64); ++TW) {
    if (fTW ? TW != std::min(fTW, a.W) : (TW != a.W && a.W % TW != 0 && TW % 8 != 0)) continue;
    for (int TH = 1; TH <= std::min(a.H, 64); ++TH) {
      if (fTH && TH != std::min(fTH, a.H)) continue;
      SGeom g{};
      g.TH = TH; g.TW = TW; g.TWh = TW + 2; g.HPX = (TH + 2) * g.TWh; g.OPX = TH * TW;
      g.MBW = ceil_div(ceil_div(g.OPX, 16), kWarps);
      if (g.MBW > 4) break;
      g.pp = (g.HPX + 11) | 1;
      {  // room for the remaining FIFO stages of a chunk in the dead P / Q tiles, when that costs little
        const int xp = kWarps * g.MBW * 16 + 12, extra = (SCfg<RP>::MB2 - kFifo) * kGC * xp;
        const int want = (ceil_div(std::max(extra, 0), 2 * RP)) | 1;
        if (want > g.pp && want <= g.pp + 32) g.pp = want;
      }
      const size_t smem = sizeof(float) * bwdf_saved_smem_floats<RP>(g);
      if ((int)smem > di.smem_optin) break;
      const int cps = std::max(1, std::min(2, (int)((228 * 1024) / (smem + 1024))));
      const long ctas = (long)a.N * ceil_div(a.H, TH) * ceil_div(a.W, TW);
      const long rounds = (ctas + (long)di.sm_count * cps - 1) / ((long)di.sm_count * cps);
      // rows of TW pixels are read as 4*TW-byte segments at any alignment: short rows waste sectors
      const double seg = (TW * 4.0) / (32.0 * ceil_div(TW * 4 + 28, 32));
      const double groups = (ceil_div(a.C, 16) + ceil_div(a.T, 16)) * (2.0 * g.MBW * (10 + 6.0 * std::max(1, RP / 16)) + 60) *
                            (0.5 + 0.5 / seg);
      const double stencil = (double)ceil_div(TH * ceil_div(TW, 8) * RP, kNT) * 600.0;
      const double tile = groups + stencil + 4.0 * RP + 600.0;
      const double occupancy = 16.0 / (cps * kWarps);
      const double cost = (double)ctas * tile / di.sm_count * occupancy + 2000.0 * rounds;
      if (cost < best_cost) { best_cost = cost; best = g; best_smem = smem; }
    }
  }
  if (best.TH == 0) return false;
  *out = best;
  *smem_out = best_smem;
  return true;
}

template <int RP, int MBW, bool CORE, int PART>
int launch_saved_part(const SGeom& g, size_t smem, long ctas, const Cp4BwdFilterArgs& a, const float* P, const float* Q,
                      cudaStream_t st) {
  auto kern = cp4_bwdf_saved_kernel<RP, MBW, CORE, PART>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<dim3((unsigned)ctas, (unsigned)g.S), kNT, smem, st>>>(g, a.X, a.dU, P, Q, a.KH, a.KW, a.KC, (float*)a.ws);
  B200CP_LAUNCH_OK("cp4_bwdf_saved_kernel");
  return B200CP_OK;
}

// part 0: the whole kernel, then the sum of the partials.  part 1 / 2: one half, no sum.  part 3: the sum only.
template <int RP, int MBW>
int launch_saved(const SGeom& g, size_t smem, const Cp4BwdFilterArgs& a, const float* P, const float* Q, cudaStream_t st,
                 int part) {
  const long ctas = (long)a.N * g.tilesH * g.tilesW;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: too many tiles");
  const size_t need = (size_t)ctas * g.nparam * sizeof(float);
  if (a.ws_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "cp4 bwd-filter: workspace of %zu bytes needed, %zu given", need, a.ws_bytes);
  int rc = B200CP_OK;
  if (part == 3) {
  } else if (a.KC) {
    if (part != 0) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: internal: the free-core kernel is not split");
    rc = launch_saved_part<RP, MBW, true, 0>(g, smem, ctas, a, P, Q, st);
  } else if (part == 0) {
    rc = launch_saved_part<RP, MBW, false, 0>(g, smem, ctas, a, P, Q, st);
  } else if (part == 1) {
    rc = launch_saved_part<RP, MBW, false, 1>(g, smem, ctas, a, P, Q, st);
  } else {
    rc = launch_saved_part<RP, MBW, false, 2>(g, smem, ctas, a, P, Q, st);
  }
  if (rc) return rc;
  if (part == 0 || part == 3)
    return cp4_reduce_partials_launch((const float*)a.ws, (int)ctas, g.nparam, a.R, a.Rs, a.r0, a.dK, st);
  return B200CP_OK;
}

template <int RP>
int run_saved(const Cp4BwdFilterArgs& a, const float* P, const float* Q, const DeviceInfo& di, cudaStream_t st, int part) {
  SGeom g{};
  size_t smem = 0;
  if (!plan_saved<RP>(a, di, &g, &smem)) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter (saved planes): no tile fits in shared memory");
  g.N = a.N; g.C = a.C; g.T = a.T; g.H = a.H; g.W = a.W; g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0;
  g.tilesH = ceil_div(a.H, g.TH); g.tilesW = ceil_div(a.W, g.TW);
  g.nparam = (a.T + a.C + (a.KC ? 9 : 6)) * a.R;
  {
    // channel slices where the tiles alone leave SMs idle: as many as fit one round of CTAs, at least 32 channels each
    const long ctas = (long)a.N * g.tilesH * g.tilesW;
    const int cps = std::max(1, std::min(2, (int)((228 * 1024) / (smem + 1024))));
    int S = 1;
    if (const char* e = getenv("B200CP_MMA_SLICES")) {
      S = std::max(1, std::min(8, atoi(e)));
    } else {
      while (S < 8 && ctas < di.sm_count && ctas * (2 * S) <= (long)di.sm_count * cps && std::max(a.T, a.C) >= 64 * S) S *= 2;
    }
    g.S = S;
    g.t_slice = (ceil_div(a.T, S) + 15) / 16 * 16;
    g.c_slice = (ceil_div(a.C, S) + 15) / 16 * 16;
  }
  g.vec = (g.TW % 4 == 0 && a.W % 4 == 0 && (g.MBW == 1 || g.MBW == 2 || g.MBW == 4) &&
           ((uintptr_t)a.X % 16 == 0) && ((uintptr_t)a.dU % 16 == 0) && !getenv("B200CP_NO_VEC")) ? 1 : 0;
  if (getenv("B200CP_DEBUG") && part != 3)
    fprintf(stderr, "[b200cp] bwd-filter (saved planes) tile TH=%d TW=%d blocks per warp %d slices %d smem=%zu RP=%d vec=%d\n",
            g.TH, g.TW, g.MBW, g.S, smem, RP, g.vec);
  switch (g.MBW) {
    case 1: return launch_saved<RP, 1>(g, smem, a, P, Q, st, part);
    case 2: return launch_saved<RP, 2>(g, smem, a, P, Q, st, part);
    case 3: return launch_saved<RP, 3>(g, smem, a, P, Q, st, part);
    case 4: return launch_saved<RP, 4>(g, smem, a, P, Q, st, part);
  }
  return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: internal: no kernel for %d blocks per warp", g.MBW);
}

template <int RP>
bool plan_bwdf(const Cp4BwdFilterArgs& a, const DeviceInfo& di, BGeom* out, size_t* smem_out) {
  BGeom best{};
  double best_cost = 1e300;
  size_t best_smem = 0;
  int fTH = 0, fTW = 0;
  if (const char* e = getenv("B200CP_MMA_TILE")) {  // "TH,TW": experiments
    if (sscanf(e, "%d,%d", &fTH, &fTW) != 2) fTH = fTW = 0;
  }
  for (int TW = 1; TW <= std::min(a.W, 64); ++TW) {
    if (fTW ? TW != std::min(fTW, a.W) : (TW != a.W && a.W % TW != 0 && TW % 8 != 0)) continue;
    for (int TH = 1; TH <= std::min(a.H, 64); ++TH) {
      if (fTH && TH != std::min(fTH, a.H)) continue;
      BGeom g{};
      g.TH = TH; g.TW = TW; g.TWh = TW + 2; g.HPX = (TH + 2) * g.TWh;
      g.MBW = ceil_div(ceil_div(g.HPX, 16), kWarps);
      if (g.MBW > 4 || g.MBW * (RP / 8) > 8) break;   // contraction accumulators: 4 * MBW * RP/8 registers
      g.pp = (kWarps * g.MBW * 16 + 11) | 1;
      const size_t smem = sizeof(float) * bwdf_mma_smem_floats<RP>(g);
      if ((int)smem > di.smem_optin) break;
      const int cps = std::max(1, std::min(2, (int)((228 * 1024) / (smem + 1024))));
      const long ctas = (long)a.N * ceil_div(a.H, TH) * ceil_div(a.W, TW);
      const long rounds = (ctas + (long)di.sm_count * cps - 1) / ((long)di.sm_count * cps);
      const double nb = RP / 8.0;
      const double contract = 2.0 * (g.MBW * (3.0 * nb + 12) + 4.0 * nb) + 40;   // per group of 16 channels
      const double reduce = 2.0 * g.MBW * (12 + nb * 9.0);
      const double groups = ceil_div(a.C, 16) * (contract + reduce + 40) + ceil_div(a.T, 16) * (contract + reduce + 40);
      const double stencil = (double)ceil_div(TH * ceil_div(TW, 8) * RP, kNT) * 450.0;
      const double tile = groups + stencil + 800.0;
      const double occupancy = 16.0 / (cps * kWarps);
      const double cost = (double)ctas * tile / di.sm_count * occupancy + 2500.0 * rounds;
      if (cost < best_cost) { best_cost = cost; best = g; best_smem = smem; }
    }
  }
  if (best.TH == 0) return false;
  *out = best;
  *smem_out = best_smem;
  return true;
}

template <int RP, int MBW, bool CORE>
int launch_bwdf_core(const BGeom& g, size_t smem, const Cp4BwdFilterArgs& a, cudaStream_t st) {
  auto kern = cp4_bwdf_mma_kernel<RP, MBW, CORE>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  const long ctas = (long)a.N * g.tilesH * g.tilesW;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: too many tiles");
  const size_t need = (size_t)ctas * g.nparam * sizeof(float);
  if (a.ws_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "cp4 bwd-filter: workspace of %zu bytes needed, %zu given", need, a.ws_bytes);
  kern<<<(unsigned)ctas, kNT, smem, st>>>(g, a.X, a.dU, a.K0, a.K1, a.KH, a.KW, a.KC, (float*)a.ws);
  B200CP_LAUNCH_OK("cp4_bwdf_mma_kernel");
  return cp4_reduce_partials_launch((const float*)a.ws, (int)ctas, g.nparam, a.R, a.Rs, a.r0, a.dK, st);
}

template <int RP, int MBW>
int launch_bwdf(const BGeom& g, size_t smem, const Cp4BwdFilterArgs& a, cudaStream_t st) {
  return a.KC ? launch_bwdf_core<RP, MBW, true>(g, smem, a, st) : launch_bwdf_core<RP, MBW, false>(g, smem, a, st);
}

template <int RP>
int run_bwdf(const Cp4BwdFilterArgs& a, const DeviceInfo& di, cudaStream_t st) {
  BGeom g{};
  size_t smem = 0;
  if (!plan_bwdf<RP>(a, di, &g, &smem)) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter (mma path): no tile fits in shared memory");
  g.N = a.N; g.C = a.C; g.T = a.T; g.H = a.H; g.W = a.W; g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0;
  g.tilesH = ceil_div(a.H, g.TH); g.tilesW = ceil_div(a.W, g.TW);
  g.nparam = (a.T + a.C + (a.KC ? 9 : 6)) * a.R;
  if (getenv("B200CP_DEBUG"))
    fprintf(stderr, "[b200cp] bwd-filter mma tile TH=%d TW=%d blocks per warp %d smem=%zu RP=%d\n", g.TH, g.TW, g.MBW, smem, RP);
  switch (g.MBW) {
    case 1: return launch_bwdf<RP, 1>(g, smem, a, st);
    case 2: return launch_bwdf<RP, 2>(g, smem, a, st);
    case 3: if constexpr (RP <= 16) return launch_bwdf<RP, 3>(g, smem, a, st); break;
    case 4: if constexpr (RP <= 16) return launch_bwdf<RP, 4>(g, smem, a, st); break;
  }
  return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: internal: no mma kernel for %d blocks per warp at rank tile %d", g.MBW, RP);
}

}  // namespace

bool cp4_bwd_filter_mma_supported(const Cp4BwdFilterArgs& a) { return a.F == 3 && a.pad == 1; }

// bytes of workspace the mma path needs for this shape (0: no device or no tile)
size_t cp4_bwd_filter_mma_workspace(const b200cp_tensor_shape& s) {
  if (s.Y != 3 || s.X != 3 || s.pad != 1) return 0;
  DeviceInfo di;
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count <= 0 || device_info(&di) != B200CP_OK) return 0;
  size_t need = 0;
  for (unsigned r0 = 0; r0 < s.Rank; r0 += 64) {
    const int rc = (int)std::min(64u, s.Rank - r0);
    Cp4BwdFilterArgs a{};
    a.N = s.N; a.C = s.C; a.T = s.T; a.H = s.H; a.W = s.W; a.F = 3; a.pad = 1; a.R = rc;
    BGeom g{};
    size_t smem = 0;
    const int rp = padded_rank(rc);
    const bool ok = rp <= 8 ? plan_bwdf<8>(a, di, &g, &smem) : rp == 16 ? plan_bwdf<16>(a, di, &g, &smem)
                    : rp == 32 ? plan_bwdf<32>(a, di, &g, &smem) : plan_bwdf<64>(a, di, &g, &smem);
    if (!ok) return 0;
    // nine spatial rows cover both the separable factors (six) and the free core of the three-factor layer
    need = std::max(need, (size_t)s.N * ceil_div(s.H, g.TH) * ceil_div(s.W, g.TW) * ((size_t)s.T + s.C + 9) * rc * sizeof(float));
  }
  return need;
}

// factor gradients from the rank planes P = K1^T X and Q = K0^T dU ([N][Rs][H][W]) the convolutions of the same
// step saved; 3x3 filters with pad 1
int cp4_bwd_filter_saved_launch(const Cp4BwdFilterArgs& a, const float* P, const float* Q, cudaStream_t st, int part) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const int rp = padded_rank(a.R);
  if (rp <= 8) return run_saved<8>(a, P, Q, di, st, part);
  if (rp == 16) return run_saved<16>(a, P, Q, di, st, part);
  if (rp == 32) return run_saved<32>(a, P, Q, di, st, part);
  return run_saved<64>(a, P, Q, di, st, part);
}

size_t cp4_bwd_filter_saved_workspace(const b200cp_tensor_shape& s) {
  if (s.Y != 3 || s.X != 3 || s.pad != 1) return 0;
  DeviceInfo di;
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count <= 0 || device_info(&di) != B200CP_OK) return 0;
  size_t need = 0;
  for (unsigned r0 = 0; r0 < s.Rank; r0 += 64) {
    const int rc = (int)std::min(64u, s.Rank - r0);
    Cp4BwdFilterArgs a{};
    a.N = s.N; a.C = s.C; a.T = s.T; a.H = s.H; a.W = s.W; a.F = 3; a.pad = 1; a.R = rc;
    SGeom g{};
    size_t smem = 0;
    const int rp = padded_rank(rc);
    const bool ok = rp <= 8 ? plan_saved<8>(a, di, &g, &smem) : rp == 16 ? plan_saved<16>(a, di, &g, &smem)
                    : rp == 32 ? plan_saved<32>(a, di, &g, &smem) : plan_saved<64>(a, di, &g, &smem);
    if (!ok) return 0;
    need = std::max(need, (size_t)s.N * ceil_div(s.H, g.TH) * ceil_div(s.W, g.TW) * ((size_t)s.T + s.C + 9) * rc * sizeof(float));
  }
  return need;
}

int cp4_bwd_filter_mma_launch(const Cp4BwdFilterArgs& a, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const int rp = padded_rank(a.R);
  if (rp <= 8) return run_bwdf<8>(a, di, st);
  if (rp == 16) return run_bwdf<16>(a, di, st);
  if (rp == 32) return run_bwdf<32>(a, di, st);
  return run_bwdf<64>(a, di, st);
}

}  // namespace b200cp
