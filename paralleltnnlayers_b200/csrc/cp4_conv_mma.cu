// CP4 conv2d forward and backward-data with warp-level tensor-core contractions (mma.sync, tf32 in three
// terms, fp32 accumulation: fp32-grade results).
//
// One CTA of 8 warps owns a TH x TW tile of output pixels of one image; the rank-R intermediate never
// leaves the SM:
//   phase 1  P[r, halo px] = sum_c Fin[c, r] * in[n, c, halo px]
//            GEMM with M = pixels (16 per mma), K = channels (8 per mma), N = ranks (8 per mma).  Each warp
//            owns some 16-pixel blocks of the halo tile and streams its own pixels of every channel through a
//            warp-private cp.async FIFO in shared memory (8 channels per group), so no CTA barrier is
//            needed in the channel loop; factors sit in shared memory already split into tf32 hi / lo.
//   phase 2  Z[r, px] = sum_{y,x} KH[y,r] KW[x,r] P[r, px + (y,x)]       (CUDA cores, weights in registers)
//   phase 3  out[n, t, px] = sum_r Fout[t, r] * Z[r, px]
//            GEMM with M = pixels, K = ranks, N = output channels; results go straight to global memory.
// Every product x*f is computed as hi(x)*hi(f) + lo(x)*hi(f) + hi(x)*lo(f) with hi = the value rounded to
// tf32 and lo = the remainder, which keeps the error near 2^-21 relative.
// Forward uses Fin = K1, Fout = K0; backward-data swaps them and flips the taps
// (formulas: Cuda_kernels/cp4Conv2dForward.cu:84-133, cp4Conv2dBackwardData.cu:57-108).
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include <cooperative_groups.h>

#include "mma_util.cuh"

namespace b200cp {

namespace {

using namespace mma;
namespace cg = cooperative_groups;

constexpr int kNT = 256, kWarps = 8;
constexpr int kGC = 8;       // channels per cp.async group = one mma k-step
constexpr int kFifo = 3;     // cp.async groups per warp (one being consumed)
constexpr int kFChunk = 128; // channels of factor planes staged at a time

struct MmaGeom {
  int N, Cin, Cout, H, W, Y, X, pad, R, Rs, r0, flip, accumulate;
  int TH, TW, THh, TWh, HPX, OPX, tilesH, tilesW;
  int MB1, MBW1, MB3, MBW3;   // 16-pixel blocks of the halo / output tile, and blocks per warp
  int xpitch;                 // FIFO row pitch (floats), = 8 mod 32
  int ppitch;                 // P row pitch  (floats)
  int zpitch;                 // Z row pitch, = 8 mod 32
  int fch;                    // channels of factor planes staged at a time (multiple of 8, <= kFChunk)
  int early_fout;             // 1: all channels fit one chunk and the output-side planes have their own space,
                              //    so both factor sets are staged at the start, behind the first pixel copies
  int S;                      // channel slices per tile = CTAs per cluster (1: no cluster)
  int cin_slice, cout_slice;  // channels per slice (multiples of 8)
};

inline int pitch_mod32(int n, int want) {  // smallest p >= n with p % 32 == want
  int p = n;
  while (p % 32 != want) ++p;
  return p;
}

// row pitches of the factor planes, chosen so that the B-fragment loads of a warp hit 32 different banks
template <int RP>
struct Planes {
  static constexpr int FIN = RP == 8 ? 24 : RP + 8;  // phase-1 B element (k = c, n = r) at [c][r]: 4 rows x 8 ranks
  static constexpr int FOUT = RP + 4;                // phase-3 B element (k = r, n = t) at [t][r]: 8 rows x 4 ranks
};

template <int RP>
size_t mma_smem_floats(const MmaGeom& g) {
  const size_t fifo = (size_t)kFifo * kGC * (kWarps * g.MBW1 * 16 + 8);
  const size_t P = (size_t)RP * g.ppitch;
  const size_t Z = (size_t)RP * (kWarps * g.MBW3 * 16 + 8);   // lives in the FIFO's space once phase 1 is over
  const size_t planes = 2 * (size_t)g.fch * Planes<RP>::FIN;  // FIN >= FOUT
  const size_t planes_out = g.early_fout ? 2 * (size_t)g.fch * Planes<RP>::FOUT : 0;
  const size_t W = (size_t)g.Y * g.X * RP;
  return std::max(fifo, Z) + P * (g.S > 1 ? 2 : 1) + planes + planes_out + W;
}

template <int RP, int FS, int MBW1, int MBW3>
__global__ void __launch_bounds__(kNT, (RP <= 16 && MBW1 <= 2) ? 3 : 2) cp4_conv_mma_kernel(const MmaGeom g, const float* __restrict__ in,
                                                             const float* __restrict__ Fin,
                                                             const float* __restrict__ Fout,
                                                             const float* __restrict__ KH,
                                                             const float* __restrict__ KW,
                                                             const float* __restrict__ KC, float* __restrict__ out,
                                                             float* __restrict__ save) {
  constexpr int NB = RP / 8;                    // rank blocks (n of phase 1, k of phase 3)
  constexpr int XP = kWarps * MBW1 * 16 + 8;    // FIFO row pitch:  8 mod 32
  constexpr int ZP = kWarps * MBW3 * 16 + 8;    // Z row pitch:     8 mod 32
  constexpr int FIN = Planes<RP>::FIN, FOUT = Planes<RP>::FOUT;
  static_assert(FIN >= FOUT, "the output-side planes reuse the input-side planes' space");
  const int kFin = g.fch * FIN, kFout = g.fch * FOUT;   // floats per plane
  const int PP = g.ppitch;                      // P row pitch:     1 mod 32
  extern __shared__ __align__(16) float smem[];
  float* Xf = smem;                             // [kFifo][kGC][XP]
  float* Zs = smem;                             // [RP][ZP]: phase 2 and 3 only, over the FIFO
  constexpr int kXZ = kFifo * kGC * XP > RP * ZP ? kFifo * kGC * XP : RP * ZP;
  float* Ps = smem + kXZ;                       // [RP][PP]
  float* Psum = Ps + (size_t)RP * PP;           // [RP][PP]: P summed over the cluster's channel slices (S > 1 only)
  float* Fh = Psum + (g.S > 1 ? (size_t)RP * PP : 0);  // input-side factor planes hi | lo
  float* Fo = g.early_fout ? Fh + 2 * kFin : Fh;  // output-side planes: own space, or the input side's after phase 1
  float* Ws = Fo + 2 * (g.early_fout ? kFout : kFin);  // [Y*X][RP]
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;      // mma "groupID" and "threadID in group"

  // Channel slices: the S CTAs of a cluster share one tile.  Each contracts its slice of the input channels,
  // the partial rank planes are summed through distributed shared memory, and each then produces its slice of
  // the output channels.  Small images with many channels have too few tiles to fill the GPU otherwise.
  int b = blockIdx.x;
  const int sl = b % g.S;
  b /= g.S;
  const int c_lo = min(g.Cin, sl * g.cin_slice), c_hi = min(g.Cin, c_lo + g.cin_slice);
  const int t_lo = min(g.Cout, sl * g.cout_slice), t_hi = min(g.Cout, t_lo + g.cout_slice);
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  const size_t HW = (size_t)g.H * g.W;
  const float* in_n = in + (size_t)n * g.Cin * HW;

  // stencil weights (phase 2)
  for (int i = tid; i < g.Y * g.X * RP; i += kNT) {
    const int r = i % RP, yx = i / RP, y = yx / g.X, x = yx - y * g.X;
    const int yy = g.flip ? g.Y - 1 - y : y, xx = g.flip ? g.X - 1 - x : x;
    // a free core [Y][X][Rs] (three-factor CP conv) takes the place of the outer product KH x KW
    Ws[i] = r >= g.R ? 0.f
            : KC   ? __ldg(KC + (size_t)(yy * g.X + xx) * g.Rs + g.r0 + r)
                   : __ldg(KH + (size_t)yy * g.Rs + g.r0 + r) * __ldg(KW + (size_t)xx * g.Rs + g.r0 + r);
  }

  auto stage_fout = [&](int t0) {
    const int tc = min(g.fch, t_hi - t0);
    const int tcp = (tc + 7) / 8 * 8;
    for (int i = tid; i < tcp * RP; i += kNT) {
      const int t = i / RP, r = i % RP;
      const float v = (r < g.R && t < tc) ? __ldg(Fout + (size_t)(t0 + t) * g.Rs + g.r0 + r) : 0.f;
      const float hi = tf32_round(v);
      Fo[t * FOUT + r] = hi;
      Fo[kFout + t * FOUT + r] = tf32_round(v - hi);
    }
  };

  // ---------------- phase 1 ----------------
  // warp-private columns: block j of this warp is halo block (j*kWarps + warp); column = warp*MBW1*16 + j*16 + i
  constexpr int WCOLS = MBW1 * 16;          // columns per warp
  constexpr int CPL = (WCOLS + 31) / 32;    // columns copied per lane
  const float* gp[CPL];                     // this lane's pixel of channel 0 (any valid address when masked)
  int gsz[CPL];                             // cp.async source size: 4, or 0 = zero fill
#pragma unroll
  for (int q = 0; q < CPL; ++q) {
    const int wc = lane + 32 * q;           // column within the warp's range
    const int jb = wc >> 4, i = wc & 15;
    const int hp = (jb * kWarps + warp) * 16 + i;
    const int hy = hp / g.TWh, hx = hp - hy * g.TWh;
    const int gy = h0 - g.pad + hy, gx = w0 - g.pad + hx;
    const bool ok = wc < WCOLS && hp < g.HPX && gy >= 0 && gy < g.H && gx >= 0 && gx < g.W;
    gp[q] = in_n + (ok ? gy * g.W + gx : 0);
    gsz[q] = ok ? 4 : 0;
  }
  float acc[MBW1][NB][4];
#pragma unroll
  for (int j = 0; j < MBW1; ++j)
#pragma unroll
    for (int nb = 0; nb < NB; ++nb)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[j][nb][e] = 0.f;

  const unsigned xw_s = (unsigned)__cvta_generic_to_shared(Xf + warp * WCOLS + lane);  // this lane's first column
  const float* xw = Xf + warp * WCOLS;
  for (int c0 = c_lo; c0 < c_hi; c0 += g.fch) {
    const int cc = min(g.fch, c_hi - c0);
    const int ccp = (cc + kGC - 1) / kGC * kGC;
    const int ng = ccp / kGC;
    auto issue = [&](int grp) {
      if (grp < ng) {
        const unsigned dst = xw_s + (unsigned)((grp % kFifo) * kGC * XP * 4);
        const size_t coff = (size_t)(c0 + grp * kGC) * HW;
        if (grp * kGC + kGC <= cc) {      // all 8 channels exist
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
                cp_async4_s(dst + (unsigned)((jc * XP + 32 * q) * 4), cin ? gp[q] + coff + (size_t)jc * HW : in_n,
                            cin ? gsz[q] : 0);
              }
            }
        }
      }
      cp_async_commit();
    };
    // the first pixel copies go out before the factors are staged: their latency hides behind that work
    // (the FIFO stages are free: the previous chunk has been consumed by every lane of this warp)
#pragma unroll
    for (int s = 0; s < kFifo - 1; ++s) issue(s);
    __syncthreads();   // every warp is done with the previous chunk's factor planes
    for (int i = tid; i < ccp * RP; i += kNT) {
      const int c = i / RP, r = i % RP;
      const float v = (r < g.R && c < cc) ? __ldg(Fin + (size_t)(c0 + c) * g.Rs + g.r0 + r) : 0.f;
      const float hi = tf32_round(v);
      Fh[c * FIN + r] = hi;
      Fh[kFin + c * FIN + r] = tf32_round(v - hi);
    }
    if (g.early_fout && c0 == c_lo) stage_fout(t_lo);
    __syncthreads();
    for (int grp = 0; grp < ng; ++grp) {
      issue(grp + kFifo - 1);
      cp_async_wait<kFifo - 1>();
      __syncwarp();
      const float* xs = xw + (grp % kFifo) * kGC * XP;
      // B fragments of this k-step: element (k = channel, n = rank)
      uint32_t bh[NB][2], bl[NB][2];
      {
        const float* f = Fh + (grp * kGC + tq) * FIN + gq;
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
          bh[nb][0] = __float_as_uint(f[nb * 8]);
          bh[nb][1] = __float_as_uint(f[nb * 8 + 4 * FIN]);
          bl[nb][0] = __float_as_uint(f[nb * 8 + kFin]);
          bl[nb][1] = __float_as_uint(f[nb * 8 + kFin + 4 * FIN]);
        }
      }
      // A fragments: element (m = pixel, k = channel) at xs[channel][column]
      uint32_t ah[MBW1][4], al[MBW1][4];
      {
        const float* xa = xs + tq * XP + gq;
#pragma unroll
        for (int j = 0; j < MBW1; ++j) {
          split_tf32(xa[j * 16], ah[j][0], al[j][0]);
          split_tf32(xa[j * 16 + 8], ah[j][1], al[j][1]);
          split_tf32(xa[j * 16 + 4 * XP], ah[j][2], al[j][2]);
          split_tf32(xa[j * 16 + 4 * XP + 8], ah[j][3], al[j][3]);
        }
      }
      __syncwarp();  // every lane has read this FIFO stage: a later group may overwrite it
#pragma unroll
      for (int j = 0; j < MBW1; ++j)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_tf32(acc[j][nb], al[j], bh[nb]);
#pragma unroll
      for (int j = 0; j < MBW1; ++j)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_tf32(acc[j][nb], ah[j], bl[nb]);
#pragma unroll
      for (int j = 0; j < MBW1; ++j)
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) mma_tf32(acc[j][nb], ah[j], bh[nb]);
    }
    cp_async_wait<0>();
  }
  // P fragments -> Ps[r][halo px]
#pragma unroll
  for (int j = 0; j < MBW1; ++j) {
    float* p = Ps + (size_t)(2 * tq) * PP + (j * kWarps + warp) * 16 + gq;
#pragma unroll
    for (int nb = 0; nb < NB; ++nb) {
      p[(nb * 8) * PP] = acc[j][nb][0];
      p[(nb * 8 + 1) * PP] = acc[j][nb][1];
      p[(nb * 8) * PP + 8] = acc[j][nb][2];
      p[(nb * 8 + 1) * PP + 8] = acc[j][nb][3];
    }
  }
  if (save != nullptr && g.S == 1) {
    // The rank plane at the tile's own pixels also goes to global memory (3x3, pad 1): the backward-filter kernel
    // of the same step reads it instead of contracting the channels again.  Straight from the fragments: a quarter
    // warp writes eight consecutive pixels of one plane.
    float* sv = save + ((size_t)n * g.Rs + g.r0) * HW;
#pragma unroll
    for (int j = 0; j < MBW1; ++j)
#pragma unroll
      for (int hlf = 0; hlf < 2; ++hlf) {
        const int hp = (j * kWarps + warp) * 16 + gq + 8 * hlf;
        const int hy = hp / g.TWh, hx = hp - hy * g.TWh;
        const int gy = h0 - 1 + hy, gx = w0 - 1 + hx;
        if (hy >= 1 && hy <= g.TH && hx >= 1 && hx <= g.TW && gy < g.H && gx < g.W) {
          float* d = sv + (size_t)gy * g.W + gx;
#pragma unroll
          for (int nb = 0; nb < NB; ++nb) {
            const int r = nb * 8 + 2 * tq;
            if (r < g.R) d[(size_t)r * HW] = acc[j][nb][2 * hlf];
            if (r + 1 < g.R) d[(size_t)(r + 1) * HW] = acc[j][nb][2 * hlf + 1];
          }
        }
      }
  }
  __syncthreads();

  const float* Pr = Ps;   // the plane phase 2 reads
  if (g.S > 1) {
    // sum the partial planes of the cluster's CTAs, in slice order on every CTA (identical sums everywhere)
    cg::cluster_group cluster = cg::this_cluster();
    cluster.sync();                                  // every CTA's partial plane is complete
    for (int i = tid; i < RP * PP; i += kNT) {
      float v = 0.f;
      for (int q = 0; q < g.S; ++q) v += cluster.map_shared_rank(Ps, q)[i];
      Psum[i] = v;
    }
    cluster.sync();                                  // nobody reads this CTA's shared memory any more
    Pr = Psum;
    if (save != nullptr && sl == 0) {                // the summed plane at the tile's own pixels (3x3, pad 1)
      float* sv = save + ((size_t)n * g.Rs + g.r0) * HW;
      for (int i = tid; i < g.R * g.OPX; i += kNT) {
        const int r = i / g.OPX, op = i - r * g.OPX;
        const int oy = op / g.TW, ox = op - oy * g.TW;
        const int gy = h0 + oy, gx = w0 + ox;
        if (gy < g.H && gx < g.W) sv[(size_t)r * HW + (size_t)gy * g.W + gx] = Psum[r * PP + (oy + 1) * g.TWh + ox + 1];
      }
    }
  }

  if (!g.early_fout) stage_fout(t_lo);

  // ---------------- phase 2 ----------------
  {
    const int r = tid % RP;           // fixed per thread (kNT is a multiple of RP)
    if (FS == 3) {
      float w[9];
#pragma unroll
      for (int t = 0; t < 9; ++t) w[t] = Ws[t * RP + r];
      constexpr int SW = 8;
      const int spr = (g.TW + SW - 1) / SW;
      const int items = g.TH * spr;
      for (int it = tid / RP; it < items; it += kNT / RP) {
        const int oy = it / spr, x0 = (it - oy * spr) * SW;
        float z[SW];
#pragma unroll
        for (int j = 0; j < SW; ++j) z[j] = 0.f;
        // reads past the tile's last column stay inside the padded row and feed only outputs that are not stored
        const float* p = Pr + (size_t)r * PP + oy * g.TWh + x0;
#pragma unroll
        for (int dy = 0; dy < 3; ++dy) {
          float v[SW + 2];
#pragma unroll
          for (int j = 0; j < SW + 2; ++j) v[j] = p[j];
          p += g.TWh;
#pragma unroll
          for (int j = 0; j < SW; ++j) {
            z[j] = fmaf(w[dy * 3 + 0], v[j], z[j]);
            z[j] = fmaf(w[dy * 3 + 1], v[j + 1], z[j]);
            z[j] = fmaf(w[dy * 3 + 2], v[j + 2], z[j]);
          }
        }
        float* zd = Zs + r * ZP + oy * g.TW + x0;
        if (x0 + SW <= g.TW) {
#pragma unroll
          for (int j = 0; j < SW; ++j) zd[j] = z[j];
        } else {
#pragma unroll
          for (int j = 0; j < SW; ++j)
            if (x0 + j < g.TW) zd[j] = z[j];
        }
      }
    } else {
      for (int op = tid / RP; op < g.OPX; op += kNT / RP) {
        const int oy = op / g.TW, ox = op - oy * g.TW;
        const float* p = Pr + (size_t)r * PP + oy * g.TWh + ox;
        float z = 0.f;
        for (int y = 0; y < g.Y; ++y)
          for (int x = 0; x < g.X; ++x) z = fmaf(Ws[(y * g.X + x) * RP + r], p[y * g.TWh + x], z);
        Zs[r * ZP + op] = z;
      }
    }
  }
  __syncthreads();

  // ---------------- phase 3 ----------------
  // this warp's output blocks: block j is output block (j*kWarps + warp).  A fragments: element (m = pixel,
  // k = rank) at Zs[rank][pixel]; B fragments: element (k = rank, n = channel) at Fh[channel][rank].
  float* out_n = out + (size_t)n * g.Cout * HW;
  float* op_ptr[MBW3][2];   // this thread's two pixels of channel 2*tq (null: outside the tile or the image)
#pragma unroll
  for (int j = 0; j < MBW3; ++j)
#pragma unroll
    for (int hlf = 0; hlf < 2; ++hlf) {
      const int op = (j * kWarps + warp) * 16 + gq + 8 * hlf;
      const int oy = op / g.TW, ox = op - oy * g.TW;
      const int gy = h0 + oy, gx = w0 + ox;
      op_ptr[j][hlf] = (op < g.OPX && gy < g.H && gx < g.W) ? out_n + (size_t)(2 * tq) * HW + gy * g.W + gx : nullptr;
    }
  constexpr bool kAllBlocks = MBW3 * NB <= 8;   // A fragments of every block fit in registers
  uint32_t zh[kAllBlocks ? MBW3 : 1][NB][4], zl[kAllBlocks ? MBW3 : 1][NB][4];
  auto load_a = [&](int j, int slot) {
    const float* za = Zs + tq * ZP + (j * kWarps + warp) * 16 + gq;
#pragma unroll
    for (int kb = 0; kb < NB; ++kb) {
      split_tf32(za[kb * 8 * ZP], zh[slot][kb][0], zl[slot][kb][0]);
      split_tf32(za[kb * 8 * ZP + 8], zh[slot][kb][1], zl[slot][kb][1]);
      split_tf32(za[(kb * 8 + 4) * ZP], zh[slot][kb][2], zl[slot][kb][2]);
      split_tf32(za[(kb * 8 + 4) * ZP + 8], zh[slot][kb][3], zl[slot][kb][3]);
    }
  };
  auto store_d = [&](const float (&d)[4], float* p0, float* p1, size_t toff, bool two) {
    if (g.accumulate) {
      if (p0) { p0[toff] += d[0]; if (two) p0[toff + HW] += d[1]; }
      if (p1) { p1[toff] += d[2]; if (two) p1[toff + HW] += d[3]; }
    } else {
      if (p0) { p0[toff] = d[0]; if (two) p0[toff + HW] = d[1]; }
      if (p1) { p1[toff] = d[2]; if (two) p1[toff + HW] = d[3]; }
    }
  };
  if (kAllBlocks) {
#pragma unroll
    for (int j = 0; j < MBW3; ++j) load_a(j, j);
  }
  for (int t0 = t_lo; t0 < t_hi; t0 += g.fch) {
    const int tc = min(g.fch, t_hi - t0);
    if (t0 > t_lo) {
      __syncthreads();
      stage_fout(t0);
      __syncthreads();
    }
    const int nbs = (tc + 7) / 8;
    if (kAllBlocks) {
#pragma unroll 2
      for (int nb = 0; nb < nbs; ++nb) {
        uint32_t bh[NB][2], bl[NB][2];
        const float* f = Fo + (nb * 8 + gq) * FOUT + tq;
#pragma unroll
        for (int kb = 0; kb < NB; ++kb) {
          bh[kb][0] = __float_as_uint(f[kb * 8]);
          bh[kb][1] = __float_as_uint(f[kb * 8 + 4]);
          bl[kb][0] = __float_as_uint(f[kb * 8 + kFout]);
          bl[kb][1] = __float_as_uint(f[kb * 8 + kFout + 4]);
        }
        float d[MBW3][4];
#pragma unroll
        for (int j = 0; j < MBW3; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
#pragma unroll
        for (int kb = 0; kb < NB; ++kb) {
#pragma unroll
          for (int j = 0; j < MBW3; ++j) mma_tf32(d[j], zl[j][kb], bh[kb]);
#pragma unroll
          for (int j = 0; j < MBW3; ++j) mma_tf32(d[j], zh[j][kb], bl[kb]);
#pragma unroll
          for (int j = 0; j < MBW3; ++j) mma_tf32(d[j], zh[j][kb], bh[kb]);
        }
        const int t = nb * 8 + 2 * tq;          // channel of d[.][0] within the chunk
        if (t < tc) {
          const size_t toff = (size_t)(t0 + nb * 8) * HW;
#pragma unroll
          for (int j = 0; j < MBW3; ++j) store_d(d[j], op_ptr[j][0], op_ptr[j][1], toff, t + 1 < tc);
        }
      }
    } else {
#pragma unroll 1
      for (int j = 0; j < MBW3; ++j) {
        load_a(j, 0);
        for (int nb = 0; nb < nbs; ++nb) {
          const float* f = Fo + (nb * 8 + gq) * FOUT + tq;
          float d[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int kb = 0; kb < NB; ++kb) {
            const uint32_t bh[2] = {__float_as_uint(f[kb * 8]), __float_as_uint(f[kb * 8 + 4])};
            const uint32_t bl[2] = {__float_as_uint(f[kb * 8 + kFout]), __float_as_uint(f[kb * 8 + kFout + 4])};
            mma_tf32(d, zl[0][kb], bh);
            mma_tf32(d, zh[0][kb], bl);
            mma_tf32(d, zh[0][kb], bh);
          }
          const int t = nb * 8 + 2 * tq;
          if (t < tc) store_d(d, op_ptr[j][0], op_ptr[j][1], (size_t)(t0 + nb * 8) * HW, t + 1 < tc);
        }
      }
    }
  }
}

template <int RP, int FS, int M1, int M3>
int launch_mma(const MmaGeom& g, const Cp4Args& a, cudaStream_t st) {
  auto kern = cp4_conv_mma_kernel<RP, FS, M1, M3>;
  const size_t smem = sizeof(float) * mma_smem_floats<RP>(g);
  static std::atomic<int> smem_set[64];
  B200CP_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_set, (int)smem));
  const long ctas = (long)a.N * g.tilesH * g.tilesW * g.S;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4: too many tiles");
  float* save = (FS == 3 && a.pad == 1) ? a.save : nullptr;
  if (a.save && !save) return fail(B200CP_ERR_UNSUPPORTED, "cp4: rank planes are saved for 3x3 filters with pad 1 only");
  if (g.S == 1) {
    kern<<<(unsigned)ctas, kNT, smem, st>>>(g, a.in, a.Fin, a.Fout, a.KH, a.KW, a.KC, a.out, save);
  } else {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3((unsigned)ctas);
    cfg.blockDim = dim3(kNT);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = (unsigned)g.S;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    B200CP_CUDA_OK(cudaLaunchKernelEx(&cfg, kern, g, a.in, a.Fin, a.Fout, a.KH, a.KW, a.KC, a.out, save));
  }
  B200CP_LAUNCH_OK("cp4_conv_mma_kernel");
  return B200CP_OK;
}

template <int RP, int FS>
int dispatch_blocks(const MmaGeom& g, const Cp4Args& a, cudaStream_t st) {
  switch (g.MBW1 * 10 + g.MBW3) {
    case 11: return launch_mma<RP, FS, 1, 1>(g, a, st);
    case 21: return launch_mma<RP, FS, 2, 1>(g, a, st);
    case 22: return launch_mma<RP, FS, 2, 2>(g, a, st);
    case 32: return launch_mma<RP, FS, 3, 2>(g, a, st);
    case 33: return launch_mma<RP, FS, 3, 3>(g, a, st);
    case 43: return launch_mma<RP, FS, 4, 3>(g, a, st);
    case 44: return launch_mma<RP, FS, 4, 4>(g, a, st);
  }
  return fail(B200CP_ERR_UNSUPPORTED, "cp4: internal: no mma kernel for %d/%d blocks per warp", g.MBW1, g.MBW3);
}

template <int RP>
bool plan_tile_search(const Cp4Args& a, const DeviceInfo& di, int fTH, int fTW, int fS, MmaGeom* out);

// The tile search runs once per shape and forced setting: the plan of the last few shapes is kept per host thread.
template <int RP>
bool plan_tile(const Cp4Args& a, const DeviceInfo& di, MmaGeom* out) {
  int fTH = 0, fTW = 0, fS = 0;
  if (const char* e = getenv("B200CP_MMA_TILE")) {  // "TH,TW": experiments
    if (sscanf(e, "%d,%d", &fTH, &fTW) != 2) fTH = fTW = 0;
  }
  if (const char* e = getenv("B200CP_MMA_SLICES")) fS = atoi(e);  // 1, 2, 4 or 8 channel slices per tile: tests
  struct Entry {
    int key[14];
    bool ok;
    MmaGeom g;
  };
  thread_local Entry cache[8];
  thread_local int used = 0, next = 0;
  const int key[14] = {a.N, a.Cin, a.Cout, a.H, a.W, a.Y, a.X, a.pad, a.R, fTH, fTW, fS, di.sm_count, di.smem_optin};
  for (int i = 0; i < used; ++i)
    if (std::memcmp(cache[i].key, key, sizeof(key)) == 0) {
      if (cache[i].ok) *out = cache[i].g;
      return cache[i].ok;
    }
  Entry& e = cache[next];
  next = (next + 1) % 8;
  used = std::min(used + 1, 8);
  std::memcpy(e.key, key, sizeof(key));
  e.ok = plan_tile_search<RP>(a, di, fTH, fTW, fS, &e.g);
  if (e.ok) *out = e.g;
  return e.ok;
}

template <int RP>
bool plan_tile_search(const Cp4Args& a, const DeviceInfo& di, int fTH, int fTW, int fS, MmaGeom* out) {
  MmaGeom best{};
  double best_cost = 1e300;
  for (int TW = 1; TW <= std::min(a.W, 64); ++TW) {
    if (fTW ? TW != std::min(fTW, a.W) : (TW != a.W && a.W % TW != 0 && TW % 8 != 0)) continue;
    for (int TH = 1; TH <= std::min(a.H, 64); ++TH) {
      if (fTH && TH != std::min(fTH, a.H)) continue;
      MmaGeom g{};
      g.TH = TH; g.TW = TW; g.THh = TH + a.Y - 1; g.TWh = TW + a.X - 1;
      g.HPX = g.THh * g.TWh; g.OPX = TH * TW;
      g.MB1 = ceil_div(g.HPX, 16); g.MB3 = ceil_div(g.OPX, 16);
      g.MBW1 = ceil_div(g.MB1, kWarps); g.MBW3 = ceil_div(g.MB3, kWarps);
      if (g.MBW1 > 4 || g.MBW1 * (RP / 8) > 16) break;   // phase-1 accumulators: 4 * MBW1 * RP/8 registers
      if (g.MBW3 > g.MBW1 || g.MBW3 < g.MBW1 - 1) continue;  // instantiated pairs
      g.xpitch = pitch_mod32(kWarps * g.MBW1 * 16, 8);
      g.ppitch = (kWarps * g.MBW1 * 16 + a.X + 8) | 1;   // odd: the ranks of a warp hit different banks; the slack
                                                          // keeps the strips' reads past the last column inside the row
      g.zpitch = pitch_mod32(kWarps * g.MBW3 * 16, 8);
      g.Y = a.Y; g.X = a.X;
      g.fch = std::min(kFChunk, (std::max(a.Cin, a.Cout) + 7) / 8 * 8);
      g.early_fout = std::max(a.Cin, a.Cout) <= g.fch ? 1 : 0;
      const int cps_max = (RP <= 16 && g.MBW1 <= 2) ? 3 : 2;   // the kernel's launch bounds
      g.S = 1; g.cin_slice = (a.Cin + 7) / 8 * 8; g.cout_slice = (a.Cout + 7) / 8 * 8;
      size_t smem = sizeof(float) * mma_smem_floats<RP>(g);
      int cps = (int)smem > di.smem_optin ? 0 : std::max(1, std::min(cps_max, (int)((228 * 1024) / (smem + 1024))));
      if (g.early_fout) {   // one more CTA per SM is worth more than staging the output-side factors early
        MmaGeom g2 = g;
        g2.early_fout = 0;
        const size_t smem2 = sizeof(float) * mma_smem_floats<RP>(g2);
        const int cps2 = (int)smem2 > di.smem_optin ? 0 : std::max(1, std::min(cps_max, (int)((228 * 1024) / (smem2 + 1024))));
        if (cps2 > cps) { g = g2; smem = smem2; cps = cps2; }
      }
      if (cps == 0) break;
      const long ctas = (long)a.N * ceil_div(a.H, TH) * ceil_div(a.W, TW);
      const long rounds = (ctas + (long)di.sm_count * cps - 1) / ((long)di.sm_count * cps);
      // issue slots per warp and tile: k-steps * blocks * (3 mma per rank block + fragment work), plus fixed work
      const double c1 = (double)ceil_div(a.Cin, 8) * (g.MBW1 * (3.0 * RP / 8 + 14) + 4.0 * RP / 8 + 12 + 10.0 * g.MBW1);
      const double c3 = (double)ceil_div(a.Cout, 8) * (g.MBW3 * (3.0 * RP / 8 + 10) + 4.0 * RP / 8);
      const double c2 = (double)ceil_div(TH * ceil_div(TW, 8) * RP, kNT) * 90.0;
      const double fixed = 150.0 + 10.0 * RP / kNT;   // set-up; staging the factor planes costs about 10 slots per 256 values
      const double tile = c1 + c2 + c3 + fixed + 10.0 * (a.Cin + a.Cout) * RP / kNT;
      // Measured on B200: the kernel is bound by dependent-issue latency, so a tile takes about the same time
      // whether one or several CTAs share the SM (about 20 % more per extra CTA).  The grid runs as full rounds of
      // sm_count * cps CTAs plus a last round in which each SM holds only ceil(rest / sm_count) of them.
      auto grid_cost = [&](long n_ctas, int per_sm, double tile_slots) {
        const long slots = (long)di.sm_count * per_sm;
        const long full = n_ctas / slots, rest = n_ctas % slots;
        const double lat_full = tile_slots * (1.0 + 0.2 * (per_sm - 1));
        const int k = (int)((rest + di.sm_count - 1) / di.sm_count);
        // a last round after full ones starts while those drain: it costs between half and all of its own latency
        const double tail = full ? 0.5 + 0.5 * (double)rest / slots : 1.0;
        return full * lat_full + (rest ? tile_slots * (1.0 + 0.2 * (k - 1)) * tail : 0.0);
      };
      const double cost = grid_cost(ctas, cps, tile);
      (void)rounds;
      if (cost < best_cost && (fS <= 1)) { best_cost = cost; best = g; }
      // channel slices over a cluster of S CTAs: the two contractions shrink by S, the stencil and the exchange
      // of the partial planes do not
      for (int S = 2; S <= 8; S *= 2) {
        // (only where the tiles alone leave SMs idle: with enough tiles the exchange and the repeated stencil cost
        // more than the shorter contractions save)
        if (fS ? S != fS : (std::min(a.Cin, a.Cout) < 16 * S || ctas >= 2 * di.sm_count)) continue;
        MmaGeom gs = g;
        gs.S = S;
        gs.cin_slice = (ceil_div(a.Cin, S) + 7) / 8 * 8;
        gs.cout_slice = (ceil_div(a.Cout, S) + 7) / 8 * 8;
        gs.fch = std::min(kFChunk, std::max(gs.cin_slice, gs.cout_slice));
        gs.early_fout = 0;
        const size_t smem_s = sizeof(float) * mma_smem_floats<RP>(gs);
        if ((int)smem_s > di.smem_optin) continue;
        const int cps_s = std::max(1, std::min(cps_max, (int)((228 * 1024) / (smem_s + 1024))));
        const long ctas_s = ctas * S;
        const double tile_s = (c1 + c3 + 10.0 * (a.Cin + a.Cout) * RP / kNT) / S + c2 + fixed + 60.0 * S + 200.0;
        const double cost_s = grid_cost(ctas_s, cps_s, tile_s);
        if (cost_s < best_cost) { best_cost = cost_s; best = gs; }
      }
    }
  }
  if (best.TH == 0) return false;
  *out = best;
  return true;
}

template <int RP>
int run_mma(const Cp4Args& a, const DeviceInfo& di, cudaStream_t st) {
  MmaGeom g{};
  if (!plan_tile<RP>(a, di, &g)) return fail(B200CP_ERR_UNSUPPORTED, "cp4 (mma path): no tile of this filter fits in shared memory");
  g.N = a.N; g.Cin = a.Cin; g.Cout = a.Cout; g.H = a.H; g.W = a.W; g.Y = a.Y; g.X = a.X; g.pad = a.pad;
  g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0; g.flip = a.flip; g.accumulate = a.accumulate;
  g.tilesH = ceil_div(a.H, g.TH); g.tilesW = ceil_div(a.W, g.TW);
  static const bool debug = getenv("B200CP_DEBUG") != nullptr;
  if (debug)
    fprintf(stderr, "[b200cp] mma tile TH=%d TW=%d blocks %d/%d per warp %d/%d slices %d smem=%zu RP=%d\n", g.TH, g.TW,
            g.MB1, g.MB3, g.MBW1, g.MBW3, g.S, sizeof(float) * mma_smem_floats<RP>(g), RP);
  if (a.Y == 3 && a.X == 3) return dispatch_blocks<RP, 3>(g, a, st);
  return dispatch_blocks<RP, 0>(g, a, st);
}

}  // namespace

int cp4_mma_launch(const Cp4Args& a, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const int rp = padded_rank(a.R);
  if (rp <= 8) return run_mma<8>(a, di, st);
  if (rp == 16) return run_mma<16>(a, di, st);
  if (rp == 32) return run_mma<32>(a, di, st);
  return run_mma<64>(a, di, st);
}

}  // namespace b200cp
