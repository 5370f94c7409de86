// CP4 conv2d on CUDA cores (exact fp32): device code shared by the forward /
// backward-data kernel and the backward-filter kernel.
//
// One CTA owns a TH x TW tile of output pixels of one image.  The rank-R
// intermediate never leaves the SM:
//   phase 1  P[r, halo px] = sum_c Fin[c, r] * in[n, c, halo px]         (registers -> smem)
//   phase 2  Z[r, px]      = sum_{y,x} KH[y,r] KW[x,r] P[r, px + (y,x)]  (smem -> registers)
//   phase 3  out[n, t, px] = sum_r Fout[t, r] * Z[r, px]                 (registers -> global)
// Forward uses Fin = K1, Fout = K0; backward-data swaps them and flips the taps
// (formulas: Cuda_kernels/cp4Conv2dForward.cu:84-133, cp4Conv2dBackwardData.cu:57-108).
// Global loads and stores are coalesced along W; factors are staged in smem and
// read as broadcast float4.
#include <algorithm>
#include <cmath>
#include <cstdlib>
#include <cstring>

#pragma once
#include "common.cuh"

namespace b200cp {

namespace {

constexpr int kFactorCap = 4096;  // most floats of smem used to stage one factor chunk
constexpr int kKC = 4;            // channels per cp.async group
#ifndef B200CP_STAGES
#define B200CP_STAGES 4
#endif
constexpr int kStages = B200CP_STAGES;  // cp.async groups in flight per thread (one being consumed)

// floats of smem reserved for a factor chunk of a layer with `maxch` channels
inline int factor_cap(int maxch, int RP) {
  return std::min(kFactorCap, (int)align_up((size_t)maxch, kKC) * RP);
}

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int sz = valid ? 4 : 0;  // src-size 0: the destination is zero-filled, nothing is read
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;\n" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;\n" ::"n"(N) : "memory");
}

struct Geom {
  int N, Cin, Cout, H, W, Y, X, pad, R, Rs, r0, flip, accumulate;
  int TH, TW, mH, mW, THh, TWh, HPX, HPXs, OPX, tilesH, tilesW, cchunk, fcap;
};

// ---------------------------------------------------------------------------
// phase 1: channel contraction of a halo tile into smem  Ps[r][hp]
// ---------------------------------------------------------------------------
// Each thread streams its own pixels of every channel through a private smem FIFO with cp.async
// (kStages groups of kKC channels in flight), so global-load latency is covered without holding
// registers; only the thread that issued a copy reads it back, so no barrier is needed.
template <int RP, int PPT>
__device__ __forceinline__ void contract_batch(const Geom& g, const float* __restrict__ src_n, int nch,
                                               const float* __restrict__ Fg, float* Fs, float* Xst, float* Ps,
                                               int h0, int w0, int base, int tid, int nt) {
  const int HW = g.H * g.W;
  const int cols = nt * PPT;
  int off[PPT];
  bool ok[PPT];
  int hp[PPT];
#pragma unroll
  for (int k = 0; k < PPT; ++k) {
    hp[k] = base + k * nt + tid;
    const int hy = hp[k] / g.TWh, hx = hp[k] - hy * g.TWh;
    const int gy = h0 - g.mH + hy, gx = w0 - g.mW + hx;
    ok[k] = hp[k] < g.HPX && gy >= 0 && gy < g.H && gx >= 0 && gx < g.W;
    off[k] = ok[k] ? gy * g.W + gx : 0;
  }
  float acc[PPT][RP];
#pragma unroll
  for (int k = 0; k < PPT; ++k)
#pragma unroll
    for (int r = 0; r < RP; ++r) acc[k][r] = 0.f;

  float* mine = Xst + tid;  // column k*nt + tid of row (stage*kKC + j)
  for (int c0 = 0; c0 < nch; c0 += g.cchunk) {
    const int cc = min(g.cchunk, nch - c0);
    const int ccp = (cc + kKC - 1) / kKC * kKC;  // rows beyond cc are zero so that 0 * stale is never NaN
    __syncthreads();
    for (int i = tid; i < ccp * RP; i += nt) {
      const int c = i / RP, r = i - c * RP;
      Fs[i] = (r < g.R && c < cc) ? __ldg(Fg + (size_t)(c0 + c) * g.Rs + g.r0 + r) : 0.f;
    }
    __syncthreads();
    const float* src = src_n + (size_t)c0 * HW;
    const int ng = ccp / kKC;
    auto issue = [&](int grp) {
      if (grp < ng) {
        float* dst = mine + (size_t)(grp % kStages) * kKC * cols;
#pragma unroll
        for (int j = 0; j < kKC; ++j) {
          const int c = grp * kKC + j;
          const float* sc = src + (size_t)min(c, cc - 1) * HW;
#pragma unroll
          for (int k = 0; k < PPT; ++k) cp_async4(dst + j * cols + k * nt, sc + off[k], ok[k] && c < cc);
        }
      }
      cp_async_commit();
    };
#pragma unroll
    for (int s = 0; s < kStages - 1; ++s) issue(s);
    for (int grp = 0; grp < ng; ++grp) {
      issue(grp + kStages - 1);
      cp_async_wait<kStages - 1>();
      const float* xs = mine + (size_t)(grp % kStages) * kKC * cols;
#pragma unroll
      for (int j = 0; j < kKC; ++j) {
        float v[PPT];
#pragma unroll
        for (int k = 0; k < PPT; ++k) v[k] = xs[j * cols + k * nt];
        const float4* f4 = reinterpret_cast<const float4*>(Fs + (grp * kKC + j) * RP);
#pragma unroll
        for (int q = 0; q < RP / 4; ++q) {
          const float4 f = f4[q];
#pragma unroll
          for (int k = 0; k < PPT; ++k) {
            acc[k][4 * q + 0] = fmaf(v[k], f.x, acc[k][4 * q + 0]);
            acc[k][4 * q + 1] = fmaf(v[k], f.y, acc[k][4 * q + 1]);
            acc[k][4 * q + 2] = fmaf(v[k], f.z, acc[k][4 * q + 2]);
            acc[k][4 * q + 3] = fmaf(v[k], f.w, acc[k][4 * q + 3]);
          }
        }
      }
    }
    cp_async_wait<0>();
  }
#pragma unroll
  for (int k = 0; k < PPT; ++k)
    if (hp[k] < g.HPX) {
#pragma unroll
      for (int r = 0; r < RP; ++r) Ps[r * g.HPXs + hp[k]] = acc[k][r];
    }
}

// all batches of a tile; the host picks NT and PPT so that one batch covers the halo tile
template <int RP, int PPT>
__device__ __forceinline__ void contract_tile(const Geom& g, const float* __restrict__ src_n, int nch,
                                              const float* __restrict__ Fg, float* Fs, float* Xst, float* Ps,
                                              int h0, int w0, int tid, int nt) {
  for (int base = 0; base < g.HPX; base += nt * PPT)
    contract_batch<RP, PPT>(g, src_n, nch, Fg, Fs, Xst, Ps, h0, w0, base, tid, nt);
}

// stencil weights Ws[(y*X+x)*RP + r] = KH[y',r] * KW[x',r]
template <int RP>
__device__ __forceinline__ void load_weights(const Geom& g, const float* __restrict__ KH,
                                             const float* __restrict__ KW, float* Ws, int tid, int nt) {
  for (int i = tid; i < g.Y * g.X * RP; i += nt) {
    const int r = i % RP, yx = i / RP, y = yx / g.X, x = yx - y * g.X;
    const int yy = g.flip ? g.Y - 1 - y : y, xx = g.flip ? g.X - 1 - x : x;
    Ws[i] = r < g.R ? __ldg(KH + (size_t)yy * g.Rs + g.r0 + r) * __ldg(KW + (size_t)xx * g.Rs + g.r0 + r) : 0.f;
  }
}

// ---------------------------------------------------------------------------
// phases 2+3: stencil in smem, expansion to the output channels
// ---------------------------------------------------------------------------
template <int RP, int PPT>
__device__ __forceinline__ void expand_batch(const Geom& g, const float* Ps, const float* Ws,
                                             const float* __restrict__ Fg, float* Fs, float* __restrict__ dst_n,
                                             int nch, int h0, int w0, int base, int tid, int nt) {
  const int HW = g.H * g.W;
  float z[PPT][RP];
  int ooff[PPT];
  bool ok[PPT];
#pragma unroll
  for (int k = 0; k < PPT; ++k) {
    const int op = base + k * nt + tid;
    const int oy = op / g.TW, ox = op - oy * g.TW;
    const int gy = h0 + oy, gx = w0 + ox;
    ok[k] = op < g.OPX && gy < g.H && gx < g.W;
    ooff[k] = gy * g.W + gx;
#pragma unroll
    for (int r = 0; r < RP; ++r) z[k][r] = 0.f;
    if (ok[k]) {
      const float* p0 = Ps + (oy + g.mH - g.pad) * g.TWh + (ox + g.mW - g.pad);
      for (int y = 0; y < g.Y; ++y)
        for (int x = 0; x < g.X; ++x) {
          const float4* w4 = reinterpret_cast<const float4*>(Ws + (y * g.X + x) * RP);
          const float* p = p0 + y * g.TWh + x;
#pragma unroll
          for (int q = 0; q < RP / 4; ++q) {
            const float4 w = w4[q];
            z[k][4 * q + 0] = fmaf(w.x, p[(4 * q + 0) * g.HPXs], z[k][4 * q + 0]);
            z[k][4 * q + 1] = fmaf(w.y, p[(4 * q + 1) * g.HPXs], z[k][4 * q + 1]);
            z[k][4 * q + 2] = fmaf(w.z, p[(4 * q + 2) * g.HPXs], z[k][4 * q + 2]);
            z[k][4 * q + 3] = fmaf(w.w, p[(4 * q + 3) * g.HPXs], z[k][4 * q + 3]);
          }
        }
    }
  }
  for (int t0 = 0; t0 < nch; t0 += g.cchunk) {
    const int tc = min(g.cchunk, nch - t0);
    __syncthreads();
    for (int i = tid; i < tc * RP; i += nt) {
      const int t = i / RP, r = i - t * RP;
      Fs[i] = r < g.R ? __ldg(Fg + (size_t)(t0 + t) * g.Rs + g.r0 + r) : 0.f;
    }
    __syncthreads();
    float* dst = dst_n + (size_t)t0 * HW;
#pragma unroll 2
    for (int t = 0; t < tc; ++t) {
      float o[PPT];
#pragma unroll
      for (int k = 0; k < PPT; ++k) o[k] = 0.f;
      const float4* f4 = reinterpret_cast<const float4*>(Fs + t * RP);
#pragma unroll
      for (int q = 0; q < RP / 4; ++q) {
        const float4 f = f4[q];
#pragma unroll
        for (int k = 0; k < PPT; ++k) {
          o[k] = fmaf(z[k][4 * q + 0], f.x, o[k]);
          o[k] = fmaf(z[k][4 * q + 1], f.y, o[k]);
          o[k] = fmaf(z[k][4 * q + 2], f.z, o[k]);
          o[k] = fmaf(z[k][4 * q + 3], f.w, o[k]);
        }
      }
#pragma unroll
      for (int k = 0; k < PPT; ++k)
        if (ok[k]) {
          float* d = dst + (size_t)t * HW + ooff[k];
          *d = g.accumulate ? *d + o[k] : o[k];
        }
    }
  }
}


// ---------------------------------------------------------------------------
// host: tile choice.  A CTA of NT threads covers the (TH+2mH)x(TW+2mW) halo tile with PPT1
// pixels per thread and the TH x TW output tile with PPT3 pixels per thread, one batch each.
// ---------------------------------------------------------------------------
struct TileChoice {
  int TH = 0, TW = 0, NT = 0, PPT1 = 0, PPT3 = 0;
  size_t smem = 0;
  double cost = 1e300;
};

inline int max_ppt(int RP) { return RP <= 16 ? 4 : RP == 32 ? 2 : 1; }

// `planes` [RP][HPX] and `oplanes` [RP][OPX] smem arrays, `extra_const` + `extra_per_opx`*OPX more floats.
// `same_ppt`: the kernel has one PPT for both phases (backward-filter).
inline TileChoice choose_tile(int N, int H, int W, int Y, int X, int pad, double w1, double w3, int RP, int fcap, int planes,
                              int oplanes, int extra_const, int extra_per_opx, bool same_ppt, const DeviceInfo& di) {
  const int mH = std::max(pad, Y - 1 - pad), mW = std::max(pad, X - 1 - pad);
  TileChoice best;
  int fTH = 0, fTW = 0, fNT = 0;
  if (const char* e = getenv("B200CP_TILE")) {  // "TH,TW,NT": restrict the search (experiments)
    if (sscanf(e, "%d,%d,%d", &fTH, &fTW, &fNT) != 3) fTH = fTW = fNT = 0;
  }
  // candidate tile widths: the full width, powers of two, and the widths that divide W exactly (no ragged last column)
  int tws[16];
  int ntw = 0;
  auto add_tw = [&](int v) {
    if (v < 8 && v != W) return;
    if (v > W || v > 128) return;
    for (int i = 0; i < ntw; ++i)
      if (tws[i] == v) return;
    if (ntw < 16) tws[ntw++] = v;
  };
  add_tw(W);
  add_tw(64); add_tw(32); add_tw(16);
  for (int parts = 2; parts <= 8; ++parts)
    if (W % parts == 0) add_tw(W / parts);
  if (ntw == 0) tws[ntw++] = std::min(W, 64);
  for (int twi = 0; twi < ntw; ++twi) {
    const int TW = tws[twi];
    if (fTW && std::min(fTW, W) != TW) continue;
    for (int TH = 1; TH <= std::min(H, 64); ++TH) {
      if (fTH && std::min(fTH, H) != TH) continue;
      const int HPX = (TH + 2 * mH) * (TW + 2 * mW), OPX = TH * TW;
      const size_t sm0 = sizeof(float) * ((size_t)fcap + (size_t)Y * X * RP +
                                          (size_t)planes * RP * align_up(HPX, 4) +
                                          (size_t)oplanes * RP * align_up(OPX, 4) + extra_const +
                                          (size_t)extra_per_opx * align_up(OPX, 4));
      if ((int)sm0 > di.smem_optin) break;
      for (int p1 = 1; p1 <= max_ppt(RP); ++p1) {
        int NT = (int)align_up((size_t)ceil_div(HPX, p1), 32);
        if (NT > 256) { if (p1 < max_ppt(RP)) continue; NT = 256; }   // several batches only as a last resort
        if (NT < 64) NT = 64;
        if (fNT && fNT != NT) continue;
        const size_t sm = sm0 + sizeof(float) * kStages * kKC * NT * p1;  // the cp.async FIFO
        if ((int)sm > di.smem_optin) continue;
        int p3 = std::max(1, std::min(p1, ceil_div(OPX, NT)));
        if (same_ppt) p3 = p1; else p3 = std::max(p3, p1 - 1);
        const double b1 = ceil_div(HPX, NT * p1) * p1, b3 = ceil_div(OPX, NT * p3) * p3;
        const long ctas = (long)N * ceil_div(H, TH) * ceil_div(W, TW);
        const int occ_smem = std::max(1, (int)((228 * 1024) / (sm + 1024)));
        const int occ = std::max(1, std::min(std::min(occ_smem, 2048 / NT), 65536 / (NT * 128)));
        const long per_sm = (ctas + di.sm_count - 1) / di.sm_count;
        const double per_cta = b1 * w1 + b3 * w3;
        const double warps = (double)std::min<long>(occ, per_sm) * NT / 32.0;
        const double lat = warps >= 16 ? 1.0 : std::sqrt(16.0 / warps);
        // narrow per-thread work (small PPT) re-reads factors from smem more often per FMA
        const double ilp = 1.0 + 0.25 / p1;
        // measured on B200: small CTAs pay their factor staging, barriers and halo set-up per few pixels
        const double small = 1.0 + 96.0 / NT;
        const double cost = (double)per_sm * per_cta * NT * lat * ilp * small;
        if (cost < best.cost) { best.TH = TH; best.TW = TW; best.NT = NT; best.PPT1 = p1; best.PPT3 = p3; best.smem = sm; best.cost = cost; }
      }
    }
  }
  if (getenv("B200CP_DEBUG"))
    fprintf(stderr, "[b200cp] tile TH=%d TW=%d NT=%d PPT=%d/%d smem=%zu RP=%d planes=%d\n", best.TH, best.TW, best.NT,
            best.PPT1, best.PPT3, best.smem, RP, planes);
  return best;
}

inline Geom make_geom(const Cp4Args& a, const TileChoice& t, int RP, int fcap) {
  Geom g;
  g.N = a.N; g.Cin = a.Cin; g.Cout = a.Cout; g.H = a.H; g.W = a.W; g.Y = a.Y; g.X = a.X; g.pad = a.pad;
  g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0; g.flip = a.flip; g.accumulate = a.accumulate;
  g.TH = t.TH; g.TW = t.TW;
  g.mH = std::max(a.pad, a.Y - 1 - a.pad);
  g.mW = std::max(a.pad, a.X - 1 - a.pad);
  g.THh = g.TH + 2 * g.mH; g.TWh = g.TW + 2 * g.mW;
  g.HPX = g.THh * g.TWh; g.HPXs = (int)align_up(g.HPX, 4); g.OPX = g.TH * g.TW;
  g.tilesH = ceil_div(a.H, g.TH); g.tilesW = ceil_div(a.W, g.TW);
  g.fcap = fcap;
  g.cchunk = fcap / RP;
  return g;
}

}  // namespace
}  // namespace b200cp
