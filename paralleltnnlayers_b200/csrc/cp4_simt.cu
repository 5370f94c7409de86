// CP4 conv2d on CUDA cores (exact fp32): forward, backward-data, backward-filter.
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

#include "common.cuh"

namespace b200cp {

namespace {

constexpr int kFactorCap = 4096;  // floats of smem used to stage one factor chunk

struct Geom {
  int N, Cin, Cout, H, W, Y, X, pad, R, Rs, r0, flip, accumulate;
  int TH, TW, mH, mW, THh, TWh, HPX, HPXs, OPX, tilesH, tilesW, cchunk;
};

// ---------------------------------------------------------------------------
// phase 1: channel contraction of a halo tile into smem  Ps[r][hp]
// ---------------------------------------------------------------------------
template <int RP, int PPT>
__device__ __forceinline__ void contract_batch(const Geom& g, const float* __restrict__ src_n, int nch,
                                               const float* __restrict__ Fg, float* Fs, float* Ps, int h0, int w0,
                                               int base, int tid, int nt) {
  const int HW = g.H * g.W;
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

  for (int c0 = 0; c0 < nch; c0 += g.cchunk) {
    const int cc = min(g.cchunk, nch - c0);
    __syncthreads();
    for (int i = tid; i < cc * RP; i += nt) {
      const int c = i / RP, r = i - c * RP;
      Fs[i] = r < g.R ? __ldg(Fg + (size_t)(c0 + c) * g.Rs + g.r0 + r) : 0.f;
    }
    __syncthreads();
    const float* src = src_n + (size_t)c0 * HW;
#pragma unroll 4
    for (int c = 0; c < cc; ++c) {
      float v[PPT];
#pragma unroll
      for (int k = 0; k < PPT; ++k) v[k] = ok[k] ? __ldg(src + (size_t)c * HW + off[k]) : 0.f;
      const float4* f4 = reinterpret_cast<const float4*>(Fs + c * RP);
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
#pragma unroll
  for (int k = 0; k < PPT; ++k)
    if (hp[k] < g.HPX) {
#pragma unroll
      for (int r = 0; r < RP; ++r) Ps[r * g.HPXs + hp[k]] = acc[k][r];
    }
}

template <int RP, int PPT>
__device__ __forceinline__ void contract_tile(const Geom& g, const float* __restrict__ src_n, int nch,
                                              const float* __restrict__ Fg, float* Fs, float* Ps, int h0, int w0,
                                              int tid, int nt) {
  int base = 0;
  for (; base + nt * PPT <= g.HPX; base += nt * PPT)
    contract_batch<RP, PPT>(g, src_n, nch, Fg, Fs, Ps, h0, w0, base, tid, nt);
  if (PPT > 1) {
    for (; base < g.HPX; base += nt) contract_batch<RP, 1>(g, src_n, nch, Fg, Fs, Ps, h0, w0, base, tid, nt);
  } else if (base < g.HPX) {
    contract_batch<RP, 1>(g, src_n, nch, Fg, Fs, Ps, h0, w0, base, tid, nt);
  }
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

template <int RP, int PPT>
__global__ void __launch_bounds__(256) cp4_conv_kernel(const Geom g, const float* __restrict__ in,
                                                       const float* __restrict__ Fin,
                                                       const float* __restrict__ Fout,
                                                       const float* __restrict__ KH,
                                                       const float* __restrict__ KW, float* __restrict__ out) {
  extern __shared__ __align__(16) float smem[];
  float* Fs = smem;                       // [cchunk][RP]
  float* Ws = Fs + kFactorCap;            // [Y*X][RP]
  float* Ps = Ws + g.Y * g.X * RP;        // [RP][HPXs]
  const int tid = threadIdx.x, nt = blockDim.x;
  int b = blockIdx.x;
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  const size_t HW = (size_t)g.H * g.W;

  load_weights<RP>(g, KH, KW, Ws, tid, nt);
  contract_tile<RP, PPT>(g, in + (size_t)n * g.Cin * HW, g.Cin, Fin, Fs, Ps, h0, w0, tid, nt);
  __syncthreads();
  float* dst_n = out + (size_t)n * g.Cout * HW;
  int base = 0;
  for (; base + nt * PPT <= g.OPX; base += nt * PPT)
    expand_batch<RP, PPT>(g, Ps, Ws, Fout, Fs, dst_n, g.Cout, h0, w0, base, tid, nt);
  if (PPT > 1) {
    for (; base < g.OPX; base += nt) expand_batch<RP, 1>(g, Ps, Ws, Fout, Fs, dst_n, g.Cout, h0, w0, base, tid, nt);
  } else if (base < g.OPX) {
    expand_batch<RP, 1>(g, Ps, Ws, Fout, Fs, dst_n, g.Cout, h0, w0, base, tid, nt);
  }
}

// ---------------------------------------------------------------------------
// host: tile choice
// ---------------------------------------------------------------------------
inline double batch_cost(int px, int nt, int ppt) {
  const int full = px / (nt * ppt);
  const int rem = px - full * nt * ppt;
  return full * ppt + ceil_div(rem, nt) * 1.1;
}

struct TileChoice {
  int TH, TW, NT;
  size_t smem;
  double cost;
};

// `planes` = number of [RP][HPX] + `oplanes` [RP][OPX] smem arrays the kernel keeps.
TileChoice choose_tile(int N, int H, int W, int Y, int X, int pad, int Cin, int Cout, int RP, int PPT, int planes,
                       int oplanes, int extra_const, int extra_per_opx, double work_scale, const DeviceInfo& di) {
  const int mH = std::max(pad, Y - 1 - pad), mW = std::max(pad, X - 1 - pad);
  TileChoice best{0, 0, 0, 0, 1e300};
  if (const char* e = getenv("B200CP_TILE")) {  // "TH,TW,NT" override for experiments
    int th, tw, nt;
    if (sscanf(e, "%d,%d,%d", &th, &tw, &nt) == 3 && th > 0 && tw > 0 && (nt == 64 || nt == 128 || nt == 256)) {
      th = std::min(th, H);
      tw = std::min(tw, W);
      const int HPX = (th + 2 * mH) * (tw + 2 * mW);
      const size_t sm = sizeof(float) * ((size_t)kFactorCap + (size_t)Y * X * RP +
                                         (size_t)planes * RP * align_up(HPX, 4) +
                                         (size_t)oplanes * RP * align_up(th * tw, 4) + extra_const +
                                         (size_t)extra_per_opx * align_up(th * tw, 4));
      if ((int)sm <= di.smem_optin) return TileChoice{th, tw, nt, sm, 0};
    }
  }
  int tws[3] = {W, 64, 32};
  for (int twi = 0; twi < 3; ++twi) {
    const int TW = tws[twi];
    if (TW > W || (twi == 0 && W > 96)) continue;
    for (int TH = 1; TH <= std::min(H, 64); ++TH) {
      const int HPX = (TH + 2 * mH) * (TW + 2 * mW), OPX = TH * TW;
      const size_t sm = sizeof(float) * ((size_t)kFactorCap + (size_t)Y * X * RP +
                                         (size_t)planes * RP * align_up(HPX, 4) +
                                         (size_t)oplanes * RP * align_up(OPX, 4) + extra_const +
                                         (size_t)extra_per_opx * align_up(OPX, 4));
      if ((int)sm > di.smem_optin) break;
      for (int NT = 128; NT <= 256; NT *= 2) {
        const long ctas = (long)N * ceil_div(H, TH) * ceil_div(W, TW);
        const int occ_smem = std::max(1, (int)((228 * 1024) / (sm + 1024)));
        const int occ = std::max(1, std::min(std::min(occ_smem, 2048 / NT), 65536 / (NT * 128)));
        const long per_sm = (ctas + di.sm_count - 1) / di.sm_count;
        const double per_cta = batch_cost(HPX, NT, PPT) * (double)Cin * RP * work_scale +
                               batch_cost(OPX, NT, PPT) * ((double)Cout * RP * work_scale + 2.5 * Y * X * RP);
        const double warps = (double)std::min<long>(occ, per_sm) * NT / 32.0;
        const double lat = warps >= 12 ? 1.0 : std::sqrt(12.0 / warps);
        const double cost = (double)per_sm * per_cta * NT * lat;
        if (cost < best.cost) best = TileChoice{TH, TW, NT, sm, cost};
      }
    }
  }
  return best;
}

Geom make_geom(const Cp4Args& a, const TileChoice& t, int RP) {
  Geom g;
  g.N = a.N; g.Cin = a.Cin; g.Cout = a.Cout; g.H = a.H; g.W = a.W; g.Y = a.Y; g.X = a.X; g.pad = a.pad;
  g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0; g.flip = a.flip; g.accumulate = a.accumulate;
  g.TH = t.TH; g.TW = t.TW;
  g.mH = std::max(a.pad, a.Y - 1 - a.pad);
  g.mW = std::max(a.pad, a.X - 1 - a.pad);
  g.THh = g.TH + 2 * g.mH; g.TWh = g.TW + 2 * g.mW;
  g.HPX = g.THh * g.TWh; g.HPXs = (int)align_up(g.HPX, 4); g.OPX = g.TH * g.TW;
  g.tilesH = ceil_div(a.H, g.TH); g.tilesW = ceil_div(a.W, g.TW);
  g.cchunk = kFactorCap / RP;
  return g;
}

template <int RP, int PPT>
int launch_conv(const Cp4Args& a, const DeviceInfo& di, cudaStream_t st) {
  const TileChoice t = choose_tile(a.N, a.H, a.W, a.Y, a.X, a.pad, a.Cin, a.Cout, RP, PPT, 1, 0, 0, 0, 1.0, di);
  if (t.NT == 0) return fail(B200CP_ERR_UNSUPPORTED, "cp4: no tile of this filter fits in shared memory");
  const Geom g = make_geom(a, t, RP);
  auto kern = cp4_conv_kernel<RP, PPT>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem));
  const long ctas = (long)a.N * g.tilesH * g.tilesW;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4: too many tiles");
  kern<<<(unsigned)ctas, t.NT, t.smem, st>>>(g, a.in, a.Fin, a.Fout, a.KH, a.KW, a.out);
  B200CP_LAUNCH_OK("cp4_conv_kernel");
  return B200CP_OK;
}

}  // namespace

int cp4_simt_launch(const Cp4Args& a, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  switch (padded_rank(a.R)) {
    case 4: return launch_conv<4, 4>(a, di, st);
    case 8: return launch_conv<8, 4>(a, di, st);
    case 16: return launch_conv<16, 4>(a, di, st);
    case 32: return launch_conv<32, 2>(a, di, st);
    default: return launch_conv<64, 1>(a, di, st);
  }
}

// ===========================================================================
// backward-filter
// ===========================================================================
//
// Per tile (one CTA):
//   Q = K0^T dU and P = K1^T X on the halo tile (phase-1 code above)
//   per rank r, per pixel:  rows_i = sum_j KW[j] P[i][j],  cols_j = sum_i KH[i] P[i][j]
//       Z  = sum_i KH[i] rows_i            -> Zs[r][px]
//       Qt = sum_{i,j} KH[i] KW[j] Q[h-i+p][w-j+p]   -> Qts[r][px]
//       dKH[i,r] += Q * rows_i,  dKW[j,r] += Q * cols_j     (warp shuffle + fixed-order smem sum)
//   dK0[t,r] = sum_px dU[t,px] Zs[r][px],  dK1[c,r] = sum_px X[c,px] Qts[r][px]
//       one warp per group of channels, lanes stride the pixels, butterfly reduction.
// Each CTA writes its partial gradients to workspace[cta][...]; a second kernel
// sums the partials in CTA order, so the result is bitwise reproducible.
// Formulas: Cuda_kernels/cp4Conv2dBackwardFilter.cu:91-104,142-155,192-205,241-254.
namespace {

struct GeomF {
  Geom g;      // Cin = C (X channels), Cout = T (dU channels)
  int F;       // filter size
  int nparam;  // (T + C + 2F) * R  floats per partial (R = ranks of this launch)
  int OPXs;
};

// Reduce M values per lane across the warp so that every value's warp-sum lands
// on exactly one lane.  After the call, lane l holds sums for indices
// idx(l, j) = j + (M >> 5) * bitrev-free mapping computed by `owner_index`.
template <int M>
__device__ __forceinline__ void warp_transpose_reduce(float (&v)[M], int lane) {
  // halving steps while more than one value per lane remains
#pragma unroll
  for (int off = 16, m = M / 2; off >= 1; off >>= 1, m >>= 1) {
    if (m >= 1) {
      const bool hi = lane & off;
#pragma unroll
      for (int i = 0; i < m; ++i) {
        const float send = hi ? v[i] : v[i + m];
        const float keep = hi ? v[i + m] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    }
  }
}
// index (0..M-1) of the j-th value lane `lane` owns after warp_transpose_reduce<M>
template <int M>
__device__ __forceinline__ int owner_index(int lane, int j) {
  int idx = 0, m = M / 2;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1, m >>= 1)
    if (m >= 1 && (lane & off)) idx += m;
  return idx + j;
}

// dK[ch, r] partial = sum over the tile's pixels of src[n, ch, px] * Vs[r][px]
template <int RP, int CG>
__device__ __forceinline__ void pixel_reduce(const Geom& g, int OPXs, const float* __restrict__ src_n, int nch,
                                             const float* Vs, const int* pixoff, float* __restrict__ part, int tid,
                                             int nt) {
  const int lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
  const size_t HW = (size_t)g.H * g.W;
  constexpr int M = CG * RP;
  constexpr int PER = M >= 32 ? M / 32 : 1;  // values per lane after the reduction
  for (int c0 = warp * CG; c0 < nch; c0 += nwarp * CG) {
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; ++i) acc[i] = 0.f;
    const float* s[CG];
#pragma unroll
    for (int j = 0; j < CG; ++j) s[j] = src_n + (size_t)min(c0 + j, nch - 1) * HW;
    for (int p = lane; p < g.OPX; p += 32) {
      const int po = pixoff[p];
      float d[CG];
#pragma unroll
      for (int j = 0; j < CG; ++j) d[j] = po >= 0 ? __ldg(s[j] + po) : 0.f;
#pragma unroll
      for (int r = 0; r < RP; ++r) {
        const float z = Vs[r * OPXs + p];
#pragma unroll
        for (int j = 0; j < CG; ++j) acc[j * RP + r] = fmaf(d[j], z, acc[j * RP + r]);
      }
    }
    warp_transpose_reduce<M>(acc, lane);
    // M < 32: after log2(M) halving steps each group of 32/M lanes holds the same sum
    const bool owner = M >= 32 || (lane & ((32 / (M < 32 ? M : 32)) - 1)) == 0;
    if (owner) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int idx = owner_index<M>(lane, j);
        const int cj = idx / RP, r = idx - cj * RP;
        if (c0 + cj < nch && r < g.R) part[(size_t)(c0 + cj) * g.R + r] = acc[j];
      }
    }
  }
}

template <int RP, int PPT, int F>
__global__ void __launch_bounds__(256) cp4_bwd_filter_kernel(const GeomF gf, const float* __restrict__ X,
                                                             const float* __restrict__ dU,
                                                             const float* __restrict__ K0,
                                                             const float* __restrict__ K1,
                                                             const float* __restrict__ KH,
                                                             const float* __restrict__ KW,
                                                             float* __restrict__ partial) {
  const Geom& g = gf.g;
  extern __shared__ __align__(16) float smem[];
  float* Fs = smem;                              // [cchunk][RP]
  float* KHs = Fs + kFactorCap;                  // [F][RP]
  float* KWs = KHs + F * RP;                     // [F][RP]
  float* red = KWs + F * RP;                     // [8 warps][2F]
  float* Ps = red + 8 * 2 * F;                   // [RP][HPXs]
  float* Qs = Ps + RP * g.HPXs;                  // [RP][HPXs]
  float* Zs = Qs + RP * g.HPXs;                  // [RP][OPXs]
  float* Qts = Zs + RP * gf.OPXs;                // [RP][OPXs]
  int* pixoff = reinterpret_cast<int*>(Qts + RP * gf.OPXs);  // [OPXs]

  const int tid = threadIdx.x, nt = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
  int b = blockIdx.x;
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  const size_t HW = (size_t)g.H * g.W;
  const float* Xn = X + (size_t)n * g.Cin * HW;
  const float* dUn = dU + (size_t)n * g.Cout * HW;
  float* part = partial + (size_t)blockIdx.x * gf.nparam;
  float* part_K0 = part;
  float* part_K1 = part_K0 + (size_t)g.Cout * g.R;
  float* part_KH = part_K1 + (size_t)g.Cin * g.R;
  float* part_KW = part_KH + (size_t)F * g.R;

  for (int i = tid; i < F * RP; i += nt) {
    const int r = i % RP, f = i / RP;
    KHs[i] = r < g.R ? __ldg(KH + (size_t)f * g.Rs + g.r0 + r) : 0.f;
    KWs[i] = r < g.R ? __ldg(KW + (size_t)f * g.Rs + g.r0 + r) : 0.f;
  }
  for (int p = tid; p < g.OPX; p += nt) {
    const int oy = p / g.TW, ox = p - oy * g.TW;
    const int gy = h0 + oy, gx = w0 + ox;
    pixoff[p] = (gy < g.H && gx < g.W) ? gy * g.W + gx : -1;
  }
  contract_tile<RP, PPT>(g, Xn, g.Cin, K1, Fs, Ps, h0, w0, tid, nt);
  contract_tile<RP, PPT>(g, dUn, g.Cout, K0, Fs, Qs, h0, w0, tid, nt);
  __syncthreads();

  // per-rank stencils and the small-factor gradients
  const int p = g.pad;
  for (int r = 0; r < g.R; ++r) {
    float kh[F], kw[F], aH[F], aW[F];
#pragma unroll
    for (int i = 0; i < F; ++i) {
      kh[i] = KHs[i * RP + r];
      kw[i] = KWs[i * RP + r];
      aH[i] = 0.f;
      aW[i] = 0.f;
    }
    const float* Pr = Ps + r * g.HPXs;
    const float* Qr = Qs + r * g.HPXs;
    for (int op = tid; op < g.OPX; op += nt) {
      const int oy = op / g.TW, ox = op - oy * g.TW;
      float zv = 0.f, qt = 0.f;
      if (pixoff[op] >= 0) {
        // window origin (tap 0,0) in halo coordinates; mH == mW == pad here
        const float* pw = Pr + oy * g.TWh + ox;
        const float* qw = Qr + oy * g.TWh + ox;
        const float q = qw[p * g.TWh + p];
        float cols[F];
#pragma unroll
        for (int j = 0; j < F; ++j) cols[j] = 0.f;
#pragma unroll
        for (int i = 0; i < F; ++i) {
          float row = 0.f, qrow = 0.f;
#pragma unroll
          for (int j = 0; j < F; ++j) {
            const float pv = pw[i * g.TWh + j];
            row = fmaf(kw[j], pv, row);
            cols[j] = fmaf(kh[i], pv, cols[j]);
            // flipped window: Q[h - i + p][w - j + p]  -> halo (oy + 2p - i, ox + 2p - j)
            qrow = fmaf(kw[j], qw[(2 * p - i) * g.TWh + (2 * p - j)], qrow);
          }
          zv = fmaf(kh[i], row, zv);
          qt = fmaf(kh[i], qrow, qt);
          aH[i] = fmaf(q, row, aH[i]);
        }
#pragma unroll
        for (int j = 0; j < F; ++j) aW[j] = fmaf(q, cols[j], aW[j]);
      }
      Zs[r * gf.OPXs + op] = zv;
      Qts[r * gf.OPXs + op] = qt;
    }
    // block reduction of aH, aW in a fixed order: lanes (shuffle tree), then warps
#pragma unroll
    for (int i = 0; i < F; ++i) {
#pragma unroll
      for (int off = 16; off >= 1; off >>= 1) {
        aH[i] += __shfl_xor_sync(0xffffffffu, aH[i], off);
        aW[i] += __shfl_xor_sync(0xffffffffu, aW[i], off);
      }
    }
    __syncthreads();  // previous rank's `red` fully consumed
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < F; ++i) {
        red[warp * 2 * F + i] = aH[i];
        red[warp * 2 * F + F + i] = aW[i];
      }
    }
    __syncthreads();
    if (tid < 2 * F) {
      float s = 0.f;
      for (int w = 0; w < nwarp; ++w) s += red[w * 2 * F + tid];
      if (tid < F) part_KH[(size_t)tid * g.R + r] = s;
      else part_KW[(size_t)(tid - F) * g.R + r] = s;
    }
  }
  __syncthreads();

  constexpr int CG = (RP >= 64) ? 1 : (RP == 32 ? 2 : 4);
  pixel_reduce<RP, CG>(g, gf.OPXs, dUn, g.Cout, Zs, pixoff, part_K0, tid, nt);
  pixel_reduce<RP, CG>(g, gf.OPXs, Xn, g.Cin, Qts, pixoff, part_K1, tid, nt);
}

// out[j] = sum over CTAs of partial[cta][j], CTA order fixed
__global__ void cp4_reduce_partials_kernel(const float* __restrict__ partial, int nparts, int nparam, int R, int Rs,
                                           int r0, float* __restrict__ dK) {
  const int j = blockIdx.x * blockDim.x + threadIdx.x;
  if (j >= nparam) return;
  float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
  int i = 0;
  for (; i + 4 <= nparts; i += 4) {
    s0 += partial[(size_t)(i + 0) * nparam + j];
    s1 += partial[(size_t)(i + 1) * nparam + j];
    s2 += partial[(size_t)(i + 2) * nparam + j];
    s3 += partial[(size_t)(i + 3) * nparam + j];
  }
  for (; i < nparts; ++i) s0 += partial[(size_t)i * nparam + j];
  const float s = (s0 + s1) + (s2 + s3);
  // j indexes [T*R | C*R | F*R | F*R] with row length R; the output rows have length Rs
  // the packed output has the same T, C, F, F row sections, with rows of length Rs
  const int row = j / R, r = j - row * R;
  dK[(size_t)row * Rs + r0 + r] = s;
}

template <int RP, int PPT, int F>
int launch_bwd_filter(const Cp4BwdFilterArgs& a, const DeviceInfo& di, cudaStream_t st) {
  const TileChoice t = choose_tile(a.N, a.H, a.W, F, F, a.pad, a.C + a.T, a.C + a.T, RP, PPT, 2, 2, 2 * F * RP + 16 * F, 1, 0.5,
                                   di);
  if (t.NT == 0) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: no tile fits in shared memory");
  Cp4Args ca{};
  ca.N = a.N; ca.Cin = a.C; ca.Cout = a.T; ca.H = a.H; ca.W = a.W; ca.Y = F; ca.X = F; ca.pad = a.pad;
  ca.R = a.R; ca.Rs = a.Rs; ca.r0 = a.r0;
  GeomF gf;
  gf.g = make_geom(ca, t, RP);
  gf.F = F;
  gf.nparam = (a.T + a.C + 2 * F) * a.R;
  gf.OPXs = (int)align_up(gf.g.OPX, 4);
  const size_t smem = sizeof(float) * ((size_t)kFactorCap + 2 * F * RP + 16 * F + 2 * (size_t)RP * gf.g.HPXs +
                                       2 * (size_t)RP * gf.OPXs + gf.OPXs);
  if ((int)smem > di.smem_optin) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: tile exceeds shared memory");
  const long ctas = (long)a.N * gf.g.tilesH * gf.g.tilesW;
  const size_t need = (size_t)ctas * gf.nparam * sizeof(float);
  if (a.ws == nullptr || a.ws_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "cp4 bwd-filter: workspace of %zu bytes needed, %zu given", need, a.ws_bytes);
  auto kern = cp4_bwd_filter_kernel<RP, PPT, F>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)ctas, t.NT, smem, st>>>(gf, a.X, a.dU, a.K0, a.K1, a.KH, a.KW, (float*)a.ws);
  B200CP_LAUNCH_OK("cp4_bwd_filter_kernel");
  cp4_reduce_partials_kernel<<<ceil_div(gf.nparam, 128), 128, 0, st>>>((const float*)a.ws, (int)ctas, gf.nparam, a.R,
                                                                      a.Rs, a.r0, a.dK);
  B200CP_LAUNCH_OK("cp4_reduce_partials_kernel");
  return B200CP_OK;
}

template <int F>
int dispatch_bwd_filter_rank(const Cp4BwdFilterArgs& a, const DeviceInfo& di, cudaStream_t st) {
  switch (padded_rank(a.R)) {
    case 4: return launch_bwd_filter<4, 4, F>(a, di, st);
    case 8: return launch_bwd_filter<8, 4, F>(a, di, st);
    case 16: return launch_bwd_filter<16, 4, F>(a, di, st);
    case 32: return launch_bwd_filter<32, 2, F>(a, di, st);
    default: return launch_bwd_filter<64, 1, F>(a, di, st);
  }
}

}  // namespace

// Upper bound of the workspace over every tile the heuristic can pick: one
// partial per CTA, and a CTA never covers fewer than one row segment of 32 pixels.
size_t cp4_bwd_filter_simt_workspace(const b200cp_tensor_shape& s) {
  const size_t R = std::min<unsigned>(s.Rank, 64);
  const size_t nparam = ((size_t)s.T + s.C + 2 * s.Y) * R;
  const size_t max_ctas = (size_t)s.N * s.H * ceil_div((int)s.W, 32);
  return max_ctas * nparam * sizeof(float);
}

int cp4_bwd_filter_simt_launch(const Cp4BwdFilterArgs& a, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  switch (a.F) {
    case 1: return dispatch_bwd_filter_rank<1>(a, di, st);
    case 3: return dispatch_bwd_filter_rank<3>(a, di, st);
    case 5: return dispatch_bwd_filter_rank<5>(a, di, st);
    case 7: return dispatch_bwd_filter_rank<7>(a, di, st);
    case 11: return dispatch_bwd_filter_rank<11>(a, di, st);
    default: return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: filter size %d not in {1,3,5,7,11}", a.F);
  }
}

// ===========================================================================
// dense filter gradient and recomposition (helpers of the reference's tests)
// ===========================================================================
namespace {

// dK[t,c,y,x] = sum_{n,h,w} dU[n,t,h,w] X[n,c,h+y-pad,w+x-pad]; one CTA per (t,c), fixed-order sum.
__global__ void cp4_bwd_filter_full_kernel(b200cp_tensor_shape s, const float* __restrict__ X,
                                           const float* __restrict__ dU, float* __restrict__ dK) {
  const int t = blockIdx.x / s.C, c = blockIdx.x % s.C;
  const int HW = s.H * s.W;
  __shared__ float red[8];
  for (unsigned yx = 0; yx < s.Y * s.X; ++yx) {
    const int y = yx / s.X, x = yx % s.X;
    float acc = 0.f;
    for (unsigned n = 0; n < s.N; ++n) {
      const float* du = dU + ((size_t)n * s.T + t) * HW;
      const float* xi = X + ((size_t)n * s.C + c) * HW;
      for (int p = threadIdx.x; p < HW; p += blockDim.x) {
        const int h = p / s.W, w = p % s.W;
        const int hh = h + y - (int)s.pad, ww = w + x - (int)s.pad;
        if (hh >= 0 && hh < (int)s.H && ww >= 0 && ww < (int)s.W) acc = fmaf(du[p], xi[hh * s.W + ww], acc);
      }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float sum = 0.f;
      for (unsigned w = 0; w < blockDim.x / 32; ++w) sum += red[w];
      dK[((size_t)(t * s.C + c) * s.Y + y) * s.X + x] = sum;
    }
  }
}

__global__ void cp4_recompose_kernel(b200cp_tensor_shape s, const float* __restrict__ K0,
                                     const float* __restrict__ K1, const float* __restrict__ KH,
                                     const float* __restrict__ KW, float* __restrict__ K) {
  const size_t total = (size_t)s.T * s.C * s.Y * s.X;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const unsigned x = i % s.X, y = (i / s.X) % s.Y, c = (i / (s.X * s.Y)) % s.C, t = i / ((size_t)s.X * s.Y * s.C);
    float acc = 0.f;
    for (unsigned r = 0; r < s.Rank; ++r)
      acc += K0[t * s.Rank + r] * K1[c * s.Rank + r] * KH[y * s.Rank + r] * KW[x * s.Rank + r];
    K[i] = acc;
  }
}

}  // namespace

int cp4_bwd_filter_full_launch(const b200cp_tensor_shape& s, const float* X, const float* dU, float* dK,
                               cudaStream_t st) {
  cp4_bwd_filter_full_kernel<<<s.T * s.C, 256, 0, st>>>(s, X, dU, dK);
  B200CP_LAUNCH_OK("cp4_bwd_filter_full_kernel");
  return B200CP_OK;
}

int cp4_recompose_launch(const b200cp_tensor_shape& s, const float* K0, const float* K1, const float* KH,
                         const float* KW, float* K, cudaStream_t st) {
  const size_t total = (size_t)s.T * s.C * s.Y * s.X;
  const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 4096);
  cp4_recompose_kernel<<<blocks, 256, 0, st>>>(s, K0, K1, KH, KW, K);
  B200CP_LAUNCH_OK("cp4_recompose_kernel");
  return B200CP_OK;
}

}  // namespace b200cp
