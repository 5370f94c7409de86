// Reshaped-CP conv2d and CP dense layer on CUDA cores (exact fp32).
//
// Both layers apply, per rank r, a Kronecker-structured channel map
//   M_r = F_1[:,:,r] (x) F_2[:,:,r] (x) ... (x) F_m[:,:,r]
// to a tile of "columns" (output pixels of one image for rCP, samples of the
// batch for the dense layer) and sum over r.  One CTA owns one tile and keeps
// every per-rank intermediate in shared memory:
//   rCP   : Xs[C][halo px] --stencil S[:,:,r]--> buf[C][px] --mode 1..m--> registers (+= over r)
//   dense : Xs[I][samples]                                  --mode 1..m--> registers (+= over r)
// A mode step views its input as [A][IK][Bn] (Bn = remaining input modes x
// columns, columns innermost) and writes [A][OK][Bn]; one thread owns 4
// adjacent columns and all OK outputs of one (a, b) position.
// The data gradient is the same kernel with the factors read transposed (and
// the stencil flipped).  Formulas: Kernels/rcp_fused_nchw.cu:4-77 and
// Kernels/dense_cp.cu:4-46 (fixed shapes there), test/layers.py:445-465,716-773.
#include <algorithm>
#include <cstring>

#include "common.cuh"

namespace b200cp {

namespace {

constexpr int kMaxOrder = 4;
constexpr int kMaxDim = 16;  // largest mode size the register tiles cover
constexpr int kNT = 256;

struct ChainGeom {
  int m;
  int din[kMaxOrder], dout[kMaxOrder];
  int fsi[kMaxOrder], fso[kMaxOrder];  // factor element (i,o,r) at F[(i*fsi + o*fso)*R + r]
  int R;
  int Cin, Cout;   // products of din / dout
  int bufElems;    // rows of the largest intermediate
  // columns
  int PIX;         // columns per tile, multiple of 4
  // rCP geometry (conv == 1)
  int conv, N, H, W, FH, FW, pad, flip;
  int TH, TW, mH, mW, TWh, HPX, HPXs, tilesH, tilesW;
  // dense geometry
  int B;
};

struct ChainPtrs {
  const float* X;
  const float* F[kMaxOrder];
  const float* S;
  float* Y;
};

template <int OKP>
__device__ __forceinline__ void load_f(const float* Fs, int i, float (&f)[OKP]) {
  const float4* p = reinterpret_cast<const float4*>(Fs + i * kMaxDim);
#pragma unroll
  for (int q = 0; q < OKP / 4; ++q) {
    const float4 v = p[q];
    f[4 * q] = v.x; f[4 * q + 1] = v.y; f[4 * q + 2] = v.z; f[4 * q + 3] = v.w;
  }
}

// one mode step, smem -> smem
template <int OKP>
__device__ __forceinline__ void mode_step(const float* src, float* dst, const float* Fs, int A, int IK, int OK,
                                          int Bn, int tid) {
  const int bq = Bn >> 2, items = A * bq;
  for (int it = tid; it < items; it += kNT) {
    const int a = it / bq, bv = it - a * bq;
    float acc[OKP][4];
#pragma unroll
    for (int o = 0; o < OKP; ++o) acc[o][0] = acc[o][1] = acc[o][2] = acc[o][3] = 0.f;
    const float* s = src + (size_t)a * IK * Bn + bv * 4;
    for (int i = 0; i < IK; ++i) {
      const float4 x = *reinterpret_cast<const float4*>(s + (size_t)i * Bn);
      float f[OKP];
      load_f<OKP>(Fs, i, f);
#pragma unroll
      for (int o = 0; o < OKP; ++o) {
        acc[o][0] = fmaf(f[o], x.x, acc[o][0]);
        acc[o][1] = fmaf(f[o], x.y, acc[o][1]);
        acc[o][2] = fmaf(f[o], x.z, acc[o][2]);
        acc[o][3] = fmaf(f[o], x.w, acc[o][3]);
      }
    }
    float* d = dst + (size_t)a * OK * Bn + bv * 4;
#pragma unroll
    for (int o = 0; o < OKP; ++o)
      if (o < OK) *reinterpret_cast<float4*>(d + (size_t)o * Bn) = make_float4(acc[o][0], acc[o][1], acc[o][2], acc[o][3]);
  }
}

// last mode step, smem -> persistent registers (accumulated over ranks)
template <int OKP, int MAXIT>
__device__ __forceinline__ void last_step(const float* src, const float* Fs, int A, int IK, int Bn, int tid,
                                          float (&acc)[MAXIT][OKP][4]) {
  const int bq = Bn >> 2, items = A * bq;
#pragma unroll
  for (int j = 0; j < MAXIT; ++j) {
    const int it = tid + j * kNT;
    if (it < items) {
      const int a = it / bq, bv = it - a * bq;
      const float* s = src + (size_t)a * IK * Bn + bv * 4;
      for (int i = 0; i < IK; ++i) {
        const float4 x = *reinterpret_cast<const float4*>(s + (size_t)i * Bn);
        float f[OKP];
        load_f<OKP>(Fs, i, f);
#pragma unroll
        for (int o = 0; o < OKP; ++o) {
          acc[j][o][0] = fmaf(f[o], x.x, acc[j][o][0]);
          acc[j][o][1] = fmaf(f[o], x.y, acc[j][o][1]);
          acc[j][o][2] = fmaf(f[o], x.z, acc[j][o][2]);
          acc[j][o][3] = fmaf(f[o], x.w, acc[j][o][3]);
        }
      }
    }
  }
}

__device__ __forceinline__ void any_mode_step(int okp, const float* src, float* dst, const float* Fs, int A, int IK,
                                              int OK, int Bn, int tid) {
  if (okp == 4) mode_step<4>(src, dst, Fs, A, IK, OK, Bn, tid);
  else if (okp == 8) mode_step<8>(src, dst, Fs, A, IK, OK, Bn, tid);
  else mode_step<16>(src, dst, Fs, A, IK, OK, Bn, tid);
}

template <int OKP, int MAXIT>
__global__ void __launch_bounds__(kNT) chain_kernel(const ChainGeom g, const ChainPtrs p) {
  extern __shared__ __align__(16) float smem[];
  float* Fs = smem;                                   // [m][kMaxDim][kMaxDim]  factors of the current rank
  float* Ss = Fs + kMaxOrder * kMaxDim * kMaxDim;     // [32*32]                 stencil of the current rank
  int* coloff = reinterpret_cast<int*>(Ss + 1024);    // [PIX] global offset of a column (-1: padding)
  int* hbase = coloff + g.PIX;                        // [PIX] halo index of a column's (0,0) tap
  float* Xs = reinterpret_cast<float*>(hbase + g.PIX);
  const int xrows = g.conv ? g.HPXs : g.PIX;
  float* bufA = Xs + (size_t)g.Cin * xrows;
  float* bufB = bufA + (size_t)g.bufElems * g.PIX;
  const int tid = threadIdx.x;

  // ---- stage the input tile -------------------------------------------------
  size_t out_base = 0;  // offset of this tile's image / first sample in Y
  if (g.conv) {
    int b = blockIdx.x;
    const int tw = b % g.tilesW;
    b /= g.tilesW;
    const int th = b % g.tilesH;
    const int n = b / g.tilesH;
    const int h0 = th * g.TH, w0 = tw * g.TW;
    const size_t HW = (size_t)g.H * g.W;
    for (int c = tid; c < g.PIX; c += kNT) {
      const int oy = c / g.TW, ox = c - oy * g.TW;
      const int gy = h0 + oy, gx = w0 + ox;
      coloff[c] = (c < g.TH * g.TW && gy < g.H && gx < g.W) ? gy * g.W + gx : -1;
      hbase[c] = (c < g.TH * g.TW) ? oy * g.TWh + ox : 0;  // halo origin is (h0 - mH, w0 - mW)
    }
    const float* Xn = p.X + (size_t)n * g.Cin * HW;
    for (int i = tid; i < g.Cin * g.HPXs; i += kNT) {
      const int c = i / g.HPXs, hp = i - c * g.HPXs;
      const int hy = hp / g.TWh, hx = hp - hy * g.TWh;
      const int gy = h0 - g.mH + hy, gx = w0 - g.mW + hx;
      const bool ok = hp < g.HPX && gy >= 0 && gy < g.H && gx >= 0 && gx < g.W;
      Xs[i] = ok ? __ldg(Xn + (size_t)c * HW + gy * g.W + gx) : 0.f;
    }
    out_base = (size_t)n * g.Cout * HW;
  } else {
    const int n0 = blockIdx.x * g.PIX;
    for (int c = tid; c < g.PIX; c += kNT) coloff[c] = (n0 + c < g.B) ? c : -1;
    for (int i = tid; i < g.Cin; i += kNT) {
#pragma unroll 4
      for (int s = 0; s < g.PIX; ++s)
        Xs[(size_t)i * g.PIX + s] = (n0 + s < g.B) ? __ldg(p.X + (size_t)(n0 + s) * g.Cin + i) : 0.f;
    }
    out_base = (size_t)n0 * g.Cout;
  }

  float acc[MAXIT][OKP][4];
#pragma unroll
  for (int j = 0; j < MAXIT; ++j)
#pragma unroll
    for (int o = 0; o < OKP; ++o) acc[j][o][0] = acc[j][o][1] = acc[j][o][2] = acc[j][o][3] = 0.f;

  const int last = g.m - 1;
  int Alast = 1;
  for (int k = 0; k < last; ++k) Alast *= g.dout[k];

  for (int r = 0; r < g.R; ++r) {
    __syncthreads();  // previous rank finished with Fs / Ss / buffers
    for (int i = tid; i < g.m * kMaxDim * kMaxDim; i += kNT) {
      const int k = i / (kMaxDim * kMaxDim), io = i - k * kMaxDim * kMaxDim, ii = io / kMaxDim, oo = io - ii * kMaxDim;
      Fs[i] = (ii < g.din[k] && oo < g.dout[k]) ? __ldg(p.F[k] + (size_t)(ii * g.fsi[k] + oo * g.fso[k]) * g.R + r) : 0.f;
    }
    if (g.conv)
      for (int i = tid; i < g.FH * g.FW; i += kNT) {
        const int y = i / g.FW, x = i - y * g.FW;
        const int yy = g.flip ? g.FH - 1 - y : y, xx = g.flip ? g.FW - 1 - x : x;
        Ss[i] = __ldg(p.S + (size_t)(yy * g.FW + xx) * g.R + r);
      }
    __syncthreads();
    const float* src = Xs;
    if (g.conv) {
      // per-rank single-channel stencil applied to every input channel
      for (int i = tid; i < g.Cin * g.PIX; i += kNT) {
        const int c = i / g.PIX, col = i - c * g.PIX;
        const float* x0 = Xs + (size_t)c * g.HPXs + hbase[col];
        float v = 0.f;
        for (int y = 0; y < g.FH; ++y)
          for (int x = 0; x < g.FW; ++x) v = fmaf(Ss[y * g.FW + x], x0[y * g.TWh + x], v);
        bufA[i] = coloff[col] >= 0 ? v : 0.f;
      }
      __syncthreads();
      src = bufA;
    }
    float* dst = (src == bufA) ? bufB : bufA;
    int A = 1, Bn = g.Cin * g.PIX;
    for (int k = 0; k < last; ++k) {
      Bn /= g.din[k];
      const int okp = g.dout[k] <= 4 ? 4 : g.dout[k] <= 8 ? 8 : 16;
      any_mode_step(okp, src, dst, Fs + k * kMaxDim * kMaxDim, A, g.din[k], g.dout[k], Bn, tid);
      __syncthreads();
      A *= g.dout[k];
      src = dst;
      dst = (src == bufA) ? bufB : bufA;
    }
    last_step<OKP, MAXIT>(src, Fs + last * kMaxDim * kMaxDim, Alast, g.din[last], g.PIX, tid, acc);
  }

  // ---- write the tile --------------------------------------------------------
  const int OK = g.dout[last];
  const int bq = g.PIX >> 2, items = Alast * bq;
#pragma unroll
  for (int j = 0; j < MAXIT; ++j) {
    const int it = tid + j * kNT;
    if (it < items) {
      const int a = it / bq, bv = it - a * bq;
#pragma unroll
      for (int o = 0; o < OKP; ++o)
        if (o < OK) {
          const int ch = a * OK + o;
#pragma unroll
          for (int v = 0; v < 4; ++v) {
            const int co = coloff[bv * 4 + v];
            if (co >= 0) {
              if (g.conv) p.Y[out_base + (size_t)ch * g.H * g.W + co] = acc[j][o][v];
              else p.Y[out_base + (size_t)co * g.Cout + ch] = acc[j][o][v];
            }
          }
        }
    }
  }
}

size_t chain_smem(const ChainGeom& g) {
  const size_t xrows = g.conv ? g.HPXs : g.PIX;
  return sizeof(float) * ((size_t)kMaxOrder * kMaxDim * kMaxDim + 1024 + 2 * (size_t)g.PIX + (size_t)g.Cin * xrows +
                          2 * (size_t)g.bufElems * g.PIX);
}

template <int OKP, int MAXIT>
int launch_chain(const ChainGeom& g, const ChainPtrs& p, long ctas, cudaStream_t st) {
  const size_t smem = chain_smem(g);
  auto kern = chain_kernel<OKP, MAXIT>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)ctas, kNT, smem, st>>>(g, p);
  B200CP_LAUNCH_OK("chain_kernel");
  return B200CP_OK;
}

int fill_modes(ChainGeom& g, int order, const int* idims, const int* odims, int R, bool transposed, const char* who) {
  if (order < 1 || order > kMaxOrder) return fail(B200CP_ERR_UNSUPPORTED, "%s: order %d not in 1..%d", who, order, kMaxOrder);
  if (R < 1) return fail(B200CP_ERR_INVALID_ARG, "%s: rank must be positive", who);
  g.m = order;
  g.R = R;
  long cin = 1, cout = 1;
  for (int k = 0; k < order; ++k) {
    const int i = idims[k], o = odims[k];
    if (i < 1 || o < 1) return fail(B200CP_ERR_INVALID_ARG, "%s: mode %d has a non-positive size", who, k);
    if (i > kMaxDim || o > kMaxDim)
      return fail(B200CP_ERR_UNSUPPORTED, "%s: mode %d size (%d -> %d) exceeds %d", who, k, i, o, kMaxDim);
    // storage is always [i][o][R]; a transposed launch contracts over o
    g.din[k] = transposed ? o : i;
    g.dout[k] = transposed ? i : o;
    g.fsi[k] = transposed ? 1 : o;
    g.fso[k] = transposed ? o : 1;
    cin *= g.din[k];
    cout *= g.dout[k];
  }
  if (cin > (1 << 20) || cout > (1 << 20)) return fail(B200CP_ERR_UNSUPPORTED, "%s: more than 2^20 channels", who);
  g.Cin = (int)cin;
  g.Cout = (int)cout;
  // rows of the largest intermediate written by a non-final mode step (and by the stencil)
  long best = 0, a = 1, b = cin;
  for (int k = 0; k + 1 < order; ++k) {
    b /= g.din[k];
    a *= g.dout[k];
    best = std::max(best, a * b);
  }
  g.bufElems = (int)best;
  return B200CP_OK;
}

int dispatch_chain(const ChainGeom& g, const ChainPtrs& p, long ctas, cudaStream_t st) {
  const int ok = g.dout[g.m - 1];
  if (ok <= 4) return launch_chain<4, 8>(g, p, ctas, st);
  if (ok <= 8) return launch_chain<8, 4>(g, p, ctas, st);
  return launch_chain<16, 2>(g, p, ctas, st);
}

int max_items(const ChainGeom& g) {
  const int ok = g.dout[g.m - 1];
  return (ok <= 4 ? 8 : ok <= 8 ? 4 : 2) * kNT;
}

}  // namespace

int rcp_chain_launch(int N, int H, int W, int order, const int* cdims, const int* tdims, int R, int FH, int FW,
                     const float* X, const float* const* A, const float* S, float* V, bool transposed,
                     cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  ChainGeom g{};
  if (int rc = fill_modes(g, order, cdims, tdims, R, transposed, "rcp")) return rc;
  if (FH < 1 || FW < 1 || FH > 31 || FW > 31 || !(FH & 1) || !(FW & 1))
    return fail(B200CP_ERR_UNSUPPORTED, "rcp: filter %dx%d must be odd and at most 31", FH, FW);
  if (N < 1 || H < 1 || W < 1) return fail(B200CP_ERR_INVALID_ARG, "rcp: non-positive N/H/W");
  {
    bool done = false;
    if (int rc = rcp_fast_launch(N, H, W, order, g.din, g.dout, g.fsi, g.fso, R, FH, FW, X, A, S, V, transposed, st, &done))
      return rc;
    if (done) return B200CP_OK;
  }
  g.conv = 1; g.N = N; g.H = H; g.W = W; g.FH = FH; g.FW = FW; g.flip = transposed ? 1 : 0;
  g.mH = (FH - 1) / 2; g.mW = (FW - 1) / 2;  // "same" padding per axis (test/test_conv2d_rcp.py:11)
  g.pad = g.mH;
  g.bufElems = std::max(g.bufElems, g.Cin);  // the stencil output [Cin][PIX] also lives in a buffer
  const int Alast = g.Cout / g.dout[g.m - 1];
  // pick the tile with the best (halo efficiency x padding efficiency x wave efficiency)
  double best = 0;
  int bestTH = 0, bestTW = 0;
  const int tws[4] = {W, 64, 32, 16};
  for (int ti = 0; ti < 4; ++ti) {
    const int TW = tws[ti];
    if (TW > W || (ti == 0 && W > 64) || (ti > 0 && TW >= W)) continue;
    for (int TH = 1; TH <= std::min(H, 32); ++TH) {
      ChainGeom t = g;
      t.TH = TH; t.TW = TW; t.PIX = (int)align_up((size_t)TH * TW, 4); t.TWh = TW + 2 * g.mW;
      t.HPX = (TH + 2 * g.mH) * t.TWh; t.HPXs = (int)align_up(t.HPX, 4);
      if ((long)Alast * (t.PIX / 4) > max_items(g)) break;
      const size_t sm = chain_smem(t);
      if ((int)sm > di.smem_optin) break;
      const long ctas = (long)N * ceil_div(H, TH) * ceil_div(W, TW);
      const long slots = (long)di.sm_count * std::max<long>(1, (228 * 1024) / (long)(sm + 1024));
      const double wave_eff = (double)ctas / (double)(ceil_div((int)ctas, (int)slots) * slots);
      const double cover = (double)H * W / ((double)ceil_div(H, TH) * TH * ceil_div(W, TW) * TW);
      const double score = cover * ((double)TH * TW / t.HPX + 1.0) * ((double)TH * TW / t.PIX) * (0.5 + 0.5 * wave_eff);
      if (score > best) { best = score; bestTH = TH; bestTW = TW; }
    }
  }
  if (!bestTH) return fail(B200CP_ERR_UNSUPPORTED, "rcp: no tile fits (channels %d -> %d)", g.Cin, g.Cout);
  g.TH = bestTH; g.TW = bestTW; g.PIX = (int)align_up((size_t)bestTH * bestTW, 4);
  g.TWh = g.TW + 2 * g.mW; g.HPX = (g.TH + 2 * g.mH) * g.TWh; g.HPXs = (int)align_up(g.HPX, 4);
  g.tilesH = ceil_div(H, g.TH); g.tilesW = ceil_div(W, g.TW);
  ChainPtrs p{};
  p.X = X; p.S = S; p.Y = V;
  for (int k = 0; k < order; ++k) p.F[k] = A[k];
  const long ctas = (long)N * g.tilesH * g.tilesW;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "rcp: too many tiles");
  return dispatch_chain(g, p, ctas, st);
}

int dense_chain_launch(int B, int order, const int* idims, const int* odims, int R, const float* X,
                       const float* const* F, float* Y, bool transposed, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  ChainGeom g{};
  if (int rc = fill_modes(g, order, idims, odims, R, transposed, "dense_cp")) return rc;
  if (B < 1) return fail(B200CP_ERR_INVALID_ARG, "dense_cp: batch must be positive");
  {
    bool done = false;
    if (int rc = dense_fast_launch(B, order, g.din, g.dout, g.fsi, g.fso, R, X, F, Y, st, &done)) return rc;
    if (done) return B200CP_OK;
  }
  g.conv = 0; g.B = B;
  const int Alast = g.Cout / g.dout[g.m - 1];
  int pix = 0;
  for (int cand = 16; cand >= 4; cand -= 4) {
    ChainGeom t = g;
    t.PIX = cand;
    if ((long)Alast * (cand / 4) > max_items(g)) continue;
    if ((int)chain_smem(t) > di.smem_optin) continue;
    // keep at least ~2 waves of tiles when the batch allows it
    if (cand > 4 && (long)ceil_div(B, cand) < 2L * di.sm_count) continue;
    pix = cand;
    break;
  }
  if (!pix) return fail(B200CP_ERR_UNSUPPORTED, "dense_cp: layer %d -> %d does not fit on chip", g.Cin, g.Cout);
  g.PIX = pix;
  ChainPtrs p{};
  p.X = X; p.Y = Y;
  for (int k = 0; k < order; ++k) p.F[k] = F[k];
  return dispatch_chain(g, p, ceil_div(B, pix), st);
}

}  // namespace b200cp
