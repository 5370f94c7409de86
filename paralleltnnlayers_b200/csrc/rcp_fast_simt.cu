// Reshaped-CP conv2d of order 3 with a 3x3 spatial core: register-tiled kernel on CUDA cores (exact fp32).
//
//   V[n,(t1,t2,t3),h,w] = sum_r sum_{i,j} S[i,j,r] sum_{c1,c2,c3} A1[c1,t1,r] A2[c2,t2,r] A3[c3,t3,r]
//                                                   X[n,(c1,c2,c3),h+i-1,w+j-1]
// (test/layers.py:716-773; the reference's fused kernel, Kernels/rcp_fused_nchw.cu:4-77, is this sum for one
// fixed order-2 shape).  One CTA owns a TH x TW tile of one image and keeps the tile of all input channels,
// with its halo, in shared memory for the whole rank loop.  Per rank:
//   phase 1  a thread owns one (c2,c3) pair and a strip of SW pixels of one tile row; for each c1 it applies
//            the rank's 3x3 filter in registers and folds the first mode (c1 -> t1) at once, then writes
//            Y1[t1][c2][c3][pixel] to shared memory;
//   phase 2  a thread owns one (pixel, t1, half of t3); it walks c2, contracts c3 -> t3 and expands into its
//            [t2][t3/2] accumulators, which stay in registers across all ranks.
// So the rank-sized intermediates never leave the SM and the only global traffic is the tile and the output.
// The data gradient is the same kernel with the factors read transposed and the filter flipped.
#include <algorithm>
#include <cstdlib>

#include "common.cuh"

namespace b200cp {

namespace {

struct RcpFastArgs {
  const float* X;
  const float* A[3];
  const float* S;
  float* V;
  int N, H, W, R;
  int fsi[3], fso[3];  // element (contracted i, produced o) of factor k at A[k][(i*fsi + o*fso)*R + r]
  int flip, tilesH, tilesW;
};

template <int I1, int O1, int I2, int O2, int I3, int O3, int TH, int TW, int SW, int NT>
struct RcpFastCfg {
  static constexpr int CIN = I1 * I2 * I3, COUT = O1 * O2 * O3;
  static constexpr int PIX = TH * TW, PIXP = PIX | 1;           // odd pitches: conflict-free scalar accesses
  static constexpr int HWP = TW + 2, HPX = (TH + 2) * HWP, HPXP = HPX | 1;
  static constexpr int COMBOS = I2 * I3, SPR = TW / SW, STRIPS = TH * SPR;
  static constexpr int OH = O3 / 2;
  static constexpr int OFF2 = I1 * O1, OFF3 = OFF2 + I2 * O2, OFFS = OFF3 + I3 * O3;
  static constexpr int FPR = (OFFS + 9 + 3) / 4 * 4;            // factor floats per rank, 16-byte multiple
  static constexpr int XS = (CIN * HPXP + 3) / 4 * 4;
  static constexpr int Y1S = O1 * COMBOS * PIXP;
  static_assert(TW % SW == 0, "strips tile a row");
  static_assert(O3 % 2 == 0 && O2 % 4 == 0 && (I1 * O1) % 4 == 0 && (I2 * O2) % 4 == 0, "vector loads of factor rows");
  static size_t smem_bytes(int R) { return sizeof(float) * ((size_t)R * FPR + XS + Y1S); }
};

template <int I1, int O1, int I2, int O2, int I3, int O3, int TH, int TW, int SW, int NT>
__global__ void __launch_bounds__(NT, 1) rcp3_fast_kernel(const RcpFastArgs a) {
  using K = RcpFastCfg<I1, O1, I2, O2, I3, O3, TH, TW, SW, NT>;
  extern __shared__ __align__(16) float sm[];
  float* Fs = sm;
  float* Xs = Fs + (size_t)a.R * K::FPR;
  float* Y1 = Xs + K::XS;
  const int tid = threadIdx.x;

  int b = blockIdx.x;
  const int tw = b % a.tilesW;
  b /= a.tilesW;
  const int th = b % a.tilesH;
  const int n = b / a.tilesH;
  const int h0 = th * TH, w0 = tw * TW;

  // factors of every rank, laid out per rank as [A1 | A2 | A3 | S]
  for (int i = tid; i < a.R * K::FPR; i += NT) {
    const int r = i / K::FPR, e = i - r * K::FPR;
    float v = 0.f;
    if (e < K::OFF2) {
      const int ii = e / O1, oo = e - ii * O1;
      v = __ldg(a.A[0] + (size_t)(ii * a.fsi[0] + oo * a.fso[0]) * a.R + r);
    } else if (e < K::OFF3) {
      const int q = e - K::OFF2, ii = q / O2, oo = q - ii * O2;
      v = __ldg(a.A[1] + (size_t)(ii * a.fsi[1] + oo * a.fso[1]) * a.R + r);
    } else if (e < K::OFFS) {
      const int q = e - K::OFF3, ii = q / O3, oo = q - ii * O3;
      v = __ldg(a.A[2] + (size_t)(ii * a.fsi[2] + oo * a.fso[2]) * a.R + r);
    } else if (e < K::OFFS + 9) {
      const int tap = e - K::OFFS;
      v = __ldg(a.S + (size_t)(a.flip ? 8 - tap : tap) * a.R + r);
    }
    Fs[i] = v;
  }
  // the tile of every input channel with a one-pixel halo; outside the image reads as zero
  {
    const float* Xn = a.X + (size_t)n * K::CIN * a.H * a.W;
    for (int i = tid; i < K::CIN * K::HPX; i += NT) {
      const int c = i / K::HPX, hp = i - c * K::HPX;
      const int hy = hp / K::HWP, hx = hp - hy * K::HWP;
      const int gy = h0 - 1 + hy, gx = w0 - 1 + hx;
      const bool ok = gy >= 0 && gy < a.H && gx >= 0 && gx < a.W;
      Xs[c * K::HPXP + hp] = ok ? __ldg(Xn + ((size_t)c * a.H + gy) * a.W + gx) : 0.f;
    }
  }

  // phase-2 role
  const bool chain = tid < K::PIX * O1 * 2;
  const int px = tid % K::PIX;
  const int t1 = (tid / K::PIX) % O1;
  const int t3h = tid / (K::PIX * O1);
  float acc[O2][K::OH];
#pragma unroll
  for (int i = 0; i < O2; ++i)
#pragma unroll
    for (int j = 0; j < K::OH; ++j) acc[i][j] = 0.f;
  __syncthreads();

  for (int r = 0; r < a.R; ++r) {
    const float* F = Fs + (size_t)r * K::FPR;
    // ---- phase 1: 3x3 filter of this rank and the first mode ----
    for (int item = tid; item < K::COMBOS * K::STRIPS; item += NT) {
      const int combo = item % K::COMBOS, strip = item / K::COMBOS;
      const int row = strip / K::SPR, col0 = (strip - row * K::SPR) * SW;
      float s[9];
#pragma unroll
      for (int t = 0; t < 9; ++t) s[t] = F[K::OFFS + t];
      float y[O1][SW];
#pragma unroll
      for (int o = 0; o < O1; ++o)
#pragma unroll
        for (int j = 0; j < SW; ++j) y[o][j] = 0.f;
#pragma unroll
      for (int c1 = 0; c1 < I1; ++c1) {
        const float* xs = Xs + (size_t)(c1 * K::COMBOS + combo) * K::HPXP + row * K::HWP + col0;
        float xr[SW];
#pragma unroll
        for (int j = 0; j < SW; ++j) xr[j] = 0.f;
#pragma unroll
        for (int dy = 0; dy < 3; ++dy) {
          float v[SW + 2];
#pragma unroll
          for (int j = 0; j < SW + 2; ++j) v[j] = xs[dy * K::HWP + j];
#pragma unroll
          for (int j = 0; j < SW; ++j) {
            xr[j] = fmaf(s[dy * 3 + 0], v[j], xr[j]);
            xr[j] = fmaf(s[dy * 3 + 1], v[j + 1], xr[j]);
            xr[j] = fmaf(s[dy * 3 + 2], v[j + 2], xr[j]);
          }
        }
        const float4* a1 = reinterpret_cast<const float4*>(F + c1 * O1);
        float w1[O1];
#pragma unroll
        for (int q = 0; q < O1 / 4; ++q) {
          const float4 t = a1[q];
          w1[4 * q] = t.x; w1[4 * q + 1] = t.y; w1[4 * q + 2] = t.z; w1[4 * q + 3] = t.w;
        }
#pragma unroll
        for (int o = 0; o < O1; ++o)
#pragma unroll
          for (int j = 0; j < SW; ++j) y[o][j] = fmaf(w1[o], xr[j], y[o][j]);
      }
#pragma unroll
      for (int o = 0; o < O1; ++o) {
        float* d = Y1 + (size_t)(o * K::COMBOS + combo) * K::PIXP + row * TW + col0;
#pragma unroll
        for (int j = 0; j < SW; ++j) d[j] = y[o][j];
      }
    }
    __syncthreads();
    // ---- phase 2: modes 2 and 3 into the register accumulators ----
    if (chain) {
      float a3[I3][K::OH];
#pragma unroll
      for (int c3 = 0; c3 < I3; ++c3)
#pragma unroll
        for (int j = 0; j < K::OH; ++j) a3[c3][j] = F[K::OFF3 + c3 * O3 + t3h * K::OH + j];
#pragma unroll 2
      for (int c2 = 0; c2 < I2; ++c2) {
        const float* y = Y1 + (size_t)((t1 * I2 + c2) * I3) * K::PIXP + px;
        float x[I3];
#pragma unroll
        for (int c3 = 0; c3 < I3; ++c3) x[c3] = y[c3 * K::PIXP];
        float tmp[K::OH];
#pragma unroll
        for (int j = 0; j < K::OH; ++j) tmp[j] = 0.f;
#pragma unroll
        for (int c3 = 0; c3 < I3; ++c3)
#pragma unroll
          for (int j = 0; j < K::OH; ++j) tmp[j] = fmaf(a3[c3][j], x[c3], tmp[j]);
        const float4* a2 = reinterpret_cast<const float4*>(F + K::OFF2 + c2 * O2);
#pragma unroll
        for (int q = 0; q < O2 / 4; ++q) {
          const float4 t = a2[q];
          const float w2[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
          for (int u = 0; u < 4; ++u)
#pragma unroll
            for (int j = 0; j < K::OH; ++j) acc[4 * q + u][j] = fmaf(w2[u], tmp[j], acc[4 * q + u][j]);
        }
      }
    }
    __syncthreads();
  }

  if (chain) {
    const int gy = h0 + px / TW, gx = w0 + px % TW;
    if (gy < a.H && gx < a.W) {
      float* Vn = a.V + (size_t)n * K::COUT * a.H * a.W + (size_t)gy * a.W + gx;
#pragma unroll
      for (int t2 = 0; t2 < O2; ++t2)
#pragma unroll
        for (int j = 0; j < K::OH; ++j) {
          const int t = (t1 * O2 + t2) * O3 + t3h * K::OH + j;
          Vn[(size_t)t * a.H * a.W] = acc[t2][j];
        }
    }
  }
}

template <int I1, int O1, int I2, int O2, int I3, int O3, int TH, int TW, int SW, int NT>
int launch_fast(RcpFastArgs a, const DeviceInfo& di, cudaStream_t st, bool* fits) {
  using K = RcpFastCfg<I1, O1, I2, O2, I3, O3, TH, TW, SW, NT>;
  const size_t smem = K::smem_bytes(a.R);
  *fits = smem <= (size_t)di.smem_optin;
  if (!*fits) return B200CP_OK;
  a.tilesH = ceil_div(a.H, TH);
  a.tilesW = ceil_div(a.W, TW);
  const long ctas = (long)a.N * a.tilesH * a.tilesW;
  if (ctas > 0x7fffffffL) { *fits = false; return B200CP_OK; }
  auto kern = rcp3_fast_kernel<I1, O1, I2, O2, I3, O3, TH, TW, SW, NT>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)ctas, NT, smem, st>>>(a);
  B200CP_LAUNCH_OK("rcp3_fast_kernel");
  return B200CP_OK;
}

}  // namespace

// Launches the register-tiled kernel when the layer has the shape it is compiled for (order 3, modes
// (4,8,8) -> (4,8,8), 3x3 core); *done tells the caller whether it did.  din/dout and the strides describe the
// factors as the chain kernel's host code does (contracted index first).
int rcp_fast_launch(int N, int H, int W, int order, const int* din, const int* dout, const int* fsi, const int* fso,
                    int R, int FH, int FW, const float* X, const float* const* A, const float* S, float* V, bool flip,
                    cudaStream_t st, bool* done) {
  *done = false;
  if (order != 3 || FH != 3 || FW != 3) return B200CP_OK;
  if (!(din[0] == 4 && dout[0] == 4 && din[1] == 8 && dout[1] == 8 && din[2] == 8 && dout[2] == 8)) return B200CP_OK;
  if (getenv("B200CP_NO_FAST")) return B200CP_OK;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  RcpFastArgs a{};
  a.X = X; a.S = S; a.V = V;
  a.N = N; a.H = H; a.W = W; a.R = R; a.flip = flip ? 1 : 0;
  for (int k = 0; k < 3; ++k) { a.A[k] = A[k]; a.fsi[k] = fsi[k]; a.fso[k] = fso[k]; }
  // 7x7 tiles waste no pixels when 7 divides the image; 8x8 tiles otherwise
  const auto cost = [&](int th, int tw) {
    const long ctas = (long)N * ceil_div(H, th) * ceil_div(W, tw);
    return (double)((ctas + di.sm_count - 1) / di.sm_count) * th * tw;
  };
  bool fits = false;
  const char* force = getenv("B200CP_RCP_TILE");  // "7" or "8": experiments and tests
  const bool seven = force ? force[0] == '7' : cost(7, 7) <= cost(8, 8);
  if (seven) {
    if (int rc = launch_fast<4, 4, 8, 8, 8, 8, 7, 7, 7, 448>(a, di, st, &fits)) return rc;
  } else {
    if (int rc = launch_fast<4, 4, 8, 8, 8, 8, 8, 8, 8, 512>(a, di, st, &fits)) return rc;
  }
  *done = fits;
  return B200CP_OK;
}

}  // namespace b200cp
