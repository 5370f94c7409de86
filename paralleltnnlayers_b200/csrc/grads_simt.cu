// Factor gradients of the rCP conv and the CP dense layer (exact fp32).
//
// Both go through the dense gradient of the recomposed weight,
//   G[t, c, y, x] = sum_{n, h, w} dV[n, t, h, w] * Xpad[n, c, h + y, w + x]
// (the quantity cp4_conv2d_backward_filter_full_gpu produces,
// Cuda_kernels/cp4Conv2dBackwardFilter.cu:47-56; for the dense layer H = W = 1
// and G = dY^T X), followed by a contraction of G with all factors but one:
//   dA_k[c_k, t_k, r] = sum_{other modes, y, x} G * S[y, x, r] * prod_{j != k} A_j[c_j, t_j, r]
//   dS[y, x, r]       = sum_{t, c} G * prod_k A_k[c_k, t_k, r]
// G is a tiled SIMT GEMM whose K dimension runs over (image, pixel); every sum
// is done in a fixed order (bitwise reproducible).
#include <algorithm>

#include "common.cuh"

namespace b200cp {

namespace {

constexpr int TM = 64, TN = 64, TK = 16, NTH = 256;

// G[tap][t][c] for one 64x64 tile of (t, c) and one tap; K loop over images and pixel chunks.
// PIXMAJOR: operands are [n][ch][HW] (pixels contiguous).  Otherwise HW == 1 and operands are [n][ch].
template <bool PIXMAJOR>
__global__ void __launch_bounds__(NTH) dense_grad_kernel(int N, int T, int C, int H, int W, int FH, int FW, int padH,
                                                         int padW, const float* __restrict__ dV,
                                                         const float* __restrict__ X, float* __restrict__ G) {
  __shared__ __align__(16) float As[TK][TM + 4];
  __shared__ __align__(16) float Bs[TK][TN + 4];
  const int tid = threadIdx.x;
  const int t0 = blockIdx.y * TM, c0 = blockIdx.x * TN;
  const int tap = blockIdx.z, ty = tap / FW, tx = tap - ty * FW;
  const int dy = ty - padH, dx = tx - padW;
  const int HW = H * W;
  const int mi = tid / 16, ni = tid % 16;  // 16x16 threads, 4x4 outputs each
  float acc[4][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[i][j] = 0.f;

  const int kchunks = PIXMAJOR ? ceil_div(HW, TK) : ceil_div(N, TK);
  const int nouter = PIXMAJOR ? N : 1;
  for (int n = 0; n < nouter; ++n)
    for (int kc = 0; kc < kchunks; ++kc) {
      __syncthreads();
      // 64 channels x 16 k values per operand = 1024 elements, 4 per thread
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int idx = tid + e * NTH;
        int ch, k;
        if (PIXMAJOR) { ch = idx / TK; k = idx % TK; } else { k = idx / TM; ch = idx % TM; }
        float a = 0.f, b = 0.f;
        if (PIXMAJOR) {
          const int p = kc * TK + k;
          if (p < HW) {
            if (t0 + ch < T) a = __ldg(dV + ((size_t)n * T + t0 + ch) * HW + p);
            const int h = p / W, w = p - h * W;
            const int hh = h + dy, ww = w + dx;
            if (c0 + ch < C && hh >= 0 && hh < H && ww >= 0 && ww < W)
              b = __ldg(X + ((size_t)n * C + c0 + ch) * HW + hh * W + ww);
          }
        } else {
          const int nn = kc * TK + k;
          if (nn < N) {
            if (t0 + ch < T) a = __ldg(dV + (size_t)nn * T + t0 + ch);
            if (c0 + ch < C) b = __ldg(X + (size_t)nn * C + c0 + ch);
          }
        }
        As[k][ch] = a;
        Bs[k][ch] = b;
      }
      __syncthreads();
#pragma unroll
      for (int k = 0; k < TK; ++k) {
        const float4 a = *reinterpret_cast<const float4*>(&As[k][mi * 4]);
        const float4 b = *reinterpret_cast<const float4*>(&Bs[k][ni * 4]);
        const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
      }
    }
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int t = t0 + mi * 4 + i, c = c0 + ni * 4 + j;
      if (t < T && c < C) G[((size_t)t * C + c) * FH * FW + tap] = acc[i][j];
    }
}

struct ContractGeom {
  int m, R, T, C, taps;
  int cd[4], td[4];
  int out_off[5];  // offsets of dA_0..dA_{m-1}, dS in the flat output index space (in units of elements / R)
};
struct ContractPtrs {
  const float* A[4];
  const float* S;   // may be null (dense layer): treated as 1, taps == 1
  float* dA[4];
  float* dS;        // may be null
};

// One CTA per output element (k, c_k, t_k, r) or (tap, r); fixed-order block reduction.
__global__ void __launch_bounds__(128) contract_factors_kernel(const ContractGeom g, const ContractPtrs p,
                                                               const float* __restrict__ G) {
  const int r = blockIdx.x % g.R;
  int e = blockIdx.x / g.R;  // element index across all outputs
  int k = 0;
  while (k < g.m && e >= g.out_off[k + 1]) ++k;
  e -= g.out_off[k];
  __shared__ float red[4];
  float acc = 0.f;
  if (k < g.m) {
    const int ck = e / g.td[k], tk = e - ck * g.td[k];
    // iterate over all (t, c) with mode k fixed, and all taps
    const int To = g.T / g.td[k], Co = g.C / g.cd[k];
    const long total = (long)To * Co * g.taps;
    for (long it = threadIdx.x; it < total; it += blockDim.x) {
      const int tap = (int)(it % g.taps);
      long rest = it / g.taps;
      int co = (int)(rest % Co), to = (int)(rest / Co);
      // expand (to, co) into full indices, inserting (tk, ck) at mode k; modes are first-slowest
      int t = 0, c = 0;
      float w = p.S ? __ldg(p.S + (size_t)tap * g.R + r) : 1.f;
      int tstride = 1, cstride = 1;
      for (int j = g.m - 1; j >= 0; --j) {
        int tj, cj;
        if (j == k) { tj = tk; cj = ck; }
        else {
          tj = to % g.td[j]; to /= g.td[j];
          cj = co % g.cd[j]; co /= g.cd[j];
          w *= __ldg(p.A[j] + ((size_t)cj * g.td[j] + tj) * g.R + r);
        }
        t += tj * tstride; tstride *= g.td[j];
        c += cj * cstride; cstride *= g.cd[j];
      }
      acc = fmaf(w, __ldg(G + ((size_t)t * g.C + c) * g.taps + tap), acc);
    }
  } else {
    const int tap = e;
    const long total = (long)g.T * g.C;
    for (long it = threadIdx.x; it < total; it += blockDim.x) {
      int c = (int)(it % g.C), t = (int)(it / g.C);
      float w = 1.f;
      int tt = t, cc = c;
      for (int j = g.m - 1; j >= 0; --j) {
        const int tj = tt % g.td[j], cj = cc % g.cd[j];
        tt /= g.td[j]; cc /= g.cd[j];
        w *= __ldg(p.A[j] + ((size_t)cj * g.td[j] + tj) * g.R + r);
      }
      acc = fmaf(w, __ldg(G + ((size_t)t * g.C + c) * g.taps + tap), acc);
    }
  }
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    const float s = (red[0] + red[1]) + (red[2] + red[3]);
    if (k < g.m) p.dA[k][(size_t)e * g.R + r] = s;
    else p.dS[(size_t)e * g.R + r] = s;
  }
}

}  // namespace

int dense_grad_launch(int N, int T, int C, int H, int W, int FH, int FW, const float* dV, const float* X, float* G,
                      cudaStream_t st) {
  dim3 grid(ceil_div(C, TN), ceil_div(T, TM), FH * FW);
  if (grid.y > 65535 || grid.z > 65535) return fail(B200CP_ERR_UNSUPPORTED, "dense gradient: too many tiles");
  if (H * W == 1 && FH * FW == 1)
    dense_grad_kernel<false><<<grid, NTH, 0, st>>>(N, T, C, H, W, FH, FW, 0, 0, dV, X, G);
  else
    dense_grad_kernel<true><<<grid, NTH, 0, st>>>(N, T, C, H, W, FH, FW, (FH - 1) / 2, (FW - 1) / 2, dV, X, G);
  B200CP_LAUNCH_OK("dense_grad_kernel");
  return B200CP_OK;
}

int contract_factors_launch(int order, const int* cdims, const int* tdims, int R, int taps, const float* const* A,
                            const float* S, const float* G, float* const* dA, float* dS, cudaStream_t st) {
  ContractGeom g{};
  ContractPtrs p{};
  g.m = order; g.R = R; g.taps = taps; g.T = 1; g.C = 1;
  int off = 0;
  for (int k = 0; k < order; ++k) {
    g.cd[k] = cdims[k]; g.td[k] = tdims[k];
    g.T *= tdims[k]; g.C *= cdims[k];
    g.out_off[k] = off;
    off += cdims[k] * tdims[k];
    p.A[k] = A[k]; p.dA[k] = dA[k];
  }
  g.out_off[order] = off;
  for (int k = order + 1; k < 5; ++k) g.out_off[k] = 0x7fffffff;
  p.S = S; p.dS = dS;
  const long elems = off + (dS ? taps : 0);
  contract_factors_kernel<<<(unsigned)(elems * R), 128, 0, st>>>(g, p, G);
  B200CP_LAUNCH_OK("contract_factors_kernel");
  return B200CP_OK;
}

}  // namespace b200cp
