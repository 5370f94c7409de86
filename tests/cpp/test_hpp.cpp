// Exercises include/b200cp.hpp the way Cuda_kernels/test/test_cp4Conv.cpp.cu:14-44 exercises the reference:
// CP::Conv2dForward against a dense convolution with the recomposed filter (computed here on the host),
// plus the backward entry points against host loops.  Prints "OK" and returns 0 on success.
#include <cstdio>
#include <cstdlib>

#include "b200cp.hpp"

static void fill(Tensor& t, unsigned seed, float scale) {
  unsigned s = seed * 2654435761u + 12345u;
  for (size_t i = 0; i < t.size(); ++i) {
    s = s * 1664525u + 1013904223u;
    t.m_data[i] = scale * (((s >> 8) & 0xffff) / 32768.0f - 1.0f);
  }
}
static float at(const Tensor& X, int n, int c, int h, int w) {
  const int C = X.shape[1], H = X.shape[2], W = X.shape[3];
  if (h < 0 || w < 0 || h >= H || w >= W) return 0.f;
  return X.m_data[((size_t)(n * C + c) * H + h) * W + w];
}

int main() {
  const unsigned n = 2, c = 6, x = 13, pad = 1, t = 5, f = 3, rank = 4;
  Tensor In{n, c, x, x}, FT{t, rank}, FC{c, rank}, FY{f, rank}, FX{f, rank}, dO{n, t, x, x};
  fill(In, 1, 1.f); fill(FT, 2, .5f); fill(FC, 3, .5f); fill(FY, 4, .5f); fill(FX, 5, .5f); fill(dO, 6, 1.f);
  Tensor K = cp4recom(FT, FC, FY, FX);
  Tensor U = CP::Conv2dForward(In, FT, FC, FY, FX, pad);
  cudaDeviceSynchronize();
  double worst = 0;
  for (unsigned nn = 0; nn < n; ++nn) for (unsigned tt = 0; tt < t; ++tt) for (unsigned h = 0; h < x; ++h) for (unsigned w = 0; w < x; ++w) {
    double ref = 0;
    for (unsigned cc = 0; cc < c; ++cc) for (unsigned y = 0; y < f; ++y) for (unsigned xx = 0; xx < f; ++xx)
      ref += (double)K.m_data[((tt * c + cc) * f + y) * f + xx] * at(In, nn, cc, (int)h + y - pad, (int)w + xx - pad);
    const double got = U.m_data[((size_t)(nn * t + tt) * x + h) * x + w];
    worst = std::fmax(worst, std::fabs(got - ref) / (1e-5 + 1e-4 * std::fabs(ref)));
  }
  if (worst > 1.0) { std::printf("forward mismatch %g\n", worst); return 1; }
  if (U.shape[0] != n || U.shape[1] != t || U.shape[2] != x || U.shape[3] != x) return 2;

  // backward data against the adjoint identity <dO, fwd(In)> == <bwd(dO), In>
  Tensor dX = CP::Conv2dBackwardData(dO, FT, FC, FY, FX, pad);
  cudaDeviceSynchronize();
  double lhs = 0, rhs = 0;
  for (size_t i = 0; i < U.size(); ++i) lhs += (double)dO.m_data[i] * U.m_data[i];
  for (size_t i = 0; i < In.size(); ++i) rhs += (double)dX.m_data[i] * In.m_data[i];
  if (std::fabs(lhs - rhs) > 1e-3 * std::fabs(lhs) + 1e-3) { std::printf("adjoint mismatch %g %g\n", lhs, rhs); return 3; }

  // factor gradients: <F, dF> == <dO, U> for each factor (U is linear in each)
  CP::FactorGrads g = CP::Conv2dBackwardFilterFactors(dO, In, FT, FC, FY, FX, pad);
  const Tensor* Fs[4] = {&FT, &FC, &FY, &FX};
  const Tensor* Gs[4] = {&g.dFT, &g.dFC, &g.dFY, &g.dFX};
  for (int k = 0; k < 4; ++k) {
    double e = 0;
    for (size_t i = 0; i < Fs[k]->size(); ++i) e += (double)Fs[k]->m_data[i] * Gs[k]->m_data[i];
    if (std::fabs(e - lhs) > 1e-3 * std::fabs(lhs) + 1e-3) { std::printf("factor %d gradient mismatch %g %g\n", k, e, lhs); return 4; }
  }
  // the per-factor reference entry point accumulates into a zero tensor
  Tensor dFC{c, rank};
  tensor_shape p = CP::shape_of(In, false, FT, FC, FY, FX, pad);
  cp4_conv2d_backward_filter_c_gpu(p, dFC.m_data, In.m_data, dO.m_data, FT.m_data, FY.m_data, FX.m_data);
  if (!AllClose(dFC, g.dFC, 1e-4f)) { std::printf("per-factor entry point mismatch\n"); return 5; }

  // the one-call step gives the three results
  CP::StepResult st = CP::Conv2dStep(In, dO, FT, FC, FY, FX, pad);
  if (!AllClose(st.Out, CP::Conv2dForward(In, FT, FC, FY, FX, pad), 1e-4f)) { std::printf("step forward mismatch\n"); return 7; }
  if (!AllClose(st.dIn, CP::Conv2dBackwardData(dO, FT, FC, FY, FX, pad), 1e-4f)) { std::printf("step backward-data mismatch\n"); return 8; }
  if (!AllClose(st.grads.dFC, g.dFC, 2e-3f) || !AllClose(st.grads.dFY, g.dFY, 2e-3f)) { std::printf("step gradient mismatch\n"); return 9; }

  auto r = CP::run_convolution(p, 3);
  if (!(r.first > 0.f) || r.second == 0) return 6;
  Tensor copy = U;
  if (!AllClose(copy, U, 1e-6f) || copy.order() != 4) return 7;
  std::printf("OK forward worst err/bound %.3f, %.1f us\n", worst, r.first);
  return 0;
}
