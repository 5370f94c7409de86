// extern "C" shim around the UNMODIFIED reference launchers, so that the test
// suite can run the reference's own kernels on a GPU and pin the CPU oracle to
// them.  TEST INFRASTRUCTURE ONLY.  Built by oracle/build_ref.py into
// oracle/_ref/ together with the reference's sources, which are compiled where
// they lie (nothing of the reference is copied into this repository).
//
// Two libraries are built because the reference defines `const_filter` and
// `conv2d_cp4_kernel` in both its forward and its backward-data file:
//   -DREF_FWD : Tensor.cu + cp4Conv2dForward.cu
//   -DREF_BWD : Tensor.cu + cp4Conv2dBackwardData.cu + cp4Conv2dBackwardFilter.cu
#include <cuda_runtime.h>

#include <cstring>

#include "Tensor.cuh"
#ifdef REF_FWD
#include "cp4Conv2dForward.cuh"
#endif
#ifdef REF_BWD
#include "cp4Conv2dBackwardData.cuh"
#include "cp4Conv2dBackwardFilter.cuh"
#endif

namespace {
tensor_shape to_shape(const unsigned* s) {  // N H W pad T C Y X Rank
  tensor_shape p;
  p.N = s[0]; p.H = s[1]; p.W = s[2]; p.pad = s[3]; p.T = s[4]; p.C = s[5]; p.Y = s[6]; p.X = s[7]; p.Rank = s[8];
  return p;
}
float* to_dev(const float* h, size_t n) {
  float* d = nullptr;
  if (cudaMalloc(&d, n * sizeof(float)) != cudaSuccess) return nullptr;
  cudaMemcpy(d, h, n * sizeof(float), cudaMemcpyHostToDevice);
  return d;
}
}  // namespace

extern "C" {

#ifdef REF_FWD
// returns 0 on success; the reference supports Rank in {1,2,4,8,16} and (T+C+Y+X)*Rank <= 16384
__attribute__((visibility("default"))) int ref_cp4_forward(const unsigned* s, const float* In, const float* FT,
                                                           const float* FC, const float* FY, const float* FX,
                                                           float* Out) {
  const tensor_shape p = to_shape(s);
  const size_t nin = (size_t)p.N * p.C * p.H * p.W, nout = (size_t)p.N * p.T * p.H * p.W;
  float *dIn = to_dev(In, nin), *dFT = to_dev(FT, p.T * p.Rank), *dFC = to_dev(FC, p.C * p.Rank),
        *dFY = to_dev(FY, p.Y * p.Rank), *dFX = to_dev(FX, p.X * p.Rank), *dOut = nullptr;
  if (cudaMalloc(&dOut, nout * sizeof(float)) != cudaSuccess) return 1;
  cudaMemset(dOut, 0, nout * sizeof(float));
  cp4_conv2d_forward_gpu(p, dIn, dFT, dFC, dFY, dFX, dOut, 1);
  const cudaError_t e = cudaDeviceSynchronize();
  cudaMemcpy(Out, dOut, nout * sizeof(float), cudaMemcpyDeviceToHost);
  cudaFree(dIn); cudaFree(dFT); cudaFree(dFC); cudaFree(dFY); cudaFree(dFX); cudaFree(dOut);
  return e == cudaSuccess ? 0 : 2;
}
// the reference's own timing: mean microseconds over `profcount` launches (its PROFCOUNT loop); negative on error
__attribute__((visibility("default"))) float ref_cp4_forward_time(const unsigned* s, const float* In, const float* FT,
                                                                  const float* FC, const float* FY, const float* FX,
                                                                  unsigned profcount) {
  const tensor_shape p = to_shape(s);
  const size_t nin = (size_t)p.N * p.C * p.H * p.W, nout = (size_t)p.N * p.T * p.H * p.W;
  float *dIn = to_dev(In, nin), *dFT = to_dev(FT, p.T * p.Rank), *dFC = to_dev(FC, p.C * p.Rank),
        *dFY = to_dev(FY, p.Y * p.Rank), *dFX = to_dev(FX, p.X * p.Rank), *dOut = nullptr;
  if (cudaMalloc(&dOut, nout * sizeof(float)) != cudaSuccess) return -1.f;
  cp4_conv2d_forward_gpu(p, dIn, dFT, dFC, dFY, dFX, dOut, 3);   // warm-up
  const float us = cp4_conv2d_forward_gpu(p, dIn, dFT, dFC, dFY, dFX, dOut, profcount);
  const cudaError_t e = cudaDeviceSynchronize();
  cudaFree(dIn); cudaFree(dFT); cudaFree(dFC); cudaFree(dFY); cudaFree(dFX); cudaFree(dOut);
  return e == cudaSuccess ? us : -1.f;
}
#endif

#ifdef REF_BWD
// the reference needs (T+C+Y+X)*Rank <= 4096 and is only safe for W % 16 == 0, H % 4 == 0
__attribute__((visibility("default"))) int ref_cp4_backward_data(const unsigned* s, const float* dU, const float* FT,
                                                                 const float* FC, const float* FY, const float* FX,
                                                                 float* Out) {
  const tensor_shape p = to_shape(s);
  const size_t nin = (size_t)p.N * p.T * p.H * p.W, nout = (size_t)p.N * p.C * p.H * p.W;
  float *dIn = to_dev(dU, nin), *dFT = to_dev(FT, p.T * p.Rank), *dFC = to_dev(FC, p.C * p.Rank),
        *dFY = to_dev(FY, p.Y * p.Rank), *dFX = to_dev(FX, p.X * p.Rank), *dOut = nullptr;
  if (cudaMalloc(&dOut, nout * sizeof(float)) != cudaSuccess) return 1;
  cudaMemset(dOut, 0, nout * sizeof(float));
  cp4_conv2d_backward_data_gpu(p, dIn, dFT, dFC, dFY, dFX, dOut, 1);
  const cudaError_t e = cudaDeviceSynchronize();
  cudaMemcpy(Out, dOut, nout * sizeof(float), cudaMemcpyDeviceToHost);
  cudaFree(dIn); cudaFree(dFT); cudaFree(dFC); cudaFree(dFY); cudaFree(dFX); cudaFree(dOut);
  return e == cudaSuccess ? 0 : 2;
}

// host loops of the reference; the gradients must be zero-filled by the caller (they are accumulated with +=)
__attribute__((visibility("default"))) int ref_cp4_backward_filter(const unsigned* s, const float* In,
                                                                   const float* dLdO, const float* FT,
                                                                   const float* FC, const float* FY, const float* FX,
                                                                   float* dFT, float* dFC, float* dFY, float* dFX) {
  const tensor_shape p = to_shape(s);
  cp4_conv2d_backward_filter_t_gpu(p, dFT, In, dLdO, FC, FY, FX, 1);
  cp4_conv2d_backward_filter_c_gpu(p, dFC, In, dLdO, FT, FY, FX, 1);
  cp4_conv2d_backward_filter_y_gpu(p, dFY, In, dLdO, FT, FC, FX, 1);
  cp4_conv2d_backward_filter_x_gpu(p, dFX, In, dLdO, FT, FC, FY, 1);
  return 0;
}

__attribute__((visibility("default"))) int ref_cp4_backward_filter_full(const unsigned* s, const float* In,
                                                                        const float* dLdO, float* FF) {
  const tensor_shape p = to_shape(s);
  cp4_conv2d_backward_filter_full_gpu(p, FF, In, dLdO, 1);
  return 0;
}
#endif

}  // extern "C"
