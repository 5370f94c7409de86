// Header-only C++ mirror of the reference's host interface (Cuda_kernels/Tensor.cuh, cp4Conv2d.cuh,
// cp4Conv2dForward.cuh, cp4Conv2dBackwardData.cuh, cp4Conv2dBackwardFilter.cuh, Utils.cuh) on top of the
// C ABI of libb200cp.  Same names, argument order and return values; errors throw std::runtime_error
// instead of calling exit().  Link with -lb200cp -lcudart.
#ifndef B200CP_HPP
#define B200CP_HPP

#include <cuda_runtime.h>

#include <cmath>
#include <cstddef>
#include <initializer_list>
#include <numeric>
#include <stdexcept>
#include <string>
#include <tuple>
#include <utility>
#include <vector>

#include "b200cp.h"

// Same fields, order and ordering operator as Cuda_kernels/Tensor.cuh:10-25.
struct tensor_shape {
  unsigned N = 0, H = 0, W = 0, pad = 0, T = 0, C = 0, Y = 0, X = 0, Rank = 0;
  friend bool operator<(const tensor_shape l, const tensor_shape r) {
    return std::tie(l.N, l.H, l.W, l.pad, l.T, l.C, l.Y, l.X, l.Rank) <
           std::tie(r.N, r.H, r.W, r.pad, r.T, r.C, r.Y, r.X, r.Rank);
  }
};

namespace b200cp_detail {
inline void check(int rc, const char* what) {
  if (rc != 0) throw std::runtime_error(std::string(what) + ": " + b200cp_last_error_string());
}
inline void cuda(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}
inline b200cp_tensor_shape abi(const tensor_shape& s) { return {s.N, s.H, s.W, s.pad, s.T, s.C, s.Y, s.X, s.Rank}; }
// mean microseconds of PROFCOUNT launches, each bracketed by events like the reference's timing loop
template <class F>
float timed(unsigned PROFCOUNT, F&& launch) {
  cudaEvent_t a, b;
  cuda(cudaEventCreate(&a), "cudaEventCreate");
  cuda(cudaEventCreate(&b), "cudaEventCreate");
  float us = 0.f;
  for (unsigned i = 0; i < (PROFCOUNT ? PROFCOUNT : 1); ++i) {
    cuda(cudaEventRecord(a), "cudaEventRecord");
    launch();
    cuda(cudaEventRecord(b), "cudaEventRecord");
    cuda(cudaEventSynchronize(b), "cudaEventSynchronize");
    float ms = 0.f;
    cuda(cudaEventElapsedTime(&ms, a, b), "cudaEventElapsedTime");
    us += ms * 1e3f;
  }
  cudaEventDestroy(a);
  cudaEventDestroy(b);
  return us / (PROFCOUNT ? PROFCOUNT : 1);
}
}  // namespace b200cp_detail

// Managed-memory tensor with the reference's public members (Cuda_kernels/Tensor.cuh:28-44).  Unlike the
// reference, assignment reallocates correctly and updates `shape`.
class Tensor {
 public:
  float* m_data = nullptr;
  std::vector<unsigned> shape;

  Tensor(std::initializer_list<unsigned> l) : shape(l) { alloc(true); }
  explicit Tensor(const std::vector<unsigned>& s) : shape(s) { alloc(true); }
  Tensor(Tensor const& o) : shape(o.shape) {
    alloc(false);
    b200cp_detail::cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    for (size_t i = 0; i < size(); ++i) m_data[i] = o.m_data[i];
  }
  Tensor(Tensor&& o) noexcept : m_data(o.m_data), shape(std::move(o.shape)) { o.m_data = nullptr; }
  Tensor& operator=(Tensor const& o) {
    if (this == &o) return *this;
    Tensor tmp(o);
    std::swap(m_data, tmp.m_data);
    std::swap(shape, tmp.shape);
    return *this;
  }
  Tensor& operator=(Tensor&& o) noexcept {
    std::swap(m_data, o.m_data);
    std::swap(shape, o.shape);
    return *this;
  }
  ~Tensor() {
    if (m_data) {
      cudaDeviceSynchronize();
      cudaFree(m_data);
    }
  }
  size_t size() const { return std::accumulate(shape.begin(), shape.end(), size_t(1), std::multiplies<size_t>()); }
  size_t order() const { return shape.size(); }

 private:
  void alloc(bool zero) {
    b200cp_detail::cuda(cudaMallocManaged(&m_data, std::max<size_t>(size(), 1) * sizeof(float)), "cudaMallocManaged");
    if (zero)
      for (size_t i = 0; i < size(); ++i) m_data[i] = 0.f;
  }
};

// ---- raw launchers (Cuda_kernels/cp4Conv2dForward.cuh:7-14 etc.): device or managed pointers, mean microseconds ----
inline float cp4_conv2d_forward_gpu(tensor_shape p, const float* In, const float* FT, const float* FC, const float* FY,
                                    const float* FX, float* Out, unsigned PROFCOUNT = 1) {
  const b200cp_tensor_shape s = b200cp_detail::abi(p);
  return b200cp_detail::timed(PROFCOUNT, [&] {
    b200cp_detail::check(b200cp_cp4_fwd(&s, In, FT, FC, FY, FX, Out, nullptr, 0), "cp4_conv2d_forward_gpu");
  });
}
inline float cp4_conv2d_backward_data_gpu(tensor_shape p, const float* dU, const float* FT, const float* FC,
                                          const float* FY, const float* FX, float* Out, unsigned PROFCOUNT = 1) {
  const b200cp_tensor_shape s = b200cp_detail::abi(p);
  return b200cp_detail::timed(PROFCOUNT, [&] {
    b200cp_detail::check(b200cp_cp4_bwd_data(&s, dU, FT, FC, FY, FX, Out, nullptr, 0), "cp4_conv2d_backward_data_gpu");
  });
}
inline float cp4_conv2d_backward_filter_full_gpu(tensor_shape p, float* FF, const float* In, const float* dLdO,
                                                 unsigned PROFCOUNT = 1) {
  const b200cp_tensor_shape s = b200cp_detail::abi(p);
  return b200cp_detail::timed(PROFCOUNT, [&] {
    b200cp_detail::check(b200cp_cp4_bwd_filter_full(&s, In, dLdO, FF, nullptr), "cp4_conv2d_backward_filter_full_gpu");
  });
}

namespace b200cp_detail {
// all four factor gradients in one pass; out = packed [T*R | C*R | Y*R | X*R] (device or managed)
inline float bwd_filter_packed(tensor_shape p, const float* In, const float* dLdO, const float* FT, const float* FC,
                               const float* FY, const float* FX, float* packed, unsigned PROFCOUNT) {
  const b200cp_tensor_shape s = abi(p);
  const size_t wsb = b200cp_cp4_bwd_filter_workspace_bytes(&s, 0);
  void* ws = nullptr;
  cuda(cudaMalloc(&ws, wsb ? wsb : 4), "cudaMalloc");
  float us = 0.f;
  try {
    us = timed(PROFCOUNT, [&] {
      check(b200cp_cp4_bwd_filter(&s, In, dLdO, FT, FC, FY, FX, packed, ws, wsb, nullptr, 0), "cp4 backward filter");
    });
  } catch (...) {
    cudaFree(ws);
    throw;
  }
  cudaFree(ws);
  return us;
}
// the reference computes one factor gradient per call, accumulating (+=) into a zero-filled tensor
inline float one_factor(tensor_shape p, int which, float* dF, const float* In, const float* dLdO, const float* FT,
                        const float* FC, const float* FY, const float* FX, unsigned PROFCOUNT) {
  const size_t n[4] = {(size_t)p.T * p.Rank, (size_t)p.C * p.Rank, (size_t)p.Y * p.Rank, (size_t)p.X * p.Rank};
  float* packed = nullptr;
  cuda(cudaMallocManaged(&packed, (n[0] + n[1] + n[2] + n[3]) * sizeof(float)), "cudaMallocManaged");
  const float us = bwd_filter_packed(p, In, dLdO, FT, FC, FY, FX, packed, PROFCOUNT);
  cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  size_t off = 0;
  for (int i = 0; i < which; ++i) off += n[i];
  for (size_t i = 0; i < n[which]; ++i) dF[i] += packed[off + i];
  cudaFree(packed);
  return us;
}
}  // namespace b200cp_detail

// Cuda_kernels/cp4Conv2dBackwardFilter.cuh:13-47.  `dF` must be host-accessible (managed), like the reference's.
// The factor being differentiated is not an argument of the reference signature; a gradient does not depend on it.
inline float cp4_conv2d_backward_filter_t_gpu(tensor_shape p, float* dFT, const float* In, const float* dLdO,
                                              const float* FC, const float* FY, const float* FX, unsigned PROFCOUNT = 1) {
  std::vector<float> z((size_t)p.T * p.Rank, 0.f);
  float* FT = nullptr;
  b200cp_detail::cuda(cudaMallocManaged(&FT, z.size() * sizeof(float)), "cudaMallocManaged");
  for (size_t i = 0; i < z.size(); ++i) FT[i] = 0.f;
  const float us = b200cp_detail::one_factor(p, 0, dFT, In, dLdO, FT, FC, FY, FX, PROFCOUNT);
  cudaFree(FT);
  return us;
}
inline float cp4_conv2d_backward_filter_c_gpu(tensor_shape p, float* dFC, const float* In, const float* dLdO,
                                              const float* FT, const float* FY, const float* FX, unsigned PROFCOUNT = 1) {
  float* FC = nullptr;
  b200cp_detail::cuda(cudaMallocManaged(&FC, (size_t)p.C * p.Rank * sizeof(float)), "cudaMallocManaged");
  for (size_t i = 0; i < (size_t)p.C * p.Rank; ++i) FC[i] = 0.f;
  const float us = b200cp_detail::one_factor(p, 1, dFC, In, dLdO, FT, FC, FY, FX, PROFCOUNT);
  cudaFree(FC);
  return us;
}
inline float cp4_conv2d_backward_filter_y_gpu(tensor_shape p, float* dFY, const float* In, const float* dLdO,
                                              const float* FT, const float* FC, const float* FX, unsigned PROFCOUNT = 1) {
  float* FY = nullptr;
  b200cp_detail::cuda(cudaMallocManaged(&FY, (size_t)p.Y * p.Rank * sizeof(float)), "cudaMallocManaged");
  for (size_t i = 0; i < (size_t)p.Y * p.Rank; ++i) FY[i] = 0.f;
  const float us = b200cp_detail::one_factor(p, 2, dFY, In, dLdO, FT, FC, FY, FX, PROFCOUNT);
  cudaFree(FY);
  return us;
}
inline float cp4_conv2d_backward_filter_x_gpu(tensor_shape p, float* dFX, const float* In, const float* dLdO,
                                              const float* FT, const float* FC, const float* FY, unsigned PROFCOUNT = 1) {
  float* FX = nullptr;
  b200cp_detail::cuda(cudaMallocManaged(&FX, (size_t)p.X * p.Rank * sizeof(float)), "cudaMallocManaged");
  for (size_t i = 0; i < (size_t)p.X * p.Rank; ++i) FX[i] = 0.f;
  const float us = b200cp_detail::one_factor(p, 3, dFX, In, dLdO, FT, FC, FY, FX, PROFCOUNT);
  cudaFree(FX);
  return us;
}

// Cuda_kernels/Utils.cuh: cp4recom and AllClose (random_fill needs cuRAND and stays with the caller)
inline Tensor cp4recom(Tensor const& FK, Tensor const& FC, Tensor const& FH, Tensor const& FW) {
  b200cp_tensor_shape s{1, 1, 1, 0, FK.shape[0], FC.shape[0], FH.shape[0], FW.shape[0], FK.shape[1]};
  Tensor Out{FK.shape[0], FC.shape[0], FH.shape[0], FW.shape[0]};
  b200cp_detail::check(b200cp_cp4_recompose(&s, FK.m_data, FC.m_data, FH.m_data, FW.m_data, Out.m_data, nullptr), "cp4recom");
  b200cp_detail::cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  return Out;
}
// max(|a-b|/|a|, |a-b|/|b|) <= tolerance for every element, counted on the device (Cuda_kernels/Utils.cu:143-180)
inline bool AllClose(Tensor const& A, Tensor const& B, float tolerance = 1e-3f) {
  if (A.size() != B.size()) return false;
  unsigned long long exceeds = 0;
  b200cp_detail::check(b200cp_allclose_count(A.m_data, B.m_data, A.size(), tolerance, &exceeds, nullptr), "AllClose");
  return exceeds == 0;
}

namespace CP {

inline tensor_shape shape_of(Tensor const& Act, bool act_is_upstream, Tensor const& FT, Tensor const& FC,
                             Tensor const& FY, Tensor const& FX, unsigned pad) {
  tensor_shape p;
  p.N = Act.shape[0];
  p.H = Act.shape[2];
  p.W = Act.shape[3];
  p.pad = pad;
  p.Rank = FT.shape[1];
  p.T = FT.shape[0];
  p.C = FC.shape[0];
  p.Y = FY.shape[0];
  p.X = FX.shape[0];
  if (Act.shape[1] != (act_is_upstream ? p.T : p.C)) throw std::runtime_error("CP: channel count does not match the factor");
  return p;
}

// Cuda_kernels/cp4Conv2d.cu:14-43
inline Tensor Conv2dForward(Tensor const& Input, Tensor const& FT, Tensor const& FC, Tensor const& FY, Tensor const& FX,
                            unsigned pad = 1) {
  const tensor_shape p = shape_of(Input, false, FT, FC, FY, FX, pad);
  Tensor Out{p.N, p.T, p.H, p.W};
  cp4_conv2d_forward_gpu(p, Input.m_data, FT.m_data, FC.m_data, FY.m_data, FX.m_data, Out.m_data);
  return Out;
}
// Cuda_kernels/cp4Conv2d.cu:48-77 (commented out in the reference)
inline Tensor Conv2dBackwardData(Tensor const& Upstream, Tensor const& FT, Tensor const& FC, Tensor const& FY,
                                 Tensor const& FX, unsigned pad = 1) {
  const tensor_shape p = shape_of(Upstream, true, FT, FC, FY, FX, pad);
  Tensor Out{p.N, p.C, p.H, p.W};
  cp4_conv2d_backward_data_gpu(p, Upstream.m_data, FT.m_data, FC.m_data, FY.m_data, FX.m_data, Out.m_data);
  return Out;
}
struct FactorGrads {
  Tensor dFT, dFC, dFY, dFX;
};
inline FactorGrads Conv2dBackwardFilterFactors(Tensor const& dLdO, Tensor const& In, Tensor const& FT, Tensor const& FC,
                                               Tensor const& FY, Tensor const& FX, unsigned pad = 1) {
  const tensor_shape p = shape_of(In, false, FT, FC, FY, FX, pad);
  FactorGrads g{Tensor{p.T, p.Rank}, Tensor{p.C, p.Rank}, Tensor{p.Y, p.Rank}, Tensor{p.X, p.Rank}};
  Tensor packed{(p.T + p.C + p.Y + p.X) * p.Rank};
  b200cp_detail::bwd_filter_packed(p, In.m_data, dLdO.m_data, FT.m_data, FC.m_data, FY.m_data, FX.m_data, packed.m_data, 1);
  b200cp_detail::cuda(cudaDeviceSynchronize(), "cudaDeviceSynchronize");
  size_t off = 0;
  for (Tensor* t : {&g.dFT, &g.dFC, &g.dFY, &g.dFX}) {
    for (size_t i = 0; i < t->size(); ++i) t->m_data[i] = packed.m_data[off + i];
    off += t->size();
  }
  return g;
}
// Cuda_kernels/cp4Conv2d.cu:83-153: the reference returns cp4recom of the four gradients
inline Tensor Conv2dBackwardFilter(Tensor const& dLdO, Tensor const& In, Tensor const& FT, Tensor const& FC,
                                   Tensor const& FY, Tensor const& FX, unsigned pad = 1) {
  FactorGrads g = Conv2dBackwardFilterFactors(dLdO, In, FT, FC, FY, FX, pad);
  return cp4recom(g.dFT, g.dFC, g.dFY, g.dFX);
}
// One training step: what Conv2dForward, Conv2dBackwardData and Conv2dBackwardFilterFactors return for the same inputs,
// from one library call that does their common work once (b200cp_cp4_step; no counterpart in the reference).
struct StepResult {
  Tensor Out, dIn;
  FactorGrads grads;
};
inline StepResult Conv2dStep(Tensor const& Input, Tensor const& Upstream, Tensor const& FT, Tensor const& FC,
                             Tensor const& FY, Tensor const& FX, unsigned pad = 1) {
  const tensor_shape p = shape_of(Input, false, FT, FC, FY, FX, pad);
  const b200cp_tensor_shape s = b200cp_detail::abi(p);
  StepResult r{Tensor{p.N, p.T, p.H, p.W}, Tensor{p.N, p.C, p.H, p.W},
               FactorGrads{Tensor{p.T, p.Rank}, Tensor{p.C, p.Rank}, Tensor{p.Y, p.Rank}, Tensor{p.X, p.Rank}}};
  Tensor packed{(p.T + p.C + p.Y + p.X) * p.Rank};
  const size_t wsb = b200cp_cp4_step_workspace_bytes(&s, 0);
  void* ws = nullptr;
  b200cp_detail::cuda(cudaMalloc(&ws, wsb ? wsb : 4), "cudaMalloc");
  const int rc = b200cp_cp4_step(&s, Input.m_data, Upstream.m_data, FT.m_data, FC.m_data, FY.m_data, FX.m_data, r.Out.m_data,
                                 r.dIn.m_data, packed.m_data, ws, wsb, nullptr, 0);
  const cudaError_t e = cudaDeviceSynchronize();
  cudaFree(ws);
  b200cp_detail::check(rc, "b200cp_cp4_step");
  b200cp_detail::cuda(e, "cudaDeviceSynchronize");
  size_t off = 0;
  for (Tensor* t : {&r.grads.dFT, &r.grads.dFC, &r.grads.dFY, &r.grads.dFX}) {
    for (size_t i = 0; i < t->size(); ++i) t->m_data[i] = packed.m_data[off + i];
    off += t->size();
  }
  return r;
}
// Cuda_kernels/cp4Conv2d.cu:158-190: forward on uninitialised device buffers -> (mean microseconds, bytes)
inline std::pair<float, unsigned> run_convolution(tensor_shape p, unsigned PROFCOUNT = 1) {
  float *In, *Out, *FT, *FC, *FX, *FY;
  const size_t nin = (size_t)p.N * p.C * p.H * p.W, nout = (size_t)p.N * p.T * p.H * p.W;
  b200cp_detail::cuda(cudaMalloc(&In, nin * 4), "cudaMalloc");
  b200cp_detail::cuda(cudaMalloc(&Out, nout * 4), "cudaMalloc");
  b200cp_detail::cuda(cudaMalloc(&FT, (size_t)p.T * p.Rank * 4), "cudaMalloc");
  b200cp_detail::cuda(cudaMalloc(&FC, (size_t)p.C * p.Rank * 4), "cudaMalloc");
  b200cp_detail::cuda(cudaMalloc(&FY, (size_t)p.Y * p.Rank * 4), "cudaMalloc");
  b200cp_detail::cuda(cudaMalloc(&FX, (size_t)p.X * p.Rank * 4), "cudaMalloc");
  cudaMemset(In, 0, nin * 4);   // the reference leaves them uninitialised; zeros keep NaNs out of the timing
  cudaMemset(FT, 0, (size_t)p.T * p.Rank * 4);
  cudaMemset(FC, 0, (size_t)p.C * p.Rank * 4);
  cudaMemset(FY, 0, (size_t)p.Y * p.Rank * 4);
  cudaMemset(FX, 0, (size_t)p.X * p.Rank * 4);
  const unsigned mem = (unsigned)(sizeof(float) * (nout + nin + (size_t)p.Rank * (p.T + p.C + p.X + p.Y)));
  float us = 0.f;
  try {
    us = cp4_conv2d_forward_gpu(p, In, FT, FC, FY, FX, Out, PROFCOUNT);
  } catch (...) {
    cudaFree(In); cudaFree(Out); cudaFree(FT); cudaFree(FC); cudaFree(FY); cudaFree(FX);
    throw;
  }
  cudaFree(In); cudaFree(Out); cudaFree(FT); cudaFree(FC); cudaFree(FY); cudaFree(FX);
  return std::make_pair(us, mem);
}

}  // namespace CP

#endif  // B200CP_HPP
