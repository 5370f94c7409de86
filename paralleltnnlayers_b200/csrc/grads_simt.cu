// Factor gradients of the rCP conv and the CP dense layer (exact fp32).
//
// Both go through the dense gradient of the recomposed weight,
//   G[y, x][t][c] = sum_{n, h, w} dV[n, t, h, w] * Xpad[n, c, h + y, w + x]
// (the quantity cp4_conv2d_backward_filter_full_gpu produces,
// Cuda_kernels/cp4Conv2dBackwardFilter.cu:47-56; for the dense layer H = W = 1
// and G = dY^T X), followed by a contraction of G with all factors but one:
//   dA_k[c_k, t_k, r] = sum_{other modes, y, x} G * S[y, x, r] * prod_{j != k} A_j[c_j, t_j, r]
//   dS[y, x, r]       = sum_{t, c} G * prod_k A_k[c_k, t_k, r]
// G is a 128x128-tiled SIMT GEMM (8x8 outputs per thread, cp.async double buffering) whose K dimension
// runs over (image, pixel); when the (t, c, tap) grid alone cannot fill the GPU the K range is split
// over CTAs and the partial tiles are summed in a fixed order, so results are bitwise reproducible.
#include <algorithm>

#include "common.cuh"

namespace b200cp {

namespace {

constexpr int BM = 128, BN = 128, NTH = 256;
constexpr int BK_CONV = 32, PITCH_CONV = BK_CONV + 4;  // [channel][k], 16-byte rows, conflict-free float4 reads
constexpr int BK_FLAT = 16;                            // [k][channel]

struct GemmArgs {
  const float* dV;
  const float* X;
  float* out;  // [split][tap][T][C]
  int N, T, C, H, W, FH, FW, padH, padW;
  int splits, per_split;  // K units (images for the conv form, rows for the flat form) per split
};

__device__ __forceinline__ void cp_async4(float* dst, const float* src, bool ok) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int sz = ok ? 4 : 0;
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async16(float* dst, const float* src, bool ok) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int sz = ok ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// Conv form: operands [n][channel][H*W], K = (image, pixel); the X operand is read shifted by the tap.
// grid = (C tiles, T tiles, taps * splits)
__global__ void __launch_bounds__(NTH, 2) grad_gemm_conv_kernel(const GemmArgs g) {
  extern __shared__ __align__(16) float sm[];
  float* As = sm;                             // [2][BM][PITCH]
  float* Bs = sm + 2 * BM * PITCH_CONV;       // [2][BN][PITCH]
  const int tid = threadIdx.x;
  const int c0 = blockIdx.x * BN, t0 = blockIdx.y * BM;
  const int taps = g.FH * g.FW;
  const int tap = blockIdx.z % taps, split = blockIdx.z / taps;
  const int dy = tap / g.FW - g.padH, dx = tap % g.FW - g.padW;
  const int HW = g.H * g.W;
  const int n_begin = split * g.per_split, n_end = min(g.N, n_begin + g.per_split);
  const int chunks = ceil_div(HW, BK_CONV);
  const int steps = (n_end - n_begin) * chunks;
  const int tn = tid % 16, tm = tid / 16;
  const int lk = tid % BK_CONV, lch = tid / BK_CONV;  // loader role: fixed k, channels lch + 8*e

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  auto load_stage = [&](int step, int buf) {
    const int n = n_begin + step / chunks, p = (step % chunks) * BK_CONV + lk;
    const bool pin = p < HW;
    const int h = p / g.W, w = p - h * g.W;
    const int hh = h + dy, ww = w + dx;
    const bool xin = pin && hh >= 0 && hh < g.H && ww >= 0 && ww < g.W;
    const float* a_src = g.dV + ((size_t)n * g.T + t0) * HW + (pin ? p : 0);
    const float* b_src = g.X + ((size_t)n * g.C + c0) * HW + (xin ? hh * g.W + ww : 0);
    float* a_dst = As + (size_t)buf * BM * PITCH_CONV + lk;
    float* b_dst = Bs + (size_t)buf * BN * PITCH_CONV + lk;
#pragma unroll
    for (int e = 0; e < BM / 8; ++e) {
      const int ch = lch + 8 * e;
      const bool aok = pin && t0 + ch < g.T, bok = xin && c0 + ch < g.C;
      cp_async4(a_dst + ch * PITCH_CONV, aok ? a_src + (size_t)ch * HW : g.dV, aok);
      cp_async4(b_dst + ch * PITCH_CONV, bok ? b_src + (size_t)ch * HW : g.X, bok);
    }
  };

  if (steps > 0) load_stage(0, 0);
  cp_async_commit();
  for (int s = 0; s < steps; ++s) {
    const int buf = s & 1;
    if (s + 1 < steps) load_stage(s + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
    const float* A = As + (size_t)buf * BM * PITCH_CONV;
    const float* B = Bs + (size_t)buf * BN * PITCH_CONV;
#pragma unroll 2
    for (int k4 = 0; k4 < BK_CONV / 4; ++k4) {
      float4 b[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) b[j] = *reinterpret_cast<const float4*>(B + (tn + 16 * j) * PITCH_CONV + k4 * 4);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        const float4 a = *reinterpret_cast<const float4*>(A + (tm + 16 * i) * PITCH_CONV + k4 * 4);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          acc[i][j] = fmaf(a.x, b[j].x, acc[i][j]);
          acc[i][j] = fmaf(a.y, b[j].y, acc[i][j]);
          acc[i][j] = fmaf(a.z, b[j].z, acc[i][j]);
          acc[i][j] = fmaf(a.w, b[j].w, acc[i][j]);
        }
      }
    }
    __syncthreads();
  }
  float* out = g.out + ((size_t)split * taps + tap) * g.T * g.C;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int t = t0 + tm + 16 * i;
    if (t >= g.T) continue;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int c = c0 + tn + 16 * j;
      if (c < g.C) out[(size_t)t * g.C + c] = acc[i][j];
    }
  }
}

// Flat form (H*W == 1): operands [n][channel], K = n.  VEC: T and C are multiples of 4 (16-byte copies).
// grid = (C tiles, T tiles, splits)
template <bool VEC>
__global__ void __launch_bounds__(NTH, 2) grad_gemm_flat_kernel(const GemmArgs g) {
  __shared__ __align__(16) float As[2][BK_FLAT][BM];
  __shared__ __align__(16) float Bs[2][BK_FLAT][BN];
  const int tid = threadIdx.x;
  const int c0 = blockIdx.x * BN, t0 = blockIdx.y * BM;
  const int split = blockIdx.z;
  const int k_begin = split * g.per_split, k_end = min(g.N, k_begin + g.per_split);
  const int steps = ceil_div(max(k_end - k_begin, 0), BK_FLAT);
  const int tn = tid % 16, tm = tid / 16;

  float acc[8][8];
#pragma unroll
  for (int i = 0; i < 8; ++i)
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[i][j] = 0.f;

  auto load_stage = [&](int step, int buf) {
    const int kb = k_begin + step * BK_FLAT;
    if (VEC) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int idx = tid + e * NTH, k = idx / 32, m4 = (idx % 32) * 4;
        const bool kin = kb + k < k_end;
        const bool aok = kin && t0 + m4 < g.T, bok = kin && c0 + m4 < g.C;
        cp_async16(&As[buf][k][m4], aok ? g.dV + (size_t)(kb + k) * g.T + t0 + m4 : g.dV, aok);
        cp_async16(&Bs[buf][k][m4], bok ? g.X + (size_t)(kb + k) * g.C + c0 + m4 : g.X, bok);
      }
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int idx = tid + e * NTH, k = idx / 128, m = idx % 128;
        const bool kin = kb + k < k_end;
        const bool aok = kin && t0 + m < g.T, bok = kin && c0 + m < g.C;
        cp_async4(&As[buf][k][m], aok ? g.dV + (size_t)(kb + k) * g.T + t0 + m : g.dV, aok);
        cp_async4(&Bs[buf][k][m], bok ? g.X + (size_t)(kb + k) * g.C + c0 + m : g.X, bok);
      }
    }
  };

  if (steps > 0) load_stage(0, 0);
  cp_async_commit();
  for (int s = 0; s < steps; ++s) {
    const int buf = s & 1;
    if (s + 1 < steps) load_stage(s + 1, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();
#pragma unroll 4
    for (int k = 0; k < BK_FLAT; ++k) {
      const float4 a0 = *reinterpret_cast<const float4*>(&As[buf][k][tm * 4]);
      const float4 a1 = *reinterpret_cast<const float4*>(&As[buf][k][64 + tm * 4]);
      const float4 b0 = *reinterpret_cast<const float4*>(&Bs[buf][k][tn * 4]);
      const float4 b1 = *reinterpret_cast<const float4*>(&Bs[buf][k][64 + tn * 4]);
      const float a[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
      const float b[8] = {b0.x, b0.y, b0.z, b0.w, b1.x, b1.y, b1.z, b1.w};
#pragma unroll
      for (int i = 0; i < 8; ++i)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
    }
    __syncthreads();
  }
  float* out = g.out + (size_t)split * g.T * g.C;
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const int t = t0 + (i < 4 ? tm * 4 + i : 64 + tm * 4 + i - 4);
    if (t >= g.T) continue;
#pragma unroll
    for (int jh = 0; jh < 2; ++jh) {
      const int c = c0 + jh * 64 + tn * 4;
      if (VEC) {
        if (c < g.C)
          *reinterpret_cast<float4*>(out + (size_t)t * g.C + c) =
              make_float4(acc[i][jh * 4], acc[i][jh * 4 + 1], acc[i][jh * 4 + 2], acc[i][jh * 4 + 3]);
      } else {
#pragma unroll
        for (int u = 0; u < 4; ++u)
          if (c + u < g.C) out[(size_t)t * g.C + c + u] = acc[i][jh * 4 + u];
      }
    }
  }
}

// G[e] = sum over splits of P[split][e], in split order
__global__ void __launch_bounds__(256) sum_splits_kernel(const float* __restrict__ P, float* __restrict__ G, size_t n,
                                                        int splits) {
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  float s = P[i];
  for (int k = 1; k < splits; ++k) s += P[(size_t)k * n + i];
  G[i] = s;
}

}  // namespace

void sum_splits_launch(const float* P, float* G, size_t n, int splits, cudaStream_t st) {
  sum_splits_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(P, G, n, splits);
}

namespace {

int pick_splits(long tiles, int kunits, int sm_count) {
  // aim at two waves of CTAs; never more splits than K units, at most 16
  int s = (int)std::min<long>(16, std::max<long>(1, (2L * sm_count + tiles - 1) / tiles));
  s = std::min(s, std::max(1, kunits));
  return s;
}

}  // namespace

// floats of scratch dense_grad_launch needs beside G itself
size_t dense_grad_scratch_floats(int N, int T, int C, int H, int W, int FH, int FW) {
  DeviceInfo di;
  if (device_info(&di)) di.sm_count = 148;
  const long tiles = (long)ceil_div(C, BN) * ceil_div(T, BM) * FH * FW;
  const int splits = pick_splits(tiles, N, di.sm_count);
  const size_t simt = splits > 1 ? (size_t)splits * T * C * FH * FW : 0;
  if (H * W == 1 && FH * FW == 1 && gemm_tc_supported(N, T, C)) return std::max(simt, gemm_tc_scratch_floats(N, T, C));
  if (H * W > 1 && conv_gemm_tc_supported(N, T, C, H, W, FH, FW))
    return std::max(simt, conv_gemm_tc_scratch_floats(N, T, C, H, W, FH, FW));
  return simt;
}

// G is written as [tap][T][C]
int dense_grad_launch(int N, int T, int C, int H, int W, int FH, int FW, const float* dV, const float* X, float* G,
                      float* scratch, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const int taps = FH * FW;
  // large flat GEMMs go to the tensor cores (16-byte aligned operands; the scratch then holds the hi / lo planes)
  if (H * W == 1 && taps == 1 && gemm_tc_supported(N, T, C) && scratch &&
      ((reinterpret_cast<uintptr_t>(dV) | reinterpret_cast<uintptr_t>(X) | reinterpret_cast<uintptr_t>(G) |
        reinterpret_cast<uintptr_t>(scratch)) & 15) == 0)
    return gemm_tc_launch(N, T, C, dV, X, G, scratch, st);
  if (H * W > 1 && scratch && conv_gemm_tc_supported(N, T, C, H, W, FH, FW) &&
      ((reinterpret_cast<uintptr_t>(G) | reinterpret_cast<uintptr_t>(scratch)) & 15) == 0)
    return conv_gemm_tc_launch(N, T, C, H, W, FH, FW, dV, X, G, scratch, st);
  const long tiles = (long)ceil_div(C, BN) * ceil_div(T, BM) * taps;
  const int splits = pick_splits(tiles, N, di.sm_count);
  GemmArgs g{};
  g.dV = dV; g.X = X;
  g.N = N; g.T = T; g.C = C; g.H = H; g.W = W; g.FH = FH; g.FW = FW;
  g.padH = (FH - 1) / 2; g.padW = (FW - 1) / 2;
  g.splits = splits;
  g.per_split = ceil_div(N, splits);
  g.out = splits > 1 ? scratch : G;
  if (splits > 1 && !scratch) return fail(B200CP_ERR_WORKSPACE, "dense gradient: split-K scratch missing");
  dim3 grid(ceil_div(C, BN), ceil_div(T, BM), taps * splits);
  if (grid.y > 65535 || grid.z > 65535) return fail(B200CP_ERR_UNSUPPORTED, "dense gradient: too many tiles");
  if (H * W == 1 && taps == 1) {
    if (T % 4 == 0 && C % 4 == 0) grad_gemm_flat_kernel<true><<<grid, NTH, 0, st>>>(g);
    else grad_gemm_flat_kernel<false><<<grid, NTH, 0, st>>>(g);
    B200CP_LAUNCH_OK("grad_gemm_flat_kernel");
  } else {
    const size_t smem = sizeof(float) * 2 * (BM + BN) * PITCH_CONV;
    B200CP_CUDA_OK(cudaFuncSetAttribute(grad_gemm_conv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    grad_gemm_conv_kernel<<<grid, NTH, smem, st>>>(g);
    B200CP_LAUNCH_OK("grad_gemm_conv_kernel");
  }
  if (splits > 1) {
    const size_t n = (size_t)taps * T * C;
    sum_splits_kernel<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(scratch, G, n, splits);
    B200CP_LAUNCH_OK("sum_splits_kernel");
  }
  return B200CP_OK;
}

}  // namespace b200cp
