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

// ---- contraction of G with all factors but one ---------------------------------------
// Index modes: the m factor modes, pair index p_j = (c_j, t_j), and (for the conv) the tap mode with
// vector S[tap, r].  For the mode q being differentiated
//   out_q[p_q][r] = sum_{rest} G[p_q, rest] * W_q[rest][r],   W_q[rest][r] = prod_{j != q} vec_j[p_j(rest)][r],
// a GEMM whose right operand is generated on the fly.  A CTA owns one q, one chunk of `rest` and 32 ranks; it
// stages 32 rest items at a time (their G offsets, W rows and G columns) in shared memory.  Partial sums per
// chunk are added in chunk order by a second kernel.
constexpr int kCNT = 256, kRB = 32, kSub = 32, kMaxNq = 256;

struct ContractGeom {
  int m, R, T, C, taps, has_s;
  int cd[4], td[4], cstride[4], tstride[4];
  int chunk[5];        // rest items per CTA for each mode
  int part_off[5];     // first partial block of each mode (in units of [n_q][R] blocks, scaled below)
};
struct ContractPtrs {
  const float* A[4];
  const float* S;   // null for the dense layer
  float* dA[4];
  float* dS;        // may be null
  float* part;      // partial sums
};

struct Digit { int size, gstride, mode, fstride; };

__device__ __forceinline__ int mode_size(const ContractGeom& g, int q) { return q < g.m ? g.cd[q] * g.td[q] : g.taps; }
__device__ __forceinline__ long rest_size(const ContractGeom& g, int q) {
  long n = 1;
  for (int j = 0; j < g.m; ++j)
    if (j != q) n *= (long)g.cd[j] * g.td[j];
  if (q != g.m) n *= g.taps;
  return n;
}

// grid = (chunks of mode q, 1, rank blocks); NP * 8 >= entries of mode q
template <int NP>
__global__ void __launch_bounds__(kCNT) contract_factors_kernel(const ContractGeom g, const ContractPtrs p,
                                                                 const float* __restrict__ G, const int q) {
  const long rest_total = rest_size(g, q);
  const long first = (long)blockIdx.x * g.chunk[q];
  if (first >= rest_total) return;
  const int nq = mode_size(g, q);
  const int tid = threadIdx.x, lane = tid % kRB, pg = tid / kRB;
  const int r = blockIdx.z * kRB + lane;

  __shared__ Digit digits[9];
  __shared__ int ndig;
  __shared__ long goff[kSub];
  __shared__ int foff[kSub][5];
  __shared__ long poff[kMaxNq];
  __shared__ float Ws[kSub * kRB];
  __shared__ float Gs[kMaxNq * (kSub + 1)];

  const long TC = (long)g.T * g.C;
  if (tid == 0) {
    int n = 0;
    if (q != g.m && g.taps > 1) digits[n++] = Digit{g.taps, 0, g.m, g.R};  // gstride of the tap handled as TC below
    for (int j = 0; j < g.m; ++j)
      if (j != q) digits[n++] = Digit{g.td[j], g.tstride[j] * g.C, j, g.R};
    for (int j = 0; j < g.m; ++j)
      if (j != q) digits[n++] = Digit{g.cd[j], g.cstride[j], j, g.td[j] * g.R};
    ndig = n;
  }
  for (int pp = tid; pp < nq; pp += kCNT) {
    if (q < g.m) {
      const int ck = pp / g.td[q], tk = pp - ck * g.td[q];
      poff[pp] = (long)tk * g.tstride[q] * g.C + (long)ck * g.cstride[q];
    } else {
      poff[pp] = (long)pp * TC;
    }
  }
  float acc[NP];
#pragma unroll
  for (int i = 0; i < NP; ++i) acc[i] = 0.f;
  __syncthreads();

  const long last = min(rest_total, first + g.chunk[q]);
  for (long base = first; base < last; base += kSub) {
    if (tid < kSub) {
      long idx = base + tid;
      long go = -1;
#pragma unroll
      for (int j = 0; j < 5; ++j) foff[tid][j] = 0;
      if (idx < last) {
        go = 0;
        for (int d = ndig - 1; d >= 0; --d) {
          const int size = digits[d].size, mode = digits[d].mode;
          const int v = (int)(idx % size);
          idx /= size;
          go += mode == g.m ? (long)v * TC : (long)v * digits[d].gstride;
          foff[tid][mode] += v * digits[d].fstride;
        }
      }
      goff[tid] = go;
    }
    __syncthreads();
    for (int idx = tid; idx < kSub * kRB; idx += kCNT) {
      const int ri = idx / kRB;  // lane == idx % kRB
      float w = 0.f;
      if (goff[ri] >= 0 && r < g.R) {
        w = 1.f;
        for (int j = 0; j < g.m; ++j)
          if (j != q) w *= __ldg(p.A[j] + foff[ri][j] + r);
        if (q != g.m && g.has_s) w *= __ldg(p.S + foff[ri][g.m] + r);
      }
      Ws[idx] = w;
    }
    for (int idx = tid; idx < nq * kSub; idx += kCNT) {
      const int pp = idx / kSub, ri = idx - pp * kSub;
      Gs[pp * (kSub + 1) + ri] = goff[ri] >= 0 ? __ldg(G + goff[ri] + poff[pp]) : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int ri = 0; ri < kSub; ++ri) {
      const float w = Ws[ri * kRB + lane];
#pragma unroll
      for (int i = 0; i < NP; ++i)
        if (i * 8 + pg < nq) acc[i] = fmaf(Gs[(i * 8 + pg) * (kSub + 1) + ri], w, acc[i]);
    }
    __syncthreads();
  }
  if (r < g.R) {
    float* out = p.part + ((size_t)g.part_off[q] + (size_t)blockIdx.x * nq) * g.R;
#pragma unroll
    for (int i = 0; i < NP; ++i)
      if (i * 8 + pg < nq) out[(size_t)(i * 8 + pg) * g.R + r] = acc[i];
  }
}

// out_q[e] = sum over chunks of part[q][chunk][e], in chunk order; grid.y = mode
__global__ void __launch_bounds__(256) contract_sum_kernel(const ContractGeom g, const ContractPtrs p) {
  const int q = blockIdx.y;
  const int n = mode_size(g, q) * g.R;
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= n) return;
  const long rest_total = rest_size(g, q);
  const int chunks = (int)((rest_total + g.chunk[q] - 1) / g.chunk[q]);
  const float* src = p.part + (size_t)g.part_off[q] * g.R + e;
  float s = 0.f;
  for (int c = 0; c < chunks; ++c) s += src[(size_t)c * n];
  float* dst = q < g.m ? p.dA[q] : p.dS;
  dst[e] = s;
}

// host mirror of the chunking; returns the number of partial floats
size_t contract_plan(ContractGeom& g, int order, const int* cdims, const int* tdims, int R, int taps, bool has_s) {
  g.m = order; g.R = R; g.taps = taps; g.has_s = has_s ? 1 : 0; g.T = 1; g.C = 1;
  for (int k = 0; k < order; ++k) { g.cd[k] = cdims[k]; g.td[k] = tdims[k]; g.T *= tdims[k]; g.C *= cdims[k]; }
  int cs = 1, ts = 1;
  for (int k = order - 1; k >= 0; --k) { g.cstride[k] = cs; g.tstride[k] = ts; cs *= cdims[k]; ts *= tdims[k]; }
  const int modes = order + (has_s ? 1 : 0);
  size_t blocks = 0;  // in units of R floats
  for (int q = 0; q < modes; ++q) {
    long rest = 1;
    for (int j = 0; j < order; ++j)
      if (j != q) rest *= (long)cdims[j] * tdims[j];
    if (q != order) rest *= taps;
    const int nq = q < order ? cdims[q] * tdims[q] : taps;
    g.chunk[q] = rest > 65536 ? 1024 : rest > 4096 ? 256 : 64;
    const long chunks = (rest + g.chunk[q] - 1) / g.chunk[q];
    g.part_off[q] = (int)blocks;
    blocks += (size_t)chunks * nq;
  }
  return blocks * R;
}

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

size_t contract_scratch_floats(int order, const int* cdims, const int* tdims, int R, int taps, bool has_s) {
  ContractGeom g{};
  return contract_plan(g, order, cdims, tdims, R, taps, has_s);
}

int contract_factors_launch(int order, const int* cdims, const int* tdims, int R, int taps, const float* const* A,
                            const float* S, const float* G, float* const* dA, float* dS, float* scratch,
                            cudaStream_t st) {
  ContractGeom g{};
  ContractPtrs p{};
  contract_plan(g, order, cdims, tdims, R, taps, S != nullptr);
  if (S && !dS) return fail(B200CP_ERR_INVALID_ARG, "factor contraction: dS missing");
  if (!scratch) return fail(B200CP_ERR_WORKSPACE, "factor contraction: scratch missing");
  const int modes = order + (S ? 1 : 0);
  for (int k = 0; k < order; ++k) { p.A[k] = A[k]; p.dA[k] = dA[k]; }
  p.S = S; p.dS = dS; p.part = scratch;
  int max_n = 1;
  for (int q = 0; q < modes; ++q) {
    long rest = 1;
    for (int j = 0; j < order; ++j)
      if (j != q) rest *= (long)cdims[j] * tdims[j];
    if (q != order) rest *= taps;
    const int nq = q < order ? cdims[q] * tdims[q] : taps;
    if (nq > kMaxNq) return fail(B200CP_ERR_UNSUPPORTED, "factor contraction: mode %d has %d > %d entries", q, nq, kMaxNq);
    const long chunks = (rest + g.chunk[q] - 1) / g.chunk[q];
    if (chunks > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "factor contraction: too many chunks");
    max_n = std::max(max_n, nq);
    dim3 grid((unsigned)chunks, 1, ceil_div(R, kRB));
    if (nq <= 16) contract_factors_kernel<2><<<grid, kCNT, 0, st>>>(g, p, G, q);
    else if (nq <= 64) contract_factors_kernel<8><<<grid, kCNT, 0, st>>>(g, p, G, q);
    else contract_factors_kernel<32><<<grid, kCNT, 0, st>>>(g, p, G, q);
    B200CP_LAUNCH_OK("contract_factors_kernel");
  }
  dim3 grid2(ceil_div(max_n * R, 256), modes);
  contract_sum_kernel<<<grid2, 256, 0, st>>>(g, p);
  B200CP_LAUNCH_OK("contract_sum_kernel");
  return B200CP_OK;
}

}  // namespace b200cp
