// The reference's "rebuild" variants: recompose the factors into the undecomposed weight and run the ordinary layer
// with it -- the comparison line of its benchmarks (test/benchmark_conv2d_cp4.py:41-42: cp4recom of
// Cuda_kernels/Utils.cu:36-98, then tf.nn.conv2d; test/benchmark_dense_cp.py:43-49: einsum of the three factors,
// then tf.matmul).  Here: the recomposition kernels of the dense and reshaped-CP layers (the CP4 one lives with the
// CP4 gradient kernels) and a dense conv2d forward for a filter K[T][C][FH][FW] -- one implicit-GEMM kernel on
// warp-level tensor instructions (mma.sync m16n8k8, three tf32 terms, fp32-grade results).  The dense layer's
// product with the recomposed matrix runs on the tcgen05 GEMM of the factor gradients.
//
//   U[n,t,h,w] = sum_{c,y,x} K[t,c,y,x] X[n,c,h+y-pad,w+x-pad]      (zero outside the image; H x W output)
//
// A CTA owns 64 output channels x 128 consecutive output pixels of one image.  Per chunk of 8 input channels it
// stages the input rows those pixels touch (zero ring included) and, per filter row, the FW x 8 x 64 slice of the
// filter split into hi / lo tf32 planes; a filter tap is then one k-step of 8 channels whose B operand is the staged
// image shifted by (y, x).  Eight warps: 2 (halves of the 64 channels) x 4 (quarters of the 128 pixels).
#include "common.cuh"
#include "mma_util.cuh"

namespace b200cp {
namespace {

constexpr int kTM = 64;    // output channels per CTA
constexpr int kTP = 128;   // output pixels per CTA
constexpr int kCK = 8;     // input channels per stage
constexpr int kWS = 72;    // filter plane row: 64 output channels + 8 (bank shift of 8 per input channel)
constexpr int kThreads = 256;

struct DenseConvGeom {
  int N, C, H, W, T, FH, FW, pad, Wp, CS;  // Wp = staged row width, CS = staged floats per input channel
};

__global__ void __launch_bounds__(kThreads, 2)
conv_dense_mma_kernel(const DenseConvGeom g, const float* __restrict__ X, const float* __restrict__ K,
                      float* __restrict__ U) {
  extern __shared__ __align__(16) float smem[];
  float* Xs = smem;                          // [8][CS]: rows h_lo-pad .., columns -pad ..
  float* Whi = Xs + kCK * g.CS;              // [FW][8][kWS]
  float* Wlo = Whi + g.FW * kCK * kWS;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;
  const int n = blockIdx.z, t0 = blockIdx.y * kTM, p0 = blockIdx.x * kTP;
  const int HW = g.H * g.W;
  const int h_lo = p0 / g.W;
  const int h_hi = min(p0 + kTP - 1, HW - 1) / g.W;
  const int nrows = h_hi - h_lo + g.FH;
  const int rowsz = nrows * g.Wp;

  int off[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = min(p0 + wn * 32 + j * 8 + gq, HW - 1);   // pixels past the image repeat the last one (not stored)
    const int ho = p / g.W;
    off[j] = (ho - h_lo) * g.Wp + (p - ho * g.W);
  }
  float acc[2][4][4];
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
      for (int e = 0; e < 4; ++e) acc[mi][j][e] = 0.f;

  const float* Xn = X + (size_t)n * g.C * HW;
  const int taps = g.FH * g.FW;
  for (int c0 = 0; c0 < g.C; c0 += kCK) {
    __syncthreads();   // the chunk before is consumed
    for (int i = tid; i < kCK * rowsz; i += kThreads) {
      const int c = i / rowsz, rem = i - c * rowsz;
      const int r = rem / g.Wp, col = rem - r * g.Wp;
      const int hi = h_lo - g.pad + r, wi = col - g.pad, cc = c0 + c;
      float v = 0.f;
      if (cc < g.C && hi >= 0 && hi < g.H && wi >= 0 && wi < g.W) v = __ldg(Xn + ((size_t)cc * g.H + hi) * g.W + wi);
      Xs[c * g.CS + rem] = v;
    }
    for (int y = 0; y < g.FH; ++y) {
      if (y) __syncthreads();   // the filter row before is consumed
      for (int i = tid; i < kTM * kCK * g.FW; i += kThreads) {
        const int x = i % g.FW, c = (i / g.FW) % kCK, t = i / (g.FW * kCK);
        float v = 0.f;
        if (t0 + t < g.T && c0 + c < g.C) v = __ldg(K + ((size_t)(t0 + t) * g.C + c0 + c) * taps + y * g.FW + x);
        uint32_t hi, lo;
        mma::split_tf32(v, hi, lo);
        Whi[(x * kCK + c) * kWS + t] = __uint_as_float(hi);
        Wlo[(x * kCK + c) * kWS + t] = __uint_as_float(lo);
      }
      __syncthreads();
      for (int x = 0; x < g.FW; ++x) {
        uint32_t ah[2][4], al[2][4];
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) {
          const int row = wm * 32 + mi * 16 + gq;
          const float* h0 = Whi + (x * kCK + tq) * kWS + row;
          const float* l0 = Wlo + (x * kCK + tq) * kWS + row;
          ah[mi][0] = __float_as_uint(h0[0]);           ah[mi][1] = __float_as_uint(h0[8]);
          ah[mi][2] = __float_as_uint(h0[4 * kWS]);     ah[mi][3] = __float_as_uint(h0[4 * kWS + 8]);
          al[mi][0] = __float_as_uint(l0[0]);           al[mi][1] = __float_as_uint(l0[8]);
          al[mi][2] = __float_as_uint(l0[4 * kWS]);     al[mi][3] = __float_as_uint(l0[4 * kWS + 8]);
        }
        const float* xb = Xs + tq * g.CS + y * g.Wp + x;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          uint32_t bh[2], bl[2];
          mma::split_tf32(xb[off[j]], bh[0], bl[0]);
          mma::split_tf32(xb[off[j] + 4 * g.CS], bh[1], bl[1]);
#pragma unroll
          for (int mi = 0; mi < 2; ++mi) {
            mma::mma_tf32(acc[mi][j], al[mi], bh);
            mma::mma_tf32(acc[mi][j], ah[mi], bl);
            mma::mma_tf32(acc[mi][j], ah[mi], bh);
          }
        }
      }
    }
  }

  float* Un = U + (size_t)n * g.T * HW;
#pragma unroll
  for (int mi = 0; mi < 2; ++mi)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int p = p0 + wn * 32 + j * 8 + 2 * tq;
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int t = t0 + wm * 32 + mi * 16 + gq + (e >> 1) * 8, pp = p + (e & 1);
        if (t < g.T && pp < HW) Un[(size_t)t * HW + pp] = acc[mi][j][e];
      }
    }
}

bool plan(const b200cp_tensor_shape& s, DenseConvGeom& g, size_t& smem) {
  g = DenseConvGeom{(int)s.N, (int)s.C, (int)s.H, (int)s.W, (int)s.T, (int)s.Y, (int)s.X, (int)s.pad, 0, 0};
  g.Wp = g.W + g.FW - 1;
  const int span = std::min(g.H, (kTP - 2) / g.W + 2);      // image rows that 128 consecutive pixels can touch
  const long per = (long)(span + g.FH - 1) * g.Wp;
  long cs = per;
  while (cs % 32 != 8) ++cs;                                // 4 channels x 8 pixels of a B fragment: 32 banks
  g.CS = (int)cs;
  smem = ((size_t)kCK * cs + 2 * (size_t)g.FW * kCK * kWS) * sizeof(float);
  return smem <= 100 * 1024 && s.N <= 65535 && ceil_div(g.T, kTM) <= 65535;
}

// W[e] = sum_r prod_k F_k[i_k, o_k, r] (* S[tap, r]), modes flattened first-mode-slowest.  Dense layer: e = i * O + o
// (test/layers.py:445,465).  Reshaped-CP conv: e = (o * I + i) * taps + tap, the [T][C][FH][FW] filter of
// einsum('hwr,' + 'c_k t_k r' ... ) in test/layers.py:716-773.
struct ModeArgs {
  const float* F[4];
  int a[4], b[4];
  int order, R, taps;
};
__global__ void __launch_bounds__(256) kron_recompose_kernel(const ModeArgs m, const float* __restrict__ S,
                                                             float* __restrict__ Wout, int I, int O) {
  const size_t total = (size_t)I * O * m.taps;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    int i, o, tap = 0;
    if (S) {
      tap = (int)(e % m.taps);
      const size_t q = e / m.taps;
      i = (int)(q % I);
      o = (int)(q / I);
    } else {
      o = (int)(e % O);
      i = (int)(e / O);
    }
    int base[4];
#pragma unroll
    for (int k = 3; k >= 0; --k) {
      if (k < m.order) {
        const int ik = i % m.a[k], ok = o % m.b[k];
        i /= m.a[k];
        o /= m.b[k];
        base[k] = (ik * m.b[k] + ok) * m.R;
      } else {
        base[k] = 0;
      }
    }
    float acc = 0.f;
    for (int r = 0; r < m.R; ++r) {
      float v = S ? S[tap * m.R + r] : 1.f;
#pragma unroll
      for (int k = 0; k < 4; ++k)
        if (k < m.order) v *= m.F[k][base[k] + r];
      acc += v;
    }
    Wout[e] = acc;
  }
}

// dst [cols][rows] = src [rows][cols]^T, 32 x 32 tiles through shared memory; grid = (col tiles, row tiles), block (32, 8)
__global__ void __launch_bounds__(256) transpose_kernel(const float* __restrict__ src, float* __restrict__ dst, int rows,
                                                        int cols) {
  __shared__ float tile[32][33];
  const int c0 = blockIdx.x * 32, r0 = blockIdx.y * 32, tx = threadIdx.x, ty = threadIdx.y;
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int r = r0 + ty + 8 * j, c = c0 + tx;
    if (r < rows && c < cols) tile[ty + 8 * j][tx] = __ldg(src + (size_t)r * cols + c);
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int c = c0 + ty + 8 * j, r = r0 + tx;
    if (r < rows && c < cols) dst[(size_t)c * rows + r] = tile[tx][ty + 8 * j];
  }
}

}  // namespace

// Y [B][O] = X [B][I] M [I][O]: X is transposed into the scratch, then the product is the flat gradient GEMM
// (A^T B with K as rows: tcgen05 with three tf32 terms where the shape fills its tiles, CUDA cores otherwise).
size_t dense_matmul_scratch_floats(int B, int I, int O) {
  return align_up((size_t)I * B, 64) + dense_grad_scratch_floats(I, B, O, 1, 1, 1, 1);
}
int dense_matmul_launch(int B, int I, int O, const float* X, const float* M, float* Y, float* scratch, cudaStream_t st) {
  if (ceil_div(B, 32) > 65535) return fail(B200CP_ERR_UNSUPPORTED, "dense matmul: batch %d too large", B);
  float* Xt = scratch;
  transpose_kernel<<<dim3(ceil_div(I, 32), ceil_div(B, 32)), dim3(32, 8), 0, st>>>(X, Xt, B, I);
  B200CP_LAUNCH_OK("transpose_kernel");
  return dense_grad_launch(I, B, O, 1, 1, 1, 1, Xt, M, Y, scratch + align_up((size_t)I * B, 64), st);
}

// dense layer: Wout [I][O]; reshaped-CP conv (S != nullptr, taps = FH * FW): Wout [T][C][FH][FW] with a = cdims, b = tdims
int kron_recompose_launch(int order, const int* a, const int* b, int R, const float* const* F, const float* S, int taps,
                          float* Wout, cudaStream_t st) {
  ModeArgs m{};
  size_t I = 1, O = 1;
  for (int k = 0; k < order; ++k) {
    m.F[k] = F[k]; m.a[k] = a[k]; m.b[k] = b[k];
    if (a[k] < 1 || b[k] < 1) return fail(B200CP_ERR_INVALID_ARG, "recompose: mode %d has size %d x %d", k, a[k], b[k]);
    I *= (size_t)a[k]; O *= (size_t)b[k];
  }
  if (R < 1 || taps < 1) return fail(B200CP_ERR_INVALID_ARG, "recompose: rank %d, taps %d", R, taps);
  if (I > 0x7fffffff || O > 0x7fffffff) return fail(B200CP_ERR_UNSUPPORTED, "recompose: more than 2^31 rows or columns");
  m.order = order; m.R = R; m.taps = S ? taps : 1;
  const size_t total = I * O * (size_t)m.taps;
  const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 64);
  kron_recompose_kernel<<<blocks, 256, 0, st>>>(m, S, Wout, (int)I, (int)O);
  B200CP_LAUNCH_OK("kron_recompose_kernel");
  return B200CP_OK;
}

bool conv_dense_supported(const b200cp_tensor_shape& s) {
  DenseConvGeom g;
  size_t smem;
  return plan(s, g, smem);
}

// U [N,T,H,W] = dense cross-correlation of X [N,C,H,W] with K [T,C,FH,FW], zero padding `pad` on the top / left
int conv_dense_launch(const b200cp_tensor_shape& s, const float* X, const float* K, float* U, cudaStream_t st) {
  DenseConvGeom g;
  size_t smem;
  if (!plan(s, g, smem))
    return fail(B200CP_ERR_UNSUPPORTED, "dense conv2d: staged rows need %zu bytes of shared memory (W=%u, filter %ux%u)",
                smem, s.W, s.Y, s.X);
  B200CP_CUDA_OK(cudaFuncSetAttribute(conv_dense_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  dim3 grid(ceil_div(g.H * g.W, kTP), ceil_div(g.T, kTM), g.N);
  conv_dense_mma_kernel<<<grid, kThreads, smem, st>>>(g, X, K, U);
  B200CP_LAUNCH_OK("conv_dense_mma_kernel");
  return B200CP_OK;
}

}  // namespace b200cp
