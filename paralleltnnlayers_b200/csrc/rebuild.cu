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
// A first pass rewrites the filter as hi / lo tf32 planes [chunk of 8 input channels][tap][T padded to 64][8], so that
// a CTA's slice of a tap is 64 rows of 32 bytes and an A fragment is one ldmatrix.  A CTA owns 64 output channels x
// 128 consecutive output pixels of one image.  Its work is a list of items (chunk of 8 input channels, group of at
// most 9 filter taps); item i + 1 is
// copied into the other half of a double buffer (cp.async: the image rows the pixels touch, zero ring included,
// once per chunk; the filter slice per item) while item i is multiplied: a tap is one k-step of 8 channels whose B
// operand is the staged image shifted by (y, x).  Eight warps: 2 (halves of the 64 channels) x 4 (quarters of the
// 128 pixels).
#include "common.cuh"
#include "mma_util.cuh"

namespace b200cp {
namespace {

constexpr int kTM = 64;    // output channels per CTA
constexpr int kTP = 128;   // output pixels per CTA
constexpr int kCK = 8;     // input channels per stage
constexpr int kWS = 8;     // staged filter row: the 8 input channels of a chunk (one ldmatrix tile row per 16 bytes)
constexpr int kTG = 9;     // filter taps per item
constexpr int kThreads = 256;
constexpr int kWBuf = kTG * kTM * kWS;   // floats of one hi (or lo) filter buffer

struct DenseConvGeom {
  int N, C, H, W, T, FH, FW, pad, Wp, CS;  // Wp = staged row width, CS = staged floats per input channel
  int TP, chunks, groups;                  // T padded to 64; chunks of 8 input channels; tap groups per chunk
  size_t plane;                            // floats of one filter plane
};

// K [T][C][taps] -> hi / lo planes [chunk][tap][TP][8], zero where t >= T or c >= C
__global__ void __launch_bounds__(256) dense_filter_split_kernel(const DenseConvGeom g, const float* __restrict__ K,
                                                                 float* __restrict__ Wg) {
  const int taps = g.FH * g.FW;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < g.plane; e += (size_t)gridDim.x * blockDim.x) {
    const int c = (int)(e % kCK);
    size_t q = e / kCK;
    const int t = (int)(q % g.TP);
    q /= g.TP;
    const int tap = (int)(q % taps), cc = (int)(q / taps) * kCK + c;
    const float v = (t < g.T && cc < g.C) ? __ldg(K + ((size_t)t * g.C + cc) * taps + tap) : 0.f;
    uint32_t hi, lo;
    mma::split_tf32(v, hi, lo);
    Wg[e] = __uint_as_float(hi);
    Wg[g.plane + e] = __uint_as_float(lo);
  }
}

// F3: 3 x 3 filter -- one item per channel chunk, the nine taps unrolled with constant offsets
template <bool F3>
__global__ void __launch_bounds__(kThreads, 2)
conv_dense_mma_kernel(const DenseConvGeom g, const float* __restrict__ X, const float* __restrict__ Wg,
                      float* __restrict__ U) {
  extern __shared__ __align__(16) float smem[];
  float* Xs = smem;                          // [2][8][CS]: rows h_lo-pad .., columns -pad ..
  float* Ws = Xs + 2 * kCK * g.CS;           // [2][hi, lo][kTG][64][kWS]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, gq = lane >> 2, tq = lane & 3;
  const int wm = warp >> 2, wn = warp & 3;
  const int n = blockIdx.z, t0 = blockIdx.y * kTM, p0 = blockIdx.x * kTP;
  const int HW = g.H * g.W;
  const int h_lo = p0 / g.W;
  const int h_hi = min(p0 + kTP - 1, HW - 1) / g.W;
  const int nrows = h_hi - h_lo + g.FH;
  const int taps = g.FH * g.FW;

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
  const unsigned xs_s = (unsigned)__cvta_generic_to_shared(Xs), ws_s = (unsigned)__cvta_generic_to_shared(Ws);

  auto load_item = [&](int item) {
    const int chunk = item / g.groups, grp = item - chunk * g.groups;
    if (grp == 0) {
      const unsigned dst = xs_s + (unsigned)((chunk & 1) * kCK * g.CS) * 4u;
      if (g.Wp < 40) {   // short rows: one element per thread and turn
        const int rowsz = nrows * g.Wp;
        for (int i = tid; i < kCK * rowsz; i += kThreads) {
          const int c = i / rowsz, rem = i - c * rowsz;
          const int r = rem / g.Wp, col = rem - r * g.Wp;
          const int hi = h_lo - g.pad + r, wi = col - g.pad, cc = chunk * kCK + c;
          const bool in = cc < g.C && hi >= 0 && hi < g.H && wi >= 0 && wi < g.W;
          mma::cp_async4_s(dst + (unsigned)(c * g.CS + rem) * 4u, in ? Xn + ((size_t)cc * g.H + hi) * g.W + wi : Xn,
                           in ? 4 : 0);
        }
      } else
      for (int row = warp; row < kCK * nrows; row += kThreads / 32) {   // long rows: a warp copies whole staged rows
        const int c = row / nrows, r = row - c * nrows;
        const int hi = h_lo - g.pad + r, cc = chunk * kCK + c;
        const bool row_in = cc < g.C && hi >= 0 && hi < g.H;
        const float* srow = Xn + ((size_t)cc * g.H + hi) * g.W - g.pad;
        const unsigned drow = dst + (unsigned)(c * g.CS + r * g.Wp) * 4u;
        for (int col = lane; col < g.Wp; col += 32) {
          const bool in = row_in && col >= g.pad && col < g.W + g.pad;
          mma::cp_async4_s(drow + (unsigned)col * 4u, in ? srow + col : Xn, in ? 4 : 0);
        }
      }
    }
    const int tap0 = grp * kTG, nt = min(kTG, taps - tap0);
    const float* src = Wg + ((size_t)(chunk * taps + tap0) * g.TP + t0) * kCK;
    const unsigned dst = ws_s + (unsigned)((item & 1) * 2 * kWBuf) * 4u;
    for (int i = tid; i < nt * kTM * 2; i += kThreads) {
      const int tl = i / (kTM * 2), rem = i - tl * kTM * 2, t = rem >> 1, half = rem & 1;
      const float* sp = src + ((size_t)tl * g.TP + t) * kCK + half * 4;
      // rows t and t + 4 of an ldmatrix tile would meet on the same banks: the two 16-byte pieces of a row swap places
      // in every second group of four rows
      const unsigned d = dst + (unsigned)((tl * kTM + t) * kWS + ((half ^ (t >> 2)) & 1) * 4) * 4u;
      mma::cp_async16_s(d, sp, 16);
      mma::cp_async16_s(d + kWBuf * 4u, sp + g.plane, 16);
    }
  };

  const int items = g.chunks * g.groups;
  load_item(0);
  mma::cp_async_commit();
  for (int item = 0; item < items; ++item) {
    if (item + 1 < items) load_item(item + 1);
    mma::cp_async_commit();
    mma::cp_async_wait<1>();
    __syncthreads();
    const int chunk = item / g.groups, grp = item - chunk * g.groups;
    const float* Xc = Xs + (chunk & 1) * kCK * g.CS + tq * g.CS;
    const float* Whi = Ws + (item & 1) * 2 * kWBuf;
    const int tap0 = grp * kTG, nt = F3 ? 9 : min(kTG, taps - tap0);
    // ldmatrix lane address: tiles (rows 0-7, k 0-3), (rows 8-15, k 0-3), (rows 0-7, k 4-7), (rows 8-15, k 4-7) = a0..a3
    const float* wl = Whi + (wm * 32 + (lane & 7) + ((lane >> 3) & 1) * 8) * kWS + (((lane >> 4) ^ (lane >> 2)) & 1) * 4;
#pragma unroll
    for (int tl = 0; tl < (F3 ? 9 : kTG); ++tl) {
      if (!F3 && tl >= nt) break;
      int y, x;
      if (F3) { y = tl / 3; x = tl % 3; } else { const int tap = tap0 + tl; y = tap / g.FW; x = tap - y * g.FW; }
      uint32_t ah[2][4], al[2][4];
#pragma unroll
      for (int mi = 0; mi < 2; ++mi) {
        const float* h0 = wl + (tl * kTM + mi * 16) * kWS;
        mma::ldmatrix_x4(ah[mi], h0);
        mma::ldmatrix_x4(al[mi], h0 + kWBuf);
      }
      const float* xb = Xc + y * g.Wp + x;
      uint32_t bh[4][2], bl[4][2];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        mma::split_tf32(xb[off[j]], bh[j][0], bl[j][0]);
        mma::split_tf32(xb[off[j] + 4 * g.CS], bh[j][1], bl[j][1]);
      }
      // term-major: the three products of one accumulator are eight instructions apart
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) mma::mma_tf32_ordered(acc[mi][j], al[mi], bh[j]);
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) mma::mma_tf32_ordered(acc[mi][j], ah[mi], bl[j]);
#pragma unroll
      for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int mi = 0; mi < 2; ++mi) mma::mma_tf32_ordered(acc[mi][j], ah[mi], bh[j]);
    }
    __syncthreads();   // the buffers of this item are free for item + 2
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
  g = DenseConvGeom{(int)s.N, (int)s.C, (int)s.H, (int)s.W, (int)s.T, (int)s.Y, (int)s.X, (int)s.pad, 0, 0, 0, 0, 0, 0};
  g.Wp = g.W + g.FW - 1;
  const int span = std::min(g.H, (kTP - 2) / g.W + 2);      // image rows that 128 consecutive pixels can touch
  const long per = (long)(span + g.FH - 1) * g.Wp;
  long cs = per;
  while (cs % 32 != 8) ++cs;                                // 4 channels x 8 pixels of a B fragment: 32 banks
  g.CS = (int)cs;
  g.TP = ceil_div(g.T, kTM) * kTM;
  g.chunks = ceil_div(g.C, kCK);
  g.groups = ceil_div(g.FH * g.FW, kTG);
  g.plane = (size_t)g.chunks * g.FH * g.FW * kCK * g.TP;
  smem = (2 * (size_t)kCK * cs + 4 * (size_t)kWBuf) * sizeof(float);
  return smem <= 200 * 1024 && s.N <= 65535 && ceil_div(g.T, kTM) <= 65535;
}

// W[e] = sum_r prod_k F_k[i_k, o_k, r] (* S[tap, r]), modes flattened first-mode-slowest.  Dense layer: e = i * O + o
// (test/layers.py:445,465).  Reshaped-CP conv: e = (o * I + i) * taps + tap, the [T][C][FH][FW] filter of
// einsum('hwr,' + 'c_k t_k r' ... ) in test/layers.py:716-773.
struct ModeArgs {
  const float* F[4];
  int a[4], b[4];
  int order, R, taps, vec;   // vec: R % 4 == 0 and every factor on a 16-byte boundary
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
    if (m.vec) {   // every factor row starts on 16 bytes: four ranks per load
      for (int r = 0; r < m.R; r += 4) {
        float4 v = S ? __ldg(reinterpret_cast<const float4*>(S + tap * m.R + r)) : make_float4(1.f, 1.f, 1.f, 1.f);
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < m.order) {
            const float4 f = __ldg(reinterpret_cast<const float4*>(m.F[k] + base[k] + r));
            v.x *= f.x; v.y *= f.y; v.z *= f.z; v.w *= f.w;
          }
        acc += v.x;   // rank order, as the scalar loop
        acc += v.y;
        acc += v.z;
        acc += v.w;
      }
    } else {
      for (int r = 0; r < m.R; ++r) {
        float v = S ? S[tap * m.R + r] : 1.f;
#pragma unroll
        for (int k = 0; k < 4; ++k)
          if (k < m.order) v *= m.F[k][base[k] + r];
        acc += v;
      }
    }
    Wout[e] = acc;
  }
}

// ---- dense layer, two or more modes: M = sum_r GA_r (x) GB_r with GA = the product of the first half of the modes,
// GB = the second half.  The half products are small ([IA][OA][R] and [IB][OB][R]); the outer product then costs one
// multiply-add per rank and element of M instead of one per rank, mode and element.
__global__ void __launch_bounds__(256) kron_half_kernel(const ModeArgs m, int k0, int k1, float* __restrict__ G, int IH,
                                                        int OH) {
  const size_t total = (size_t)IH * OH * m.R;
  for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < total; e += (size_t)gridDim.x * blockDim.x) {
    const int r = (int)(e % m.R);
    size_t q = e / m.R;
    int o = (int)(q % OH), i = (int)(q / OH);
    float v = 1.f;
    for (int k = k1 - 1; k >= k0; --k) {
      const int ik = i % m.a[k], ok = o % m.b[k];
      i /= m.a[k];
      o /= m.b[k];
      v *= __ldg(m.F[k] + (size_t)(ik * m.b[k] + ok) * m.R + r);
    }
    G[e] = v;
  }
}

constexpr int kOutIB = 4, kOutOA = 8, kOutOB = 64, kOutR = 32;
// M[(iA * IB + iB)][(oA * OB + oB)] = sum_r GA[iA][oA][r] GB[iB][oB][r], ranks added in order.
// grid = (oA blocks * iB blocks, IA); 256 threads: thread = (oB within 64, oA pair); 2 oA x 4 iB outputs per thread.
__global__ void __launch_bounds__(256) kron_outer_kernel(const float* __restrict__ GA, const float* __restrict__ GB,
                                                         float* __restrict__ M, int IA, int OA, int IB, int OB, int R) {
  __shared__ float sa[kOutOA][kOutR];
  __shared__ float sb[kOutIB][kOutOB][kOutR + 1];
  const int nib = (IB + kOutIB - 1) / kOutIB;
  const int iA = blockIdx.y, ib0 = ((int)blockIdx.x % nib) * kOutIB, oa0 = ((int)blockIdx.x / nib) * kOutOA;
  const int tid = threadIdx.x, obl = tid % kOutOB, oq = tid / kOutOB;
  for (int ob0 = 0; ob0 < OB; ob0 += kOutOB) {
    float acc[2][kOutIB];
#pragma unroll
    for (int u = 0; u < 2; ++u)
#pragma unroll
      for (int v = 0; v < kOutIB; ++v) acc[u][v] = 0.f;
    for (int r0 = 0; r0 < R; r0 += kOutR) {
      __syncthreads();
      for (int i = tid; i < kOutOA * kOutR; i += 256) {
        const int oa = i / kOutR, r = i % kOutR;
        sa[oa][r] = (oa0 + oa < OA && r0 + r < R) ? __ldg(GA + ((size_t)iA * OA + oa0 + oa) * R + r0 + r) : 0.f;
      }
      for (int i = tid; i < kOutIB * kOutOB * kOutR; i += 256) {
        const int r = i % kOutR, ob = (i / kOutR) % kOutOB, ib = i / (kOutR * kOutOB);
        sb[ib][ob][r] = (ib0 + ib < IB && ob0 + ob < OB && r0 + r < R)
                            ? __ldg(GB + ((size_t)(ib0 + ib) * OB + ob0 + ob) * R + r0 + r) : 0.f;
      }
      __syncthreads();
#pragma unroll 8
      for (int r = 0; r < kOutR; ++r) {
        const float a0 = sa[oq][r], a1 = sa[oq + 4][r];
#pragma unroll
        for (int v = 0; v < kOutIB; ++v) {
          const float b = sb[v][obl][r];
          acc[0][v] = fmaf(a0, b, acc[0][v]);
          acc[1][v] = fmaf(a1, b, acc[1][v]);
        }
      }
    }
    const int ob = ob0 + obl;
    if (ob < OB) {
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int oa = oa0 + oq + 4 * u;
        if (oa >= OA) continue;
#pragma unroll
        for (int v = 0; v < kOutIB; ++v)
          if (ib0 + v < IB) M[((size_t)iA * IB + ib0 + v) * ((size_t)OA * OB) + (size_t)oa * OB + ob] = acc[u][v];
      }
    }
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
  uintptr_t bits = reinterpret_cast<uintptr_t>(S);
  for (int k = 0; k < order; ++k) bits |= reinterpret_cast<uintptr_t>(F[k]);
  m.vec = R % 4 == 0 && (bits & 15) == 0;
  const size_t total = I * O * (size_t)m.taps;
  const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 148 * 64);
  kron_recompose_kernel<<<blocks, 256, 0, st>>>(m, S, Wout, (int)I, (int)O);
  B200CP_LAUNCH_OK("kron_recompose_kernel");
  return B200CP_OK;
}

// floats of scratch for the two half products of dense_recompose_launch (0: the direct kernel is used)
size_t dense_recompose_scratch_floats(int order, const int* a, const int* b, int R) {
  if (order < 2) return 0;
  const int h = (order + 1) / 2;
  size_t A = 1, B = 1;
  for (int k = 0; k < order; ++k) (k < h ? A : B) *= (size_t)a[k] * b[k];
  return align_up(A * R, 64) + align_up(B * R, 64);
}

// M [I][O] of the dense layer; with a scratch of dense_recompose_scratch_floats() floats the two-stage form runs
int dense_recompose_launch(int order, const int* a, const int* b, int R, const float* const* F, float* M, float* scratch,
                           cudaStream_t st) {
  if (order < 2 || scratch == nullptr) return kron_recompose_launch(order, a, b, R, F, nullptr, 1, M, st);
  ModeArgs m{};
  const int h = (order + 1) / 2;
  size_t IA = 1, OA = 1, IB = 1, OB = 1;
  for (int k = 0; k < order; ++k) {
    m.F[k] = F[k]; m.a[k] = a[k]; m.b[k] = b[k];
    if (a[k] < 1 || b[k] < 1) return fail(B200CP_ERR_INVALID_ARG, "recompose: mode %d has size %d x %d", k, a[k], b[k]);
    (k < h ? IA : IB) *= (size_t)a[k];
    (k < h ? OA : OB) *= (size_t)b[k];
  }
  if (R < 1) return fail(B200CP_ERR_INVALID_ARG, "recompose: rank %d", R);
  if (IA * IB > 0x7fffffff || OA * OB > 0x7fffffff || IA > 65535)
    return fail(B200CP_ERR_UNSUPPORTED, "recompose: more than 2^31 rows or columns");
  m.order = order; m.R = R; m.taps = 1;
  float* GA = scratch;
  float* GB = scratch + align_up(IA * OA * R, 64);
  const size_t na = IA * OA * R, nb = IB * OB * R;
  kron_half_kernel<<<(unsigned)std::min<size_t>((na + 255) / 256, 148 * 16), 256, 0, st>>>(m, 0, h, GA, (int)IA, (int)OA);
  B200CP_LAUNCH_OK("kron_half_kernel");
  kron_half_kernel<<<(unsigned)std::min<size_t>((nb + 255) / 256, 148 * 16), 256, 0, st>>>(m, h, order, GB, (int)IB, (int)OB);
  B200CP_LAUNCH_OK("kron_half_kernel");
  dim3 grid((unsigned)(ceil_div((int)OA, kOutOA) * ceil_div((int)IB, kOutIB)), (unsigned)IA);
  kron_outer_kernel<<<grid, 256, 0, st>>>(GA, GB, M, (int)IA, (int)OA, (int)IB, (int)OB, R);
  B200CP_LAUNCH_OK("kron_outer_kernel");
  return B200CP_OK;
}

bool conv_dense_supported(const b200cp_tensor_shape& s) {
  DenseConvGeom g;
  size_t smem;
  return plan(s, g, smem);
}

// floats of scratch: the hi / lo planes of the re-laid filter
size_t conv_dense_scratch_floats(const b200cp_tensor_shape& s) {
  DenseConvGeom g;
  size_t smem;
  plan(s, g, smem);
  return 2 * g.plane;
}

// U [N,T,H,W] = dense cross-correlation of X [N,C,H,W] with K [T,C,FH,FW], zero padding `pad` on the top / left;
// scratch: conv_dense_scratch_floats() floats, 16-byte aligned
int conv_dense_launch(const b200cp_tensor_shape& s, const float* X, const float* K, float* U, float* scratch,
                      cudaStream_t st) {
  DenseConvGeom g;
  size_t smem;
  if (!plan(s, g, smem))
    return fail(B200CP_ERR_UNSUPPORTED, "dense conv2d: staged rows need %zu bytes of shared memory (W=%u, filter %ux%u)",
                smem, s.W, s.Y, s.X);
  if (reinterpret_cast<uintptr_t>(scratch) & 15)
    return fail(B200CP_ERR_INVALID_ARG, "dense conv2d: the workspace must be 16-byte aligned");
  dense_filter_split_kernel<<<(unsigned)std::min<size_t>((g.plane + 255) / 256, 148 * 16), 256, 0, st>>>(g, K, scratch);
  B200CP_LAUNCH_OK("dense_filter_split_kernel");
  dim3 grid(ceil_div(g.H * g.W, kTP), ceil_div(g.T, kTM), g.N);
  if (g.FH == 3 && g.FW == 3) {
    B200CP_CUDA_OK(cudaFuncSetAttribute(conv_dense_mma_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_dense_mma_kernel<true><<<grid, kThreads, smem, st>>>(g, X, scratch, U);
  } else {
    B200CP_CUDA_OK(cudaFuncSetAttribute(conv_dense_mma_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    conv_dense_mma_kernel<false><<<grid, kThreads, smem, st>>>(g, X, scratch, U);
  }
  B200CP_LAUNCH_OK("conv_dense_mma_kernel");
  return B200CP_OK;
}

}  // namespace b200cp
