// CP4 conv2d backward-filter (and the dense filter gradient / recomposition helpers) on CUDA cores.
#include <mutex>

#include "cp4_simt.cuh"

namespace b200cp {

// ===========================================================================
// backward-filter
// ===========================================================================
//
// Per tile (one CTA):
//   Q = K0^T dU and P = K1^T X on the halo tile (phase-1 code above)
//   per rank r, per pixel:  rows_i = sum_j KW[j] P[i][j],  cols_j = sum_i KH[i] P[i][j]
//       Z  = sum_i KH[i] rows_i            -> Zs[r][px]
//       Qt = sum_{i,j} KH[i] KW[j] Q[h-i+p][w-j+p]   -> Qts[r][px]
//       dKH[i,r] += Q * rows_i,  dKW[j,r] += Q * cols_j     (warp shuffle + fixed-order smem sum)
//   dK0[t,r] = sum_px dU[t,px] Zs[r][px],  dK1[c,r] = sum_px X[c,px] Qts[r][px]
//       one warp per group of channels, lanes stride the pixels, butterfly reduction.
// Each CTA writes its partial gradients to workspace[cta][...]; a second kernel
// sums the partials in CTA order, so the result is bitwise reproducible.
// Formulas: Cuda_kernels/cp4Conv2dBackwardFilter.cu:91-104,142-155,192-205,241-254.
namespace {

constexpr int kRedFloats = 8 * 64;  // block-reduction staging: 8 warps x 64 sums (>= 8 x 2F for F <= 11)

struct GeomF {
  Geom g;      // Cin = C (X channels), Cout = T (dU channels)
  int F;       // filter size
  int nparam;  // (T + C + 2F) * R  floats per partial (R = ranks of this launch)
  int OPXs;
};

// Reduce M values per lane across the warp so that every value's warp-sum lands
// on exactly one lane.  After the call, lane l holds sums for indices
// idx(l, j) = j + (M >> 5) * bitrev-free mapping computed by `owner_index`.
template <int M>
__device__ __forceinline__ void warp_transpose_reduce(float (&v)[M], int lane) {
  // halving steps while more than one value per lane remains
#pragma unroll
  for (int off = 16, m = M / 2; off >= 1; off >>= 1, m >>= 1) {
    if (m >= 1) {
      const bool hi = lane & off;
#pragma unroll
      for (int i = 0; i < m; ++i) {
        const float send = hi ? v[i] : v[i + m];
        const float keep = hi ? v[i + m] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
      }
    } else {
      v[0] += __shfl_xor_sync(0xffffffffu, v[0], off);
    }
  }
}
// index (0..M-1) of the j-th value lane `lane` owns after warp_transpose_reduce<M>
template <int M>
__device__ __forceinline__ int owner_index(int lane, int j) {
  int idx = 0, m = M / 2;
#pragma unroll
  for (int off = 16; off >= 1; off >>= 1, m >>= 1)
    if (m >= 1 && (lane & off)) idx += m;
  return idx + j;
}

// dK[ch, r] partial = sum over the tile's pixels of src[n, ch, px] * Vs[r][px]
template <int RP, int CG>
__device__ __forceinline__ void pixel_reduce(const Geom& g, int OPXs, const float* __restrict__ src_n, int nch,
                                             const float* Vs, const int* pixoff, float* __restrict__ part, int tid,
                                             int nt) {
  const int lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
  const size_t HW = (size_t)g.H * g.W;
  constexpr int M = CG * RP;
  constexpr int PER = M >= 32 ? M / 32 : 1;  // values per lane after the reduction
  for (int c0 = warp * CG; c0 < nch; c0 += nwarp * CG) {
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; ++i) acc[i] = 0.f;
    const float* s[CG];
#pragma unroll
    for (int j = 0; j < CG; ++j) s[j] = src_n + (size_t)min(c0 + j, nch - 1) * HW;
    // eight pixel rows of the warp are fetched before any is used, so the loads overlap
    for (int pb = 0; pb < g.OPX; pb += 32 * 8) {
      float d[8][CG];
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int p = pb + it * 32 + lane;
        const int po = p < g.OPX ? pixoff[p] : -1;
#pragma unroll
        for (int j = 0; j < CG; ++j) d[it][j] = po >= 0 ? __ldg(s[j] + po) : 0.f;
      }
#pragma unroll
      for (int it = 0; it < 8; ++it) {
        const int p = min(pb + it * 32 + lane, g.OPX - 1);  // d is zero beyond the tile
#pragma unroll
        for (int r = 0; r < RP; ++r) {
          const float z = Vs[r * OPXs + p];
#pragma unroll
          for (int j = 0; j < CG; ++j) acc[j * RP + r] = fmaf(d[it][j], z, acc[j * RP + r]);
        }
      }
    }
    warp_transpose_reduce<M>(acc, lane);
    // M < 32: after log2(M) halving steps each group of 32/M lanes holds the same sum
    const bool owner = M >= 32 || (lane & ((32 / (M < 32 ? M : 32)) - 1)) == 0;
    if (owner) {
#pragma unroll
      for (int j = 0; j < PER; ++j) {
        const int idx = owner_index<M>(lane, j);
        const int cj = idx / RP, r = idx - cj * RP;
        if (c0 + cj < nch && r < g.R) part[(size_t)(c0 + cj) * g.R + r] = acc[j];
      }
    }
  }
}

// 3x3 stencil phase: one pass over the thread's pixels per chunk of RC ranks; the dKH / dKW contributions stay in
// registers and are reduced once per chunk (butterfly over the warp, then warps in a fixed order).
template <int RP>
__device__ __forceinline__ void stencil_phase_3x3(const GeomF& gf, const float* Ps, const float* Qs, float* Zs, float* Qts,
                                                  const float* KHs, const float* KWs, const int* pixoff, float* red,
                                                  float* part_KH, float* part_KW, int tid, int nt) {
  const Geom& g = gf.g;
  constexpr int RC = RP < 8 ? RP : 8;
  constexpr int M = RC * 8;  // per rank: 3 row sums, 3 column sums, 2 unused (power-of-two butterfly)
  const int lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
  const int p = g.pad;
  for (int rc = 0; rc < RP; rc += RC) {
    float acc[M];
#pragma unroll
    for (int i = 0; i < M; ++i) acc[i] = 0.f;
    for (int op = tid; op < g.OPX; op += nt) {
      const int oy = op / g.TW, ox = op - oy * g.TW;
      const bool in = pixoff[op] >= 0;
      const int wo = oy * g.TWh + ox;
#pragma unroll
      for (int rr = 0; rr < RC; ++rr) {
        const int r = rc + rr;
        float zv = 0.f, qt = 0.f;
        if (in) {
          const float* pw = Ps + r * g.HPXs + wo;
          const float* qw = Qs + r * g.HPXs + wo;
          float kh[3], kw[3], cols[3] = {0.f, 0.f, 0.f};
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            kh[i] = KHs[i * RP + r];
            kw[i] = KWs[i * RP + r];
          }
          const float q = qw[p * g.TWh + p];
#pragma unroll
          for (int i = 0; i < 3; ++i) {
            float row = 0.f, qrow = 0.f;
#pragma unroll
            for (int j = 0; j < 3; ++j) {
              const float pv = pw[i * g.TWh + j];
              row = fmaf(kw[j], pv, row);
              cols[j] = fmaf(kh[i], pv, cols[j]);
              qrow = fmaf(kw[j], qw[(2 * p - i) * g.TWh + (2 * p - j)], qrow);
            }
            zv = fmaf(kh[i], row, zv);
            qt = fmaf(kh[i], qrow, qt);
            acc[rr * 8 + i] = fmaf(q, row, acc[rr * 8 + i]);
          }
#pragma unroll
          for (int j = 0; j < 3; ++j) acc[rr * 8 + 3 + j] = fmaf(q, cols[j], acc[rr * 8 + 3 + j]);
        }
        Zs[r * gf.OPXs + op] = zv;
        Qts[r * gf.OPXs + op] = qt;
      }
    }
    warp_transpose_reduce<M>(acc, lane);
#pragma unroll
    for (int j = 0; j < M / 32; ++j) red[warp * M + owner_index<M>(lane, j)] = acc[j];
    __syncthreads();
    if (tid < M) {
      float sum = 0.f;
      for (int w = 0; w < nwarp; ++w) sum += red[w * M + tid];
      const int r = rc + tid / 8, k = tid & 7;
      if (r < g.R && k < 6) {
        if (k < 3) part_KH[(size_t)k * g.R + r] = sum;
        else part_KW[(size_t)(k - 3) * g.R + r] = sum;
      }
    }
    __syncthreads();
  }
}

// FMAX bounds the register arrays of the stencil phase; EXACT means F == FMAX at compile time.
template <int RP, int PPT, int FMAX, bool EXACT>
__global__ void __launch_bounds__(256) cp4_bwd_filter_kernel(const GeomF gf, const float* __restrict__ X,
                                                             const float* __restrict__ dU,
                                                             const float* __restrict__ K0,
                                                             const float* __restrict__ K1,
                                                             const float* __restrict__ KH,
                                                             const float* __restrict__ KW,
                                                             float* __restrict__ partial) {
  const Geom& g = gf.g;
  const int F = EXACT ? FMAX : gf.F;
  extern __shared__ __align__(16) float smem[];
  float* Fs = smem;                              // [cchunk][RP]
  float* KHs = Fs + g.fcap;                      // [F][RP]
  float* KWs = KHs + F * RP;                     // [F][RP]
  float* red = KWs + F * RP;                     // [8 warps][max(2F, 64)]
  float* Ps = red + kRedFloats;                  // [RP][HPXs]
  float* Qs = Ps + RP * g.HPXs;                  // [RP][HPXs]
  float* Zs = Qs + RP * g.HPXs;                  // [RP][OPXs]
  float* Qts = Zs + RP * gf.OPXs;                // [RP][OPXs]
  int* pixoff = reinterpret_cast<int*>(Qts + RP * gf.OPXs);  // [OPXs]
  float* Xst = reinterpret_cast<float*>(pixoff + gf.OPXs);   // [kStages*kKC][nt*PPT]  cp.async FIFO

  const int tid = threadIdx.x, nt = blockDim.x;
  const int lane = tid & 31, warp = tid >> 5, nwarp = nt >> 5;
  int b = blockIdx.x;
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  const size_t HW = (size_t)g.H * g.W;
  const float* Xn = X + (size_t)n * g.Cin * HW;
  const float* dUn = dU + (size_t)n * g.Cout * HW;
  float* part = partial + (size_t)blockIdx.x * gf.nparam;
  float* part_K0 = part;
  float* part_K1 = part_K0 + (size_t)g.Cout * g.R;
  float* part_KH = part_K1 + (size_t)g.Cin * g.R;
  float* part_KW = part_KH + (size_t)F * g.R;

  for (int i = tid; i < F * RP; i += nt) {
    const int r = i % RP, f = i / RP;
    KHs[i] = r < g.R ? __ldg(KH + (size_t)f * g.Rs + g.r0 + r) : 0.f;
    KWs[i] = r < g.R ? __ldg(KW + (size_t)f * g.Rs + g.r0 + r) : 0.f;
  }
  for (int p = tid; p < g.OPX; p += nt) {
    const int oy = p / g.TW, ox = p - oy * g.TW;
    const int gy = h0 + oy, gx = w0 + ox;
    pixoff[p] = (gy < g.H && gx < g.W) ? gy * g.W + gx : -1;
  }
#ifdef B200CP_TRACE
  float* trace = (blockIdx.x == gridDim.x / 2 && tid == 0) ? partial + (size_t)gridDim.x * gf.nparam : nullptr;
  const long long tr0 = clock64();
#define TRACE(i) do { if (trace) trace[i] = (float)(clock64() - tr0); } while (0)
#else
#define TRACE(i) do {} while (0)
#endif
  TRACE(0);
  contract_tile<RP, PPT>(g, Xn, g.Cin, K1, Fs, Xst, Ps, h0, w0, tid, nt);
  TRACE(1);
  contract_tile<RP, PPT>(g, dUn, g.Cout, K0, Fs, Xst, Qs, h0, w0, tid, nt);
  __syncthreads();
  TRACE(2);

  // per-rank stencils and the small-factor gradients
  const int p = g.pad;
  if (EXACT && FMAX == 3) {
    stencil_phase_3x3<RP>(gf, Ps, Qs, Zs, Qts, KHs, KWs, pixoff, red, part_KH, part_KW, tid, nt);
  } else
  for (int r = 0; r < g.R; ++r) {
    float kh[FMAX], kw[FMAX], aH[FMAX], aW[FMAX];
#pragma unroll
    for (int i = 0; i < FMAX; ++i) {
      const bool on = EXACT || i < F;
      kh[i] = on ? KHs[i * RP + r] : 0.f;
      kw[i] = on ? KWs[i * RP + r] : 0.f;
      aH[i] = 0.f;
      aW[i] = 0.f;
    }
    const float* Pr = Ps + r * g.HPXs;
    const float* Qr = Qs + r * g.HPXs;
    for (int op = tid; op < g.OPX; op += nt) {
      const int oy = op / g.TW, ox = op - oy * g.TW;
      float zv = 0.f, qt = 0.f;
      if (pixoff[op] >= 0) {
        // window origin (tap 0,0) in halo coordinates; mH == mW == pad here
        const float* pw = Pr + oy * g.TWh + ox;
        const float* qw = Qr + oy * g.TWh + ox;
        const float q = qw[p * g.TWh + p];
        float cols[FMAX];
#pragma unroll
        for (int j = 0; j < FMAX; ++j) cols[j] = 0.f;
#pragma unroll
        for (int i = 0; i < FMAX; ++i) {
          if (EXACT || i < F) {
            float row = 0.f, qrow = 0.f;
#pragma unroll
            for (int j = 0; j < FMAX; ++j) {
              if (EXACT || j < F) {
                const float pv = pw[i * g.TWh + j];
                row = fmaf(kw[j], pv, row);
                cols[j] = fmaf(kh[i], pv, cols[j]);
                // flipped window: Q[h - i + p][w - j + p]  -> halo (oy + 2p - i, ox + 2p - j)
                qrow = fmaf(kw[j], qw[(2 * p - i) * g.TWh + (2 * p - j)], qrow);
              }
            }
            zv = fmaf(kh[i], row, zv);
            qt = fmaf(kh[i], qrow, qt);
            aH[i] = fmaf(q, row, aH[i]);
          }
        }
#pragma unroll
        for (int j = 0; j < FMAX; ++j) aW[j] = fmaf(q, cols[j], aW[j]);
      }
      Zs[r * gf.OPXs + op] = zv;
      Qts[r * gf.OPXs + op] = qt;
    }
    // block reduction of aH, aW in a fixed order: lanes (shuffle tree), then warps
#pragma unroll
    for (int i = 0; i < FMAX; ++i) {
      if (EXACT || i < F) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
          aH[i] += __shfl_xor_sync(0xffffffffu, aH[i], off);
          aW[i] += __shfl_xor_sync(0xffffffffu, aW[i], off);
        }
      }
    }
    __syncthreads();  // previous rank's `red` fully consumed
    if (lane == 0) {
#pragma unroll
      for (int i = 0; i < FMAX; ++i)
        if (EXACT || i < F) {
          red[warp * 2 * F + i] = aH[i];
          red[warp * 2 * F + F + i] = aW[i];
        }
    }
    __syncthreads();
    if (tid < 2 * F) {
      float sum = 0.f;
      for (int w = 0; w < nwarp; ++w) sum += red[w * 2 * F + tid];
      if (tid < F) part_KH[(size_t)tid * g.R + r] = sum;
      else part_KW[(size_t)(tid - F) * g.R + r] = sum;
    }
  }
  __syncthreads();

  TRACE(3);
  constexpr int CG = (RP >= 64) ? 1 : (RP == 32 ? 2 : 4);
  pixel_reduce<RP, CG>(g, gf.OPXs, dUn, g.Cout, Zs, pixoff, part_K0, tid, nt);
  TRACE(4);
  pixel_reduce<RP, CG>(g, gf.OPXs, Xn, g.Cin, Qts, pixoff, part_K1, tid, nt);
  TRACE(5);
}

// The two parts of one warp's exchange (`seq` is the exchange's sequence number, its parity the slot).
__device__ __forceinline__ void exchange_post(const ExchangeArgs& ex, bool live, int j, float v, unsigned seq) {
  const int slot = (int)(seq & 1u);
  if (live)
    for (int p = 0; p < ex.world; ++p) exchange_store(ex.data[p] + ((size_t)slot * ex.world + ex.rank) * ex.row + j, v, seq);
}
// the sum over the ranks of entry j, in rank order (the same bits on every rank); NaN for the whole warp when a
// rank's word did not arrive within the limit
__device__ __forceinline__ float exchange_gather(const ExchangeArgs& ex, bool live, int j, unsigned seq) {
  const int slot = (int)(seq & 1u);
  bool missed = false;
  float t = 0.f;
  if (live) {
    const unsigned long long* own = ex.data[ex.rank] + (size_t)slot * ex.world * ex.row + j;
    const long long t0 = clock64();
    for (int p = 0; p < ex.world && !missed; ++p) {
      float v;
      while (!exchange_load(own + (size_t)p * ex.row, seq, &v)) {
        if (clock64() - t0 > ex.wait_cycles) {   // give up, never hang
          missed = true;
          atomicExch(ex.status, 1 + ex.rank);
          break;
        }
        __nanosleep(20);
      }
      t += v;
    }
  }
  missed = __any_sync(0xffffffffu, missed);
  return missed ? __int_as_float(0x7fc00000) : t;
}

// out[j] = sum over CTAs of partial[cta][j].  32 parameters x 32 slices per block: slice s adds the
// partials of its contiguous CTA range in order, then the slices are added in order (reproducible).
// EXCHANGE: the sums then go through the peer-memory exchange of a data-parallel step in the same kernel -- the first
// warp of every CTA stores its 32 sums, each with the sequence number in one 8-byte word, into every rank's region,
// reads all ranks' words of the same entries from its own region (spinning, bounded, until they carry the sequence
// number; a wait that runs out gives NaN and a status word) and adds them in rank order, so every rank gets the
// same bits.
// In pipelined mode (ex.mode == 1) the kernel only posts its sums and completes the *previous* step's exchange, whose
// flags have long arrived: the exchange latency then costs the step nothing.
template <bool EXCHANGE>
__global__ void __launch_bounds__(1024) cp4_reduce_partials_kernel(const float* __restrict__ partial, int nparts_high,
                                                                   int nparam, int R, int Rs, int r0,
                                                                   float* __restrict__ dK, const ExchangeArgs ex,
                                                                   int split, int nparts_low) {
  __shared__ float red[32][33];
  grid_dependency_wait();   // the partials are the previous kernel's output
  const int j = blockIdx.x * 32 + threadIdx.x, sl = threadIdx.y;
  const int nparts = j < split ? nparts_low : nparts_high;   // entries below `split` come from fewer CTAs
  const int per = (nparts + 31) / 32;
  const int i0 = sl * per, i1 = min(nparts, i0 + per);
  float s0 = 0.f;
  if (j < nparam) {
    // eight loads in flight, then added in index order
    for (int i = i0; i < i1; i += 8) {
      float v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) v[u] = i + u < i1 ? __ldg(partial + (size_t)(i + u) * nparam + j) : 0.f;
#pragma unroll
      for (int u = 0; u < 8; ++u) s0 += v[u];
    }
  }
  red[sl][threadIdx.x] = s0;
  __syncthreads();
  if (sl != 0) return;
  float s = 0.f;
#pragma unroll
  for (int k = 0; k < 32; ++k) s += red[k][threadIdx.x];
  // the packed output has the same T, C, F, F row sections, with rows of length Rs
  const int row = j / R, r = j - row * R;
  float* out = dK + (size_t)row * Rs + r0 + r;
  if (!EXCHANGE) {
    if (j < nparam) *out = s;
    return;
  }
  // ---- exchange (one warp; lane = entry of the CTA's 32) -----------------------------------------------------------
  const int lane = threadIdx.x, cta = blockIdx.x;
  const bool live = j < nparam;
  const unsigned last = ex.seqs[cta];
  if (ex.mode == 1 && ex.prev_out != nullptr) {
    // pipelined: the previous step's exchange is completed here, a whole step after it was posted
    const float t = exchange_gather(ex, live, j, last);
    if (live) ex.prev_out[(size_t)row * Rs + r0 + r] = t;
  }
  const unsigned seq = last + 1;
  exchange_post(ex, live, j, s, seq);
  if (ex.mode == 0) {
    const float t = exchange_gather(ex, live, j, seq);
    if (live) *out = t;
  }
  __syncwarp();
  if (lane == 0) ex.seqs[cta] = seq;   // the sequence advances either way: the next exchange lines up with the peers' again
}

// Completes the last posted exchange of a pipelined sequence: one warp per 32 entries.
__global__ void __launch_bounds__(32) exchange_finish_kernel(const ExchangeArgs ex, int nparam, int R, int Rs, int r0,
                                                             float* __restrict__ dK) {
  grid_dependency_wait();
  const int lane = threadIdx.x, cta = blockIdx.x, j = cta * 32 + lane;
  const float t = exchange_gather(ex, j < nparam, j, ex.seqs[cta]);
  if (j < nparam) {
    const int row = j / R, r = j - row * R;
    dK[(size_t)row * Rs + r0 + r] = t;
  }
}

TileChoice bwdf_tile(int N, int H, int W, int F, int pad, int C, int T, int RP, const DeviceInfo& di) {
  // halo pass over C + T channels, reductions over C + T channels (about 1.6x a contraction each), stencils
  const double w1 = (double)(C + T) * RP, w3 = 1.6 * (C + T) * RP + 6.0 * F * F * RP;
  return choose_tile(N, H, W, F, F, pad, w1, w3, RP, factor_cap(std::max(C, T), RP), 2, 2, 2 * F * RP + kRedFloats, 1, true,
                     di);
}

template <int RP, int PPT, int FMAX, bool EXACT>
int launch_bwd_filter(const Cp4BwdFilterArgs& a, const TileChoice& t, const DeviceInfo& di, cudaStream_t st) {
  const int F = a.F;
  Cp4Args ca{};
  ca.N = a.N; ca.Cin = a.C; ca.Cout = a.T; ca.H = a.H; ca.W = a.W; ca.Y = F; ca.X = F; ca.pad = a.pad;
  ca.R = a.R; ca.Rs = a.Rs; ca.r0 = a.r0;
  GeomF gf;
  gf.g = make_geom(ca, t, RP, factor_cap(std::max(a.C, a.T), RP));
  gf.F = F;
  gf.nparam = (a.T + a.C + 2 * F) * a.R;
  gf.OPXs = (int)align_up(gf.g.OPX, 4);
  const size_t smem = sizeof(float) * ((size_t)gf.g.fcap + 2 * F * RP + kRedFloats + 2 * (size_t)RP * gf.g.HPXs +
                                       2 * (size_t)RP * gf.OPXs + gf.OPXs + (size_t)kStages * kKC * t.NT * PPT);
  if ((int)smem > di.smem_optin) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: tile exceeds shared memory");
  const long ctas = (long)a.N * gf.g.tilesH * gf.g.tilesW;
  const size_t need = (size_t)ctas * gf.nparam * sizeof(float);
  if (a.ws == nullptr || a.ws_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "cp4 bwd-filter: workspace of %zu bytes needed, %zu given", need, a.ws_bytes);
  auto kern = cp4_bwd_filter_kernel<RP, PPT, FMAX, EXACT>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
  kern<<<(unsigned)ctas, t.NT, smem, st>>>(gf, a.X, a.dU, a.K0, a.K1, a.KH, a.KW, (float*)a.ws);
  B200CP_LAUNCH_OK("cp4_bwd_filter_kernel");
  cp4_reduce_partials_kernel<false><<<ceil_div(gf.nparam, 32), dim3(32, 32), 0, st>>>((const float*)a.ws, (int)ctas,
                                                                                   gf.nparam, a.R, a.Rs, a.r0, a.dK,
                                                                                   ExchangeArgs{}, 0, 0);
  B200CP_LAUNCH_OK("cp4_reduce_partials_kernel");
  return B200CP_OK;
}

template <int RP, int FMAX, bool EXACT>
int dispatch_bwd_filter_ppt(const Cp4BwdFilterArgs& a, const DeviceInfo& di, cudaStream_t st) {
  const TileChoice t = bwdf_tile(a.N, a.H, a.W, a.F, a.pad, a.C, a.T, RP, di);
  if (t.NT == 0) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: no tile fits in shared memory");
  switch (t.PPT1) {
    case 1: return launch_bwd_filter<RP, 1, FMAX, EXACT>(a, t, di, st);
    case 2: if constexpr (RP <= 32) return launch_bwd_filter<RP, 2, FMAX, EXACT>(a, t, di, st); break;
    case 3: if constexpr (RP <= 16) return launch_bwd_filter<RP, 3, FMAX, EXACT>(a, t, di, st); break;
    case 4: if constexpr (RP <= 16) return launch_bwd_filter<RP, 4, FMAX, EXACT>(a, t, di, st); break;
  }
  return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: internal: no kernel for PPT %d at rank tile %d", t.PPT1, RP);
}

template <int FMAX, bool EXACT>
int dispatch_bwd_filter_rank(const Cp4BwdFilterArgs& a, const DeviceInfo& di, cudaStream_t st) {
  switch (padded_rank(a.R)) {
    case 4: return dispatch_bwd_filter_ppt<4, FMAX, EXACT>(a, di, st);
    case 8: return dispatch_bwd_filter_ppt<8, FMAX, EXACT>(a, di, st);
    case 16: return dispatch_bwd_filter_ppt<16, FMAX, EXACT>(a, di, st);
    case 32: return dispatch_bwd_filter_ppt<32, FMAX, EXACT>(a, di, st);
    default: return dispatch_bwd_filter_ppt<64, FMAX, EXACT>(a, di, st);
  }
}

}  // namespace

int cp4_reduce_partials_launch(const float* partial, int nparts, int nparam, int R, int Rs, int r0, float* dK,
                               cudaStream_t st, bool after_own_kernel, const ExchangeArgs* exchange, int split,
                               int nparts_low) {
  if (exchange != nullptr) {
    if (ceil_div(nparam, 32) > exchange->ctas)
      return fail(B200CP_ERR_INVALID_ARG, "fused exchange: %d gradient entries, the context has flags for %d", nparam,
                  exchange->ctas * 32);
    B200CP_CUDA_OK(launch_kernel(cp4_reduce_partials_kernel<true>, dim3(ceil_div(nparam, 32)), dim3(32, 32), 0, st,
                                 after_own_kernel, partial, nparts, nparam, R, Rs, r0, dK, *exchange, split, nparts_low));
  } else {
    B200CP_CUDA_OK(launch_kernel(cp4_reduce_partials_kernel<false>, dim3(ceil_div(nparam, 32)), dim3(32, 32), 0, st,
                                 after_own_kernel, partial, nparts, nparam, R, Rs, r0, dK, ExchangeArgs{}, split, nparts_low));
  }
  B200CP_LAUNCH_OK("cp4_reduce_partials_kernel");
  return B200CP_OK;
}

int exchange_finish_launch(const ExchangeArgs& ex, int nparam, int R, int Rs, int r0, float* dK, cudaStream_t st) {
  B200CP_CUDA_OK(launch_kernel(exchange_finish_kernel, dim3(ceil_div(nparam, 32)), dim3(32), 0, st, true, ex, nparam, R, Rs, r0, dK));
  B200CP_LAUNCH_OK("exchange_finish_kernel");
  return B200CP_OK;
}

// One partial gradient set per CTA.  With a device present the tile the launch will pick is
// known exactly; without one (argument checks on a CPU-only host) an upper bound is returned.
size_t cp4_bwd_filter_simt_workspace(const b200cp_tensor_shape& s) {
  const size_t R = std::min<unsigned>(s.Rank, 64);
  const size_t nparam = ((size_t)s.T + s.C + 2 * s.Y) * R;
  DeviceInfo di;
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) == cudaSuccess && dev_count > 0 && device_info(&di) == B200CP_OK) {
    // ranks are processed in chunks of 64; the last chunk may use a narrower rank tile (and another spatial tile)
    size_t need = 0;
    for (unsigned r0 = 0; r0 < s.Rank; r0 += 64) {
      const int rc = (int)std::min(64u, s.Rank - r0);
      const TileChoice t = bwdf_tile(s.N, s.H, s.W, s.Y, s.pad, s.C, s.T, padded_rank(rc), di);
      if (!t.NT) { need = 0; break; }
      need = std::max(need, (size_t)s.N * ceil_div(s.H, t.TH) * ceil_div(s.W, t.TW) *
                                ((size_t)s.T + s.C + 2 * s.Y) * rc * sizeof(float));
    }
    if (need) return need;
  }
  cudaGetLastError();
  const size_t max_ctas = (size_t)s.N * s.H * ceil_div((int)s.W, 16);
  return max_ctas * nparam * sizeof(float);
}

int cp4_bwd_filter_simt_launch(const Cp4BwdFilterArgs& a, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  if (a.F == 3) return dispatch_bwd_filter_rank<3, true>(a, di, st);
  if (a.F >= 1 && a.F <= 11 && (a.F & 1)) return dispatch_bwd_filter_rank<11, false>(a, di, st);
  return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: filter size %d is not odd and <= 11", a.F);
}

// ===========================================================================
// backward-filter without any allocation: the per-CTA partial gradients go to a fixed array that
// lives in the library's device image instead of a caller-provided workspace.
// ===========================================================================
namespace {
constexpr size_t kStaticScratchBytes = size_t(8) << 20;  // 8 MiB per device that loads the library
}
static __device__ __align__(256) float g_bwdf_static_scratch[kStaticScratchBytes / sizeof(float)];

size_t cp4_bwd_filter_static_scratch_bytes() { return kStaticScratchBytes; }

// In host code `g_bwdf_static_scratch` is only a handle of the symbol, not a device address; the address on
// the current device comes from cudaGetSymbolAddress, once per device (kept in a small table).
int cp4_bwd_filter_static_launch(const Cp4BwdFilterArgs& a_in, cudaStream_t st) {
  static std::mutex mu;
  static float* table[64] = {nullptr};
  int dev = 0;
  B200CP_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200CP_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
  float* ptr = nullptr;
  {
    std::lock_guard<std::mutex> lk(mu);
    if (!table[dev]) {
      void* p = nullptr;
      B200CP_CUDA_OK(cudaGetSymbolAddress(&p, g_bwdf_static_scratch));
      table[dev] = static_cast<float*>(p);
    }
    ptr = table[dev];
  }
  Cp4BwdFilterArgs a = a_in;
  a.ws = ptr;
  a.ws_bytes = kStaticScratchBytes;
  return cp4_bwd_filter_simt_launch(a, st);
}

// ===========================================================================
// dense filter gradient and recomposition (helpers of the reference's tests)
// ===========================================================================
namespace {

// dK[t,c,y,x] = sum_{n,h,w} dU[n,t,h,w] X[n,c,h+y-pad,w+x-pad]; one CTA per (t,c), fixed-order sum.
__global__ void cp4_bwd_filter_full_kernel(b200cp_tensor_shape s, const float* __restrict__ X,
                                           const float* __restrict__ dU, float* __restrict__ dK) {
  const int t = blockIdx.x / s.C, c = blockIdx.x % s.C;
  const int HW = s.H * s.W;
  __shared__ float red[8];
  for (unsigned yx = 0; yx < s.Y * s.X; ++yx) {
    const int y = yx / s.X, x = yx % s.X;
    float acc = 0.f;
    for (unsigned n = 0; n < s.N; ++n) {
      const float* du = dU + ((size_t)n * s.T + t) * HW;
      const float* xi = X + ((size_t)n * s.C + c) * HW;
      for (int p = threadIdx.x; p < HW; p += blockDim.x) {
        const int h = p / s.W, w = p % s.W;
        const int hh = h + y - (int)s.pad, ww = w + x - (int)s.pad;
        if (hh >= 0 && hh < (int)s.H && ww >= 0 && ww < (int)s.W) acc = fmaf(du[p], xi[hh * s.W + ww], acc);
      }
    }
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
      float sum = 0.f;
      for (unsigned w = 0; w < blockDim.x / 32; ++w) sum += red[w];
      dK[((size_t)(t * s.C + c) * s.Y + y) * s.X + x] = sum;
    }
  }
}

__global__ void cp4_recompose_kernel(b200cp_tensor_shape s, const float* __restrict__ K0,
                                     const float* __restrict__ K1, const float* __restrict__ KH,
                                     const float* __restrict__ KW, float* __restrict__ K) {
  const size_t total = (size_t)s.T * s.C * s.Y * s.X;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.x * blockDim.x) {
    const unsigned x = i % s.X, y = (i / s.X) % s.Y, c = (i / (s.X * s.Y)) % s.C, t = i / ((size_t)s.X * s.Y * s.C);
    float acc = 0.f;
    for (unsigned r = 0; r < s.Rank; ++r)
      acc += K0[t * s.Rank + r] * K1[c * s.Rank + r] * KH[y * s.Rank + r] * KW[x * s.Rank + r];
    K[i] = acc;
  }
}

}  // namespace

int cp4_bwd_filter_full_launch(const b200cp_tensor_shape& s, const float* X, const float* dU, float* dK,
                               cudaStream_t st) {
  cp4_bwd_filter_full_kernel<<<s.T * s.C, 256, 0, st>>>(s, X, dU, dK);
  B200CP_LAUNCH_OK("cp4_bwd_filter_full_kernel");
  return B200CP_OK;
}

int cp4_recompose_launch(const b200cp_tensor_shape& s, const float* K0, const float* K1, const float* KH,
                         const float* KW, float* K, cudaStream_t st) {
  const size_t total = (size_t)s.T * s.C * s.Y * s.X;
  const unsigned blocks = (unsigned)std::min<size_t>((total + 255) / 256, 4096);
  cp4_recompose_kernel<<<blocks, 256, 0, st>>>(s, K0, K1, KH, KW, K);
  B200CP_LAUNCH_OK("cp4_recompose_kernel");
  return B200CP_OK;
}

// ---- AllClose (Cuda_kernels/Utils.cu:143-180) --------------------------------------------------------------
// Number of elements whose relative difference max(|a-b|/|a|, |a-b|/|b|) (the absolute difference where a or b is
// zero) exceeds `tol`: a grid-stride loop, a warp and block sum, one atomic per block.
namespace {
__global__ void __launch_bounds__(256) relative_delta_count_kernel(const float* __restrict__ A, const float* __restrict__ B,
                                                                   size_t n, float tol, unsigned long long* count) {
  unsigned mine = 0;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    const float a = A[i], b = B[i], d = fabsf(a - b);
    const float err = (a == 0.f || b == 0.f) ? d : fmaxf(d / fabsf(a), d / fabsf(b));
    mine += !(err <= tol);   // a NaN difference counts as exceeding
  }
  __shared__ unsigned warp_sum[8];
  for (int o = 16; o; o >>= 1) mine += __shfl_down_sync(0xffffffffu, mine, o);
  if ((threadIdx.x & 31) == 0) warp_sum[threadIdx.x >> 5] = mine;
  __syncthreads();
  if (threadIdx.x == 0) {
    unsigned s = 0;
    for (int w = 0; w < 8; ++w) s += warp_sum[w];
    if (s) atomicAdd(count, (unsigned long long)s);
  }
}
}  // namespace

int allclose_count_launch(const float* A, const float* B, size_t n, float tol, unsigned long long* count_dev,
                          cudaStream_t st) {
  B200CP_CUDA_OK(cudaMemsetAsync(count_dev, 0, sizeof(unsigned long long), st));
  if (n == 0) return B200CP_OK;
  const unsigned blocks = (unsigned)std::min<size_t>((n + 255) / 256, 148 * 8);
  relative_delta_count_kernel<<<blocks, 256, 0, st>>>(A, B, n, tol, count_dev);
  B200CP_LAUNCH_OK("relative_delta_count_kernel");
  return B200CP_OK;
}

}  // namespace b200cp
