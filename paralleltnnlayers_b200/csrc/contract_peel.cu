// Factor gradients of the reshaped-CP conv and the CP dense layer from the dense gradient G.
//
// Index modes: the m factor modes with pair index p_j = c_j * t_dim_j + t_j (the factor's own [c][t] layout, vector
// vec_j[p_j][r] = A_j[c_j][t_j][r]) and, for the conv, the tap mode with vector S[tap][r].  For every mode q
//   d vec_q[p_q][r] = sum_{rest} G[p_q, rest] * prod_{j != q} vec_j[p_j(rest)][r].
// Done mode by mode this reads G once per mode and multiplies every element by every other factor each time.
// Instead the modes are peeled off one at a time from the inside.  With the mode list u_0 .. u_{L-1} and
//   S_L = G,   S_k[p_{u_0} .. p_{u_{k-1}}][r] = sum_{p_{u_k}} S_{k+1}[.., p_{u_k}][r] * vec_{u_k}[p_{u_k}][r],
// the gradient of mode u_k needs only S_{k+1} and the running product of the outer vectors:
//   d vec_{u_k}[p][r] = sum_{rows} S_{k+1}[row, p][r] * prod_{j < k} vec_{u_j}[p_{u_j}(row)][r].
// The first peel (over G itself, which has no rank index) is the only heavy step: 2 * |G| * R multiply-adds, G read
// once.  Every later level works on a tensor smaller by the size of the peeled mode.
//
// Sums over rows are accumulated per CTA in registers over a fixed, strided set of row batches and written as
// partial blocks that a second kernel adds in CTA order, so the result does not depend on scheduling.
#include <algorithm>

#include "common.cuh"

namespace b200cp {

namespace {

constexpr int kPT = 256;      // threads per CTA: lane = rank within a block of 32, warp = row / entry group
constexpr int kRB = 32;       // ranks per CTA
constexpr int kRows0 = 64;    // rows of G per batch in the first peel
constexpr int kMaxNb = 256;   // entries of one mode (c_dim * t_dim)
constexpr int kGridCap = 592; // CTAs per level (fixed: the order of the partial sums must not depend on the device)

struct PeelMode {
  int nc, nt;      // p = c * nt + t
  long gc, gt;     // G offset per c and per t (first peel only)
  const float* vec;  // [nc * nt][R]
};

struct PeelGeom {
  int R, nouter, nb, nbp;  // nbp: nb padded to the kernel's entry count
  long rows;               // product of the outer mode sizes
  PeelMode outer[4];       // in list order; the peeled mode is the innermost index of the source
  PeelMode b;
  const float* src;        // G (first peel) or S_{k+1}[rows][nb][R]
  float* next;             // S_k[rows][R] (null when there is no outer mode)
  float* part;             // [gridDim.x][nb][R] partial gradients of the peeled mode
};

// ---- first peel: the source is G, without a rank index -------------------------------------------------------------
// Rows are enumerated with the t digits of the outer modes slow and their c digits fast, so that consecutive rows
// are neighbours in G and a batch is read with full sectors.
template <int NPW>  // entries of the peeled mode per warp: nbp = 8 * NPW
__global__ void __launch_bounds__(kPT) peel_first_kernel(const PeelGeom g) {
  extern __shared__ __align__(16) float smem_f[];
  const int nbp = 8 * NPW;
  float* Gs = smem_f;                       // [kRows0][nbp]
  float* Vs = Gs + kRows0 * nbp;            // [nbp][kRB]
  float* Ls = Vs + nbp * kRB;               // [kRows0][kRB]
  int* goff = reinterpret_cast<int*>(Ls + kRows0 * kRB);  // [kRows0] G offset of the row, -1 past the end
  int* orow = goff + kRows0;                // [kRows0] row index in the layout of `next`
  int* pjs = orow + kRows0;                 // [kRows0][4] entry index of each outer mode
  int* slab = pjs + kRows0 * 4;             // [kRows0 * nc] (row << 16) | c for the load order of one t slab

  const int tid = threadIdx.x, lane = tid & 31, wg = tid >> 5;
  const int r = blockIdx.y * kRB + lane;
  const bool rok = r < g.R;

  for (int i = tid; i < nbp * kRB; i += kPT) {
    const int p = i / kRB, rr = blockIdx.y * kRB + (i - p * kRB);
    Vs[i] = (p < g.nb && rr < g.R) ? __ldg(g.b.vec + (size_t)p * g.R + rr) : 0.f;
  }
  // load order within one t slab of the peeled mode: row slow, c fast (c is the contiguous index of G)
  for (int i = tid; i < kRows0 * g.b.nc; i += kPT) {
    const int row = i / g.b.nc;
    slab[i] = (row << 16) | (i - row * g.b.nc);
  }
  float acc2[NPW];
#pragma unroll
  for (int i = 0; i < NPW; ++i) acc2[i] = 0.f;

  // entries past nb stay zero for the whole kernel
  if (g.nb < nbp)
    for (int i = tid; i < kRows0 * (nbp - g.nb); i += kPT) {
      const int row = i / (nbp - g.nb), e = g.nb + i - row * (nbp - g.nb);
      Gs[row * nbp + e] = 0.f;
    }
  const int rows = (int)g.rows;  // the host checks that rows and the G offsets fit 31 bits
  const int batches = (rows + kRows0 - 1) / kRows0;
  for (int bt = blockIdx.x; bt < batches; bt += gridDim.x) {
    __syncthreads();  // the previous batch has been consumed (and, the first time, Vs / slab are written)
    if (tid < kRows0) {
      int idx = bt * kRows0 + tid, go = -1, orw = 0;
      int pj[4] = {0, 0, 0, 0};
      if (idx < rows) {
        go = 0;
#pragma unroll
        for (int j = 3; j >= 0; --j) {  // c digits, fastest first
          if (j < g.nouter) {
            const int v = idx % g.outer[j].nc;
            idx /= g.outer[j].nc;
            go += v * (int)g.outer[j].gc;
            pj[j] = v * g.outer[j].nt;
          }
        }
#pragma unroll
        for (int j = 3; j >= 0; --j) {  // t digits
          if (j < g.nouter) {
            const int v = idx % g.outer[j].nt;
            idx /= g.outer[j].nt;
            go += v * (int)g.outer[j].gt;
            pj[j] += v;
          }
        }
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < g.nouter) orw = orw * (g.outer[j].nc * g.outer[j].nt) + pj[j];
      }
      goff[tid] = go;
      orow[tid] = orw;
#pragma unroll
      for (int j = 0; j < 4; ++j) pjs[tid * 4 + j] = pj[j];
    }
    __syncthreads();
    // product of the outer vectors per row
    for (int i = tid; i < kRows0 * kRB; i += kPT) {
      const int row = i / kRB;
      float w = 0.f;
      if (goff[row] >= 0 && rok) {
        w = 1.f;
#pragma unroll
        for (int j = 0; j < 4; ++j)
          if (j < g.nouter) w *= __ldg(g.outer[j].vec + (size_t)pjs[row * 4 + j] * g.R + r);
      }
      Ls[i] = w;
    }
    // the batch of G, one t slab of the peeled mode at a time: [row][c], c fastest
    {
      const int nc = g.b.nc, nt = g.b.nt, per_t = kRows0 * nc;
      const int gc = (int)g.b.gc, gt = (int)g.b.gt;
      for (int t = 0; t < nt; ++t)
        for (int i = tid; i < per_t; i += kPT) {
          const int rc = slab[i], row = rc >> 16, c = rc & 0xffff;
          const int go = goff[row];
          Gs[row * nbp + c * nt + t] = go >= 0 ? __ldg(g.src + go + t * gt + c * gc) : 0.f;
        }
    }
    __syncthreads();
    // next[row][r] = sum_p G[row][p] * vec_b[p][r]: each warp takes kRows0 / 8 rows
    if (g.next != nullptr) {
      float acc1[kRows0 / 8];
#pragma unroll
      for (int i = 0; i < kRows0 / 8; ++i) acc1[i] = 0.f;
      for (int p4 = 0; p4 < nbp; p4 += 4) {
        const float v0 = Vs[(p4 + 0) * kRB + lane], v1 = Vs[(p4 + 1) * kRB + lane];
        const float v2 = Vs[(p4 + 2) * kRB + lane], v3 = Vs[(p4 + 3) * kRB + lane];
#pragma unroll
        for (int i = 0; i < kRows0 / 8; ++i) {
          const float4 gq = *reinterpret_cast<const float4*>(Gs + (wg * (kRows0 / 8) + i) * nbp + p4);
          acc1[i] = fmaf(gq.x, v0, acc1[i]);
          acc1[i] = fmaf(gq.y, v1, acc1[i]);
          acc1[i] = fmaf(gq.z, v2, acc1[i]);
          acc1[i] = fmaf(gq.w, v3, acc1[i]);
        }
      }
      if (rok) {
#pragma unroll
        for (int i = 0; i < kRows0 / 8; ++i) {
          const int row = wg * (kRows0 / 8) + i;
          if (goff[row] >= 0) g.next[(size_t)orow[row] * g.R + r] = acc1[i];
        }
      }
    }
    // d vec_b[p][r] += sum_rows G[row][p] * L[row][r]: each warp takes NPW entries
#pragma unroll 4
    for (int row = 0; row < kRows0; ++row) {
      const float l = Ls[row * kRB + lane];
#pragma unroll
      for (int i4 = 0; i4 < NPW / 4; ++i4) {
        const float4 gq = *reinterpret_cast<const float4*>(Gs + row * nbp + wg * NPW + i4 * 4);
        acc2[i4 * 4 + 0] = fmaf(gq.x, l, acc2[i4 * 4 + 0]);
        acc2[i4 * 4 + 1] = fmaf(gq.y, l, acc2[i4 * 4 + 1]);
        acc2[i4 * 4 + 2] = fmaf(gq.z, l, acc2[i4 * 4 + 2]);
        acc2[i4 * 4 + 3] = fmaf(gq.w, l, acc2[i4 * 4 + 3]);
      }
    }
  }
  if (rok) {
    float* out = g.part + (size_t)blockIdx.x * g.nb * g.R;
#pragma unroll
    for (int i = 0; i < NPW; ++i) {
      const int p = wg * NPW + i;
      if (p < g.nb) out[(size_t)p * g.R + r] = acc2[i];
    }
  }
}

// ---- later peels: the source has a rank index, everything is element-wise in r ----------------------------------------
// src[row][p][r]; warp wg takes the entries p = wg, wg + 8, ...; one row at a time per CTA.
template <int NPW>
__global__ void __launch_bounds__(kPT) peel_rank_kernel(const PeelGeom g) {
  __shared__ float red[8][kRB];
  const int tid = threadIdx.x, lane = tid & 31, wg = tid >> 5;
  const int r = blockIdx.y * kRB + lane;
  const bool rok = r < g.R;
  float v[NPW], acc2[NPW];
#pragma unroll
  for (int i = 0; i < NPW; ++i) {
    const int p = wg + 8 * i;
    v[i] = (p < g.nb && rok) ? __ldg(g.b.vec + (size_t)p * g.R + r) : 0.f;
    acc2[i] = 0.f;
  }
  for (long row = blockIdx.x; row < g.rows; row += gridDim.x) {
    float l = 1.f;
    if (rok) {
      long o = row;
      for (int j = g.nouter - 1; j >= 0; --j) {
        const int n = g.outer[j].nc * g.outer[j].nt;
        const int pj = (int)(o % n);
        o /= n;
        l *= __ldg(g.outer[j].vec + (size_t)pj * g.R + r);
      }
    }
    const float* s = g.src + (size_t)row * g.nb * g.R + r;
    float a1 = 0.f;
#pragma unroll
    for (int i = 0; i < NPW; ++i) {
      const int p = wg + 8 * i;
      const float x = (p < g.nb && rok) ? __ldg(s + (size_t)p * g.R) : 0.f;
      a1 = fmaf(x, v[i], a1);
      acc2[i] = fmaf(x, l, acc2[i]);
    }
    if (g.next != nullptr) {
      red[wg][lane] = a1;
      __syncthreads();
      if (wg == 0 && rok) {
        float t = red[0][lane];
#pragma unroll
        for (int w = 1; w < 8; ++w) t += red[w][lane];
        g.next[(size_t)row * g.R + r] = t;
      }
      __syncthreads();
    }
  }
  if (rok) {
    float* out = g.part + (size_t)blockIdx.x * g.nb * g.R;
#pragma unroll
    for (int i = 0; i < NPW; ++i) {
      const int p = wg + 8 * i;
      if (p < g.nb) out[(size_t)p * g.R + r] = acc2[i];
    }
  }
}

// dst[e] = sum over CTAs of part[cta][e]: 32 elements per block, eight interleaved slices of the CTA range summed
// side by side and then added in slice order (a fixed association, whatever the schedule)
__global__ void __launch_bounds__(256) peel_sum_kernel(const float* __restrict__ part, float* __restrict__ dst, int n,
                                                       int ctas) {
  __shared__ float red[8][32];
  const int lane = threadIdx.x & 31, sl = threadIdx.x >> 5;
  const int e = blockIdx.x * 32 + lane;
  float s = 0.f;
  if (e < n)
    for (int c = sl; c < ctas; c += 8) s += __ldg(part + (size_t)c * n + e);
  red[sl][lane] = s;
  __syncthreads();
  if (sl == 0 && e < n) {
    float t = red[0][lane];
#pragma unroll
    for (int w = 1; w < 8; ++w) t += red[w][lane];
    dst[e] = t;
  }
}

struct PeelPlan {
  int L;                 // modes in the list: [tap] + factor modes
  int nmode[5];          // entries per mode
  long rows[5];          // rows[k] = product of nmode[0 .. k-1]: outer size when mode k is peeled
  int grid[5];           // CTAs of the level that peels mode k
  size_t s_floats[2];    // the two ping-pong buffers of the S tensors
  size_t part_floats;    // the largest partial block
};

int entries_per_warp(int nb) { return nb <= 32 ? 4 : nb <= 64 ? 8 : nb <= 128 ? 16 : 32; }

void peel_plan(PeelPlan& pl, int order, const int* cdims, const int* tdims, int R, int taps, bool has_s) {
  pl.L = 0;
  if (has_s) pl.nmode[pl.L++] = taps;
  for (int k = 0; k < order; ++k) pl.nmode[pl.L++] = cdims[k] * tdims[k];
  long rows = 1;
  for (int k = 0; k < pl.L; ++k) { pl.rows[k] = rows; rows *= pl.nmode[k]; }
  pl.s_floats[0] = pl.s_floats[1] = 0;
  pl.part_floats = 0;
  for (int k = pl.L - 1; k >= 0; --k) {
    const bool first = k == pl.L - 1;
    const long units = first ? (pl.rows[k] + kRows0 - 1) / kRows0 : pl.rows[k];
    pl.grid[k] = (int)std::min<long>(kGridCap, std::max<long>(1, units));
    pl.part_floats = std::max(pl.part_floats, (size_t)pl.grid[k] * pl.nmode[k] * R);
    // S_k (written by the level that peels mode k, read by the level that peels mode k - 1); S_1 is the gradient of mode 0
    if (k >= 2) {
      size_t& slot = pl.s_floats[(pl.L - 1 - k) & 1];
      slot = std::max(slot, (size_t)pl.rows[k] * R);
    }
  }
}

}  // namespace

size_t contract_scratch_floats(int order, const int* cdims, const int* tdims, int R, int taps, bool has_s) {
  PeelPlan pl;
  peel_plan(pl, order, cdims, tdims, R, taps, has_s);
  return pl.s_floats[0] + pl.s_floats[1] + pl.part_floats + 8;
}

// G is [tap][T][C] with T = (t_0 .. t_{m-1}) and C = (c_0 .. c_{m-1}) row-major; A[k] is [c_k][t_k][R], S is [taps][R]
int contract_factors_launch(int order, const int* cdims, const int* tdims, int R, int taps, const float* const* A,
                            const float* S, const float* G, float* const* dA, float* dS, float* scratch,
                            cudaStream_t st) {
  if (S && !dS) return fail(B200CP_ERR_INVALID_ARG, "factor contraction: dS missing");
  if (!scratch) return fail(B200CP_ERR_WORKSPACE, "factor contraction: scratch missing");
  if (!S && taps != 1) return fail(B200CP_ERR_INVALID_ARG, "factor contraction: a tap mode needs its vector");
  PeelPlan pl;
  peel_plan(pl, order, cdims, tdims, R, taps, S != nullptr);
  long T = 1, C = 1;
  for (int k = 0; k < order; ++k) { T *= tdims[k]; C *= cdims[k]; }
  // the mode list with the G strides of each mode
  PeelMode modes[5];
  float* grads[5];
  int L = 0;
  if (S) {
    modes[L] = PeelMode{taps, 1, T * C, 0, S};
    grads[L++] = dS;
  }
  {
    long cs = 1, ts = 1;
    for (int k = order - 1; k >= 0; --k) {
      modes[(S ? 1 : 0) + k] = PeelMode{cdims[k], tdims[k], cs, ts * C, A[k]};
      grads[(S ? 1 : 0) + k] = dA[k];
      cs *= cdims[k];
      ts *= tdims[k];
    }
    L += order;
  }
  for (int k = 0; k < L; ++k)
    if (modes[k].nc * modes[k].nt > kMaxNb)
      return fail(B200CP_ERR_UNSUPPORTED, "factor contraction: a mode has %d > %d entries", modes[k].nc * modes[k].nt, kMaxNb);
  float* sbuf[2] = {scratch, scratch + ((pl.s_floats[0] + 3) & ~size_t(3))};
  float* part = sbuf[1] + ((pl.s_floats[1] + 3) & ~size_t(3));
  const float* src = G;
  for (int k = L - 1; k >= 0; --k) {
    const bool first = k == L - 1;
    PeelGeom g{};
    g.R = R; g.nouter = k; g.nb = modes[k].nc * modes[k].nt; g.rows = pl.rows[k];
    for (int j = 0; j < k; ++j) g.outer[j] = modes[j];
    g.b = modes[k];
    g.src = src;
    // the tensor left after this peel: the gradient of mode 0 itself when only that mode is left
    g.next = k == 0 ? nullptr : k == 1 ? grads[0] : sbuf[(L - 1 - k) & 1];
    g.part = part;
    const int npw = entries_per_warp(g.nb);
    g.nbp = 8 * npw;
    dim3 grid(pl.grid[k], ceil_div(R, kRB));
    // partial blocks are per (CTA, rank block): the rank blocks write disjoint columns of the same [nb][R] block
    if (first) {
      const size_t smem = sizeof(float) * ((size_t)kRows0 * g.nbp + (size_t)g.nbp * kRB + kRows0 * kRB) +
                          sizeof(int) * (6 * kRows0 + kRows0 * g.b.nc);
      if (g.rows > 0x7fffffffL / 2 || (long)taps * T * C > 0x7fffffffL)
        return fail(B200CP_ERR_UNSUPPORTED, "factor contraction: the dense gradient has too many entries");
#define LAUNCH_FIRST(N)                                                                                       \
  do {                                                                                                        \
    B200CP_CUDA_OK(cudaFuncSetAttribute(peel_first_kernel<N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
    peel_first_kernel<N><<<grid, kPT, smem, st>>>(g);                                                         \
  } while (0)
      if (npw == 4) LAUNCH_FIRST(4);
      else if (npw == 8) LAUNCH_FIRST(8);
      else if (npw == 16) LAUNCH_FIRST(16);
      else LAUNCH_FIRST(32);
#undef LAUNCH_FIRST
      B200CP_LAUNCH_OK("peel_first_kernel");
    } else {
      if (npw == 4) peel_rank_kernel<4><<<grid, kPT, 0, st>>>(g);
      else if (npw == 8) peel_rank_kernel<8><<<grid, kPT, 0, st>>>(g);
      else if (npw == 16) peel_rank_kernel<16><<<grid, kPT, 0, st>>>(g);
      else peel_rank_kernel<32><<<grid, kPT, 0, st>>>(g);
      B200CP_LAUNCH_OK("peel_rank_kernel");
    }
    if (k >= 1) {
      const int n = g.nb * R;
      peel_sum_kernel<<<ceil_div(n, 32), 256, 0, st>>>(part, grads[k], n, pl.grid[k]);
      B200CP_LAUNCH_OK("peel_sum_kernel");
    } else if (L == 1) {
      // a single mode: its gradient is the sum of the partial blocks as well
      const int n = g.nb * R;
      peel_sum_kernel<<<ceil_div(n, 32), 256, 0, st>>>(part, grads[0], n, pl.grid[0]);
      B200CP_LAUNCH_OK("peel_sum_kernel");
    }
    src = g.next;
    if (k == 1) break;  // the tensor left is the gradient of mode 0, already in place
  }
  return B200CP_OK;
}

}  // namespace b200cp
