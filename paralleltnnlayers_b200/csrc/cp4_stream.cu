// CP4 conv2d forward / backward-data as a row stream: one persistent CTA per SM walks a contiguous range of image
// rows, and three kinds of warps work on different rows at the same time, so that the loads of one row, the channel
// contraction of the next and the stencil + output contraction of a third overlap instead of following each other.
//
//   producer warp    one 4-D TMA box (W pixels, 1 row, all input channels, 1 image) per input row into a ring of
//                    stages; rows above / below the image are never loaded (their rank row is zero)
//   rank warps (A)   warp w owns the 8 pixels [8w, 8w+8) of every row:
//                    P[r, px] = sum_c Fin[c, r] in[c, px]   mma.sync m16n8k8, M = 16 ranks, N = 8 pixels, K = channels;
//                    A fragments (the factor, tf32 hi | lo planes [rank][channel]) by ldmatrix, B fragments two 4-byte
//                    shared loads per 8 channels from the stage (conflict-free: W = 8 or 24 modulo 32).  The rank row
//                    goes into a ring of rows in shared memory (and, optionally, to the saved rank plane).
//   output warps (B) warp w owns the same 8 pixels of every output row: the 3x3 stencil over three ring rows is
//                    computed directly in the B-fragment layout of the next product (lane (g, t) holds ranks
//                    t, t+4, t+8, t+12 of pixel g), then out[ch, px] = sum_r Fout[ch, r] Z[r, px]  (M = 16 channels per
//                    mma, K = ranks), and the D fragments are stored as 8-byte words: a quarter warp writes 32
//                    contiguous bytes of one channel row.
//
// Every product is hi*hi + lo*hi + hi*lo (fp32-grade).  Forward: Fin = K1, Fout = K0; backward-data swaps them and
// flips the taps (Cuda_kernels/cp4Conv2dForward.cu:84-133, cp4Conv2dBackwardData.cu:57-108).  A convolution given no
// output only writes its rank plane P (what the stand-alone backward-filter needs of it): the producer then loads
// its own rows only and the output warps skip it.  One launch can carry
// two convolutions (the forward and the backward-data of a training step): their rows form one list that is cut into
// equal ranges.  A range that starts inside an image recomputes the rank rows of its two neighbours (one row above,
// one below).  The warps meet only through mbarriers; every wait is bounded, and a wait that runs out sets a status
// word and lets the CTA leave through its normal exit.
#include <algorithm>
#include <atomic>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "b200cp_test.h"
#include "mma_util.cuh"
#include "tc_common.cuh"

namespace b200cp {

// defined with the row-band kernel: (W, H, C, N) view of an NCHW tensor with box (W, rows, cb, 1)
int band_tensor_map(const float* ptr, int N, int C, int H, int W, int rows, int cb, CUtensorMap* out);

__device__ int g_stream_status = 0;  // 0 ok; otherwise (code << 16) | block index of the first wait that ran out

namespace {

using namespace mma;
using tc::fence_barrier_init;
using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::smem_u32;
using tc::tma_load_4d;
using tc::tma_prefetch_desc;

constexpr int kMaxNB = 7;                       // 8-pixel blocks per row (W <= 56)
constexpr int kMaxRing = 8;                     // stages of the input ring, rows of the rank ring
constexpr int kRP = 16;                         // ranks per launch (padded)

struct StreamProb {            // one convolution of the launch
  const float *in, *Fin, *Fout, *KH, *KW, *KC;
  float *out, *save;
  int Cin, Cout, flip, accumulate;
};

struct StreamGeom {
  int N, H, W, R, Rs, r0, nconv;
  int NB;                      // W / 8: warps per group
  int XS, PS;                  // input stages, rank-ring rows
  int xstage_floats;           // max Cin * W
  int pslot_floats;            // (W + 2) * 16
  int FP1, FP2;                // pitches of the factor planes
  int CoutPad;                 // rows of the Fout planes (multiple of 64)
  int oP, oF1, oF2, oW, oBar;  // byte offsets from the shared-memory base (input ring at 0)
};

__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n"
      ".reg .pred p;\n"
      "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(done)
      : "r"(bar), "r"(parity)
      : "memory");
  return done != 0;
}
// The first probe costs one instruction; only a wait that has to spin reads the clock.  Gives up after about a
// second, or as soon as another thread of the CTA has given up.
__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (;;) {
    if (try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > 1500000000ll) {
      *abort_flag = 1;
      return false;
    }
  }
}
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t a = smem_u32(bar);
  if (try_wait(a, parity)) return true;
  return wait_slow(a, parity, abort_flag);
}

// a ring position: slot index and the parity of the phase awaited there
struct RingPos {
  int slot;
  uint32_t par;
  __device__ __forceinline__ void next(int n) {
    if (++slot == n) { slot = 0; par ^= 1u; }
  }
};

// the rows [ga, gb) of the launch's row list, one (convolution, image) segment at a time
struct Segment {
  int conv, n, y0, len;
};
// (row indices are 32-bit: the launcher refuses row lists of 2^31 rows or more)
__device__ __forceinline__ bool next_segment(int& cur, int end, const StreamGeom& g, Segment& s) {
  if (cur >= end) return false;
  const int img = cur / g.H;
  s.y0 = cur - img * g.H;
  s.len = min(g.H - s.y0, end - cur);
  s.conv = img >= g.N ? 1 : 0;
  s.n = img - s.conv * g.N;
  cur += s.len;
  return true;
}

// P ring: [slot][W + 2 pixel columns][16 ranks], pixel x at column x + 1, columns 0 and W + 1 zero for good.  The 16
// ranks of a pixel are stored so that the four ranks an output lane needs (t, t+4, t+8, t+12) are one 16-byte word:
// rank r sits at (r & 3) * 4 + (r >> 2).
__device__ __forceinline__ int rank_pos(int r) { return (r & 3) * 4 + (r >> 2); }

// NB: 8-pixel blocks per row (W = 8 NB).  NKS1 / NMB2 > 0: every convolution of the launch has 8 NKS1 input and
// 16 NMB2 output channels and the factor fragments stay in registers (at most 64 each); 0: any channel counts, the
// fragments are read with ldmatrix as they are used.
template <int NB, int NKS1, int NMB2>
__global__ void __launch_bounds__((2 * NB + 1) * 32, 1)
cp4_stream_kernel(const StreamGeom g, const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                  const StreamProb p0, const StreamProb p1) {
  constexpr bool kRegs = NKS1 > 0;
  constexpr int W = 8 * NB;
  constexpr int PSLOT = (W + 2) * kRP;       // floats per rank-ring row
  constexpr int FP2 = kRP + 4;
  constexpr int kWorkers = 2 * NB * 32;      // threads of the rank and output warps
  // all pointers below are derived from this array by pointer arithmetic, so every access is a shared-space access
  extern __shared__ __align__(1024) uint8_t sm[];
  float* Xr = reinterpret_cast<float*>(sm);              // [XS][Cin][W]      input rows (TMA boxes, dense)
  float* Pr = reinterpret_cast<float*>(sm + g.oP);       // [PS][W + 2][16]   rank rows
  float* F1 = reinterpret_cast<float*>(sm + g.oF1);      // [conv][2][16][FP1]       hi | lo of Fin^T
  float* F2 = reinterpret_cast<float*>(sm + g.oF2);      // [conv][2][CoutPad][FP2]  hi | lo of Fout
  float* Ws = reinterpret_cast<float*>(sm + g.oW);       // [conv][9][16]     tap weights, ranks in rank_pos order
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + g.oBar);   // input stage landed          (tx bytes)
  uint64_t* empty = full + kMaxRing;                            // input stage read            (NB warps)
  uint64_t* pfull = empty + kMaxRing;                           // rank row written            (NB warps)
  uint64_t* pempty = pfull + kMaxRing;                          // rank row no longer needed   (NB warps)
  volatile int* abort_flag = reinterpret_cast<volatile int*>(pempty + kMaxRing);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const int H = g.H, FP1 = g.FP1;
  const int XS = g.XS, PS = g.PS;
  if (smem_u32(sm) & 127) {   // cannot happen with the launch this file does; never run on a misaligned base
    if (tid == 0) atomicCAS(&g_stream_status, 0, (2 << 16) | (int)(blockIdx.x & 0xffff));
    return;
  }

  if (tid == 0) {
    for (int i = 0; i < kMaxRing; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], NB);
      mbar_init(&pfull[i], NB);
      mbar_init(&pempty[i], NB);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&map0);
    if (g.nconv > 1) tma_prefetch_desc(&map1);
  }
  __syncthreads();
  grid_launch_dependents();

  // rows [ga, gb) of the list: the first (G mod grid) CTAs take one row more
  const int G = g.nconv * g.N * H;
  const int per = G / (int)gridDim.x, rem = G - per * (int)gridDim.x;
  const int ga = (int)blockIdx.x * per + min((int)blockIdx.x, rem);
  const int gb = ga + per + ((int)blockIdx.x < rem ? 1 : 0);
  int cur = ga;
  Segment s;

  if (warp == 2 * NB) {
    // ================= producer: the first rows are on their way while the other warps stage the factors ===========
    if (lane == 0) {
      RingPos x{0, 1u};   // parity of the "empty" phase awaited: the wrap before the first wait flips it to 0
      int issued = 0;
      bool ok = true;
      while (ok && next_segment(cur, gb, g, s)) {
        const StreamProb& p = s.conv ? p1 : p0;
        const CUtensorMap* map = s.conv ? &map1 : &map0;
        const uint32_t bytes = (uint32_t)p.Cin * (uint32_t)W * 4u;
        // a convolution without an output only writes its rank plane: its own rows, no neighbours
        const bool po = p.out == nullptr;
        const int ya = po ? s.y0 : max(s.y0 - 1, 0), yb = po ? s.y0 + s.len : min(s.y0 + s.len + 1, H);
        for (int y = ya; y < yb; ++y) {
          if (issued >= XS && !wait_or_abort(&empty[x.slot], x.par, abort_flag)) { ok = false; break; }
          mbar_expect_tx(&full[x.slot], bytes);
          tma_load_4d(Xr + (size_t)x.slot * g.xstage_floats, map, &full[x.slot], 0, y, 0, s.n);
          ++issued;
          x.next(XS);
        }
      }
    }
  } else {
    // factor planes, stencil weights and the two zero columns of every rank-ring row; the global loads of a thread
    // are all issued before the first value is used
    {
      // only the convolutions this CTA's rows belong to (one, except for the CTA whose range crosses from the first
      // convolution's rows into the second's)
      const int cv_first = ga >= g.N * H ? 1 : 0, cv_last = gb - 1 >= g.N * H ? 1 : 0;
      for (int cv = cv_first; cv <= cv_last; ++cv) {
        const StreamProb& p = cv ? p1 : p0;
        float* f1 = F1 + (size_t)cv * 2 * kRP * FP1;
        float* f2 = F2 + (size_t)cv * 2 * g.CoutPad * FP2;
        const int n1 = kRP * p.Cin, n2 = g.CoutPad * kRP;
        for (int i0 = 0; i0 < max(n1, n2); i0 += 4 * kWorkers) {
          float v1[4], v2[4];
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * kWorkers + tid;
            const int c = i / kRP, r = i - c * kRP;     // r fastest: contiguous reads of Fin[c][:] and Fout[t][:]
            v1[k] = (i < n1 && r < g.R) ? __ldg(p.Fin + (size_t)c * g.Rs + g.r0 + r) : 0.f;
            v2[k] = (i < n2 && r < g.R && c < p.Cout && p.out != nullptr) ? __ldg(p.Fout + (size_t)c * g.Rs + g.r0 + r) : 0.f;
          }
#pragma unroll
          for (int k = 0; k < 4; ++k) {
            const int i = i0 + k * kWorkers + tid;
            const int c = i / kRP, r = i - c * kRP;
            if (i < n1) {
              const float hi = tf32_round(v1[k]);
              f1[r * FP1 + c] = hi;
              f1[kRP * FP1 + r * FP1 + c] = tf32_round(v1[k] - hi);
            }
            if (i < n2) {
              const float hi = tf32_round(v2[k]);
              f2[c * FP2 + r] = hi;
              f2[g.CoutPad * FP2 + c * FP2 + r] = tf32_round(v2[k] - hi);
            }
          }
        }
        for (int i = tid; i < 9 * kRP; i += kWorkers) {
          const int r = i % kRP, yx = i / kRP, y = yx / 3, x = yx - y * 3;
          const int yy = p.flip ? 2 - y : y, xx = p.flip ? 2 - x : x;
          // a free core [3][3][Rs] (three-factor CP conv) takes the place of the outer product KH x KW
          Ws[cv * 9 * kRP + yx * kRP + rank_pos(r)] =
              r >= g.R ? 0.f
              : p.KC   ? __ldg(p.KC + (size_t)(yy * 3 + xx) * g.Rs + g.r0 + r)
                       : __ldg(p.KH + (size_t)yy * g.Rs + g.r0 + r) * __ldg(p.KW + (size_t)xx * g.Rs + g.r0 + r);
        }
      }
      for (int i = tid; i < PS * 2 * kRP; i += kWorkers) {
        const int slot = i / (2 * kRP), q = i - slot * 2 * kRP;
        Pr[slot * PSLOT + (q < kRP ? q : (W + 1) * kRP + q - kRP)] = 0.f;
      }
    }
    asm volatile("bar.sync 1, %0;" ::"n"(kWorkers) : "memory");

    if (warp < NB) {
      // ================= rank rows: P = Fin^T in =====================================================================
      const int w = warp;
      RingPos x{0, 0u}, pr{0, 1u};
      int written = 0;
      bool ok = true;
      // ldmatrix row address of this lane: tile lane/8 = (rows 0-7 | 8-15) x (k 0-3 | 4-7)
      const int frow = ((lane & 7) + ((lane >> 3) & 1) * 8) * FP1 + (lane >> 4) * 4;
      const int xlane = tq * W + w * 8 + gq;
      // ranks gq and gq + 8 of pixels 8w + 2tq and 8w + 2tq + 1
      const int pst = (w * 8 + 2 * tq + 1) * kRP + rank_pos(gq);
      uint32_t fh[kRegs ? NKS1 : 1][4], fl[kRegs ? NKS1 : 1][4];
      while (ok && next_segment(cur, gb, g, s)) {
        const StreamProb& p = s.conv ? p1 : p0;
        const float* f1 = F1 + (size_t)s.conv * 2 * kRP * FP1 + frow;
        const int nks = kRegs ? NKS1 : (p.Cin >> 3);
        if (kRegs) {
#pragma unroll
          for (int ks = 0; ks < (kRegs ? NKS1 : 1); ++ks) {
            ldmatrix_x4(fh[ks], f1 + ks * 8);
            ldmatrix_x4(fl[ks], f1 + ks * 8 + kRP * FP1);
          }
        }
        float* sv = p.save == nullptr ? nullptr
                    : p.save + (((size_t)s.n * g.Rs + g.r0 + gq) * H + s.y0) * W + w * 8 + 2 * tq;
        const bool sv0 = gq < g.R, sv1 = gq + 8 < g.R;
        const bool po = p.out == nullptr;   // plane only: no rank ring, no output warps
        for (int j = po ? 1 : 0; j <= (po ? s.len : s.len + 1) && ok; ++j) {
          const int y = s.y0 - 1 + j;
          float a0[4] = {0.f, 0.f, 0.f, 0.f}, a1[4] = {0.f, 0.f, 0.f, 0.f}, a2[4] = {0.f, 0.f, 0.f, 0.f};
          float b0[4] = {0.f, 0.f, 0.f, 0.f}, b1[4] = {0.f, 0.f, 0.f, 0.f}, b2[4] = {0.f, 0.f, 0.f, 0.f};
          if (y >= 0 && y < H) {     // uniform over the CTA: rows outside the image are zero and were never loaded
            ok = wait_or_abort(&full[x.slot], x.par, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            const float* xs = Xr + (size_t)x.slot * g.xstage_floats + xlane;
            if (kRegs) {
              float xv[kRegs ? NKS1 : 1][2];
#pragma unroll
              for (int ks = 0; ks < (kRegs ? NKS1 : 1); ++ks) {
                xv[ks][0] = xs[ks * 8 * W];
                xv[ks][1] = xs[ks * 8 * W + 4 * W];
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(&empty[x.slot]);   // every lane of this warp holds its values of the stage
#pragma unroll
              for (int ks = 0; ks < (kRegs ? NKS1 : 1); ++ks) {
                uint32_t bh[2], bl[2];
                split_tf32(xv[ks][0], bh[0], bl[0]);
                split_tf32(xv[ks][1], bh[1], bl[1]);
                // six accumulator chains (three terms x even / odd k-step): consecutive mma on one accumulator are six
                // instructions apart
                if (ks & 1) {
                  mma_tf32_ordered(b0, fh[ks], bh);
                  mma_tf32_ordered(b1, fl[ks], bh);
                  mma_tf32_ordered(b2, fh[ks], bl);
                } else {
                  mma_tf32_ordered(a0, fh[ks], bh);
                  mma_tf32_ordered(a1, fl[ks], bh);
                  mma_tf32_ordered(a2, fh[ks], bl);
                }
              }
#pragma unroll
              for (int e = 0; e < 4; ++e) { a0[e] += b0[e]; a1[e] += b1[e]; a2[e] += b2[e]; }
            } else {
              const float* fk = f1;
              float x0 = xs[0], x1 = xs[4 * W];
#pragma unroll 2
              for (int ks = 0; ks < nks; ++ks) {
                uint32_t bh[2], bl[2];
                split_tf32(x0, bh[0], bl[0]);
                split_tf32(x1, bh[1], bl[1]);
                xs += 8 * W;
                if (ks + 1 < nks) { x0 = xs[0]; x1 = xs[4 * W]; }
                uint32_t ah[4], al[4];
                ldmatrix_x4(ah, fk);
                ldmatrix_x4(al, fk + kRP * FP1);
                fk += 8;
                mma_tf32_ordered(a0, ah, bh);
                mma_tf32_ordered(a1, al, bh);
                mma_tf32_ordered(a2, ah, bl);
              }
              __syncwarp();
              if (lane == 0) mbar_arrive(&empty[x.slot]);
            }
            x.next(XS);
          }
          const float v0 = a0[0] + (a1[0] + a2[0]), v1 = a0[1] + (a1[1] + a2[1]);
          const float v2 = a0[2] + (a1[2] + a2[2]), v3 = a0[3] + (a1[3] + a2[3]);
          if (sv != nullptr && j >= 1 && j <= s.len) {   // the rows this range owns
            if (sv0) *reinterpret_cast<float2*>(sv) = make_float2(v0, v1);
            if (sv1) *reinterpret_cast<float2*>(sv + (size_t)8 * H * W) = make_float2(v2, v3);
            sv += W;
          }
          if (po) continue;
          if (written >= PS) {
            ok = wait_or_abort(&pempty[pr.slot], pr.par, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
          }
          float* pd = Pr + pr.slot * PSLOT + pst;
          pd[0] = v0;
          pd[kRP] = v1;
          pd[2] = v2;          // rank gq + 8 sits two places after rank gq
          pd[kRP + 2] = v3;
          __syncwarp();
          if (lane == 0) mbar_arrive(&pfull[pr.slot]);
          pr.next(PS);
          ++written;
        }
      }
    } else {
      // ================= output rows: stencil, out = Fout Z ==========================================================
      const int w = warp - NB;
      RingPos wp{0, 0u};          // next rank row to wait for
      int waited = 0, base = 0;   // rank rows waited for so far; index of the segment's first rank row
      int fslot = 0;              // next rank row to hand back
      int rs0 = 0;                // slot of the rank row above the current output row
      bool ok = true;
      const int frow = ((lane & 7) + ((lane >> 3) & 1) * 8) * FP2 + (lane >> 4) * 4;
      const int plane = (w * 8 + gq) * kRP + tq * 4;   // pixel 8w + gq - 1, ranks tq, tq+4, tq+8, tq+12
      uint32_t fh[kRegs ? NMB2 : 1][2][4], fl[kRegs ? NMB2 : 1][2][4];
      while (ok && next_segment(cur, gb, g, s)) {
        const StreamProb& p = s.conv ? p1 : p0;
        if (p.out == nullptr) continue;   // plane only: nothing for the output warps, and no rank rows in the ring
        const int kF2 = g.CoutPad * FP2;
        const float* f2 = F2 + (size_t)s.conv * 2 * kF2 + frow;
        const int nmb = kRegs ? NMB2 : ((p.Cout + 15) >> 4);
        if (kRegs) {
#pragma unroll
          for (int m = 0; m < (kRegs ? NMB2 : 1); ++m)
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              ldmatrix_x4(fh[m][ks], f2 + m * 16 * FP2 + ks * 8);
              ldmatrix_x4(fl[m][ks], f2 + m * 16 * FP2 + ks * 8 + kF2);
            }
        }
        const float4* wsv = reinterpret_cast<const float4*>(Ws + s.conv * 9 * kRP + tq * 4);
        float4 wt[kRegs ? 1 : 9];
        if (!kRegs) {
#pragma unroll
          for (int t = 0; t < 9; ++t) wt[t] = wsv[t * 4];
        }
        const size_t cstride = (size_t)H * W;
        float* op = p.out + (((size_t)s.n * p.Cout + gq) * H + s.y0) * W + w * 8 + 2 * tq;
        for (int o = 0; o < s.len && ok; ++o) {
          while (waited <= base + o + 2) {
            ok = wait_or_abort(&pfull[wp.slot], wp.par, abort_flag);
            ok = __all_sync(0xffffffffu, ok);
            if (!ok) break;
            wp.next(PS);
            ++waited;
          }
          if (!ok) break;
          int rs1 = rs0 + 1; if (rs1 == PS) rs1 = 0;
          int rs2 = rs1 + 1; if (rs2 == PS) rs2 = 0;
          const float* q[3] = {Pr + rs0 * PSLOT + plane, Pr + rs1 * PSLOT + plane, Pr + rs2 * PSLOT + plane};
          float z[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int dy = 0; dy < 3; ++dy)
#pragma unroll
            for (int dx = 0; dx < 3; ++dx) {
              const float4 pv = *reinterpret_cast<const float4*>(q[dy] + dx * kRP);
              const float4 wv = kRegs ? wsv[(dy * 3 + dx) * 4] : wt[kRegs ? 0 : dy * 3 + dx];
              z[0] = fmaf(wv.x, pv.x, z[0]);
              z[1] = fmaf(wv.y, pv.y, z[1]);
              z[2] = fmaf(wv.z, pv.z, z[2]);
              z[3] = fmaf(wv.w, pv.w, z[3]);
            }
          uint32_t zh[4], zl[4];
#pragma unroll
          for (int j = 0; j < 4; ++j) split_tf32(z[j], zh[j], zl[j]);
          // the row above is not needed again; after the last output row of the segment neither are the other two
          __syncwarp();
          {
            const int nfree = o == s.len - 1 ? 3 : 1;
            for (int k = 0; k < nfree; ++k) {
              if (lane == 0) mbar_arrive(&pempty[fslot]);
              if (++fslot == PS) fslot = 0;
            }
          }
          rs0 = rs1;
          if (kRegs) {
            float acc[kRegs ? NMB2 : 1][4];
#pragma unroll
            for (int m = 0; m < (kRegs ? NMB2 : 1); ++m)
#pragma unroll
              for (int e = 0; e < 4; ++e) acc[m][e] = 0.f;
#pragma unroll
            for (int ks = 0; ks < 2; ++ks) {
              const uint32_t bh[2] = {zh[2 * ks], zh[2 * ks + 1]}, bl[2] = {zl[2 * ks], zl[2 * ks + 1]};
#pragma unroll
              for (int m = 0; m < (kRegs ? NMB2 : 1); ++m) mma_tf32_ordered(acc[m], fl[m][ks], bh);
#pragma unroll
              for (int m = 0; m < (kRegs ? NMB2 : 1); ++m) mma_tf32_ordered(acc[m], fh[m][ks], bl);
#pragma unroll
              for (int m = 0; m < (kRegs ? NMB2 : 1); ++m) mma_tf32_ordered(acc[m], fh[m][ks], bh);
            }
            float* o0 = op;
#pragma unroll
            for (int m = 0; m < (kRegs ? NMB2 : 1); ++m) {
              float* o1 = o0 + 8 * cstride;
              float2 u0 = make_float2(acc[m][0], acc[m][1]), u1 = make_float2(acc[m][2], acc[m][3]);
              if (p.accumulate) {
                const float2 c0 = *reinterpret_cast<const float2*>(o0), c1 = *reinterpret_cast<const float2*>(o1);
                u0.x += c0.x; u0.y += c0.y; u1.x += c1.x; u1.y += c1.y;
              }
              *reinterpret_cast<float2*>(o0) = u0;
              *reinterpret_cast<float2*>(o1) = u1;
              o0 = o1 + 8 * cstride;
            }
          } else {
            for (int mc = 0; mc < nmb; mc += 4) {
              float acc[4][4];
#pragma unroll
              for (int m = 0; m < 4; ++m)
#pragma unroll
                for (int e = 0; e < 4; ++e) acc[m][e] = 0.f;
#pragma unroll
              for (int ks = 0; ks < 2; ++ks) {
                const uint32_t bh[2] = {zh[2 * ks], zh[2 * ks + 1]}, bl[2] = {zl[2 * ks], zl[2 * ks + 1]};
                uint32_t ah[4][4], al[4][4];
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                  ldmatrix_x4(ah[m], f2 + (mc + m) * 16 * FP2 + ks * 8);
                  ldmatrix_x4(al[m], f2 + (mc + m) * 16 * FP2 + ks * 8 + kF2);
                }
#pragma unroll
                for (int m = 0; m < 4; ++m) mma_tf32_ordered(acc[m], al[m], bh);
#pragma unroll
                for (int m = 0; m < 4; ++m) mma_tf32_ordered(acc[m], ah[m], bl);
#pragma unroll
                for (int m = 0; m < 4; ++m) mma_tf32_ordered(acc[m], ah[m], bh);
              }
#pragma unroll
              for (int m = 0; m < 4; ++m) {
                // only the stores are guarded: channels past Cout were computed on zero factor rows
                const int t0 = (mc + m) * 16 + gq;
                float* o0 = op + (size_t)(mc + m) * 16 * cstride;
                float* o1 = o0 + 8 * cstride;
                float2 u0 = make_float2(acc[m][0], acc[m][1]), u1 = make_float2(acc[m][2], acc[m][3]);
                if (t0 < p.Cout) {
                  if (p.accumulate) {
                    const float2 c0 = *reinterpret_cast<const float2*>(o0);
                    u0.x += c0.x; u0.y += c0.y;
                  }
                  *reinterpret_cast<float2*>(o0) = u0;
                }
                if (t0 + 8 < p.Cout) {
                  if (p.accumulate) {
                    const float2 c1 = *reinterpret_cast<const float2*>(o1);
                    u1.x += c1.x; u1.y += c1.y;
                  }
                  *reinterpret_cast<float2*>(o1) = u1;
                }
              }
            }
          }
          op += W;
        }
        base += s.len + 2;
        rs0 += 2;                 // past the segment's last two rank rows
        if (rs0 >= PS) rs0 -= PS;
      }
    }
  }
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(&g_stream_status, 0, (1 << 16) | (int)(blockIdx.x & 0xffff));
    // loads that may still be in flight towards this CTA's shared memory get time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) {}
  }
}

const bool g_stream_off = [] {
  const char* e = getenv("B200CP_STREAM");
  return e && e[0] == '0';
}();
std::atomic<long long> g_stream_launches{0};   // launches of the row-stream kernel by this process (tests read it)
std::atomic<int> g_stream_force{-1};   // test hook: 0 off, 1 on, -1 the environment's choice

struct StreamPlan {
  StreamGeom g;
  size_t smem;
};

bool stream_shape_ok(const Cp4Args& a) {
  if (a.Y != 3 || a.X != 3 || a.pad != 1) return false;
  if (a.W % 8 != 0 || a.W > 8 * kMaxNB || (a.W % 32 != 8 && a.W % 32 != 24)) return false;
  if (a.H < 1 || a.R < 1 || a.R > kRP) return false;
  if (a.Cin % 8 != 0 || a.Cin > 256 || a.Cout < 1) return false;   // the box of a row holds all input channels
  if (reinterpret_cast<uintptr_t>(a.in) & 15) return false;                    // tensor map
  if (reinterpret_cast<uintptr_t>(a.out) & 7) return false;                    // 8-byte stores
  if (a.out == nullptr && (a.save == nullptr || a.accumulate)) return false;   // no output: the rank plane is the result
  if (a.save && (reinterpret_cast<uintptr_t>(a.save) & 7)) return false;
  return true;
}

bool plan_stream(const Cp4Args* convs, int nconv, const DeviceInfo& di, StreamPlan* out) {
  const Cp4Args& a = convs[0];
  int cin = 0, cout = 0;
  for (int i = 0; i < nconv; ++i) { cin = std::max(cin, convs[i].Cin); cout = std::max(cout, convs[i].Cout); }
  StreamGeom g{};
  g.N = a.N; g.H = a.H; g.W = a.W; g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0; g.nconv = nconv;
  g.NB = a.W / 8;
  g.xstage_floats = cin * a.W;
  g.pslot_floats = (a.W + 2) * kRP;
  g.FP1 = cin + 4;
  g.FP2 = kRP + 4;
  g.CoutPad = (cout + 63) / 64 * 64;
  // rank rows in the ring: three are read per output row and one is being written; deeper rings measured slower
  // (step at N=32, C=T=64, 56x56, R=16: 60.6 us with 4, 61.1 with 6, 61.4 with 8)
  g.PS = 4;
  static_assert(4 <= kMaxRing, "the rank ring has a barrier pair per row");
  const size_t pring = (size_t)g.PS * g.pslot_floats * 4;
  const size_t f1 = (size_t)nconv * 2 * kRP * g.FP1 * 4;
  const size_t f2 = (size_t)nconv * 2 * g.CoutPad * g.FP2 * 4;
  const size_t ws = (size_t)nconv * 9 * kRP * 4;
  const size_t bars = (size_t)4 * kMaxRing * 8 + 16;
  const size_t fixed = pring + f1 + f2 + ws + bars + 512;
  const size_t stage = (size_t)g.xstage_floats * 4;
  if (fixed + 3 * stage > (size_t)di.smem_optin) return false;
  // input rows in flight: four measured best (step at N=32, C=T=64, 56x56, R=16: 59.1 us with 3, 58.8 with 4, 59.0 with
  // 5, 59.6 with 6, 60.6 with 8 -- every CTA asks for its rows at the same time, and deeper rings only lengthen the
  // queue in front of the memory system)
  g.XS = (int)std::min<size_t>(4, ((size_t)di.smem_optin - fixed) / stage);
  size_t o = align_up((size_t)g.XS * stage, 128);
  g.oP = (int)o; o += pring;
  g.oF1 = (int)o; o += f1;
  g.oF2 = (int)o; o += f2;
  g.oW = (int)o; o += ws;
  o = align_up(o, 16);
  g.oBar = (int)o; o += bars;
  out->g = g;
  out->smem = o;
  return o <= (size_t)di.smem_optin;
}

template <int NB, int NKS1, int NMB2>
int launch_stream(const StreamPlan& pl, unsigned grid, const CUtensorMap* m, const StreamProb* p, cudaStream_t st) {
  auto kern = cp4_stream_kernel<NB, NKS1, NMB2>;
  static std::atomic<int> smem_set[64];
  B200CP_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_set, (int)pl.smem));
  kern<<<grid, (2 * NB + 1) * 32, pl.smem, st>>>(pl.g, m[0], m[1], p[0], p[1]);
  B200CP_LAUNCH_OK("cp4_stream_kernel");
  return B200CP_OK;
}

StreamProb make_prob(const Cp4Args& a) {
  StreamProb p{};
  p.in = a.in; p.Fin = a.Fin; p.Fout = a.Fout; p.KH = a.KH; p.KW = a.KW; p.KC = a.KC; p.out = a.out; p.save = a.save;
  p.Cin = a.Cin; p.Cout = a.Cout; p.flip = a.flip; p.accumulate = a.accumulate;
  return p;
}

}  // namespace

// One or two convolutions (same image size, batch and rank range) in one launch.  *done = false: not a shape this
// kernel takes; the caller uses another path.
int cp4_stream_launch(const Cp4Args* convs, int nconv, cudaStream_t st, bool* done) {
  *done = false;
  const int force = g_stream_force.load(std::memory_order_relaxed);
  if (force == 0 || (force < 0 && g_stream_off)) return B200CP_OK;
  if (nconv < 1 || nconv > 2) return B200CP_OK;
  const Cp4Args& a = convs[0];
  for (int i = 0; i < nconv; ++i) {
    const Cp4Args& c = convs[i];
    if (!stream_shape_ok(c) || c.N != a.N || c.H != a.H || c.W != a.W || c.R != a.R || c.Rs != a.Rs || c.r0 != a.r0) return B200CP_OK;
  }
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  StreamPlan pl;
  if (!plan_stream(convs, nconv, di, &pl)) return B200CP_OK;
  CUtensorMap m[2];
  StreamProb p[2];
  std::memset(m, 0, sizeof(m));
  for (int i = 0; i < 2; ++i) {
    const Cp4Args& c = convs[i < nconv ? i : 0];
    if (int rc = band_tensor_map(c.in, c.N, c.Cin, c.H, c.W, 1, c.Cin, &m[i])) return rc;
    p[i] = make_prob(c);
  }
  const long long rows = (long long)nconv * a.N * a.H;
  if (rows >= 0x7fffffffLL) return B200CP_OK;
  const unsigned grid = (unsigned)std::min<long long>(di.sm_count, rows);
  static const bool debug = getenv("B200CP_DEBUG") != nullptr;
  if (debug)
    fprintf(stderr, "[b200cp] stream NB=%d XS=%d PS=%d smem=%zu grid=%u convs=%d\n", pl.g.NB, pl.g.XS, pl.g.PS, pl.smem, grid, nconv);
  // factor fragments in registers when every convolution has the same 8 * 8 input and 16 * 4 output channels
  bool regs = true;
  for (int i = 0; i < nconv; ++i) regs = regs && convs[i].Cin == 64 && convs[i].Cout == 64;
  int rc = B200CP_ERR_UNSUPPORTED;
  switch (pl.g.NB * 2 + (regs ? 1 : 0)) {
#define STREAM_CASE(NBV) \
    case NBV * 2: rc = launch_stream<NBV, 0, 0>(pl, grid, m, p, st); break; \
    case NBV * 2 + 1: rc = launch_stream<NBV, 8, 4>(pl, grid, m, p, st); break;
    STREAM_CASE(1) STREAM_CASE(3) STREAM_CASE(5) STREAM_CASE(7)
#undef STREAM_CASE
    default: return B200CP_OK;
  }
  if (rc) return rc;
  g_stream_launches.fetch_add(1, std::memory_order_relaxed);
  *done = true;
  return B200CP_OK;
}

long long stream_launches() { return g_stream_launches.load(std::memory_order_relaxed); }

void stream_force(int on) { g_stream_force.store(on); }

int stream_device_status(int* out) {
  int v = 0, zero = 0;
  B200CP_CUDA_OK(cudaDeviceSynchronize());
  B200CP_CUDA_OK(cudaMemcpyFromSymbol(&v, g_stream_status, sizeof(int)));
  if (v) B200CP_CUDA_OK(cudaMemcpyToSymbol(g_stream_status, &zero, sizeof(int)));
  *out = v;
  return B200CP_OK;
}

}  // namespace b200cp

extern "C" void b200cp_test_set_stream(int on) { b200cp::stream_force(on); }
extern "C" long long b200cp_test_stream_launches(void) { return b200cp::stream_launches(); }
