// CP4 factor gradients from the rank planes P = K1^T X and Q = K0^T dU that the two convolutions of a training step
// saved, over full-width row bands (3x3 filters, pad 1, W a multiple of 4, at most 16 ranks, at most 128 channels).
//
// One launch, two kinds of CTA per band of TH image rows of one image:
//   kind 0  Z  = stencil(P) on the band;            dK0[t, r] += sum_px dU[t, px] Z[r, px]
//   kind 1  Qt = flipped stencil(Q) on the band;     dK1[c, r] += sum_px X[c, px] Qt[r, px]
//           dKH[i, r] += sum_px Q[px] * sum_j KW[j, r] P[px + (i-1, j-1)],   dKW likewise with KH
// (formulas: Cuda_kernels/cp4Conv2dBackwardFilter.cu:91-104, 142-155, 192-205, 241-254, with the channel
// contractions already done by the convolutions).
//
// Data movement is all bulk-asynchronous: the halo band of a plane is one contiguous range per rank (one
// cp.async.bulk each; rows outside the image are zeroed by the CTA: the padding); the band of X / dU streams through a
// ring of [channels][32 pixels] chunks, one cp.async.bulk.tensor box each, written with the 128-byte swizzle so that
// ldmatrix reads it without bank conflicts.  The ring lives in the planes' space once the stencil has consumed them.
//
// The pixel sums are warp-level tensor-core products (mma.sync m16n8k8, tf32 in three terms, fp32 accumulate):
// M = 16 channels (A fragments by ldmatrix from the chunk), N = 8 ranks (B fragments by ldmatrix from the stencilled
// plane), K = 8 pixels.  A warp owns 16 channels and every KS-th pixel step; its accumulators live in registers for
// the whole band.  The KS partial sums of a channel block are added in a fixed order, each CTA writes its rows of a
// per-band partial vector, and cp4_reduce_partials_kernel adds the bands in order: bitwise reproducible.
// All mbarrier waits are bounded; a wait that runs out sets a status word and the CTA leaves through its normal exit.
#include <algorithm>
#include <cstdlib>
#include <cstring>

#include "common.cuh"
#include "mma_util.cuh"
#include "tc_common.cuh"

namespace b200cp {

__device__ int g_grad_band_status = 0;

namespace {

using namespace mma;
using tc::fence_barrier_init;
using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::smem_u32;

constexpr int kCons = 9;                  // warps that run the stencil; the first eight also run the pixel sums
constexpr int kMma = 8;
constexpr int kWarps = kCons + 1;         // + the producer warp
constexpr int kNT = kWarps * 32;
constexpr int kMaxStages = 8;
constexpr int kChunk = 32;                // pixels per ring stage: 128 bytes per channel row = the swizzle span

struct GradGeom {
  int N, H, W, C, T, R, Rs, r0;
  int TH, NPH, OPX, bands, tiles;         // band rows, halo pixels, own pixels, bands per image, CTAs per kind
  int PP, ZP;                             // row pitches (floats) of the halo planes and of the stencilled plane
  int nchunk;                             // pixel chunks per band
  int stages, stage_bytes, chmax;         // ring depth, bytes per stage, channel rows per stage (max(T, C) padded to 16)
  int nparam;                             // floats of a band's partial vector: (T + C + 6) * R
  int oP, oQ, oZ, oW, oRed, oBar;         // byte offsets: Q plane first (ring space from the start), then P; Z; weights
  long long* trace;                       // diagnostics: 32 cycle stamps per CTA for the first 1024 CTAs (null: off)
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
__device__ __noinline__ bool wait_slow(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
  const long long t0 = clock64();
  for (;;) {
    if (try_wait(bar, parity)) return true;
    if (*abort_flag) return false;
    if (clock64() - t0 > 1500000000ll) {   // about a second: give up, never hang
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
__device__ __forceinline__ void bulk_load(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(sdst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCons * 32) : "memory"); }
__device__ __forceinline__ void mma_sync() { asm volatile("bar.sync 2, %0;" ::"n"(kMma * 32) : "memory"); }

// NMB: blocks of 16 channels per warp (1 or 2).  KS = pixel steps interleaved over warps = 8 warps / channel-block groups.
template <int NMB>
__global__ void __launch_bounds__(kNT, 2)
cp4_grad_band_kernel(const GradGeom g, const __grid_constant__ CUtensorMap mapU, const __grid_constant__ CUtensorMap mapX,
                     const float* __restrict__ Pg, const float* __restrict__ Qg, const float* __restrict__ KH,
                     const float* __restrict__ KW, float* __restrict__ ws) {
  constexpr int RP = 16;
  extern __shared__ __align__(1024) uint8_t sm[];
  // Two plane slots.  Kind 0 keeps P in the second one (the first is ring space from the start).  Kind 1 keeps P in
  // the first and Q in the second: P is consumed first (the Q x P correlations), so the ring's first stages load
  // while the stencil of Q still runs.
  float* Zs = reinterpret_cast<float*>(sm + g.oZ);    // [RP][ZP] Z (kind 0) or Qt (kind 1) on the band's own pixels
  float* Ws = reinterpret_cast<float*>(sm + g.oW);    // [9][RP] stencil weights, then [3][RP] KH, [3][RP] KW
  float* red = reinterpret_cast<float*>(sm + g.oRed); // [threads][9] spatial correlations, later the warps' channel sums
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + g.oBar);
  uint64_t* empty = full + kMaxStages;
  uint64_t* planes_full = empty + kMaxStages;
  uint64_t* planes_free = planes_full + 1;
  uint64_t* first_free = planes_free + 1;             // kind 1: the first plane slot (P) is consumed
  volatile int* abort_flag = reinterpret_cast<volatile int*>(first_free + 1);

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  // The longer-running kind comes first in the grid: the CTAs that do not fit the first round then follow the
  // shorter ones.
  const int kind = (int)blockIdx.x < g.tiles ? 1 : 0;
  const int b = (int)blockIdx.x - (1 - kind) * g.tiles;
  const int band = b % g.bands, n = b / g.bands;
  float* Ps = reinterpret_cast<float*>(sm + (kind ? g.oQ : g.oP));   // [RP][PP] halo band of P
  float* Qs = reinterpret_cast<float*>(sm + g.oP);                   // [RP][PP] halo band of Q (kind 1 only)
  const int h0 = band * g.TH;
  const int W = g.W, HW = g.H * g.W, PP = g.PP, ZP = g.ZP;
  const int S = g.stages;
  const int ra = h0 == 0 ? 1 : 0, rb = min(g.TH + 2, g.H - h0 + 1);   // halo rows [ra, rb) lie inside the image
  const int own_rows = min(g.TH, g.H - h0);
  const int nch = kind ? g.C : g.T;                   // channels of the streamed tensor
  const int mbs = (nch + 15) >> 4;                    // blocks of 16 channels
  // warps per channel-block group and pixel-step interleave: 8 warps cover mbs / NMB groups KS ways
  const int groups = (mbs + NMB - 1) / NMB;
  const int KS = groups <= 2 ? 4 : groups <= 4 ? 2 : 1;   // groups * KS <= 8 warps (the planner keeps groups <= 8)
  float* part = ws + (size_t)b * g.nparam;
  if (smem_u32(sm) & 1023) {
    if (tid == 0) atomicCAS(&g_grad_band_status, 0, (2 << 16) | (int)(blockIdx.x & 0xffff));
    return;
  }

  long long* tr = (g.trace != nullptr && blockIdx.x < 1024 && tid == 0) ? g.trace + (size_t)blockIdx.x * 32 : nullptr;
  auto stamp = [&](int k) { if (tr) tr[k] = clock64(); };
  stamp(0);
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kMma);
    }
    mbar_init(planes_full, 1);
    mbar_init(planes_free, kCons);
    mbar_init(first_free, kCons);
    *abort_flag = 0;
    fence_barrier_init();
    tc::tma_prefetch_desc(kind ? &mapX : &mapU);
  }
  __syncthreads();
  grid_launch_dependents();
  grid_dependency_wait();   // the rank planes are the previous kernel's output

  float acc[NMB][3][2][4];   // [channel block][term][rank block][fragment]
  if (warp == kCons) {
    // ================= producer =========================================================================================
    const uint32_t bytes = (uint32_t)((rb - ra) * W) * 4u;
    if (lane == 0) mbar_expect_tx(planes_full, bytes * (uint32_t)g.R * (kind ? 2u : 1u));
    __syncwarp();
    {
      const size_t off = ((size_t)n * g.Rs + g.r0) * HW + (size_t)(h0 - 1 + ra) * W;
      if (lane < g.R) {
        bulk_load(Ps + lane * PP + ra * W, Pg + off + (size_t)lane * HW, bytes, planes_full);
        if (kind) bulk_load(Qs + lane * PP + ra * W, Qg + off + (size_t)lane * HW, bytes, planes_full);
      }
    }
    // the ring: stage s at s * stage_bytes from the start of the planes' space.  The stages inside the first plane
    // slot are free from the start for kind 0 (it has no second plane) and once the correlations have consumed P for
    // kind 1; the others wait until the stencil has consumed the planes.
    const CUtensorMap* map = kind ? &mapX : &mapU;
    const int nfirst = (g.oP - g.oQ) / g.stage_bytes;
    bool first_done = kind == 0, planes_done = false;
    int slot = 0;
    uint32_t par = 1;
    for (int s = 0; s < g.nchunk; ++s) {
      if (s >= S) {
        if (!wait_or_abort(&empty[slot], par, abort_flag)) break;
      } else if (slot < nfirst) {
        if (!first_done) {
          if (!wait_or_abort(first_free, 0, abort_flag)) break;
          first_done = true;
        }
      } else if (!planes_done) {
        if (!wait_or_abort(planes_free, 0, abort_flag)) break;
        planes_done = true;
      }
      if (lane == 0) {
        mbar_expect_tx(&full[slot], (uint32_t)g.stage_bytes);
        tc::tma_load_3d(sm + g.oQ + (size_t)slot * g.stage_bytes, map, &full[slot], h0 * W + s * kChunk, 0, n);
      }
      if (++slot == S) { slot = 0; par ^= 1; }
    }
  } else {
    // ================= consumers ==========================================================================================
    constexpr int NTC = kCons * 32;
    for (int i = tid; i < 9 * RP; i += NTC) {
      const int r = i % RP, yx = i / RP, y = yx / 3, x = yx - y * 3;
      // kind 1 applies the taps flipped (the transpose of the forward stencil)
      const int yy = kind ? 2 - y : y, xx = kind ? 2 - x : x;
      Ws[i] = r < g.R ? __ldg(KH + (size_t)yy * g.Rs + g.r0 + r) * __ldg(KW + (size_t)xx * g.Rs + g.r0 + r) : 0.f;
    }
    for (int i = tid; i < 6 * RP; i += NTC) {
      const int r = i % RP, k = i / RP;
      const float* src = k < 3 ? KH + (size_t)k * g.Rs : KW + (size_t)(k - 3) * g.Rs;
      Ws[9 * RP + i] = r < g.R ? __ldg(src + g.r0 + r) : 0.f;
    }
    // what the bulk copies never write must read as zero: halo rows outside the image, ranks past R
    {
      const int zr = ra + (g.TH + 2 - rb);
      const int per = zr * W;
      for (int i = tid; i < RP * per; i += NTC) {
        const int r = i / per, q = i - r * per;
        const int row = q / W, col = q - row * W;
        const int hr = row < ra ? row : rb + (row - ra);
        Ps[r * PP + hr * W + col] = 0.f;
        if (kind) Qs[r * PP + hr * W + col] = 0.f;
      }
      const int live = (rb - ra) * W;
      for (int i = tid; i < (RP - g.R) * live; i += NTC) {
        const int r = g.R + i / live, q = i - (i / live) * live;
        Ps[r * PP + ra * W + q] = 0.f;
        if (kind) Qs[r * PP + ra * W + q] = 0.f;
      }
      // Z beyond the band's own pixels (the tail of the last chunk, rows outside the image) multiplies real data
      for (int i = tid; i < RP * (ZP - own_rows * W); i += NTC) {
        const int r = i / (ZP - own_rows * W), q = i - r * (ZP - own_rows * W);
        Zs[r * ZP + own_rows * W + q] = 0.f;
      }
    }
    stamp(1);
    bool ok = wait_or_abort(planes_full, 0, abort_flag);
    consumers_sync();
    stamp(2);
    ok = ok && !*abort_flag;

    // ---- stencil: strips of 8 pixels, one rank per thread ------------------------------------------------------------
    float sp[9] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};   // this thread's share of the nine Q x P correlations of its rank
    if (ok) {
      static_assert(NTC % RP == 0, "a thread keeps one rank");
      const int spr = (W + 7) >> 3;
      const int nitems = own_rows * spr;
      const int r = tid % RP;
      float w[9];
#pragma unroll
      for (int t = 0; t < 9; ++t) w[t] = Ws[t * RP + r];
      const float* src = kind ? Qs : Ps;
      constexpr int STEP = NTC / RP;
      const int dy_step = STEP / spr, dx_step = STEP % spr;
      // pass 0 (kind 1 only): the nine Q x P correlations, after which P's slot joins the ring; pass 1: the stencil
      for (int pass = kind ? 0 : 1; pass < 2; ++pass) {
        int oy = (tid / RP) / spr, sx = (tid / RP) % spr;
        for (int it = tid / RP; it < nitems; it += STEP) {
          const int x0 = sx * 8;
          const bool hi_ok = x0 + 4 < W, lft = x0 > 0, rgt = x0 + 8 < W;
          if (pass) {
            float z[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) z[j] = 0.f;
            const float* pr = src + r * PP + oy * W + x0;
#pragma unroll
            for (int dy = 0; dy < 3; ++dy) {
              float v[10];
              const float4 a = *reinterpret_cast<const float4*>(pr);
              const float4 c = hi_ok ? *reinterpret_cast<const float4*>(pr + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
              v[0] = lft ? pr[-1] : 0.f;
              v[9] = rgt ? pr[8] : 0.f;
              v[1] = a.x; v[2] = a.y; v[3] = a.z; v[4] = a.w;
              v[5] = c.x; v[6] = c.y; v[7] = c.z; v[8] = c.w;
              pr += W;
#pragma unroll
              for (int j = 0; j < 8; ++j) {
                z[j] = fmaf(w[dy * 3 + 0], v[j], z[j]);
                z[j] = fmaf(w[dy * 3 + 1], v[j + 1], z[j]);
                z[j] = fmaf(w[dy * 3 + 2], v[j + 2], z[j]);
              }
            }
            float* zd = Zs + r * ZP + oy * W + x0;
            *reinterpret_cast<float4*>(zd) = make_float4(z[0], z[1], z[2], z[3]);
            if (hi_ok) *reinterpret_cast<float4*>(zd + 4) = make_float4(z[4], z[5], z[6], z[7]);
          } else {
            // spatial factors: the nine correlations S[dy][dx] = sum_px Q[px] P[px + (dy-1, dx-1)] of the strip; the
            // factor gradients are their contractions with the other factor (dKH[i] = sum_j KW[j] S[i][j], dKW[j] =
            // sum_i KH[i] S[i][j]), formed once per CTA
            const float* qc = Qs + r * PP + (oy + 1) * W + x0;
            const float4 qa = *reinterpret_cast<const float4*>(qc);
            const float4 qb = hi_ok ? *reinterpret_cast<const float4*>(qc + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
            const float q[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
            const float* pp = Ps + r * PP + oy * W + x0;
#pragma unroll
            for (int dy = 0; dy < 3; ++dy) {
              float v[10];
              const float4 a = *reinterpret_cast<const float4*>(pp);
              const float4 c = hi_ok ? *reinterpret_cast<const float4*>(pp + 4) : make_float4(0.f, 0.f, 0.f, 0.f);
              v[0] = lft ? pp[-1] : 0.f;
              v[9] = rgt ? pp[8] : 0.f;
              v[1] = a.x; v[2] = a.y; v[3] = a.z; v[4] = a.w;
              v[5] = c.x; v[6] = c.y; v[7] = c.z; v[8] = c.w;
              pp += W;
#pragma unroll
              for (int dx = 0; dx < 3; ++dx) {
                float t = 0.f;
#pragma unroll
                for (int j = 0; j < 8; ++j) t = fmaf(q[j], v[j + dx], t);
                sp[dy * 3 + dx] += t;
              }
            }
          }
          oy += dy_step;
          sx += dx_step;
          if (sx >= spr) { sx -= spr; ++oy; }
        }
        if (pass == 0) {
          tc::fence_proxy_async();   // this thread's zero fill of P's slot is ordered before the bulk copies that reuse it
          __syncwarp();
          if (lane == 0) mbar_arrive(first_free);
        }
      }
    }
    if (kind && !ok) {   // the producer may be waiting for P's slot
      __syncwarp();
      if (lane == 0) mbar_arrive(first_free);
    }
    if (kind) {
#pragma unroll
      for (int k = 0; k < 9; ++k) red[tid * 9 + k] = sp[k];
    }
    tc::fence_proxy_async();   // this thread's writes into the planes' space are ordered before the bulk copies that reuse it
    __syncwarp();
    if (lane == 0) mbar_arrive(planes_free);   // this warp reads the halo planes no more: their space joins the ring
    consumers_sync();                          // Z is complete; the spatial sums are in place
    stamp(3);
    if (kind && ok && tid < 6 * RP) {
      // the correlations of rank r summed over the threads that worked on it, in thread order, then contracted with
      // the other spatial factor: k < 3 is dKH[k], k >= 3 is dKW[k - 3]
      const int r = tid % RP, k = tid / RP;
      float s = 0.f;
#pragma unroll
      for (int o = 0; o < 3; ++o) {
        const int idx = k < 3 ? k * 3 + o : o * 3 + (k - 3);            // S[k][o] or S[o][k - 3]
        float c = 0.f;
        for (int t = r; t < NTC; t += RP) c += red[t * 9 + idx];
        s = fmaf(Ws[((k < 3 ? 12 : 9) + o) * RP + r], c, s);            // KW[o] for dKH, KH[o] for dKW
      }
      if (r < g.R) part[(size_t)(g.T + g.C + k) * g.R + r] = s;
    }

    // ---- pixel sums ----------------------------------------------------------------------------------------------------
    if (warp < kMma) {
      const int grp = warp / KS, kp = warp - grp * KS;   // channel-block group and pixel-step phase of this warp
      const bool active = grp < groups;
#pragma unroll
      for (int m = 0; m < NMB; ++m)
#pragma unroll
        for (int t = 0; t < 3; ++t)
#pragma unroll
          for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[m][t][nb][e] = 0.f;
      // ldmatrix lane addresses.  A (chunk, 128-byte swizzle): tile lane/8 = (channels 0-7 | 8-15) x (pixels 0-3 | 4-7);
      // 16-byte piece j of channel row c sits at piece j ^ (c % 8).  B (Z plane): tile = (ranks 0-7 | 8-15) x (pixels 0-3 | 4-7).
      const int arow = (lane & 7) + ((lane >> 3) & 1) * 8, ahalf = lane >> 4;
      const int brow = (lane & 7) + ((lane >> 4) & 1) * 8, bhalf = (lane >> 3) & 1;
      const float* zrow = Zs + brow * ZP + bhalf * 4;
      int slot = 0;
      uint32_t par = 0;
      for (int s = 0; s < g.nchunk && ok; ++s) {
        ok = wait_or_abort(&full[slot], par, abort_flag);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) break;
        if (s < 16) stamp(8 + s);
        if (active) {
          const uint8_t* st = sm + g.oQ + (size_t)slot * g.stage_bytes;
          for (int ks = kp; ks < kChunk / 8; ks += KS) {
            uint32_t zr4[4], zh[2][2], zl[2][2];
            ldmatrix_x4(zr4, zrow + s * kChunk + ks * 8);
            split_tf32_bits(zr4[0], zh[0][0], zl[0][0]);
            split_tf32_bits(zr4[1], zh[0][1], zl[0][1]);
            split_tf32_bits(zr4[2], zh[1][0], zl[1][0]);
            split_tf32_bits(zr4[3], zh[1][1], zl[1][1]);
#pragma unroll
            for (int m = 0; m < NMB; ++m) {
              const int ch = (grp * NMB + m) * 16 + arow;
              const int piece = (ks * 2 + ahalf) ^ (ch & 7);
              uint32_t xr[4], xh[4], xl[4];
              ldmatrix_x4(xr, reinterpret_cast<const float*>(st + ch * 128 + piece * 16));
#pragma unroll
              for (int e = 0; e < 4; ++e) split_tf32_bits(xr[e], xh[e], xl[e]);
#pragma unroll
              for (int nb = 0; nb < 2; ++nb) mma_tf32_ordered(acc[m][0][nb], xl, zh[nb]);
#pragma unroll
              for (int nb = 0; nb < 2; ++nb) mma_tf32_ordered(acc[m][1][nb], xh, zl[nb]);
#pragma unroll
              for (int nb = 0; nb < 2; ++nb) mma_tf32_ordered(acc[m][2][nb], xh, zh[nb]);
            }
          }
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);
        if (++slot == S) { slot = 0; par ^= 1; }
      }
      stamp(4);
      // the KS partial sums of a channel block meet in shared memory and are added in phase order
      mma_sync();
      float* rw = red + warp * (NMB * 256);
      if (active) {
#pragma unroll
        for (int m = 0; m < NMB; ++m)
#pragma unroll
          for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
              const int row = gq + (e >> 1) * 8, col = nb * 8 + 2 * tq + (e & 1);
              rw[m * 256 + row * 16 + col] = acc[m][0][nb][e] + acc[m][1][nb][e] + acc[m][2][nb][e];
            }
      }
      mma_sync();
      if (ok) {
        const int rows = groups * NMB * 16;   // channel rows held in the scratch
        float* prow = part + (size_t)(kind ? g.T : 0) * g.R;
        for (int i = tid; i < rows * 16; i += kMma * 32) {
          const int chn = i >> 4, r = i & 15;
          const int gi = chn / (NMB * 16), within = chn - gi * (NMB * 16);
          float sum = 0.f;
          for (int k = 0; k < KS; ++k) sum += red[(gi * KS + k) * (NMB * 256) + within * 16 + r];
          if (chn < nch && r < g.R) prow[(size_t)chn * g.R + r] = sum;
        }
      }
    }
  }
  stamp(5);
  if (tr) { unsigned smid; asm("mov.u32 %0, %%smid;" : "=r"(smid)); tr[6] = smid; tr[7] = kind; }
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(&g_grad_band_status, 0, (1 << 16) | (int)(blockIdx.x & 0xffff));
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) {}
  }
}

int pitch_mod(int n, int mod, int want) {
  int p = (n + 3) / 4 * 4;
  while (p % mod != want) p += 4;
  return p;
}

struct MapKey {
  const void* ptr;
  int N, C, H, W, rows;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  MapKey key{};
  CUtensorMap map;
  bool used = false;
};
thread_local MapSlot t_maps[16];
thread_local int t_map_next = 0;

// (H*W, C, N) view of an NCHW tensor, box (32 pixels, rows channels, 1), 128-byte swizzle
int chunk_map(const float* ptr, int N, int C, int H, int W, int rows, CUtensorMap* out) {
  MapKey k;
  std::memset(&k, 0, sizeof(k));
  k.ptr = ptr; k.N = N; k.C = C; k.H = H; k.W = W; k.rows = rows;
  for (auto& s : t_maps)
    if (s.used && s.key == k) {
      *out = s.map;
      return B200CP_OK;
    }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B200CP_ERR_NO_DEVICE, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t gdim[3] = {(cuuint64_t)H * W, (cuuint64_t)C, (cuuint64_t)N};
  const cuuint64_t gstr[2] = {(cuuint64_t)H * W * 4, (cuuint64_t)C * H * W * 4};
  const cuuint32_t box[3] = {(cuuint32_t)kChunk, (cuuint32_t)rows, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  CUtensorMap m;
  const CUresult cr = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(ptr), gdim, gstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(B200CP_ERR_CUDA, "cuTensorMapEncodeTiled (chunk map) failed with code %d", (int)cr);
  MapSlot& s = t_maps[t_map_next];
  t_map_next = (t_map_next + 1) % 16;
  s.key = k; s.map = m; s.used = true;
  *out = m;
  return B200CP_OK;
}

const bool g_grad_band_off = [] {
  const char* e = getenv("B200CP_GRAD_BAND");
  return e && e[0] == '0';
}();
const int g_grad_band_th = [] {
  const char* e = getenv("B200CP_GRAD_BAND_TH");
  return e ? atoi(e) : 0;
}();

bool plan_grad_search(const Cp4BwdFilterArgs& a, const DeviceInfo& di, GradGeom* out, size_t* smem_out, int* nmb_out);

// The search runs once per shape (and pointer alignment class): a training loop asks for the same plan every step.
bool plan_grad(const Cp4BwdFilterArgs& a, const DeviceInfo& di, GradGeom* out, size_t* smem_out, int* nmb_out) {
  struct Entry {
    int key[12];
    bool ok;
    GradGeom g;
    size_t smem;
    int nmb;
  };
  thread_local Entry cache[4];
  thread_local int used = 0, next = 0;
  const int aligned = !((reinterpret_cast<uintptr_t>(a.X) & 15) || (reinterpret_cast<uintptr_t>(a.dU) & 15));
  const int key[12] = {a.N, a.C, a.T, a.H, a.W, a.F, a.pad, a.R, a.KC ? 1 : 0, aligned, di.sm_count, di.smem_optin};
  for (int i = 0; i < used; ++i)
    if (std::memcmp(cache[i].key, key, sizeof(key)) == 0) {
      if (cache[i].ok) { *out = cache[i].g; *smem_out = cache[i].smem; *nmb_out = cache[i].nmb; }
      return cache[i].ok;
    }
  Entry& e = cache[next];
  next = (next + 1) % 4;
  used = std::min(used + 1, 4);
  std::memcpy(e.key, key, sizeof(key));
  e.ok = plan_grad_search(a, di, &e.g, &e.smem, &e.nmb);
  if (e.ok) { *out = e.g; *smem_out = e.smem; *nmb_out = e.nmb; }
  return e.ok;
}

bool plan_grad_search(const Cp4BwdFilterArgs& a, const DeviceInfo& di, GradGeom* out, size_t* smem_out, int* nmb_out) {
  if (g_grad_band_off) return false;
  if (a.F != 3 || a.pad != 1 || a.KC) return false;
  if (a.W % 4 != 0 || (a.H * a.W) % 4 != 0 || a.R > 16 || a.R < 1) return false;
  const int chmax = (std::max(a.C, a.T) + 15) / 16 * 16;
  if (chmax > 256) return false;
  if ((reinterpret_cast<uintptr_t>(a.X) & 15) || (reinterpret_cast<uintptr_t>(a.dU) & 15)) return false;
  const int mbs = chmax / 16;
  const int NMB = mbs > 8 ? 2 : 1;
  GradGeom best{};
  size_t best_smem = 0;
  double best_cost = 1e300;
  for (int TH = 1; TH <= std::min(a.H, 62); ++TH) {
    if (g_grad_band_th && TH != std::min(g_grad_band_th, a.H)) continue;
    GradGeom g{};
    g.TH = TH;
    g.NPH = (TH + 2) * a.W;
    g.OPX = TH * a.W;
    g.bands = ceil_div(a.H, TH);
    g.tiles = a.N * g.bands;
    g.nchunk = ceil_div(g.OPX, kChunk);
    g.PP = pitch_mod(g.NPH, 32, 4);                        // 16-byte loads of a quarter warp (one rank per lane) do not collide
    g.ZP = pitch_mod(g.nchunk * kChunk + 4, 8, 4);         // ldmatrix rows 16 bytes apart modulo 32
    g.chmax = chmax;
    g.stage_bytes = chmax * 128;
    const size_t plane = align_up((size_t)16 * g.PP * 4, 1024);
    const size_t planes = std::max(2 * plane, (size_t)3 * g.stage_bytes);   // at least three stages
    g.stages = (int)std::min<size_t>(kMaxStages, planes / g.stage_bytes);
    g.oQ = 0;
    g.oP = (int)plane;
    size_t o = align_up(planes, 1024);
    g.oZ = (int)o; o += (size_t)16 * g.ZP * 4;
    g.oW = (int)o; o += (size_t)15 * 16 * 4;
    o = align_up(o, 16);
    g.oRed = (int)o; o += std::max((size_t)kCons * 32 * 9 * 4, (size_t)kMma * NMB * 256 * 4);
    o = align_up(o, 16);
    g.oBar = (int)o; o += 256;
    if ((int)o > di.smem_optin || (o + 1024) * 2 > (size_t)228 * 1024) continue;   // two CTAs per SM
    const long ctas = 2L * g.tiles;
    const long waves = (ctas + 2L * di.sm_count - 1) / (2L * di.sm_count);
    const double tile = (double)TH * a.W * (chmax + 60.0) + (double)(TH + 2) * a.W * 40.0 + 9000.0;
    const double cost = (double)waves * tile;
    if (cost < best_cost) { best_cost = cost; best = g; best_smem = o; }
  }
  if (best.TH == 0) return false;
  *out = best;
  *smem_out = best_smem;
  *nmb_out = NMB;
  return true;
}

}  // namespace

bool cp4_grad_band_supported(const Cp4BwdFilterArgs& a) {
  DeviceInfo di;
  if (device_info(&di) != B200CP_OK) return false;
  GradGeom g;
  size_t smem;
  int nmb;
  return plan_grad(a, di, &g, &smem, &nmb);
}

size_t cp4_grad_band_workspace(const b200cp_tensor_shape& s) {
  if (s.Y != 3 || s.X != 3 || s.pad != 1) return 0;
  const int R = (int)std::min(s.Rank, 16u);   // larger ranks go through the kernel in slices of 16
  DeviceInfo di;
  int dev_count = 0;
  if (cudaGetDeviceCount(&dev_count) != cudaSuccess || dev_count <= 0 || device_info(&di) != B200CP_OK) return 0;
  Cp4BwdFilterArgs a{};
  a.N = s.N; a.C = s.C; a.T = s.T; a.H = s.H; a.W = s.W; a.F = 3; a.pad = 1; a.R = R;
  GradGeom g;
  size_t smem;
  int nmb;
  if (!plan_grad(a, di, &g, &smem, &nmb)) return 0;
  return (size_t)g.tiles * ((size_t)s.T + s.C + 6) * R * sizeof(float);
}

// Factor gradients from the saved rank planes; *done = false: not a shape this kernel takes.
int cp4_grad_band_launch(const Cp4BwdFilterArgs& a, const float* P, const float* Q, cudaStream_t st, bool* done,
                         bool after_own_kernel, const ExchangeArgs* exchange) {
  *done = false;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  GradGeom g;
  size_t smem;
  int nmb;
  if (!plan_grad(a, di, &g, &smem, &nmb)) return B200CP_OK;
  if ((reinterpret_cast<uintptr_t>(P) & 15) || (reinterpret_cast<uintptr_t>(Q) & 15)) return B200CP_OK;
  g.N = a.N; g.H = a.H; g.W = a.W; g.C = a.C; g.T = a.T; g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0;
  g.nparam = (a.T + a.C + 6) * a.R;
  g.trace = band_trace_buffer();
  const size_t need = (size_t)g.tiles * g.nparam * sizeof(float);
  if (a.ws_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "cp4 bwd-filter (bands): workspace of %zu bytes needed, %zu given", need, a.ws_bytes);
  CUtensorMap mU, mX;
  if (int rc = chunk_map(a.dU, a.N, a.T, a.H, a.W, g.chmax, &mU)) return rc;
  if (int rc = chunk_map(a.X, a.N, a.C, a.H, a.W, g.chmax, &mX)) return rc;
  static const bool debug = getenv("B200CP_DEBUG") != nullptr;
  if (debug)
    fprintf(stderr, "[b200cp] grad band TH=%d bands=%d chunks=%d stages=%d stage=%d smem=%zu NMB=%d\n", g.TH, g.bands, g.nchunk,
            g.stages, g.stage_bytes, smem, nmb);
  const long ctas = 2L * g.tiles;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: too many tiles");
  if (nmb == 1) {
    auto kern = cp4_grad_band_kernel<1>;
    static std::atomic<int> smem_set[64];
    B200CP_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_set, (int)smem));
    B200CP_CUDA_OK(launch_kernel(kern, dim3((unsigned)ctas), dim3(kNT), smem, st, after_own_kernel, g, mU, mX, P, Q, a.KH, a.KW,
                                 (float*)a.ws));
  } else {
    auto kern = cp4_grad_band_kernel<2>;
    static std::atomic<int> smem_set[64];
    B200CP_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_set, (int)smem));
    B200CP_CUDA_OK(launch_kernel(kern, dim3((unsigned)ctas), dim3(kNT), smem, st, after_own_kernel, g, mU, mX, P, Q, a.KH, a.KW,
                                 (float*)a.ws));
  }
  B200CP_LAUNCH_OK("cp4_grad_band_kernel");
  if (int rc = cp4_reduce_partials_launch((const float*)a.ws, g.tiles, g.nparam, a.R, a.Rs, a.r0, a.dK, st, true, exchange))
    return rc;
  *done = true;
  return B200CP_OK;
}

int grad_band_device_status(int* out) {
  int v = 0, zero = 0;
  B200CP_CUDA_OK(cudaDeviceSynchronize());
  B200CP_CUDA_OK(cudaMemcpyFromSymbol(&v, g_grad_band_status, sizeof(int)));
  if (v) B200CP_CUDA_OK(cudaMemcpyToSymbol(g_grad_band_status, &zero, sizeof(int)));
  *out = v;
  return B200CP_OK;
}

}  // namespace b200cp
