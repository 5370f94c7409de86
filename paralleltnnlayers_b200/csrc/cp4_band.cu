// CP4 conv2d forward / backward-data over full-width row bands: TMA tile loads, warp-level tensor-core
// contractions (mma.sync m16n8k8, tf32 in three terms, fp32 accumulation), 8-byte stores.
//
// One CTA of 9 warps owns a band of TH image rows of one image, all W columns.  The band with its one-row halo is a
// *contiguous* pixel range of every channel, so one 4-D TMA box (W, TH+2, CB channels, 1 image) per pipeline stage
// brings it in; rows above and below the image arrive as zeros (the tensor map's out-of-range fill), which is the
// zero padding.  No thread computes a global address or a predicate for the input.
//
//   phase 1  P[r, halo px] = sum_c Fin[c, r] * in[c, halo px]         M = ranks (16 per mma), N = 8 pixels, K = 8 channels
//            A fragments: the factor, staged once as tf32 hi | lo planes [rank][channel], read with ldmatrix;
//            B fragments: two 4-byte shared loads per 8 pixels x 8 channels from the TMA stage (conflict-free for
//            the band heights the planner picks), split into hi / lo in registers.
//   phase 2  Z[r, px] = 3x3 stencil of P per rank (CUDA cores, weights in registers, 16-byte shared loads / stores);
//            the image's left and right edge are two predicated loads per strip.
//   phase 3  out[t, px] = sum_r Fout[t, r] * Z[r, px]                  M = channels, N = 8 pixels, K = ranks
//            A fragments: Fout hi | lo [channel][rank] by ldmatrix; B fragments from Z; the D fragments hold pixel
//            pairs, stored as 8-byte words (a quarter warp writes 32 contiguous bytes of one channel).
//
// Every product is hi*hi + lo*hi + hi*lo (fp32-grade).  Forward: Fin = K1, Fout = K0; backward-data swaps them and
// flips the taps (Cuda_kernels/cp4Conv2dForward.cu:84-133, cp4Conv2dBackwardData.cu:57-108).  One launch can carry
// two convolutions (the forward and the backward-data of a training step): the first half of the grid runs one,
// the second half the other.  All mbarrier waits are bounded; a wait that runs out sets a status word and the CTA
// leaves through its normal exit.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"
#include "b200cp_test.h"
#include "mma_util.cuh"
#include "tc_common.cuh"

namespace b200cp {

__device__ int g_band_status = 0;  // 0 ok; otherwise (code << 16) | block index of the first wait that ran out

namespace {

using namespace mma;
using tc::fence_barrier_init;
using tc::mbar_arrive;
using tc::mbar_expect_tx;
using tc::mbar_init;
using tc::smem_u32;
using tc::tma_load_4d;
using tc::tma_prefetch_desc;

constexpr int kCons = 9;                  // warps that run phase 1 (the tensor-core channel contraction)
constexpr int kWarps = kCons + 1;         // + the producer warp; all ten run phases 2 and 3
constexpr int kNT = kWarps * 32;
constexpr int kMaxStages = 6;

struct BandProb {            // one convolution of the launch
  const float *in, *Fin, *Fout, *KH, *KW, *KC;
  float *out, *save;
  int Cin, Cout, flip, accumulate;
};

struct BandGeom {
  int N, H, W, R, Rs, r0;
  int TH, NPH, OPX, bands, tiles;   // band rows, halo pixels = (TH+2)*W, own pixels = TH*W, bands per image, CTAs per conv
  int CB;                           // channels per stage (multiple of 8)
  int stages;                       // ring depth
  int tensor;                       // 1: one 4-D tensor-map load per stage; 0: one 1-D bulk copy per channel
  int NB3;                          // n-blocks (8 pixels) of phase 3
  int obuf;                         // output tiles in shared memory (2: a tile drains while the next one fills)
  int NMB, ncols;                   // tcgen05 phase 3: blocks of 128 own pixels, TMEM columns allocated
  int XP, PP, ZP, OP, FP1, FP2;     // row pitches (floats): stage channel, P plane, Z plane, output tile, factor planes
  int CoutPad;                      // rows of the Fout planes (multiple of 16, maximum over the two convolutions)
  int stage_floats;
  int oZ, oF1, oF2, oW, oBar;       // byte offsets from the shared-memory base (ring, P and the output tile at 0)
  int stagger;                      // cycles the producers of the second CTA per SM wait before their first load
  int sm_count;
  long long* trace;                 // diagnostics: 64 cycle stamps per CTA for the first 512 CTAs (null: off)
};

// Bounded wait on an mbarrier phase.  The first probe costs one instruction; only a wait that has to spin reads the
// clock.  Gives up after about a second, or as soon as another thread of the CTA has given up.
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

// ---- bulk asynchronous copies (the TMA engine without a tensor map) -------------------------------------------------
__device__ __forceinline__ void bulk_load(void* sdst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
               ::"r"(smem_u32(sdst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void consumers_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCons * 32) : "memory"); }

// NBW1: halo n-blocks (8 pixels) per consumer warp in phase 1; warp w owns blocks w, w + 9, w + 18, ...  Blocks past
// the band are computed on whatever the shared memory holds there and never stored: no mma sits under a branch.
// TC3: phase 3 on the fifth-generation tensor cores (tcgen05.mma, accumulators in TMEM) instead of mma.sync.
template <int RP, int NBW1, bool TC3>
__global__ void __launch_bounds__(kNT, RP <= 16 ? 2 : 1)
cp4_band_kernel(const BandGeom g, const __grid_constant__ CUtensorMap map0, const __grid_constant__ CUtensorMap map1,
                const BandProb p0, const BandProb p1) {
  constexpr int MB = RP / 16;    // rank m-blocks of phase 1
  constexpr int KS3 = RP / 8;    // k-steps of phase 3
  constexpr int NG = RP == 16 ? 5 : 3;   // phase-3 n-blocks a warp keeps in registers at a time
  // all pointers below are derived from this array by pointer arithmetic, so every access is a shared-space access;
  // the planner's offsets are multiples of 128 bytes and dynamic shared memory starts on a 1024-byte boundary
  extern __shared__ __align__(1024) uint8_t sm[];
  float* ring = reinterpret_cast<float*>(sm);         // [stages][CB][XP] during phase 1, then:
  float* Ps = ring;                                   //   [RP][PP]   rank plane on the halo band
  float* Os = ring;                                   //   [2][16][OP] output tiles of one channel block (P is dead by then)
  float* Zs = reinterpret_cast<float*>(sm + g.oZ);    //   [RP][ZP]   stencilled plane on the band's own pixels
  float* F1 = reinterpret_cast<float*>(sm + g.oF1);   // [2][RP][FP1]       hi | lo of Fin^T
  float* F2 = reinterpret_cast<float*>(sm + g.oF2);   // [2][CoutPad][FP2]  hi | lo of Fout
  float* Ws = reinterpret_cast<float*>(sm + g.oW);    // [9][RP]
  uint64_t* full = reinterpret_cast<uint64_t*>(sm + g.oBar);
  uint64_t* empty = full + kMaxStages;
  uint64_t* d2bar = empty + kMaxStages;               // [4] tcgen05 phase 3: accumulator of a pixel block complete
  volatile int* abort_flag = reinterpret_cast<volatile int*>(d2bar + 4);
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d2bar + 4) + 1;

  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int gq = lane >> 2, tq = lane & 3;
  const bool second = (int)blockIdx.x >= g.tiles;
  const BandProb p = second ? p1 : p0;
  const CUtensorMap* map = second ? &map1 : &map0;
  const int b = (int)blockIdx.x - (second ? g.tiles : 0);
  const int band = b % g.bands, n = b / g.bands;
  const int h0 = band * g.TH;
  const int W = g.W, HW = g.H * g.W, XP = g.XP, PP = g.PP, ZP = g.ZP, OP = g.OP, FP1 = g.FP1, FP2 = g.FP2;
  const int nst = (p.Cin + g.CB - 1) / g.CB;
  const int S = g.stages;
  // halo rows [ra, rb) of the band lie inside the image (halo row i is image row h0 - 1 + i)
  const int ra = h0 == 0 ? 1 : 0, rb = min(g.TH + 2, g.H - h0 + 1);
  if (smem_u32(sm) & (TC3 ? 1023 : 127)) {   // cannot happen with the launch this file does; never run on a misaligned base
    if (tid == 0) atomicCAS(&g_band_status, 0, (2 << 16) | (int)(blockIdx.x & 0xffff));
    return;
  }

  long long* tr = (g.trace != nullptr && blockIdx.x < 512 && (tid == 0 || tid == 256)) ? g.trace + (size_t)blockIdx.x * 64 + (tid ? 32 : 0) : nullptr;
  auto stamp = [&](int k) { if (tr) tr[k] = clock64(); };
  stamp(0);
  if (tid == 0) {
    for (int i = 0; i < S; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], kCons);
    }
    if (TC3)
      for (int i = 0; i < 4; ++i) mbar_init(&d2bar[i], 1);
    *abort_flag = 0;
    fence_barrier_init();
    if (g.tensor) tma_prefetch_desc(map);
  }
  __syncthreads();

  float acc[MB][NBW1][4];
  if (warp == kCons) {
    // ================= producer: streams the band's channels through the ring =====================================
    if (TC3) {   // this warp also owns the CTA's tensor memory: allocated here, released at the very end
      tc::tmem_alloc(tmem_slot, (uint32_t)g.ncols);
      tc::tc_fence_before_sync();
    }
    const uint32_t row_bytes = (uint32_t)W * 4u;
    const float* src0 = p.in + ((size_t)n * p.Cin * g.H + (size_t)(h0 - 1 + ra)) * W;   // channel 0, first row inside
    if (g.stagger > 0 && (int)blockIdx.x >= g.sm_count && (int)blockIdx.x < 2 * g.sm_count) {
      // Two CTAs share an SM and would otherwise load, compute and store in lockstep, leaving the memory system idle
      // while both compute: the second one asks for its input later, when the first one's has arrived.
      const long long t0 = clock64();
      while (clock64() - t0 < g.stagger) {}
    }
    int slot = 0;
    uint32_t par = 1;   // parity of the "empty" phase awaited: the wrap before the first wait flips it to 0
    for (int s = 0; s < nst; ++s) {
      if (s >= S && !wait_or_abort(&empty[slot], par, abort_flag)) break;   // all nine warps have left the stage
      float* dst = ring + (size_t)slot * g.stage_floats;
      if (g.tensor) {
        if (lane == 0) {
          mbar_expect_tx(&full[slot], (uint32_t)g.stage_floats * 4u);
          tma_load_4d(dst, map, &full[slot], 0, h0 - 1, s * g.CB, n);
        }
      } else {
        const int nch = min(g.CB, p.Cin - s * g.CB);
        const uint32_t bytes = (uint32_t)(rb - ra) * row_bytes;
        if (lane == 0) mbar_expect_tx(&full[slot], bytes * (uint32_t)nch);
        __syncwarp();
        if (lane < nch)
          bulk_load(dst + (size_t)lane * XP + ra * W, src0 + (size_t)(s * g.CB + lane) * HW, bytes, &full[slot]);
      }
      if (++slot == S) { slot = 0; par ^= 1; }
    }
  } else {
    // ================= consumers ======================================================================================
    // factor planes and stencil weights (the first stages are in flight meanwhile)
    {
      const int CinPad = nst * g.CB;
      const int kF1 = RP * FP1;
      constexpr int NTC = kCons * 32;
#pragma unroll 4
      for (int i = tid; i < RP * CinPad; i += NTC) {
        const int c = i / RP, r = i - c * RP;     // r fastest: contiguous reads of Fin[c][:]
        const float v = (r < g.R && c < p.Cin) ? __ldg(p.Fin + (size_t)c * g.Rs + g.r0 + r) : 0.f;
        const float hi = tf32_round(v);
        F1[r * FP1 + c] = hi;
        F1[kF1 + r * FP1 + c] = tf32_round(v - hi);
      }
      if (!TC3) {
        const int kF2 = g.CoutPad * FP2;
#pragma unroll 4
        for (int i = tid; i < g.CoutPad * RP; i += NTC) {
          const int t = i / RP, r = i - t * RP;
          const float v = (r < g.R && t < p.Cout) ? __ldg(p.Fout + (size_t)t * g.Rs + g.r0 + r) : 0.f;
          const float hi = tf32_round(v);
          F2[t * FP2 + r] = hi;
          F2[kF2 + t * FP2 + r] = tf32_round(v - hi);
        }
      }
      for (int i = tid; i < 9 * RP; i += NTC) {
        const int r = i % RP, yx = i / RP, y = yx / 3, x = yx - y * 3;
        const int yy = p.flip ? 2 - y : y, xx = p.flip ? 2 - x : x;
        // a free core [3][3][Rs] (three-factor CP conv) takes the place of the outer product KH x KW
        Ws[i] = r >= g.R ? 0.f
                : p.KC   ? __ldg(p.KC + (size_t)(yy * 3 + xx) * g.Rs + g.r0 + r)
                         : __ldg(p.KH + (size_t)yy * g.Rs + g.r0 + r) * __ldg(p.KW + (size_t)xx * g.Rs + g.r0 + r);
      }
      if (!g.tensor) {
        // what the bulk copies of this band never write must read as zero: halo rows outside the image (the
        // padding) in every slot, and the channels past Cin in the last stage's slot
        const int zr = ra + (g.TH + 2 - rb);   // rows outside: [0, ra) and [rb, TH + 2)
        if (zr > 0) {
          const int per = zr * W;
          for (int i = tid; i < S * g.CB * per; i += NTC) {
            const int ch = i / per, q = i - ch * per;
            const int row = q / W, col = q - row * W;
            const int hr = row < ra ? row : rb + (row - ra);
            ring[(size_t)(ch / g.CB) * g.stage_floats + (size_t)(ch % g.CB) * XP + hr * W + col] = 0.f;
          }
        }
        const int tail = nst * g.CB - p.Cin;   // channels of the last stage that do not exist
        if (tail > 0) {
          float* z0 = ring + (size_t)((nst - 1) % S) * g.stage_floats + (size_t)(g.CB - tail) * XP;
          for (int i = tid; i < tail * XP; i += NTC) z0[i] = 0.f;
        }
      }
    }
    consumers_sync();
    stamp(1);

    // ---- phase 1 --------------------------------------------------------------------------------------------------
#pragma unroll
    for (int m = 0; m < MB; ++m)
#pragma unroll
      for (int i = 0; i < NBW1; ++i)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[m][i][e] = 0.f;

    const int kF1 = RP * FP1;
    // ldmatrix row address of this lane: tile lane/8 = (rows 0-7 | 8-15) x (k 0-3 | 4-7)
    const float* fk = F1 + ((lane & 7) + ((lane >> 3) & 1) * 8) * FP1 + (lane >> 4) * 4;
    // B fragment of n-block i: channels tq and tq + 4, pixel (warp + 9 i) * 8 + gq  ->  fixed offsets 72 i from here
    const int xlane = tq * XP + warp * 8 + gq;
    const int XP4 = 4 * XP;
    const int nks = g.CB >> 3, total = nst * nks;
    // The loop runs over k-steps of 8 channels.  The raw values of step k + 1 are loaded while the tensor pipe
    // works on step k; a stage is handed back to the producer as soon as its last values sit in registers.
    int slot = 0, ks = 0;
    uint32_t par = 0;
    bool ok = wait_or_abort(&full[0], 0, abort_flag);
    ok = __all_sync(0xffffffffu, ok);
    const float* xs = ring + xlane;
    float xr[NBW1][2];
    if (ok) {
#pragma unroll
      for (int i = 0; i < NBW1; ++i) {
        xr[i][0] = xs[i * (kCons * 8)];
        xr[i][1] = xs[i * (kCons * 8) + XP4];
      }
    }
    for (int kk = 0; kk < total && ok; ++kk) {
      if (kk < 16) stamp(8 + kk);
      uint32_t bh[NBW1][2], bl[NBW1][2];
#pragma unroll
      for (int i = 0; i < NBW1; ++i) {
        split_tf32(xr[i][0], bh[i][0], bl[i][0]);
        split_tf32(xr[i][1], bh[i][1], bl[i][1]);
      }
      uint32_t ah[MB][4], al[MB][4];
#pragma unroll
      for (int m = 0; m < MB; ++m) {
        ldmatrix_x4(ah[m], fk + m * 16 * FP1);
        ldmatrix_x4(al[m], fk + m * 16 * FP1 + kF1);
      }
      fk += 8;
      const bool stage_done = ++ks == nks;
      if (stage_done) {
        __syncwarp();
        if (lane == 0) mbar_arrive(&empty[slot]);   // every lane of this warp holds its values of the stage
      }
#pragma unroll
      for (int i = 0; i < NBW1; ++i)
#pragma unroll
        for (int m = 0; m < MB; ++m) mma_tf32_ordered(acc[m][i], al[m], bh[i]);
#pragma unroll
      for (int i = 0; i < NBW1; ++i)
#pragma unroll
        for (int m = 0; m < MB; ++m) mma_tf32_ordered(acc[m][i], ah[m], bl[i]);
#pragma unroll
      for (int i = 0; i < NBW1; ++i)
#pragma unroll
        for (int m = 0; m < MB; ++m) mma_tf32_ordered(acc[m][i], ah[m], bh[i]);
      if (kk + 1 < total) {
        if (stage_done) {
          ks = 0;
          if (++slot == S) { slot = 0; par ^= 1; }
          ok = wait_or_abort(&full[slot], par, abort_flag);
          ok = __all_sync(0xffffffffu, ok);
          if (!ok) break;
          xs = ring + (size_t)slot * g.stage_floats + xlane;
        } else {
          xs += 8 * XP;
        }
#pragma unroll
        for (int i = 0; i < NBW1; ++i) {
          xr[i][0] = xs[i * (kCons * 8)];
          xr[i][1] = xs[i * (kCons * 8) + XP4];
        }
      }
    }
    stamp(2);
  }
  __syncthreads();   // the ring is free: every stage has landed and has been read
  const bool aborted = *abort_flag != 0;   // uniform: no thread is inside a wait at this point
  uint32_t tmem_base = 0;
  if (TC3) {
    tc::tc_fence_after_sync();
    tmem_base = *tmem_slot;
    // Fout as the B operand of tcgen05.mma (K-major core matrices, no swizzle): element (t, r) at
    // (t/8) * RP*32 + (r/4) * 128 + (t%8) * 16 + (r%4) * 4 bytes, hi | lo.  It takes the place of the phase-1 factor
    // planes, which nobody reads any more.
    uint8_t* b2 = sm + g.oF1;
    const int plane = g.CoutPad * RP * 4;
    for (int i = tid; i < g.CoutPad * RP; i += kNT) {
      const int t = i / RP, r = i - t * RP;
      const float v = (r < g.R && t < p.Cout) ? __ldg(p.Fout + (size_t)t * g.Rs + g.r0 + r) : 0.f;
      const float hi = tf32_round(v);
      const int o = (t >> 3) * (RP * 32) + (r >> 2) * 128 + (t & 7) * 16 + (r & 3) * 4;
      *reinterpret_cast<float*>(b2 + o) = hi;
      *reinterpret_cast<float*>(b2 + plane + o) = tf32_round(v - hi);
    }
  }

  // P fragments -> Ps[r][halo px]
  const int own_rows = min(g.TH, g.H - h0);            // band rows inside the image
  if (warp < kCons && !aborted) {
    float* pw = Ps + gq * PP + warp * 8 + 2 * tq;      // rank gq, this lane's pixel pair of the warp's first n-block
#pragma unroll
    for (int i = 0; i < NBW1; ++i) {
      if ((warp + kCons * i) * 8 + 2 * tq < g.NPH) {
#pragma unroll
        for (int m = 0; m < MB; ++m) {
          *reinterpret_cast<float2*>(pw + m * 16 * PP + i * (kCons * 8)) = make_float2(acc[m][i][0], acc[m][i][1]);
          *reinterpret_cast<float2*>(pw + (m * 16 + 8) * PP + i * (kCons * 8)) = make_float2(acc[m][i][2], acc[m][i][3]);
        }
      }
    }
  }
  __syncthreads();
  stamp(3);
  // the band's own rows of the plane also go to global memory when the caller wants them (the factor gradients of
  // the same training step start from them): 16 bytes per lane, whole lines per warp instruction
  if (p.save != nullptr && !aborted) {
    const unsigned n4 = (unsigned)(own_rows * W) >> 2;   // float4 per rank
    const unsigned inv = n4 ? (1u << 20) / n4 + 1 : 0;
    float* sv = p.save + ((size_t)n * g.Rs + g.r0) * HW + (size_t)h0 * W;
#pragma unroll 5
    for (unsigned idx = tid; idx < (unsigned)g.R * n4; idx += kNT) {
      const unsigned r = (idx * inv) >> 20, i = idx - r * n4;
      *reinterpret_cast<float4*>(sv + (size_t)r * HW + 4 * i) = *reinterpret_cast<const float4*>(Ps + r * PP + W + 4 * i);
    }
  }

  // ---- phase 2: 3x3 stencil per rank, strips of 8 pixels ----------------------------------------------------------
  if (!aborted) {
    static_assert(kNT % RP == 0, "a thread keeps one rank: its nine weights stay in registers");
    const int spr = (W + 7) >> 3;
    const int nitems = g.TH * spr;
    const int r = tid % RP;
    float w[9];
#pragma unroll
    for (int t = 0; t < 9; ++t) w[t] = Ws[t * RP + r];
    int oy = (tid / RP) / spr, sx = (tid / RP) % spr;
    constexpr int STEP = kNT / RP;
    const int dy_step = STEP / spr, dx_step = STEP % spr;
    for (int it = tid / RP; it < nitems; it += STEP) {
      const int x0 = sx * 8;
      const bool hi_ok = x0 + 4 < W, lft = x0 > 0, rgt = x0 + 8 < W;
      float z[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) z[j] = 0.f;
      const float* pr = Ps + r * PP + oy * W + x0;
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
      if (TC3) {
        // Z as the A operand of tcgen05.mma, already split: blocks of 128 pixels x 8 ranks, pixels contiguous
        // ("MN-major"), rows of 32 pixels = 128 bytes per rank, the four 32-byte chunks of a row permuted by the
        // rank (the 128-byte swizzle with 32-byte atoms); hi plane, then lo plane
        uint8_t* zp = reinterpret_cast<uint8_t*>(Zs) + (r >> 3) * 4096 + (r & 7) * 128;
        const int planeZ = g.NMB * KS3 * 4096;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          if (h == 0 || hi_ok) {
            const int q = oy * W + x0 + 4 * h;
            const int o = (q >> 7) * (KS3 * 4096) + ((q & 127) >> 5) * 1024 + ((((q & 31) >> 3) ^ (r & 3)) << 5) + (q & 7) * 4;
            float4 hi4, lo4;
            hi4.x = tf32_round(z[4 * h + 0]); hi4.y = tf32_round(z[4 * h + 1]);
            hi4.z = tf32_round(z[4 * h + 2]); hi4.w = tf32_round(z[4 * h + 3]);
            lo4.x = z[4 * h + 0] - hi4.x; lo4.y = z[4 * h + 1] - hi4.y; lo4.z = z[4 * h + 2] - hi4.z; lo4.w = z[4 * h + 3] - hi4.w;
            *reinterpret_cast<float4*>(zp + o) = hi4;
            *reinterpret_cast<float4*>(zp + planeZ + o) = lo4;
          }
        }
      } else {
        float* zd = Zs + r * ZP + oy * W + x0;
        *reinterpret_cast<float4*>(zd) = make_float4(z[0], z[1], z[2], z[3]);
        if (hi_ok) *reinterpret_cast<float4*>(zd + 4) = make_float4(z[4], z[5], z[6], z[7]);
      }
      oy += dy_step;
      sx += dx_step;
      if (sx >= spr) { sx -= spr; ++oy; }
    }
  }
  if (TC3) {
    tc::fence_proxy_async();     // this thread's writes of Z and of the Fout operand become visible to the tensor core
    tc::tc_fence_before_sync();
  }
  __syncthreads();
  stamp(4);

  if (TC3) {
    // ---- phase 3 on tcgen05 ------------------------------------------------------------------------------------------
    // out[px, t] = sum_r Z[px, r] Fout[t, r] per block of 128 own pixels: M = 128, N = CoutPad, K = 8 ranks per
    // instruction, three instructions per K step (lo*hi + hi*lo + hi*hi), accumulators in tensor memory, one column
    // range per pixel block.  One thread issues everything; each block's completion arrives on its own mbarrier and
    // the warps read their lane quarter out (tcgen05.ld) and store it: a warp instruction writes 32 consecutive pixels
    // of one channel, i.e. one whole line.
    const int vpx = own_rows * W;
    if (!aborted && warp == kCons && lane == 0) {
      tc::tc_fence_after_sync();
      const uint32_t idesc = tc::make_idesc_tf32((uint32_t)g.CoutPad, 1, 0);
      const uint64_t dA = tc::make_smem_desc(0, 1024, 512, tc::kSwizzle128B_32B);
      const uint64_t dB = tc::make_smem_desc(0, 128, RP * 32, tc::kSwizzleNone);
      const uint32_t zhi = smem_u32(Zs), zlo = zhi + (uint32_t)(g.NMB * KS3 * 4096);
      const uint32_t bhi = smem_u32(sm + g.oF1), blo = bhi + (uint32_t)(g.CoutPad * RP * 4);
      for (int mb = 0; mb < g.NMB; ++mb) {
        const uint32_t tD = tmem_base + (uint32_t)(mb * g.CoutPad);
#pragma unroll
        for (int ks = 0; ks < KS3; ++ks) {
          const uint32_t ao = (uint32_t)((mb * KS3 + ks) * 4096), bo = (uint32_t)(ks * 256);
          const uint64_t ah = dA + (uint64_t)((zhi + ao) >> 4), al = dA + (uint64_t)((zlo + ao) >> 4);
          const uint64_t bh = dB + (uint64_t)((bhi + bo) >> 4), bl = dB + (uint64_t)((blo + bo) >> 4);
          tc::mma_tf32_ss(tD, al, bh, idesc, ks != 0);
          tc::mma_tf32_ss(tD, ah, bl, idesc, true);
          tc::mma_tf32_ss(tD, ah, bh, idesc, true);
        }
        tc::mma_commit(&d2bar[mb]);
      }
    }
    if (!aborted) {
      const int qd = warp & 3;                       // the TMEM lane quarter this warp may read
      const int nq = (kWarps - qd + 3) >> 2;         // warps that share it
      float* outp = p.out + (size_t)n * p.Cout * HW + (size_t)h0 * W;
      for (int mb = warp >> 2; mb < g.NMB; mb += nq) {
        if (mb * 128 + qd * 32 >= vpx) continue;     // nothing of this quarter lies inside the band
        if (mb < 4) stamp(16 + 4 * mb);
        bool ok3 = wait_or_abort(&d2bar[mb], 0, abort_flag);
        ok3 = __all_sync(0xffffffffu, ok3);
        if (!ok3) break;
        if (mb < 4) stamp(17 + 4 * mb);
        tc::tc_fence_after_sync();
        const int px = mb * 128 + qd * 32 + lane;
        float* o = outp + px;
        const uint32_t ta = tmem_base + ((uint32_t)(qd * 32) << 16) + (uint32_t)(mb * g.CoutPad);
        for (int c0 = 0; c0 < g.CoutPad; c0 += 16) {
          float v[16];
          tc::tmem_ld16(ta + (uint32_t)c0, v);
          if (px < vpx) {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (c0 + i < p.Cout) o[(size_t)(c0 + i) * HW] = v[i];
          }
        }
        if (mb < 4) stamp(18 + 4 * mb);
      }
    }
    stamp(5);
    tc::tc_fence_before_sync();
    __syncthreads();
    if (warp == kCons) {
      tc::tc_fence_after_sync();
      tc::tmem_dealloc(tmem_base, (uint32_t)g.ncols);
    }
    if (*abort_flag) {
      if (tid == 0) atomicCAS(&g_band_status, 0, (1 << 16) | (int)(blockIdx.x & 0xffff));
      const long long t0 = clock64();
      while (clock64() - t0 < 400000) {}
    }
    return;
  }

  // ---- phase 3 ----------------------------------------------------------------------------------------------------
  // n-block nb = warp + 10 i covers own pixels [8 nb, 8 nb + 8); a group of NG blocks per warp covers 80 NG
  // consecutive pixels.  Per group and per block of 16 output channels: mma -> registers -> one of two output tiles in
  // shared memory -> barrier -> all threads copy the tile out, 16 bytes per lane, so every warp instruction writes
  // whole lines.  With two tiles one barrier per round is enough: whoever refills a tile has passed the barrier of
  // the round in between, which every thread reaches only after its reads of that tile.
  if (!aborted) {
    const int kF2 = g.CoutPad * FP2;
    const int vpx = own_rows * W;                       // own pixels inside the image
    float* outp = p.out + (size_t)n * p.Cout * HW + (size_t)h0 * W;
    const float* f2row = F2 + ((lane & 7) + ((lane >> 3) & 1) * 8) * FP2 + (lane >> 4) * 4;
    const int nbw3 = (g.NB3 + kWarps - 1) / kWarps;
    const int mbs = (p.Cout + 15) >> 4;
    int round = 0;
    for (int i0 = 0; i0 < nbw3; i0 += NG) {
      const int px_lo = i0 * kWarps * 8;
      const unsigned n4 = (unsigned)max(0, min(vpx, (i0 + NG) * kWarps * 8) - px_lo) >> 2;   // float4 per channel
      const unsigned inv = n4 ? (1u << 20) / n4 + 1 : 0;   // idx / n4 == (idx * inv) >> 20 for idx < 8192
      uint32_t zh[NG][KS3][2], zl[NG][KS3][2];
      {
        const float* zb = Zs + tq * ZP + (warp + kWarps * i0) * 8 + gq;
#pragma unroll
        for (int j = 0; j < NG; ++j)
#pragma unroll
          for (int ks = 0; ks < KS3; ++ks) {
            split_tf32(zb[ks * 8 * ZP + j * (kWarps * 8)], zh[j][ks][0], zl[j][ks][0]);
            split_tf32(zb[(ks * 8 + 4) * ZP + j * (kWarps * 8)], zh[j][ks][1], zl[j][ks][1]);
          }
      }
      for (int m = 0; m < mbs; ++m, ++round) {
        uint32_t ah[KS3][4], al[KS3][4];
        const float* fm = f2row + m * 16 * FP2;
#pragma unroll
        for (int ks = 0; ks < KS3; ++ks) {
          ldmatrix_x4(ah[ks], fm + ks * 8);
          ldmatrix_x4(al[ks], fm + ks * 8 + kF2);
        }
        float d[NG][4];
#pragma unroll
        for (int j = 0; j < NG; ++j) d[j][0] = d[j][1] = d[j][2] = d[j][3] = 0.f;
#pragma unroll
        for (int ks = 0; ks < KS3; ++ks) {
#pragma unroll
          for (int j = 0; j < NG; ++j) mma_tf32_ordered(d[j], al[ks], zh[j][ks]);
#pragma unroll
          for (int j = 0; j < NG; ++j) mma_tf32_ordered(d[j], ah[ks], zl[j][ks]);
#pragma unroll
          for (int j = 0; j < NG; ++j) mma_tf32_ordered(d[j], ah[ks], zh[j][ks]);
        }
        if (round < 4) stamp(16 + 4 * round);
        float* ot = Os + (g.obuf == 2 ? (round & 1) * 16 * OP : 0);
        if (g.obuf == 1 && round > 0) __syncthreads();   // one tile only: everybody has copied the previous round out
        float* o = ot + gq * OP + warp * 8 + 2 * tq;
#pragma unroll
        for (int j = 0; j < NG; ++j) {
          *reinterpret_cast<float2*>(o + j * (kWarps * 8)) = make_float2(d[j][0], d[j][1]);
          *reinterpret_cast<float2*>(o + 8 * OP + j * (kWarps * 8)) = make_float2(d[j][2], d[j][3]);
        }
        if (round < 4) stamp(17 + 4 * round);
        __syncthreads();   // tile full
        if (round < 4) stamp(18 + 4 * round);
        const unsigned cnt = (unsigned)min(16, p.Cout - m * 16) * n4;
        float* om = outp + (size_t)(m * 16) * HW + px_lo;
        if (p.accumulate) {
          for (unsigned idx = tid; idx < cnt; idx += kNT) {
            const unsigned c = (idx * inv) >> 20, i = idx - c * n4;
            const float4 a = *reinterpret_cast<const float4*>(ot + c * OP + 4 * i);
            float4* q = reinterpret_cast<float4*>(om + (size_t)c * HW + 4 * i);
            const float4 v = *q;
            *q = make_float4(a.x + v.x, a.y + v.y, a.z + v.z, a.w + v.w);
          }
        } else {
#pragma unroll 5
          for (unsigned idx = tid; idx < cnt; idx += kNT) {
            const unsigned c = (idx * inv) >> 20, i = idx - c * n4;
            *reinterpret_cast<float4*>(om + (size_t)c * HW + 4 * i) = *reinterpret_cast<const float4*>(ot + c * OP + 4 * i);
          }
        }
        if (round < 4) stamp(19 + 4 * round);
      }
    }
  }
  stamp(5);
  if (tr) { unsigned smid; asm("mov.u32 %0, %%smid;" : "=r"(smid)); tr[6] = smid; }
  if (aborted) {
    if (tid == 0) atomicCAS(&g_band_status, 0, (1 << 16) | (int)(blockIdx.x & 0xffff));
    // bulk copies that may still be in flight towards this CTA's shared memory get time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) {}
  }
}

// ---- tensor maps: (W, H, C, N) view of an NCHW tensor, box (W, TH + 2, CB, 1) --------------------------------------
struct MapKey {
  const void* ptr;
  int N, C, H, W, rows, cb;
  bool operator==(const MapKey& o) const { return std::memcmp(this, &o, sizeof(MapKey)) == 0; }
};
struct MapSlot {
  MapKey key{};
  CUtensorMap map;
  bool used = false;
};
// a few recent maps per host thread: a training loop calls with the same buffers again and again
thread_local MapSlot t_maps[16];
thread_local int t_map_next = 0;

int band_map(const float* ptr, int N, int C, int H, int W, int rows, int cb, CUtensorMap* out) {
  MapKey k;
  std::memset(&k, 0, sizeof(k));
  k.ptr = ptr; k.N = N; k.C = C; k.H = H; k.W = W; k.rows = rows; k.cb = cb;
  for (auto& s : t_maps)
    if (s.used && s.key == k) {
      *out = s.map;
      return B200CP_OK;
    }
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B200CP_ERR_NO_DEVICE, "cuTensorMapEncodeTiled entry point not available");
  const cuuint64_t gdim[4] = {(cuuint64_t)W, (cuuint64_t)H, (cuuint64_t)C, (cuuint64_t)N};
  const cuuint64_t gstr[3] = {(cuuint64_t)W * 4, (cuuint64_t)H * W * 4, (cuuint64_t)C * H * W * 4};
  const cuuint32_t box[4] = {(cuuint32_t)W, (cuuint32_t)rows, (cuuint32_t)cb, 1};
  const cuuint32_t estr[4] = {1, 1, 1, 1};
  CUtensorMap m;
  const CUresult cr = enc(&m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 4, const_cast<float*>(ptr), gdim, gstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(B200CP_ERR_CUDA, "cuTensorMapEncodeTiled (band map) failed with code %d", (int)cr);
  MapSlot& s = t_maps[t_map_next];
  t_map_next = (t_map_next + 1) % 16;
  s.key = k; s.map = m; s.used = true;
  *out = m;
  return B200CP_OK;
}

int pitch_mod32(int n, int want) {   // smallest multiple-of-4 pitch >= n with pitch % 32 == want
  int p = (n + 3) / 4 * 4;
  while (p % 32 != want) p += 4;
  return p;
}

int pitch_mod16(int n, int want) {   // smallest multiple-of-4 pitch >= n with pitch % 16 == want
  int p = (n + 3) / 4 * 4;
  while (p % 16 != want) p += 4;
  return p;
}

std::atomic<long long*> g_band_trace{nullptr};
std::atomic<int> g_band_tensor{[] {   // input loads: 1 = 4-D tensor-map boxes, 0 = 1-D bulk copies per channel (default)
  const char* e = getenv("B200CP_BAND_TENSOR");
  return e ? atoi(e) : 0;
}()};
std::atomic<int> g_band_th{[] {   // forced band height: B200CP_BAND_TH at load, b200cp_test_set_band_rows later
  const char* e = getenv("B200CP_BAND_TH");
  return e ? atoi(e) : 0;
}()};

struct BandPlan {
  BandGeom g;
  int RP, NBW1;
  bool tc3;
  size_t smem;
  int per_sm;
};

int next_pow2_cols(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

// Phase 3 on tcgen05 (B200CP_BAND_TC3=1, or the test hook) or on mma.sync (default).  Measured at N=32, C=T=64,
// 56x56, R=16: 23.3 us against 21.9 us -- the accumulators leave tensor memory one pixel per lane, so the stores are
// 4 bytes per lane, and the stencil has to write its result split and swizzled; the mma.sync form copies its
// staged tile out 16 bytes per lane.
std::atomic<int> g_band_tc3{[] {
  const char* e = getenv("B200CP_BAND_TC3");
  return e ? atoi(e) : 0;
}()};
// Cycles by which the producer of the second CTA of every SM delays its first load (B200CP_BAND_STAGGER).  Two CTAs
// that start together load, compute and store in lockstep; a shift of about 1.5 us lets one compute while the
// other's input arrives (measured: 22.5 -> 21.0 us per convolution at the size above).
const int g_band_stagger = [] {
  const char* e = getenv("B200CP_BAND_STAGGER");
  return e ? atoi(e) : 3000;
}();

bool fill_plan(int RP, int N, int H, int W, int Cin_max, int Cout_max, int TH, int tensor, bool want_tc3,
               const DeviceInfo& di, BandPlan* out) {
  BandGeom g{};
  g.N = N; g.H = H; g.W = W;
  g.TH = TH;
  g.NPH = (TH + 2) * W;
  g.OPX = TH * W;
  g.tensor = tensor;
  if (tensor) {
    // the box lands densely: the channel pitch is the halo band itself, and most heights collide in shared memory
    // (the B-fragment loads of a warp hit 32 different banks only when the pitch is 8 or 24 modulo 32)
    if (g.NPH % 32 != 8 && g.NPH % 32 != 24) return false;
    g.XP = g.NPH;
  } else {
    g.XP = pitch_mod32(g.NPH + 4, 8);
  }
  g.NB3 = ceil_div(g.OPX, 8);
  const int NBW1 = ceil_div(ceil_div(g.NPH, 8), kCons);
  if (NBW1 > 8 || (RP / 16) * NBW1 * 4 > 64) return false;   // phase-1 accumulators per thread
  g.bands = ceil_div(H, TH);
  g.tiles = N * g.bands;
  g.CB = 8;   // stage: about 16 KB
  while (g.CB < 32 && 2 * g.CB * g.XP * 4 <= 17 * 1024 && 2 * g.CB <= (Cin_max + 7) / 8 * 8) g.CB *= 2;
  g.stage_floats = g.CB * g.XP;
  g.PP = pitch_mod32(g.NPH, 4);
  g.ZP = pitch_mod32(g.OPX + 4, 8);
  const int NG = RP == 16 ? 5 : 3;
  g.OP = pitch_mod16(NG * kWarps * 8, 8);   // 8 or 24 modulo 32: the 8-byte fragment stores of a warp do not collide
  const int CinPad = ceil_div(Cin_max, g.CB) * g.CB;
  g.FP1 = CinPad + 4;
  g.FP2 = RP + 4;
  g.CoutPad = (Cout_max + 15) / 16 * 16;
  // tcgen05 phase 3: the accumulators of all pixel blocks must fit the CTA's share of tensor memory
  g.NMB = ceil_div(g.OPX, 128);
  g.ncols = next_pow2_cols(g.NMB * g.CoutPad);
  const int cap0 = RP <= 16 ? 2 : 1;
  const bool tc3 = want_tc3 && RP == 16 && g.CoutPad <= 256 && g.ncols * cap0 <= 512;
  const size_t planeP = align_up((size_t)RP * g.PP * 4, 1024);
  const size_t planeZ = tc3 ? (size_t)2 * g.NMB * (RP / 8) * 4096 : align_up((size_t)RP * g.ZP * 4, 128);
  const size_t tile = tc3 ? 0 : (size_t)16 * g.OP * 4;
  // blocks past the band read up to this far behind the last stage
  const size_t slack = (size_t)std::max(0, kCons * 8 * NBW1 - g.XP) * 4 + 128;
  const size_t f1 = (size_t)2 * RP * g.FP1 * 4;
  const size_t f2 = (size_t)2 * g.CoutPad * (tc3 ? RP : g.FP2) * 4;   // tcgen05: dense operand in place of the F1 planes
  const size_t fixed = (tc3 ? align_up(std::max(f1, f2), 128) : f1 + f2) + (size_t)9 * RP * 4 + 128 + 256;
  const int nst = ceil_div(Cin_max, g.CB);
  const int cap = RP <= 16 ? 2 : 1;   // the kernel's launch bounds
  // ring depth: as deep as two resident CTAs allow, at least three stages.  After phase 1 the ring's space holds the
  // planes: P (then the output tiles) from its start, Z at its end.
  int S = std::min(kMaxStages, std::max(2, nst));
  size_t ring = 0, total = 0;
  for (;; --S) {
    ring = align_up(std::max((size_t)S * g.stage_floats * 4 + slack, std::max(planeP, tile) + planeZ), 1024);
    total = ring + fixed;
    if (S <= 3 || total + 1024 <= (size_t)(228 * 1024) / cap) break;
  }
  // a second output tile (one drains while the next fills) where it costs no residency
  const size_t ring2 = std::max(ring, align_up(2 * tile + planeZ, 1024));
  if (!tc3 && (ring2 + fixed + 1024 <= (size_t)(228 * 1024) / cap || (ring2 + fixed) / 1024 == total / 1024)) {
    ring = ring2;
    total = ring + fixed;
  }
  if ((int)total > di.smem_optin) return false;
  g.stages = S;
  g.oZ = (int)(ring - planeZ);
  g.obuf = 2 * tile <= (size_t)g.oZ ? 2 : 1;
  size_t o = ring;
  g.oF1 = (int)o;
  if (tc3) {
    g.oF2 = g.oF1;
    o += align_up(std::max(f1, f2), 128);
  } else {
    o += f1;
    g.oF2 = (int)o; o += f2;
  }
  g.oW = (int)o; o += (size_t)9 * RP * 4;
  o = align_up(o, 16);
  g.oBar = (int)o; o += 256;
  out->g = g;
  out->RP = RP;
  out->NBW1 = NBW1;
  out->tc3 = tc3;
  out->smem = o;
  out->per_sm = std::max(1, std::min(cap, (int)((228 * 1024) / (out->smem + 1024))));
  return true;
}

// band height: least estimated time.  A band costs its two contractions (halo rows for the first) plus a fixed part;
// the busiest SM runs ceil(tiles / SMs) of them, and two resident CTAs overlap each other's phases.
bool plan_band_search(int RP, int N, int H, int W, int Cin, int Cout, int nconv, int tensor, bool want_tc3, int forced,
                      const DeviceInfo& di, BandPlan* best);

// The search runs once per shape: a training loop asks for the same few plans again and again.
bool plan_band(int RP, int N, int H, int W, int Cin, int Cout, int nconv, bool accumulate, const DeviceInfo& di,
               BandPlan* best) {
  const int tensor = g_band_tensor.load(std::memory_order_relaxed);
  const bool want_tc3 = !accumulate && g_band_tc3.load(std::memory_order_relaxed) != 0;
  const int forced = g_band_th.load(std::memory_order_relaxed);
  struct Entry {
    int key[12];
    bool ok;
    BandPlan plan;
  };
  thread_local Entry cache[8];
  thread_local int used = 0, next = 0;
  const int key[12] = {RP, N, H, W, Cin, Cout, nconv, tensor, want_tc3 ? 1 : 0, forced, di.sm_count, di.smem_optin};
  for (int i = 0; i < used; ++i)
    if (std::memcmp(cache[i].key, key, sizeof(key)) == 0) {
      if (cache[i].ok) *best = cache[i].plan;
      return cache[i].ok;
    }
  Entry& e = cache[next];
  next = (next + 1) % 8;
  used = std::min(used + 1, 8);
  std::memcpy(e.key, key, sizeof(key));
  e.ok = plan_band_search(RP, N, H, W, Cin, Cout, nconv, tensor, want_tc3, forced, di, &e.plan);
  if (e.ok) *best = e.plan;
  return e.ok;
}

bool plan_band_search(int RP, int N, int H, int W, int Cin, int Cout, int nconv, int tensor, bool want_tc3, int forced,
                      const DeviceInfo& di, BandPlan* best) {
  if (forced) {
    // the first height from the forced one upwards that the kernel can take
    for (int TH = std::min(forced, H); TH <= std::min(H, 62); ++TH)
      if (fill_plan(RP, N, H, W, Cin, Cout, TH, tensor, want_tc3, di, best)) return true;
    return false;
  }
  double best_cost = 1e300;
  bool found = false;
  for (int TH = 1; TH <= std::min(H, 62); ++TH) {
    BandPlan pl;
    if (!fill_plan(RP, N, H, W, Cin, Cout, TH, tensor, want_tc3, di, &pl)) continue;
    const long tiles = (long)nconv * pl.g.tiles;
    const long per_sm = (tiles + di.sm_count - 1) / di.sm_count;
    const double tile = (double)(TH + 2) * W * (Cin + 24.0) + (double)TH * W * (Cout + 40.0) + 6000.0;
    const double cost = per_sm * tile * (pl.per_sm >= 2 ? 1.0 : 1.35);
    if (cost < best_cost) { best_cost = cost; *best = pl; found = true; }
  }
  return found;
}

template <int RP, int NBW1, bool TC3>
int launch_band(const BandPlan& pl, const CUtensorMap& m0, const CUtensorMap& m1, const BandProb& p0, const BandProb& p1,
                int nconv, cudaStream_t st) {
  auto kern = cp4_band_kernel<RP, NBW1, TC3>;
  static std::atomic<int> smem_set[64];
  B200CP_CUDA_OK(ensure_dynamic_smem(reinterpret_cast<const void*>(kern), smem_set, (int)pl.smem));
  const long ctas = (long)nconv * pl.g.tiles;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4: too many tiles");
  kern<<<(unsigned)ctas, kNT, pl.smem, st>>>(pl.g, m0, m1, p0, p1);
  B200CP_LAUNCH_OK("cp4_band_kernel");
  return B200CP_OK;
}

const bool g_band_off = [] {
  const char* e = getenv("B200CP_BAND");
  return e && e[0] == '0';
}();

// Ranks above 16 need two rank m-blocks per warp and one CTA per SM; at N=64, C=T=128, 28x28, R=32 that measures
// 37.2 us per convolution against 32.8 us for the tile kernel, so the bands take them only on request
// (B200CP_BAND_MAX_RANK=32, or the test hook).
std::atomic<int> g_band_max_rank{[] {
  const char* e = getenv("B200CP_BAND_MAX_RANK");
  return e ? std::max(1, std::min(32, atoi(e))) : 16;
}()};

bool band_shape_ok(const Cp4Args& a) {
  if (g_band_off) return false;
  if (a.R > g_band_max_rank.load(std::memory_order_relaxed)) return false;
  if (a.Y != 3 || a.X != 3 || a.pad != 1) return false;
  if (a.W % 4 != 0 || a.W > 256 || a.H < 1 || a.R > 32) return false;
  if ((reinterpret_cast<uintptr_t>(a.in) & 15) || (reinterpret_cast<uintptr_t>(a.out) & 15)) return false;   // bulk copies
  if (a.save && (reinterpret_cast<uintptr_t>(a.save) & 15)) return false;
  return true;
}

BandProb make_prob(const Cp4Args& a) {
  BandProb p{};
  p.in = a.in; p.Fin = a.Fin; p.Fout = a.Fout; p.KH = a.KH; p.KW = a.KW; p.KC = a.KC; p.out = a.out; p.save = a.save;
  p.Cin = a.Cin; p.Cout = a.Cout; p.flip = a.flip; p.accumulate = a.accumulate;
  return p;
}

}  // namespace

// One or two convolutions (same image size, batch and rank range) in one launch.  *done = false: not a shape this
// kernel takes; the caller uses another path.
int cp4_band_launch(const Cp4Args* convs, int nconv, cudaStream_t st, bool* done) {
  *done = false;
  if (nconv < 1 || nconv > 2) return B200CP_OK;
  const Cp4Args& a = convs[0];
  for (int i = 0; i < nconv; ++i) {
    const Cp4Args& c = convs[i];
    if (!band_shape_ok(c) || c.N != a.N || c.H != a.H || c.W != a.W || c.R != a.R || c.Rs != a.Rs || c.r0 != a.r0) return B200CP_OK;
  }
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  const int RP = a.R <= 16 ? 16 : 32;
  int cin = 0, cout = 0;
  for (int i = 0; i < nconv; ++i) { cin = std::max(cin, convs[i].Cin); cout = std::max(cout, convs[i].Cout); }
  BandPlan pl;
  bool accumulate = false;
  for (int i = 0; i < nconv; ++i) accumulate = accumulate || convs[i].accumulate;
  if (!plan_band(RP, a.N, a.H, a.W, cin, cout, nconv, accumulate, di, &pl)) return B200CP_OK;
  pl.g.R = a.R; pl.g.Rs = a.Rs; pl.g.r0 = a.r0;
  pl.g.trace = g_band_trace.load(std::memory_order_relaxed);
  pl.g.sm_count = di.sm_count;
  pl.g.stagger = g_band_stagger;
  CUtensorMap m[2];
  BandProb p[2];
  std::memset(m, 0, sizeof(m));
  for (int i = 0; i < 2; ++i) {
    const Cp4Args& c = convs[i < nconv ? i : 0];
    if (pl.g.tensor)
      if (int rc = band_map(c.in, c.N, c.Cin, c.H, c.W, pl.g.TH + 2, pl.g.CB, &m[i])) return rc;
    p[i] = make_prob(c);
  }
  static const bool debug = getenv("B200CP_DEBUG") != nullptr;
  if (debug)
    fprintf(stderr, "[b200cp] band TH=%d bands=%d CB=%d stages=%d tensor=%d obuf=%d tc3=%d NMB=%d ncols=%d RP=%d NBW1=%d smem=%zu per_sm=%d convs=%d\n",
            pl.g.TH, pl.g.bands, pl.g.CB, pl.g.stages, pl.g.tensor, pl.g.obuf, (int)pl.tc3, pl.g.NMB, pl.g.ncols, pl.RP, pl.NBW1, pl.smem, pl.per_sm, nconv);
  int rc = B200CP_ERR_UNSUPPORTED;
#define BAND_CASE(RPV, NB) case NB: rc = launch_band<RPV, NB, false>(pl, m[0], m[1], p[0], p[1], nconv, st); break;
#define BAND_CASE_TC(NB) case NB: rc = launch_band<16, NB, true>(pl, m[0], m[1], p[0], p[1], nconv, st); break;
  if (pl.tc3) {
    switch (pl.NBW1) { BAND_CASE_TC(1) BAND_CASE_TC(2) BAND_CASE_TC(3) BAND_CASE_TC(4) BAND_CASE_TC(5) BAND_CASE_TC(6)
                       BAND_CASE_TC(7) BAND_CASE_TC(8) }
  } else if (pl.RP == 16) {
    switch (pl.NBW1) { BAND_CASE(16, 1) BAND_CASE(16, 2) BAND_CASE(16, 3) BAND_CASE(16, 4) BAND_CASE(16, 5) BAND_CASE(16, 6)
                       BAND_CASE(16, 7) BAND_CASE(16, 8) }
  } else {
    switch (pl.NBW1) { BAND_CASE(32, 1) BAND_CASE(32, 2) BAND_CASE(32, 3) BAND_CASE(32, 4) BAND_CASE(32, 5) BAND_CASE(32, 6)
                       BAND_CASE(32, 7) BAND_CASE(32, 8) }
  }
#undef BAND_CASE
#undef BAND_CASE_TC
  if (rc) return rc;
  *done = true;
  return B200CP_OK;
}

// (W, H, C, N) view of an NCHW tensor with box (W, rows, cb, 1), from the per-thread cache of recent maps
int band_tensor_map(const float* ptr, int N, int C, int H, int W, int rows, int cb, CUtensorMap* out) {
  return band_map(ptr, N, C, H, W, rows, cb, out);
}

void band_set_max_rank(int r) { g_band_max_rank.store(std::max(1, std::min(32, r))); }
void band_force_rows(int rows) { g_band_th.store(rows > 0 ? rows : 0); }
void band_force_tensor(int on) { g_band_tensor.store(on ? 1 : 0); }
void band_force_tc3(int on) { g_band_tc3.store(on ? 1 : 0); }
void band_set_trace(long long* p) { g_band_trace.store(p); }
long long* band_trace_buffer() { return g_band_trace.load(std::memory_order_relaxed); }

int band_device_status(int* out) {
  int v = 0, zero = 0;
  B200CP_CUDA_OK(cudaDeviceSynchronize());
  B200CP_CUDA_OK(cudaMemcpyFromSymbol(&v, g_band_status, sizeof(int)));
  if (v) B200CP_CUDA_OK(cudaMemcpyToSymbol(g_band_status, &zero, sizeof(int)));
  *out = v;
  return B200CP_OK;
}

}  // namespace b200cp

extern "C" void b200cp_test_set_band_rows(int rows) { b200cp::band_force_rows(rows); }
extern "C" void b200cp_test_set_band_max_rank(int rank) { b200cp::band_set_max_rank(rank); }
extern "C" void b200cp_test_set_band_tensor_loads(int on) { b200cp::band_force_tensor(on); }
extern "C" void b200cp_test_set_band_tcgen05(int on) { b200cp::band_force_tc3(on); }
extern "C" void b200cp_test_set_band_trace(void* device_buffer) { b200cp::band_set_trace(static_cast<long long*>(device_buffer)); }
