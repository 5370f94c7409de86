// CP4 conv2d forward / backward-data on the 5th-generation tensor cores (tcgen05, TMEM, TMA).
//
// One CTA owns a band of TH full-width rows of one image, addressed as a flat pixel range so
// that the halo is a contiguous range too.  The rank-R intermediate stays on chip:
//
//   TMA      in[n, c-chunk, flat px] -> smem, 128B span / 32B atom swizzle, pixels contiguous (MN-major A operand)
//   SIMT     split every fp32 into hi = tf32(x) and lo = x - hi (3-term split, fp32-grade accuracy)
//   tcgen05  P[px, r]  = sum_c in[px, c] * Fin[c, r]          accumulators in TMEM
//   SIMT     TMEM -> smem Ps[r][px]; per-rank Y x X stencil -> Z[px, r] (hi / lo) as a K-major A operand
//   tcgen05  out[px, t] = sum_r Z[px, r] * Fout[t, r]          accumulators in TMEM
//   SIMT     TMEM -> registers -> coalesced global stores
//
// Forward uses Fin = K1, Fout = K0; backward-data swaps them and flips the taps.  Zero padding
// comes from the TMA out-of-bounds fill (rows) and a per-pixel column mask in the stencil.
// Every mbarrier wait is bounded; on a timeout the CTA records it in a status word and exits.
#include <algorithm>
#include <mutex>

#include "common.cuh"
#include "tc_common.cuh"

namespace b200cp {

PFN_encodeTiled get_encode_tiled() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<PFN_encodeTiled>(p);
  });
  return fn;
}

__device__ int g_tc_status = 0;  // 0 ok; otherwise (code << 16) | block index of the first failure

namespace {

using namespace tc;

constexpr int kKC = 16;          // channels per TMA stage
constexpr int kStagesHi = 4;     // TMA stages in flight
constexpr int kStageBytes = 4 * kKC * 128;  // four 32-pixel groups of kKC rows of 128 B
constexpr int kWorkers = 256;    // 8 worker warps: tf32 split, TMEM read-out, stencil, stores
constexpr int kNT = kWorkers + 64;  // + warp 8 (issues every tcgen05.mma) + warp 9 (issues every TMA load)
constexpr int kD1Stride = 96;    // TMEM columns between the two GEMM-1 accumulator sets
constexpr int kD2Col = 192;      // first TMEM column of the GEMM-2 accumulator

struct TcGeom {
  int N, Cin, Cout, H, W, HW, Y, X, pad, R, Rs, r0, flip, terms;
  int RP, Cpad, Tpad, TH, bands, NKC, Mmax, ncols;
  // byte offsets from the 1024-aligned smem base
  int oXhi, oXlo, oA2hi, oA2lo, oB1hi, oB1lo, oB2hi, oB2lo, oWs, oPs, oBar;
  size_t smem;
};

__device__ __forceinline__ int floor4(int v) { return v - (((v % 4) + 4) % 4); }

// Bounded wait shared by the three roles: gives up after about a second, or as soon as another
// role has given up (the flag), so that every thread reaches the common exit.
__device__ __forceinline__ bool wait_or_abort(uint64_t* bar, uint32_t parity, volatile int* abort_flag) {
  const uint32_t a = smem_u32(bar);
  const long long t0 = clock64();
  for (int it = 0;; ++it) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(done)
        : "r"(a), "r"(parity)
        : "memory");
    if (done) return true;
    if ((it & 31) == 31) {
      if (*abort_flag) return false;
      if (clock64() - t0 > 1500000000ll) {
        *abort_flag = 1;
        return false;
      }
    }
  }
}

// barrier 1 over the 256 worker threads with an OR-reduction of `pred`
__device__ __forceinline__ bool workers_sync_or(bool pred) {
  uint32_t r;
  asm volatile(
      "{\n"
      ".reg .pred p, q;\n"
      "setp.ne.u32 q, %1, 0;\n"
      "bar.red.or.pred p, 1, 256, q;\n"
      "selp.u32 %0, 1, 0, p;\n"
      "}\n"
      : "=r"(r)
      : "r"((uint32_t)pred)
      : "memory");
  return r != 0;
}

// Z[4 ranks] of one output pixel: per-rank Y x X stencil over Ps, columns outside the image masked
template <int FS>
__device__ __forceinline__ void stencil4(const TcGeom& g, const float* __restrict__ Ws, const float* __restrict__ p0,
                                         int RP, int rbase, int w, float (&z)[4]) {
  const int Y = FS ? FS : g.Y, X = FS ? FS : g.X;
  z[0] = z[1] = z[2] = z[3] = 0.f;
#pragma unroll
  for (int y = 0; y < (FS ? FS : 1); ++y) {
    for (int yy = FS ? y : 0; yy < (FS ? y + 1 : Y); ++yy) {
#pragma unroll
      for (int x = 0; x < (FS ? FS : 1); ++x) {
        for (int xx = FS ? x : 0; xx < (FS ? x + 1 : X); ++xx) {
          const int wx = w + xx - g.pad;
          const float msk = (wx >= 0 && wx < g.W) ? 1.f : 0.f;
          const float4 wt = *reinterpret_cast<const float4*>(Ws + (yy * X + xx) * RP + rbase);
          const float* p = p0 + yy * g.W + xx;
          z[0] = fmaf(wt.x * msk, p[0], z[0]);
          z[1] = fmaf(wt.y * msk, p[g.Mmax], z[1]);
          z[2] = fmaf(wt.z * msk, p[2 * g.Mmax], z[2]);
          z[3] = fmaf(wt.w * msk, p[3 * g.Mmax], z[3]);
        }
      }
    }
  }
}

// Warp-specialised: warp 9 streams the input through TMA, warps 0-7 split each stage into tf32 hi / lo,
// warp 8 issues the MMAs; the roles meet only through mbarriers, so loads, conversion and tensor work overlap.
template <int RP, int FS>
__global__ void __launch_bounds__(kNT) cp4_tc_kernel(const TcGeom g, const __grid_constant__ CUtensorMap xmap,
                                                     const float* __restrict__ Fin, const float* __restrict__ Fout,
                                                     const float* __restrict__ KH, const float* __restrict__ KW,
                                                     float* __restrict__ out, float* __restrict__ dbgP) {
  // pointer arithmetic on the shared array keeps every access a shared-space access (a round trip through an
  // integer would turn them into generic loads and stores); the pad aligns the base to the swizzle atom
  extern __shared__ __align__(1024) uint8_t smem_raw[];
  uint8_t* sm = smem_raw + ((1024u - (smem_u32(smem_raw) & 1023u)) & 1023u);
  float* Ws = reinterpret_cast<float*>(sm + g.oWs);
  float* Ps = reinterpret_cast<float*>(sm + g.oPs);
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + g.oBar);
  uint64_t* full = bars;                      // [kStagesHi] TMA landed                      (tx bytes)
  uint64_t* ready = full + kStagesHi;         // [kStagesHi] stage split into hi / lo        (8 warp arrivals)
  uint64_t* freeb = ready + kStagesHi;        // [kStagesHi] MMAs that read the stage done   (commit)
  uint64_t* lofree = freeb + kStagesHi;       // [2] MMAs that read the lo buffer done       (commit)
  uint64_t* d1full = lofree + 2;              // [2] GEMM-1 accumulator complete             (commit)
  uint64_t* d1free = d1full + 2;              // [2] GEMM-1 accumulator read out             (8 warp arrivals)
  uint64_t* a2ready = d1free + 2;             // GEMM-2 operand written                      (8 warp arrivals)
  uint64_t* d2full = a2ready + 1;             // GEMM-2 accumulator complete                 (commit)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d2full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int band = blockIdx.x % g.bands, n = blockIdx.x / g.bands;
  const int h0 = band * g.TH, h1 = min(g.H, h0 + g.TH);
  const int q0 = h0 * g.W, q1 = h1 * g.W;
  const int ha = q0 - g.pad * g.W - g.pad;
  const int hb = q1 + (g.Y - 1 - g.pad) * g.W + (g.X - 1 - g.pad);  // one past the last halo position
  const int s0 = floor4(ha);
  const int MB = (max(hb - s0, 1) + 127) >> 7;
  const int NS = MB * g.NKC;
  const int OB = (q1 - q0 + 127) >> 7;

  // ---- set-up ------------------------------------------------------------------------------------
  if (tid == 0) {
    for (int i = 0; i < kStagesHi; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&ready[i], kWorkers / 32);
      mbar_init(&freeb[i], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&lofree[i], 1);
      mbar_init(&d1full[i], 1);
      mbar_init(&d1free[i], kWorkers / 32);
    }
    mbar_init(a2ready, kWorkers / 32);
    mbar_init(d2full, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&xmap);
  }
  if (warp == 8) tmem_alloc(tmem_slot, (uint32_t)g.ncols);
  // factor operands (K-major, no swizzle): element (n, k) at (n/8)*SBO + (k/4)*128 + (n%8)*16 + (k%4)*4
  {
    uint8_t *b1h = sm + g.oB1hi, *b1l = sm + g.oB1lo, *b2h = sm + g.oB2hi, *b2l = sm + g.oB2lo;
    const int sbo1 = g.Cpad * 32, sbo2 = RP * 32;
    for (int i = tid; i < RP * g.Cpad; i += kNT) {
      const int c = i / RP, r = i - c * RP;  // r fastest: coalesced reads of Fin[c][:]
      const float v = (r < g.R && c < g.Cin) ? __ldg(Fin + (size_t)c * g.Rs + g.r0 + r) : 0.f;
      const float h = tf32_hi(v);
      const int o = (r >> 3) * sbo1 + (c >> 2) * 128 + (r & 7) * 16 + (c & 3) * 4;
      *reinterpret_cast<float*>(b1h + o) = h;
      *reinterpret_cast<float*>(b1l + o) = v - h;
    }
    for (int i = tid; i < g.Tpad * RP; i += kNT) {
      const int t = i / RP, r = i - t * RP;
      const float v = (r < g.R && t < g.Cout) ? __ldg(Fout + (size_t)t * g.Rs + g.r0 + r) : 0.f;
      const float h = tf32_hi(v);
      const int o = (t >> 3) * sbo2 + (r >> 2) * 128 + (t & 7) * 16 + (r & 3) * 4;
      *reinterpret_cast<float*>(b2h + o) = h;
      *reinterpret_cast<float*>(b2l + o) = v - h;
    }
    for (int i = tid; i < g.Y * g.X * RP; i += kNT) {
      const int r = i % RP, yx = i / RP, y = yx / g.X, x = yx - y * g.X;
      const int yy = g.flip ? g.Y - 1 - y : y, xx = g.flip ? g.X - 1 - x : x;
      Ws[i] = r < g.R ? __ldg(KH + (size_t)yy * g.Rs + g.r0 + r) * __ldg(KW + (size_t)xx * g.Rs + g.r0 + r) : 0.f;
    }
  }
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tD2 = tmem_base + kD2Col;
  // diagnostic cycle stamps of one CTA: worker thread 0 at [0, 512), the MMA thread at [512, 1024), the TMA thread at [1024, 1536)
  float* dbgT = (dbgP != nullptr && blockIdx.x == gridDim.x / 2 && (tid == 0 || tid == 256 || tid == 288))
                    ? dbgP + RP * g.Mmax + (tid == 0 ? 0 : tid == 256 ? 512 : 1024) : nullptr;
  const long long tstart = clock64();
  auto stamp = [&](int idx) { if (dbgT) dbgT[idx] = (float)(clock64() - tstart); };

  if (warp == 9) {
    // ================= TMA producer ===================================================================
    if (lane == 0) {
      for (int t = 0; t < NS; ++t) {
        const int b = t / g.NKC, kc = t - b * g.NKC, slot = t % kStagesHi;
        if (t >= kStagesHi && !wait_or_abort(&freeb[slot], ((t / kStagesHi) - 1) & 1, abort_flag)) break;
        if (t < 100) stamp(t);
        uint8_t* dst = sm + g.oXhi + slot * kStageBytes;
        mbar_expect_tx(&full[slot], kStageBytes);
#pragma unroll
        for (int grp = 0; grp < 4; ++grp)
          tma_load_3d(dst + grp * (kKC * 128), &xmap, &full[slot], s0 + b * 128 + grp * 32, kc * kKC, n);
      }
    }
  } else if (warp == 8) {
    // ================= MMA issuer ======================================================================
    if (lane == 0) {
      const uint32_t idesc1 = make_idesc_tf32(RP, 1, 0);
      const uint32_t idesc2 = make_idesc_tf32((uint32_t)g.Tpad, 0, 0);
      // MN-major tf32 operand: rows of 32 pixels (128 B), one row per channel, 32-byte chunks swizzled within
      // groups of 4 rows (the only MN-major layout tf32 has).  LBO: next 32-pixel group, SBO: next 4 rows.
      const uint64_t dA0 = make_smem_desc(0, kKC * 128, 512, kSwizzle128B_32B);
      const uint64_t dB1 = make_smem_desc(0, 128, g.Cpad * 32, kSwizzleNone);
      const uint32_t xhi = smem_u32(sm + g.oXhi), xlo = smem_u32(sm + g.oXlo);
      const uint32_t b1h = smem_u32(sm + g.oB1hi), b1l = smem_u32(sm + g.oB1lo);
      bool ok = true;
      for (int s = 0; s < NS && ok; ++s) {
        const int b = s / g.NKC, kc = s - b * g.NKC, slot = s % kStagesHi, l = s & 1;
        const uint32_t tD1 = tmem_base + (b & 1) * kD1Stride;
        if (kc == 0 && b >= 2) ok = wait_or_abort(&d1free[b & 1], ((b >> 1) - 1) & 1, abort_flag);
        if (s < 40) stamp(6 * s + 5);
        ok = ok && wait_or_abort(&ready[slot], (s / kStagesHi) & 1, abort_flag);
        if (!ok) break;
        if (s < 40) stamp(6 * s);
        tc_fence_after_sync();
        if (s < 40) stamp(6 * s + 1);
#pragma unroll
        for (int kk = 0; kk < kKC / 8; ++kk) {
          const uint64_t dah = dA0 + (uint64_t)((xhi + slot * kStageBytes + kk * 1024) >> 4);
          const uint64_t dal = dA0 + (uint64_t)((xlo + l * kStageBytes + kk * 1024) >> 4);
          const uint32_t koff = (uint32_t)(kc * (kKC / 4) + kk * 2) * 128;
          const uint64_t dbh = dB1 + (uint64_t)((b1h + koff) >> 4);
          const uint64_t dbl = dB1 + (uint64_t)((b1l + koff) >> 4);
          // one accumulator per (term, K half): the MMAs of a stage do not depend on each other
          const uint32_t tA = tD1 + (RP == 16 ? kk * 48 : 0);
          const bool first = (kc == 0) && (RP == 16 || kk == 0);
          mma_tf32_ss(tA, dah, dbh, idesc1, !first);
          if (g.terms == 3) {
            mma_tf32_ss(tA + (RP == 16 ? 16 : 0), dal, dbh, idesc1, RP == 16 ? !first : true);
            mma_tf32_ss(tA + (RP == 16 ? 32 : 0), dah, dbl, idesc1, RP == 16 ? !first : true);
          }
        }
        if (s < 40) stamp(6 * s + 2);
        mma_commit(&freeb[slot]);
        if (s < 40) stamp(6 * s + 3);
        if (g.terms == 3) mma_commit(&lofree[l]);
        if (kc == g.NKC - 1) mma_commit(&d1full[b & 1]);
        if (s < 40) stamp(6 * s + 4);
      }
      // GEMM 2, one block of 128 output pixels at a time
      const uint64_t dA2 = make_smem_desc(0, 2048, 128, kSwizzleNone);
      const uint64_t dB2 = make_smem_desc(0, 128, RP * 32, kSwizzleNone);
      const uint32_t a2h = smem_u32(sm + g.oA2hi), a2l = smem_u32(sm + g.oA2lo);
      const uint32_t b2h = smem_u32(sm + g.oB2hi), b2l = smem_u32(sm + g.oB2lo);
      for (int ob = 0; ob < OB && ok; ++ob) {
        ok = wait_or_abort(a2ready, ob & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
#pragma unroll
        for (int kk = 0; kk < RP / 8; ++kk) {
          const uint64_t dah = dA2 + (uint64_t)((a2h + kk * 4096) >> 4), dal = dA2 + (uint64_t)((a2l + kk * 4096) >> 4);
          const uint64_t dbh = dB2 + (uint64_t)((b2h + kk * 256) >> 4), dbl = dB2 + (uint64_t)((b2l + kk * 256) >> 4);
          mma_tf32_ss(tD2, dah, dbh, idesc2, kk != 0);
          if (g.terms == 3) {
            mma_tf32_ss(tD2, dal, dbh, idesc2, true);
            mma_tf32_ss(tD2, dah, dbl, idesc2, true);
          }
        }
        mma_commit(d2full);
      }
    }
  } else {
    // ================= workers ============================================================================
    bool ok = true;
    const int qd = warp & 3, hf = warp >> 2;
    // TMEM accumulator of block b -> Ps[r][b*128 + position]
    auto epilogue1 = [&](int b) {
      ok = ok && wait_or_abort(&d1full[b & 1], (b >> 1) & 1, abort_flag);
      if (ok) {
        tc_fence_after_sync();
        const uint32_t tD1 = tmem_base + (b & 1) * kD1Stride + ((uint32_t)(qd * 32) << 16);
        const int m = b * 128 + qd * 32 + lane;
#pragma unroll
        for (int c8 = 0; c8 < RP / 16; ++c8) {
          const int col = hf * (RP / 2) + c8 * 8;
          float v[8];
          tmem_ld8(tD1 + col, v);
          if (RP == 16) {  // six partial accumulators: (term, K half) at columns 16 * i
            const int nacc = g.terms == 3 ? 6 : 2;
            for (int a = 1; a < nacc; ++a) {
              float u[8];
              tmem_ld8(tD1 + col + (g.terms == 3 ? 16 * a : 48 * a), u);
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] += u[i];
            }
          }
#pragma unroll
          for (int i = 0; i < 8; ++i) Ps[(size_t)(col + i) * g.Mmax + m] = v[i];
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&d1free[b & 1]);
      }
    };
    stamp(0);
    for (int s = 0; s < NS && ok; ++s) {
      const int b = s / g.NKC, kc = s - b * g.NKC, slot = s % kStagesHi, l = s & 1;
      ok = wait_or_abort(&full[slot], (s / kStagesHi) & 1, abort_flag);
      if (s < 60) stamp(16 + 4 * s);
      if (ok && g.terms == 3 && s >= 2) ok = wait_or_abort(&lofree[l], ((s >> 1) - 1) & 1, abort_flag);
      if (s < 60) stamp(16 + 4 * s + 1);
      if (!ok) break;
      float4* hi4 = reinterpret_cast<float4*>(sm + g.oXhi + slot * kStageBytes);
      float4* lo4 = reinterpret_cast<float4*>(sm + g.oXlo + l * kStageBytes);
#pragma unroll
      for (int i = tid; i < kStageBytes / 16; i += kWorkers) {
        const float4 v = hi4[i];
        float4 h, d;
        h.x = tf32_hi(v.x); h.y = tf32_hi(v.y); h.z = tf32_hi(v.z); h.w = tf32_hi(v.w);
        d.x = v.x - h.x; d.y = v.y - h.y; d.z = v.z - h.z; d.w = v.w - h.w;
        hi4[i] = h;
        if (g.terms == 3) lo4[i] = d;
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(&ready[slot]);
      if (s < 60) stamp(16 + 4 * s + 2);
      if (kc == g.NKC - 1 && b >= 1) epilogue1(b - 1);
      if (s < 60) stamp(16 + 4 * s + 3);  // one block behind, so the tensor pipe is never waited on
    }
    if (ok) epilogue1(MB - 1);
    stamp(1);
    ok = !workers_sync_or(!ok);
    if (ok && dbgP != nullptr && blockIdx.x == 0)
      for (int i = tid; i < RP * g.Mmax; i += kWorkers) dbgP[i] = Ps[i];

    // ---- stencil + GEMM 2 + store, one block of 128 output pixels at a time ------------------------------------
    const int j = tid & 127, rhalf = tid >> 7;
    uint8_t *a2h = sm + g.oA2hi, *a2l = sm + g.oA2lo;
    for (int ob = 0; ob < OB && ok; ++ob) {
      const int q = q0 + ob * 128 + j;
      const bool valid = q < q1;
      const int w = q % g.W;
      const float* pbase = Ps + (q - g.pad * g.W - g.pad - s0);
#pragma unroll
      for (int r4 = 0; r4 < RP / 8; ++r4) {
        const int rbase = rhalf * (RP / 2) + r4 * 4;
        float z[4] = {0.f, 0.f, 0.f, 0.f};
        if (valid) stencil4<FS>(g, Ws, pbase + (size_t)rbase * g.Mmax, RP, rbase, w, z);
        float4 h, d;
        h.x = tf32_hi(z[0]); h.y = tf32_hi(z[1]); h.z = tf32_hi(z[2]); h.w = tf32_hi(z[3]);
        d.x = z[0] - h.x; d.y = z[1] - h.y; d.z = z[2] - h.z; d.w = z[3] - h.w;
        // K-major, no swizzle: element (m, k) at m*16 + (k/4)*2048 + (k%4)*4
        const int o = j * 16 + (rbase >> 2) * 2048;
        *reinterpret_cast<float4*>(a2h + o) = h;
        *reinterpret_cast<float4*>(a2l + o) = d;
      }
      fence_proxy_async();
      __syncwarp();
      if (lane == 0) mbar_arrive(a2ready);
      if (ob < 8) stamp(300 + 4 * ob);
      ok = wait_or_abort(d2full, ob & 1, abort_flag);
      if (ob < 8) stamp(300 + 4 * ob + 1);
      if (!ok) break;
      tc_fence_after_sync();
      {
        const int ch = hf;
        const int qq = q0 + ob * 128 + qd * 32 + lane;
        float* dst = out + (size_t)n * g.Cout * g.HW + qq;
        for (int c16 = ch; c16 < g.Tpad / 16; c16 += 2) {
          float v[16];
          tmem_ld16(tD2 + ((uint32_t)(qd * 32) << 16) + c16 * 16, v);
          if (qq < q1) {
#pragma unroll
            for (int i = 0; i < 16; ++i) {
              const int t = c16 * 16 + i;
              if (t < g.Cout) dst[(size_t)t * g.HW] = v[i];
            }
          }
        }
      }
      tc_fence_before_sync();
      // no barrier here: the next GEMM 2 starts only after all eight warps have arrived on a2ready again,
      // which each does after its own read-out above
      if (ob < 8) stamp(300 + 4 * ob + 2);
    }
  }

  // ---- exit ---------------------------------------------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    if (tid == 0) atomicCAS(&g_tc_status, 0, (1 << 16) | (int)(blockIdx.x & 0xffff));
    // give bulk copies that may still be in flight towards this CTA's shared memory time to land
    const long long t0 = clock64();
    while (clock64() - t0 < 400000) {}
  }
  if (warp == 8) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, (uint32_t)g.ncols);
  }
}

int next_pow2(int v) {
  int p = 32;
  while (p < v) p <<= 1;
  return p;
}

}  // namespace

// Shapes the tensor path takes: flat-pixel TMA needs H*W % 4 == 0; operands of both GEMMs must fit in smem.
bool cp4_tc_supported(const Cp4Args& a, const DeviceInfo& di, TcPlan* plan) {
  const int HW = a.H * a.W;
  if (a.R > 64 || HW % 4 != 0 || HW < 128 || a.W < a.X || a.accumulate) return false;
  if (a.pad > a.Y - 1 || a.pad > a.X - 1) return false;
  const int RP = a.R <= 16 ? 16 : a.R <= 32 ? 32 : 64;
  const int Cpad = (int)align_up((size_t)a.Cin, kKC), Tpad = (int)align_up((size_t)a.Cout, 32);
  if (Tpad > 256) return false;
  const size_t fac = (size_t)2 * RP * (Cpad + Tpad) * 4;
  const size_t a2 = (size_t)2 * 128 * RP * 4;
  const size_t xreg = (size_t)(kStagesHi + 2) * kStageBytes;
  const size_t fixed = std::max(xreg, a2) + fac + (size_t)a.Y * a.X * RP * 4 + 256 + 1024;
  // band height: as many rows as fit, balanced against the number of CTAs
  int bestTH = 0;
  double bestCost = 1e300;
  int forced = 0;
  if (const char* e = getenv("B200CP_TC_TH")) forced = atoi(e);
  for (int TH = 1; TH <= a.H; ++TH) {
    if (forced && TH != std::min(forced, a.H)) continue;
    const int span = (TH + a.Y - 1) * a.W + a.X - 1 + 3;
    const int Mmax = (int)align_up((size_t)span, 128);
    const size_t sm = fixed + (size_t)RP * Mmax * 4;
    if ((int)sm > di.smem_optin) break;
    const int bands = ceil_div(a.H, TH);
    const long ctas = (long)a.N * bands;
    const int occ = std::max(1, std::min((int)((228 * 1024) / (sm + 1024)), 512 / next_pow2(kD2Col + Tpad)));
    const long waves = (ctas + (long)di.sm_count * occ - 1) / ((long)di.sm_count * occ);
    // measured on B200: a GEMM-1 stage costs about 1.5k cycles of the MMA-issuing thread, an output block about 6k
    // (stencil, GEMM 2, stores); resident CTAs overlap each other's phases
    const int MBf = Mmax / 128, OBf = ceil_div(std::min(TH, a.H) * a.W, 128);
    const double per = MBf * (Cpad / (double)kKC) * 1.5 * (RP / 16.0 > 2 ? 2.0 : 1.0) + OBf * (4.0 + RP / 8.0 + Tpad / 64.0) + 3.0;
    const double cost = (double)waves * per * (occ > 1 ? 1.0 + 0.15 * (occ - 1) : 1.0);
    if (cost < bestCost) { bestCost = cost; bestTH = TH; }
  }
  if (!bestTH) return false;
  if (plan) {
    plan->TH = bestTH;
    plan->RP = RP;
  }
  return true;
}

int cp4_tc_launch(const Cp4Args& a, int terms, float* dbgP, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  TcPlan plan;
  if (!cp4_tc_supported(a, di, &plan))
    return fail(B200CP_ERR_UNSUPPORTED,
                "cp4 tensor path needs R <= 64, H*W %% 4 == 0, H*W >= 128, out channels <= 256 and operands that fit "
                "in shared memory (N=%d Cin=%d Cout=%d H=%d W=%d R=%d)", a.N, a.Cin, a.Cout, a.H, a.W, a.R);
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B200CP_ERR_NO_DEVICE, "cuTensorMapEncodeTiled entry point not available");
  TcGeom g{};
  g.N = a.N; g.Cin = a.Cin; g.Cout = a.Cout; g.H = a.H; g.W = a.W; g.HW = a.H * a.W; g.Y = a.Y; g.X = a.X;
  g.pad = a.pad; g.R = a.R; g.Rs = a.Rs; g.r0 = a.r0; g.flip = a.flip; g.terms = terms;
  g.RP = plan.RP;
  g.Cpad = (int)align_up((size_t)a.Cin, kKC);
  g.Tpad = (int)align_up((size_t)a.Cout, 32);
  g.TH = plan.TH;
  g.bands = ceil_div(a.H, g.TH);
  g.NKC = g.Cpad / kKC;
  g.Mmax = (int)align_up((size_t)((g.TH + a.Y - 1) * a.W + a.X - 1 + 3), 128);
  g.ncols = next_pow2(kD2Col + g.Tpad);
  const int a2 = 128 * g.RP * 4;
  int o = 0;
  g.oXhi = 0;
  g.oXlo = kStagesHi * kStageBytes;
  g.oA2hi = 0;                // the GEMM-2 operand reuses the (then idle) input stages
  g.oA2lo = a2;
  o = std::max((kStagesHi + 2) * kStageBytes, 2 * a2);
  g.oB1hi = o; o += g.RP * g.Cpad * 4;
  g.oB1lo = o; o += g.RP * g.Cpad * 4;
  g.oB2hi = o; o += g.Tpad * g.RP * 4;
  g.oB2lo = o; o += g.Tpad * g.RP * 4;
  g.oWs = o; o += a.Y * a.X * g.RP * 4;
  g.oPs = o; o += g.RP * g.Mmax * 4;
  g.oBar = (int)align_up((size_t)o, 16); o = g.oBar + 256;
  g.smem = (size_t)o + 1024;  // slack for the 1024-byte alignment of the base
  if ((int)g.smem > di.smem_optin) return fail(B200CP_ERR_UNSUPPORTED, "cp4 tensor path: tile exceeds shared memory");

  CUtensorMap map;
  const cuuint64_t gdim[3] = {(cuuint64_t)g.HW, (cuuint64_t)a.Cin, (cuuint64_t)a.N};
  const cuuint64_t gstr[2] = {(cuuint64_t)g.HW * 4, (cuuint64_t)g.HW * a.Cin * 4};
  const cuuint32_t box[3] = {32, (cuuint32_t)kKC, 1};
  const cuuint32_t estr[3] = {1, 1, 1};
  if (reinterpret_cast<uintptr_t>(a.in) & 15)
    return fail(B200CP_ERR_INVALID_ARG, "cp4 tensor path: the input must be 16-byte aligned");
  const CUresult cr = enc(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float*>(a.in), gdim, gstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(B200CP_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)cr);

  const long ctas = (long)a.N * g.bands;
  if (getenv("B200CP_DEBUG"))
    fprintf(stderr, "[b200cp] tc TH=%d bands=%d RP=%d Cpad=%d Tpad=%d Mmax=%d ncols=%d smem=%zu ctas=%ld terms=%d\n", g.TH,
            g.bands, g.RP, g.Cpad, g.Tpad, g.Mmax, g.ncols, g.smem, ctas, terms);
#define LAUNCH_TC(RPV)                                                                                            \
  do {                                                                                                            \
    auto kern = (a.Y == 3 && a.X == 3) ? cp4_tc_kernel<RPV, 3> : cp4_tc_kernel<RPV, 0>;                           \
    B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));         \
    kern<<<(unsigned)ctas, kNT, g.smem, st>>>(g, map, a.Fin, a.Fout, a.KH, a.KW, a.out, dbgP);                    \
  } while (0)
  if (g.RP == 16) LAUNCH_TC(16);
  else if (g.RP == 32) LAUNCH_TC(32);
  else LAUNCH_TC(64);
#undef LAUNCH_TC
  B200CP_LAUNCH_OK("cp4_tc_kernel");
  return B200CP_OK;
}

// Reads (and clears) the status word of the tensor-path kernels; synchronises the device.
int tc_device_status(int* out) {
  int v = 0, zero = 0;
  B200CP_CUDA_OK(cudaDeviceSynchronize());
  B200CP_CUDA_OK(cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)));
  if (v) B200CP_CUDA_OK(cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)));
  *out = v;
  return B200CP_OK;
}

}  // namespace b200cp

// ---------------------------------------------------------------------------------------------------------
// Self-test of the tcgen05 building blocks: D[128 x 16] = A[128 x 8] * B[16 x 8]^T with one MMA.
//   mode 0: A K-major, no swizzle          (the layout of the GEMM-2 operand)
//   mode 1: A MN-major, 128-byte span with 32-byte swizzle atoms   (what TMA writes for the GEMM-1 operand)
// ---------------------------------------------------------------------------------------------------------
namespace b200cp {
namespace {
__global__ void __launch_bounds__(128) tc_selftest_kernel(int mode, const float* __restrict__ A,
                                                          const float* __restrict__ B, float* __restrict__ D,
                                                          int* __restrict__ status) {
  using namespace tc;
  __shared__ __align__(1024) uint8_t sa[8192];
  __shared__ __align__(1024) uint8_t sb[1024];
  __shared__ __align__(8) uint64_t bar;
  __shared__ uint32_t slot;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  for (int i = tid; i < 2048; i += 128) reinterpret_cast<float*>(sa)[i] = 0.f;
  __syncthreads();
  for (int i = tid; i < 128 * 8; i += 128) {
    const int m = i / 8, k = i % 8;
    int o;
    if (mode == 0) o = m * 16 + (k >> 2) * 2048 + (k & 3) * 4;
    else o = (m >> 5) * 1024 + k * 128 + ((((m & 31) >> 3) ^ (k & 3)) << 5) + (m & 7) * 4;
    *reinterpret_cast<float*>(sa + o) = A[i];
  }
  for (int i = tid; i < 16 * 8; i += 128) {
    const int n = i / 8, k = i % 8;
    *reinterpret_cast<float*>(sb + (n >> 3) * 256 + (k >> 2) * 128 + (n & 7) * 16 + (k & 3) * 4) = B[i];
  }
  if (tid == 0) {
    mbar_init(&bar, 1);
    fence_barrier_init();
  }
  if (warp == 1) tmem_alloc(&slot, 32);
  fence_proxy_async();
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tbase = slot;
  if (tid == 0) {
    const uint64_t da = mode == 0 ? make_smem_desc(smem_u32(sa), 2048, 128, kSwizzleNone)
                                  : make_smem_desc(smem_u32(sa), 1024, 512, kSwizzle128B_32B);
    const uint64_t db = make_smem_desc(smem_u32(sb), 128, 256, kSwizzleNone);
    mma_tf32_ss(tbase, da, db, make_idesc_tf32(16, mode == 0 ? 0 : 1, 0), false);
    mma_commit(&bar);
  }
  const bool ok = mbar_wait(&bar, 0);
  if (__syncthreads_or(!ok)) {
    if (tid == 0) *status = 1;
  } else {
    tc_fence_after_sync();
    float v[16];
    tmem_ld16(tbase + ((uint32_t)(warp * 32) << 16), v);
#pragma unroll
    for (int i = 0; i < 16; ++i) D[(warp * 32 + lane) * 16 + i] = v[i];
    if (tid == 0) *status = 0;
  }
  tc_fence_before_sync();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tbase, 32);
  }
}
}  // namespace

int tc_selftest_launch(int mode, const float* A, const float* B, float* D, int* status, cudaStream_t st) {
  tc_selftest_kernel<<<1, 128, 0, st>>>(mode, A, B, D, status);
  B200CP_LAUNCH_OK("tc_selftest_kernel");
  return B200CP_OK;
}
}  // namespace b200cp
