// G[m][n] = sum_k A[k][m] * B[k][n] on the tcgen05 tensor cores with fp32-grade accuracy: the gradient GEMM of the CP
// dense layer (G = dY^T X: A = dY [batch][out], B = X [batch][in], K = batch), which is the one GEMM-shaped step
// of the hot path large enough to keep a 128 x 256 tile busy.
//
// Both operands are "MN-major" (contiguous along m / n, K = rows), which tcgen05 takes directly for tf32:
//   * a first pass splits each operand once into hi = tf32(x) and lo = x - hi (two planes per operand),
//   * TMA streams 16-row slabs of the four planes into shared memory (32-float boxes, 128-byte span with
//     32-byte swizzle atoms -- the only MN-major tf32 layout), four stages deep,
//   * one thread issues, per 8 rows of K and per 128-row half of the 256 x 256 tile, the three products
//     hi*hi + lo*hi + hi*lo as 128 x 256 x 8 tcgen05.mma into two fp32 accumulators in TMEM (2 x 256 columns),
//   * four warps read the finished accumulators out of TMEM and store the tile.
// The kernel is bound by the L2 -> shared-memory stream of the operand planes (8 bytes per element and K row),
// which is why the tile is as large as TMEM allows: 256 x 256 moves a third less per product than 128 x 256.
// Roles (TMA warp, MMA warp, four read-out warps) meet only through mbarriers; every wait is bounded and a
// wait that runs out sets a status word and lets the CTA leave through its normal exit (TMEM released).
#include <algorithm>
#include <cstdio>
#include <cstdlib>

#include "common.cuh"
#include "tc_common.cuh"

namespace b200cp {

__device__ int g_gemm_tc_status = 0;  // 0 ok; otherwise (code << 16) | (linear block index & 0xffff)

namespace {

using namespace tc;

constexpr int kBM = 256, kBN = 256, kKS = 16;          // tile and the K rows of one stage
constexpr int kMH = kBM / 128;                         // accumulators (tcgen05.mma has M = 128 per CTA)
constexpr int kStages = 3;
constexpr int kGroupBytes = kKS * 128;                 // one TMA box: 32 floats x kKS rows
constexpr int kAPlane = (kBM / 32) * kGroupBytes;      // 16 KB
constexpr int kBPlane = (kBN / 32) * kGroupBytes;      // 16 KB
constexpr int kStageBytes = 2 * (kAPlane + kBPlane);   // A hi, A lo, B hi, B lo = 64 KB
constexpr int kTmemCols = kMH * kBN;                   // 512: all of TMEM (one CTA per SM by its shared memory)
constexpr int kThreads = 192;                          // warp 0 TMA, warp 1 MMA, warps 2..5 read-out
constexpr size_t kSmem = (size_t)kStages * kStageBytes + 1024 + 256;

__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* map, uint64_t* bar, int x, int y) {
  asm volatile(
      "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
      ::"r"(smem_u32(smem_dst)), "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
      : "memory");
}

// Bounded wait shared by the roles: gives up after about a second, or as soon as another role has given up.
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

// hi = tf32(x) (round to nearest), lo = x - hi (exact); n4 = number of float4
__global__ void __launch_bounds__(256) split_tf32_kernel(const float4* __restrict__ src, float4* __restrict__ hi,
                                                         float4* __restrict__ lo, size_t n4) {
  for (size_t i = (size_t)blockIdx.x * 256 + threadIdx.x; i < n4; i += (size_t)gridDim.x * 256) {
    const float4 v = __ldg(src + i);
    float4 h, d;
    h.x = tf32_hi(v.x); h.y = tf32_hi(v.y); h.z = tf32_hi(v.z); h.w = tf32_hi(v.w);
    d.x = v.x - h.x; d.y = v.y - h.y; d.z = v.z - h.z; d.w = v.w - h.w;
    hi[i] = h;
    lo[i] = d;
  }
}

struct GemmTcGeom {
  int M, N, K;
  int NS;            // stages of kKS rows per CTA (per K split)
  int splits;        // blockIdx.z = tap * splits + split; the tile goes to G + (split * taps + tap) * M * N
  int taps, FW, padH, padW, Wp;  // conv form: the B rows of tap (y, x) are shifted by (y - padH) * Wp + (x - padW)
};

// NCHW -> [n][padded pixel][channel] hi / lo planes with a zero ring of (padH, padW) pixels: the layout in which a
// filter tap is a shift of the row index, which TMA takes at any value (only the contiguous coordinate has an
// alignment rule).  grid = (pixel tiles, channel tiles, N), block = (32, 8).
__global__ void __launch_bounds__(256) pad_transpose_split_kernel(const float* __restrict__ src, float* __restrict__ hi,
                                                                  float* __restrict__ lo, int CH, int H, int W,
                                                                  int padH, int padW) {
  __shared__ float tile[32][33];
  const int Hp = H + 2 * padH, Wp = W + 2 * padW, PP = Hp * Wp;
  const int n = blockIdx.z, p0 = blockIdx.x * 32, c0 = blockIdx.y * 32;
  const int tx = threadIdx.x, ty = threadIdx.y;
  {
    const int p = p0 + tx, ph = p / Wp, pw = p - ph * Wp;
    const int h = ph - padH, w = pw - padW;
    const bool in = p < PP && h >= 0 && h < H && w >= 0 && w < W;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int c = c0 + ty + 8 * j;
      tile[ty + 8 * j][tx] = (in && c < CH) ? __ldg(src + (((size_t)n * CH + c) * H + h) * W + w) : 0.f;
    }
  }
  __syncthreads();
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const int p = p0 + ty + 8 * j, c = c0 + tx;
    if (p < PP && c < CH) {
      const float v = tile[tx][ty + 8 * j];
      const float h = tf32_hi(v);
      const size_t o = ((size_t)n * PP + p) * CH + c;
      hi[o] = h;
      lo[o] = v - h;
    }
  }
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_tc_kernel(const GemmTcGeom g, const __grid_constant__ CUtensorMap mAhi, const __grid_constant__ CUtensorMap mAlo,
               const __grid_constant__ CUtensorMap mBhi, const __grid_constant__ CUtensorMap mBlo,
               float* __restrict__ G) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sm = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(sm + kStages * kStageBytes);
  uint64_t* full = bars;               // [kStages] TMA landed                     (tx bytes)
  uint64_t* empty = full + kStages;    // [kStages] MMAs that read the stage done  (commit)
  uint64_t* accfull = empty + kStages; // accumulator complete                     (commit)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(accfull + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int n0 = blockIdx.x * kBN, m0 = blockIdx.y * kBM;
  const int tap = blockIdx.z / g.splits, split = blockIdx.z - tap * g.splits;
  const int k0 = split * g.NS * kKS;
  const int bshift = (tap / g.FW - g.padH) * g.Wp + (tap % g.FW - g.padW);
  G += ((size_t)split * g.taps + tap) * g.M * g.N;

  if (tid == 0) {
    for (int i = 0; i < kStages; ++i) {
      mbar_init(&full[i], 1);
      mbar_init(&empty[i], 1);
    }
    mbar_init(accfull, 1);
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&mAhi);
    tma_prefetch_desc(&mAlo);
    tma_prefetch_desc(&mBhi);
    tma_prefetch_desc(&mBlo);
  }
  if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ================= TMA producer =====================================================================
    if (lane == 0) {
      for (int s = 0; s < g.NS; ++s) {
        const int slot = s % kStages;
        if (s >= kStages && !wait_or_abort(&empty[slot], ((s / kStages) - 1) & 1, abort_flag)) break;
        uint8_t* dst = sm + slot * kStageBytes;
        mbar_expect_tx(&full[slot], kStageBytes);
        const int k = k0 + s * kKS;  // rows past K (and shifted rows outside the tensor) read as zero
#pragma unroll
        for (int grp = 0; grp < kBM / 32; ++grp) {
          tma_load_2d(dst + grp * kGroupBytes, &mAhi, &full[slot], m0 + grp * 32, k);
          tma_load_2d(dst + kAPlane + grp * kGroupBytes, &mAlo, &full[slot], m0 + grp * 32, k);
        }
#pragma unroll
        for (int grp = 0; grp < kBN / 32; ++grp) {
          tma_load_2d(dst + 2 * kAPlane + grp * kGroupBytes, &mBhi, &full[slot], n0 + grp * 32, k + bshift);
          tma_load_2d(dst + 2 * kAPlane + kBPlane + grp * kGroupBytes, &mBlo, &full[slot], n0 + grp * 32, k + bshift);
        }
      }
    }
  } else if (warp == 1) {
    // ================= MMA issuer ========================================================================
    if (lane == 0) {
      const uint32_t idesc = make_idesc_tf32(kBN, 1, 1);
      // MN-major tf32 operand: rows of 32 floats (128 B), one row per k, 32-byte chunks swizzled within groups
      // of 4 rows.  LBO: next group of 32 columns, SBO: next 4 rows; 8 rows of K per instruction = 1024 bytes.
      const uint64_t d0 = make_smem_desc(0, kGroupBytes, 512, kSwizzle128B_32B);
      const uint32_t base = smem_u32(sm);
      bool ok = true;
      for (int s = 0; s < g.NS && ok; ++s) {
        const int slot = s % kStages;
        ok = wait_or_abort(&full[slot], (s / kStages) & 1, abort_flag);
        if (!ok) break;
        tc_fence_after_sync();
        const uint32_t st = base + slot * kStageBytes;
#pragma unroll
        for (int kk = 0; kk < kKS / 8; ++kk) {
          const uint64_t ah = d0 + (uint64_t)((st + kk * 1024) >> 4);
          const uint64_t al = d0 + (uint64_t)((st + kAPlane + kk * 1024) >> 4);
          const uint64_t bh = d0 + (uint64_t)((st + 2 * kAPlane + kk * 1024) >> 4);
          const uint64_t bl = d0 + (uint64_t)((st + 2 * kAPlane + kBPlane + kk * 1024) >> 4);
#pragma unroll
          for (int h = 0; h < kMH; ++h) {  // the 128-row halves: 4 groups of 32 columns further on in the A planes
            const uint64_t ho = (uint64_t)((h * 4 * kGroupBytes) >> 4);
            mma_tf32_ss(tmem_base + h * kBN, al + ho, bh, idesc, !(s == 0 && kk == 0));
            mma_tf32_ss(tmem_base + h * kBN, ah + ho, bl, idesc, true);
            mma_tf32_ss(tmem_base + h * kBN, ah + ho, bh, idesc, true);
          }
        }
        mma_commit(&empty[slot]);
      }
      if (ok) mma_commit(accfull);
    }
  } else {
    // ================= read-out: TMEM -> global ===========================================================
    const int qd = warp & 3;  // the TMEM lane quarter this warp may read
    if (wait_or_abort(accfull, 0, abort_flag)) {
      tc_fence_after_sync();
#pragma unroll 1
      for (int hc = 0; hc < kMH * (kBN / 16); ++hc) {
        const int h = hc / (kBN / 16), c = hc % (kBN / 16);
        const int m = m0 + h * 128 + qd * 32 + lane;
        float* dst = G + (size_t)m * g.N + n0;
        float v[16];
        tmem_ld16(tmem_base + ((uint32_t)(qd * 32) << 16) + h * kBN + c * 16, v);
        if (m < g.M) {
          if (n0 + c * 16 + 16 <= g.N) {
#pragma unroll
            for (int i = 0; i < 4; ++i)
              *reinterpret_cast<float4*>(dst + c * 16 + i * 4) = make_float4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
          } else {
#pragma unroll
            for (int i = 0; i < 16; ++i)
              if (n0 + c * 16 + i < g.N) dst[c * 16 + i] = v[i];
          }
        }
      }
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (tid == 0 && *abort_flag)
    atomicCAS(&g_gemm_tc_status, 0,
              (1 << 16) | (((blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x) & 0xffff));
  if (warp == 1) {
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

bool enabled() {  // B200CP_GEMM_TC=0 keeps the CUDA-core GEMM (read per call: tests switch it)
  const char* e = getenv("B200CP_GEMM_TC");
  return !(e && e[0] == '0');
}

int encode_plane(PFN_encodeTiled enc, CUtensorMap* map, const float* base, int cols, int rows) {
  const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
  const cuuint64_t gstr[1] = {(cuuint64_t)cols * 4};
  const cuuint32_t box[2] = {32, (cuuint32_t)kKS};
  const cuuint32_t estr[2] = {1, 1};
  const CUresult cr = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float*>(base), gdim, gstr, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (cr != CUDA_SUCCESS) return fail(B200CP_ERR_CUDA, "cuTensorMapEncodeTiled failed with code %d", (int)cr);
  return B200CP_OK;
}

}  // namespace

// The tensor path takes a flat GEMM with 16-byte rows that is large enough to fill a good part of a 256 x 256 tile.
bool gemm_tc_supported(int K, int M, int N) {
  return enabled() && M % 4 == 0 && N % 4 == 0 && M >= 128 && N >= kBN && K >= 256 && get_encode_tiled() != nullptr;
}

// floats of scratch: the hi / lo planes of both operands
size_t gemm_tc_scratch_floats(int K, int M, int N) { return 2 * (size_t)K * ((size_t)M + (size_t)N); }

// G[M][N] = A^T B with A [K][M], B [K][N]; scratch holds gemm_tc_scratch_floats() floats, 16-byte aligned
int gemm_tc_launch(int K, int M, int N, const float* A, const float* B, float* G, float* scratch, cudaStream_t st) {
  PFN_encodeTiled enc = get_encode_tiled();
  if (!enc) return fail(B200CP_ERR_NO_DEVICE, "cuTensorMapEncodeTiled entry point not available");
  if ((reinterpret_cast<uintptr_t>(A) | reinterpret_cast<uintptr_t>(B) | reinterpret_cast<uintptr_t>(G) |
       reinterpret_cast<uintptr_t>(scratch)) & 15)
    return fail(B200CP_ERR_INVALID_ARG, "tensor-core gradient GEMM: operands must be 16-byte aligned");
  const size_t na = (size_t)K * M, nb = (size_t)K * N;
  float *Ahi = scratch, *Alo = Ahi + na, *Bhi = Alo + na, *Blo = Bhi + nb;
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  split_tf32_kernel<<<(unsigned)std::min<size_t>((na / 4 + 255) / 256, (size_t)di.sm_count * 16), 256, 0, st>>>(
      reinterpret_cast<const float4*>(A), reinterpret_cast<float4*>(Ahi), reinterpret_cast<float4*>(Alo), na / 4);
  B200CP_LAUNCH_OK("split_tf32_kernel");
  split_tf32_kernel<<<(unsigned)std::min<size_t>((nb / 4 + 255) / 256, (size_t)di.sm_count * 16), 256, 0, st>>>(
      reinterpret_cast<const float4*>(B), reinterpret_cast<float4*>(Bhi), reinterpret_cast<float4*>(Blo), nb / 4);
  B200CP_LAUNCH_OK("split_tf32_kernel");
  CUtensorMap mAhi, mAlo, mBhi, mBlo;
  if (int rc = encode_plane(enc, &mAhi, Ahi, M, K)) return rc;
  if (int rc = encode_plane(enc, &mAlo, Alo, M, K)) return rc;
  if (int rc = encode_plane(enc, &mBhi, Bhi, N, K)) return rc;
  if (int rc = encode_plane(enc, &mBlo, Blo, N, K)) return rc;
  GemmTcGeom g{M, N, K, ceil_div(K, kKS), 1, 1, 1, 0, 0, 0};
  dim3 grid(ceil_div(N, kBN), ceil_div(M, kBM));
  if (grid.y > 65535) return fail(B200CP_ERR_UNSUPPORTED, "tensor-core gradient GEMM: too many tiles");
  B200CP_CUDA_OK(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
  gemm_tc_kernel<<<grid, kThreads, kSmem, st>>>(g, mAhi, mAlo, mBhi, mBlo, G);
  B200CP_LAUNCH_OK("gemm_tc_kernel");
  return B200CP_OK;
}

// ---- conv form: G[tap][t][c] = sum_{n,h,w} dV[n,t,h,w] * Xpad[n,c,h+y,w+x] ------------------------------------------------
// Both operands are rewritten once as [n][padded pixel][channel] hi / lo planes (K = padded pixel index, rows);
// the nine taps are then nine GEMMs over the same planes with the X rows shifted, each split over K so that the
// (tile, tap, split) grid fills the GPU; a last kernel adds the splits in order.
namespace {
struct ConvGemmPlan {
  int Hp, Wp, taps, splits, NS;
  long K;
  size_t plane_a, plane_b, partial;
};
bool conv_plan(ConvGemmPlan& p, int N, int T, int C, int H, int W, int FH, int FW) {
  if (!(enabled() && T % 4 == 0 && C % 4 == 0 && T >= 128 && C >= 128 && FH % 2 == 1 && FW % 2 == 1)) return false;
  p.Hp = H + FH - 1; p.Wp = W + FW - 1; p.taps = FH * FW;
  p.K = (long)N * p.Hp * p.Wp;
  if (p.K < 1024 || p.K > 0x7fffff00L) return false;
  const long tiles = (long)ceil_div(C, kBN) * ceil_div(T, kBM) * p.taps;
  const int stages = (int)((p.K + kKS - 1) / kKS);
  // one wave of CTAs (one CTA per SM by its shared memory); at least 32 stages per split
  int splits = (int)std::max<long>(1, std::min<long>(148 / std::max<long>(1, tiles), stages / 32));
  p.NS = ceil_div(stages, splits);
  p.splits = ceil_div(stages, p.NS);
  p.plane_a = (size_t)p.K * T;
  p.plane_b = (size_t)p.K * C;
  p.partial = p.splits > 1 ? (size_t)p.splits * p.taps * T * C : 0;
  return get_encode_tiled() != nullptr;
}
}  // namespace

bool conv_gemm_tc_supported(int N, int T, int C, int H, int W, int FH, int FW) {
  ConvGemmPlan p;
  return conv_plan(p, N, T, C, H, W, FH, FW);
}

size_t conv_gemm_tc_scratch_floats(int N, int T, int C, int H, int W, int FH, int FW) {
  ConvGemmPlan p;
  if (!conv_plan(p, N, T, C, H, W, FH, FW)) return 0;
  return 2 * (p.plane_a + p.plane_b) + p.partial;
}

// G is written as [tap][T][C]; dV [N][T][H][W], X [N][C][H][W]
int conv_gemm_tc_launch(int N, int T, int C, int H, int W, int FH, int FW, const float* dV, const float* X, float* G,
                        float* scratch, cudaStream_t st) {
  ConvGemmPlan p;
  if (!conv_plan(p, N, T, C, H, W, FH, FW)) return fail(B200CP_ERR_UNSUPPORTED, "tensor-core conv gradient: shape not taken");
  PFN_encodeTiled enc = get_encode_tiled();
  if ((reinterpret_cast<uintptr_t>(G) | reinterpret_cast<uintptr_t>(scratch)) & 15)
    return fail(B200CP_ERR_INVALID_ARG, "tensor-core conv gradient: buffers must be 16-byte aligned");
  float *Ahi = scratch, *Alo = Ahi + p.plane_a, *Bhi = Alo + p.plane_a, *Blo = Bhi + p.plane_b;
  float* part = Blo + p.plane_b;
  const int padH = (FH - 1) / 2, padW = (FW - 1) / 2, PP = p.Hp * p.Wp;
  if (N > 65535) return fail(B200CP_ERR_UNSUPPORTED, "tensor-core conv gradient: batch too large");
  pad_transpose_split_kernel<<<dim3(ceil_div(PP, 32), ceil_div(T, 32), N), dim3(32, 8), 0, st>>>(dV, Ahi, Alo, T, H, W,
                                                                                                 padH, padW);
  B200CP_LAUNCH_OK("pad_transpose_split_kernel");
  pad_transpose_split_kernel<<<dim3(ceil_div(PP, 32), ceil_div(C, 32), N), dim3(32, 8), 0, st>>>(X, Bhi, Blo, C, H, W,
                                                                                                 padH, padW);
  B200CP_LAUNCH_OK("pad_transpose_split_kernel");
  CUtensorMap mAhi, mAlo, mBhi, mBlo;
  if (int rc = encode_plane(enc, &mAhi, Ahi, T, (int)p.K)) return rc;
  if (int rc = encode_plane(enc, &mAlo, Alo, T, (int)p.K)) return rc;
  if (int rc = encode_plane(enc, &mBhi, Bhi, C, (int)p.K)) return rc;
  if (int rc = encode_plane(enc, &mBlo, Blo, C, (int)p.K)) return rc;
  GemmTcGeom g{T, C, (int)p.K, p.NS, p.splits, p.taps, FW, padH, padW, p.Wp};
  dim3 grid(ceil_div(C, kBN), ceil_div(T, kBM), p.taps * p.splits);
  if (grid.y > 65535 || grid.z > 65535) return fail(B200CP_ERR_UNSUPPORTED, "tensor-core conv gradient: too many tiles");
  B200CP_CUDA_OK(cudaFuncSetAttribute(gemm_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem));
  gemm_tc_kernel<<<grid, kThreads, kSmem, st>>>(g, mAhi, mAlo, mBhi, mBlo, p.splits > 1 ? part : G);
  B200CP_LAUNCH_OK("gemm_tc_kernel");
  if (p.splits > 1) {
    const size_t n = (size_t)p.taps * T * C;
    sum_splits_launch(part, G, n, p.splits, st);
    B200CP_LAUNCH_OK("sum_splits_kernel");
  }
  return B200CP_OK;
}

// Reads (and clears) the status word of the GEMM kernel; the caller has synchronised the device.
int gemm_tc_status(int* out) {
  int v = 0, zero = 0;
  B200CP_CUDA_OK(cudaMemcpyFromSymbol(&v, g_gemm_tc_status, sizeof(int)));
  if (v) B200CP_CUDA_OK(cudaMemcpyToSymbol(g_gemm_tc_status, &zero, sizeof(int)));
  *out = v;
  return B200CP_OK;
}

}  // namespace b200cp
