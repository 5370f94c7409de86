// CP4 conv2d forward and backward-data on CUDA cores (exact fp32).
#include "cp4_simt.cuh"

namespace b200cp {
namespace {

template <int RP, int PPT1, int PPT3>
__global__ void __launch_bounds__(256) cp4_conv_kernel(const Geom g, const float* __restrict__ in,
                                                       const float* __restrict__ Fin,
                                                       const float* __restrict__ Fout,
                                                       const float* __restrict__ KH,
                                                       const float* __restrict__ KW, float* __restrict__ out) {
  extern __shared__ __align__(16) float smem[];
  float* Fs = smem;                       // [cchunk][RP]
  float* Ws = Fs + g.fcap;                // [Y*X][RP]
  float* Ps = Ws + g.Y * g.X * RP;        // [RP][HPXs]
  float* Xst = Ps + RP * g.HPXs;          // [kStages*kKC][nt*PPT1]  cp.async FIFO
  const int tid = threadIdx.x, nt = blockDim.x;
  int b = blockIdx.x;
  const int tw = b % g.tilesW;
  b /= g.tilesW;
  const int th = b % g.tilesH;
  const int n = b / g.tilesH;
  const int h0 = th * g.TH, w0 = tw * g.TW;
  const size_t HW = (size_t)g.H * g.W;

  load_weights<RP>(g, KH, KW, Ws, tid, nt);
  contract_tile<RP, PPT1>(g, in + (size_t)n * g.Cin * HW, g.Cin, Fin, Fs, Xst, Ps, h0, w0, tid, nt);
  __syncthreads();
  float* dst_n = out + (size_t)n * g.Cout * HW;
  for (int base = 0; base < g.OPX; base += nt * PPT3)
    expand_batch<RP, PPT3>(g, Ps, Ws, Fout, Fs, dst_n, g.Cout, h0, w0, base, tid, nt);
}

template <int RP, int P1, int P3>
int launch_conv(const Cp4Args& a, const TileChoice& t, cudaStream_t st) {
  const Geom g = make_geom(a, t, RP, factor_cap(std::max(a.Cin, a.Cout), RP));
  auto kern = cp4_conv_kernel<RP, P1, P3>;
  B200CP_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)t.smem));
  const long ctas = (long)a.N * g.tilesH * g.tilesW;
  if (ctas > 0x7fffffffL) return fail(B200CP_ERR_UNSUPPORTED, "cp4: too many tiles");
  kern<<<(unsigned)ctas, t.NT, t.smem, st>>>(g, a.in, a.Fin, a.Fout, a.KH, a.KW, a.out);
  B200CP_LAUNCH_OK("cp4_conv_kernel");
  return B200CP_OK;
}

template <int RP>
int dispatch_conv(const Cp4Args& a, const DeviceInfo& di, cudaStream_t st) {
  const double w1 = (double)a.Cin * RP, w3 = (double)a.Cout * RP + 2.5 * a.Y * a.X * RP;
  const TileChoice t = choose_tile(a.N, a.H, a.W, a.Y, a.X, a.pad, w1, w3, RP, factor_cap(std::max(a.Cin, a.Cout), RP), 1,
                                   0, 0, 0, false, di);
  if (t.NT == 0) return fail(B200CP_ERR_UNSUPPORTED, "cp4: no tile of this filter fits in shared memory");
  const int key = t.PPT1 * 10 + t.PPT3;
  if constexpr (RP <= 16) {
    switch (key) {
      case 11: return launch_conv<RP, 1, 1>(a, t, st);
      case 21: return launch_conv<RP, 2, 1>(a, t, st);
      case 22: return launch_conv<RP, 2, 2>(a, t, st);
      case 32: return launch_conv<RP, 3, 2>(a, t, st);
      case 33: return launch_conv<RP, 3, 3>(a, t, st);
      case 43: return launch_conv<RP, 4, 3>(a, t, st);
      case 44: return launch_conv<RP, 4, 4>(a, t, st);
    }
  } else if constexpr (RP == 32) {
    switch (key) {
      case 11: return launch_conv<RP, 1, 1>(a, t, st);
      case 21: return launch_conv<RP, 2, 1>(a, t, st);
      case 22: return launch_conv<RP, 2, 2>(a, t, st);
    }
  } else {
    if (key == 11) return launch_conv<RP, 1, 1>(a, t, st);
  }
  return fail(B200CP_ERR_UNSUPPORTED, "cp4: internal: no kernel for PPT %d/%d at rank tile %d", t.PPT1, t.PPT3, RP);
}

}  // namespace

int cp4_simt_launch(const Cp4Args& a, cudaStream_t st) {
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  switch (padded_rank(a.R)) {
    case 4: return dispatch_conv<4>(a, di, st);
    case 8: return dispatch_conv<8>(a, di, st);
    case 16: return dispatch_conv<16>(a, di, st);
    case 32: return dispatch_conv<32>(a, di, st);
    default: return dispatch_conv<64>(a, di, st);
  }
}

}  // namespace b200cp
