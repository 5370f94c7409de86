// extern "C" surface of libb200cp: argument validation, rank chunking, host-buffer helpers.
#include <algorithm>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "b200cp_test.h"

namespace b200cp {

std::atomic<unsigned long long> g_launches{0};

char* last_error_buffer() {
  static thread_local char buf[512] = {0};
  return buf;
}

int fail(int status, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(last_error_buffer(), 512, fmt, ap);
  va_end(ap);
  return status;
}

int device_info(DeviceInfo* out) {
  static std::mutex mu;
  static DeviceInfo cache[64];
  int dev = 0;
  B200CP_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200CP_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(mu);
  if (cache[dev].sm_count == 0) {
    DeviceInfo d;
    B200CP_CUDA_OK(cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev));
    B200CP_CUDA_OK(cudaDeviceGetAttribute(&d.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev));
    B200CP_CUDA_OK(cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev));
    if (d.cc_major != 10)
      return fail(B200CP_ERR_NO_DEVICE, "this library is built for sm_100a only; device %d is sm_%d0", dev, d.cc_major);
    cache[dev] = d;
  }
  *out = cache[dev];
  return B200CP_OK;
}

namespace {

int check_shape(const b200cp_tensor_shape* s, const char* who) {
  if (!s) return fail(B200CP_ERR_INVALID_ARG, "%s: shape is null", who);
  if (!s->N || !s->H || !s->W || !s->T || !s->C || !s->Y || !s->X || !s->Rank)
    return fail(B200CP_ERR_INVALID_ARG, "%s: zero dimension in shape N=%u H=%u W=%u T=%u C=%u Y=%u X=%u Rank=%u", who,
                s->N, s->H, s->W, s->T, s->C, s->Y, s->X, s->Rank);
  if ((size_t)s->H * s->W >= (1u << 30) || s->Y > 31 || s->X > 31)
    return fail(B200CP_ERR_UNSUPPORTED, "%s: image or filter too large (H*W=%zu, Y=%u, X=%u)", who,
                (size_t)s->H * s->W, s->Y, s->X);
  return B200CP_OK;
}

int check_ptrs(const char* who, std::initializer_list<const void*> ps) {
  for (const void* p : ps) {
    if (!p) return fail(B200CP_ERR_INVALID_ARG, "%s: null pointer argument", who);
    if (reinterpret_cast<uintptr_t>(p) & 3) return fail(B200CP_ERR_INVALID_ARG, "%s: pointer not 4-byte aligned", who);
  }
  return B200CP_OK;
}

int path_of(int flags) { return flags & B200CP_PATH_MASK; }

// B200CP_PATH_AUTO takes the warp-level tensor path (mma.sync): at every measured size it is at least as fast as the
// tcgen05 path, which needs larger tiles than these layers offer per SM.  B200CP_AUTO_TC=1 prefers tcgen05 where
// the shape allows it; B200CP_AUTO_MMA=0 falls back to the CUDA-core kernels.
const bool g_auto_tc = [] {
  const char* e = getenv("B200CP_AUTO_TC");
  return e && e[0] == '1';
}();
const bool g_auto_mma = [] {
  const char* e = getenv("B200CP_AUTO_MMA");
  return !(e && e[0] == '0');
}();

Cp4Args conv_args(const b200cp_tensor_shape* s, const float* in, const float* K0, const float* K1, const float* KH,
                  const float* KW, float* out, bool backward, const float* KC, float* save) {
  Cp4Args a{};
  a.N = s->N; a.H = s->H; a.W = s->W; a.Y = s->Y; a.X = s->X; a.pad = s->pad;
  a.Cin = backward ? s->T : s->C;
  a.Cout = backward ? s->C : s->T;
  a.Fin = backward ? K0 : K1;
  a.Fout = backward ? K1 : K0;
  a.KH = KH; a.KW = KW; a.KC = KC; a.in = in; a.out = out; a.save = save;
  a.flip = backward ? 1 : 0;
  a.Rs = s->Rank;
  a.R = s->Rank;
  return a;
}

bool takes_mma(int path, const float* KC, const float* save) {
  return KC || save || path == B200CP_PATH_MMA || (path == B200CP_PATH_AUTO && g_auto_mma);
}

int run_conv(const b200cp_tensor_shape* s, const float* in, const float* K0, const float* K1, const float* KH,
             const float* KW, float* out, cudaStream_t st, int flags, bool backward, const float* KC = nullptr,
             float* save = nullptr) {
  const int path = path_of(flags);
  Cp4Args a = conv_args(s, in, K0, K1, KH, KW, out, backward, KC, save);
  if (KC && path != B200CP_PATH_AUTO && path != B200CP_PATH_MMA)
    return fail(B200CP_ERR_UNSUPPORTED, "the three-factor CP conv runs on the mma path only (flags AUTO or MMA)");
  if (path == B200CP_PATH_TC3X || path == B200CP_PATH_TC1X) return cp4_tc_launch(a, path == B200CP_PATH_TC3X ? 3 : 1, nullptr, st);
  if (path == B200CP_PATH_AUTO && g_auto_tc && !KC && !save) {
    DeviceInfo di;
    if (int rc = device_info(&di)) return rc;
    if (cp4_tc_supported(a, di, nullptr)) return cp4_tc_launch(a, 3, nullptr, st);
  }
  const bool mma = takes_mma(path, KC, save);
  if (mma && s->Rank <= 32) {   // row bands with TMA loads where the shape allows them
    bool done = false;
    if (int rc = cp4_stream_launch(&a, 1, st, &done)) return rc;
    if (done) return B200CP_OK;
    if (int rc = cp4_band_launch(&a, 1, st, &done)) return rc;
    if (done) return B200CP_OK;
  }
  for (unsigned r0 = 0; r0 < s->Rank; r0 += 64) {
    a.r0 = r0;
    a.R = std::min(64u, s->Rank - r0);
    a.accumulate = r0 > 0;
    if (int rc = (mma ? cp4_mma_launch(a, st) : cp4_simt_launch(a, st))) return rc;
  }
  return B200CP_OK;
}

// ---- cached device buffers of the *_host helpers --------------------------
// Slots of the host-buffer step.  With two, the copy-out of a step waits for its kernels while the copy-in of the next
// step but one waits for that copy-out (it reuses the buffers): each direction of the host link idles for a kernel
// time per step.  A third and fourth slot let the copy-in run ahead.
constexpr int kHostSlots = 4;
struct HostCtx {
  std::vector<void*> bufs;
  std::vector<size_t> sizes;
  // copy-in, compute and copy-out streams: the two copy directions and the kernels overlap
  cudaStream_t s_in = nullptr, s_cmp = nullptr, s_out = nullptr;
  // per slot: X and factors in, dU in, forward / backward-data / backward-filter done, results out
  cudaEvent_t ev[kHostSlots][6] = {};
  bool pending[kHostSlots] = {};
  // pinned staging of the four factor matrices of a slot: they go to the device as one copy
  float* stage[kHostSlots] = {};
  size_t stage_bytes[kHostSlots] = {};
};
std::mutex g_host_mu;
HostCtx g_host_ctx[64];

int host_buffer(HostCtx& c, size_t slot, size_t bytes, float** out) {
  if (c.bufs.size() <= slot) {
    c.bufs.resize(slot + 1, nullptr);
    c.sizes.resize(slot + 1, 0);
  }
  if (c.sizes[slot] < bytes) {
    if (c.bufs[slot]) B200CP_CUDA_OK(cudaFree(c.bufs[slot]));
    c.bufs[slot] = nullptr;
    c.sizes[slot] = 0;
    B200CP_CUDA_OK(cudaMalloc(&c.bufs[slot], bytes));
    c.sizes[slot] = bytes;
  }
  *out = static_cast<float*>(c.bufs[slot]);
  return B200CP_OK;
}

}  // namespace
}  // namespace b200cp

using namespace b200cp;

extern "C" {

int b200cp_cp4_fwd(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1, const float* KH,
                   const float* KW, float* U, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_fwd")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_fwd", {X, K0, K1, KH, KW, U})) return rc;
  return run_conv(s, X, K0, K1, KH, KW, U, static_cast<cudaStream_t>(stream), flags, false);
}

int b200cp_cp4_bwd_data(const b200cp_tensor_shape* s, const float* dU, const float* K0, const float* K1,
                        const float* KH, const float* KW, float* dX, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_bwd_data")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_bwd_data", {dU, K0, K1, KH, KW, dX})) return rc;
  return run_conv(s, dU, K0, K1, KH, KW, dX, static_cast<cudaStream_t>(stream), flags, true);
}

// 3x3 / pad 1 / at most 16 ranks: the stand-alone backward-filter can write the two rank planes with plane-only
// convolutions and form the gradients from them with the step's band kernel; that needs room for the planes
static size_t bwd_filter_plane_bytes(const b200cp_tensor_shape* s) {
  return align_up((size_t)s->N * s->Rank * s->H * s->W * sizeof(float), 256);
}
static bool bwd_filter_by_planes(const b200cp_tensor_shape* s, int flags) {
  const int path = path_of(flags);
  return s->Y == 3 && s->X == 3 && s->pad == 1 && s->Rank <= 16 &&
         (path == B200CP_PATH_MMA || (path == B200CP_PATH_AUTO && g_auto_mma));
}

size_t b200cp_cp4_bwd_filter_workspace_bytes(const b200cp_tensor_shape* s, int flags) {
  if (check_shape(s, "b200cp_cp4_bwd_filter_workspace_bytes")) return 0;
  if (path_of(flags) == B200CP_PATH_SIMT) return cp4_bwd_filter_simt_workspace(*s);
  size_t need = std::max(cp4_bwd_filter_simt_workspace(*s), cp4_bwd_filter_mma_workspace(*s));
  if (bwd_filter_by_planes(s, flags)) need = std::max(need, 2 * bwd_filter_plane_bytes(s) + cp4_grad_band_workspace(*s));
  return need;
}

int b200cp_cp4_bwd_filter(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                          const float* K1, const float* KH, const float* KW, float* dK_packed, void* workspace,
                          size_t workspace_bytes, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_bwd_filter")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_bwd_filter", {X, dU, K0, K1, KH, KW, dK_packed})) return rc;
  if (s->Y != s->X || (s->Y & 1) == 0 || s->pad != (s->Y - 1) / 2)
    return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_bwd_filter: needs Y == X odd and pad == (Y-1)/2 (Y=%u X=%u pad=%u)",
                s->Y, s->X, s->pad);
  const int path = path_of(flags);
  if (path == B200CP_PATH_TC3X || path == B200CP_PATH_TC1X)
    return fail(B200CP_ERR_UNSUPPORTED, "cp4 bwd-filter: the tcgen05 path is not available for this operation");
  if (!workspace) return fail(B200CP_ERR_WORKSPACE, "b200cp_cp4_bwd_filter: workspace is null");
  Cp4BwdFilterArgs a{};
  a.N = s->N; a.C = s->C; a.T = s->T; a.H = s->H; a.W = s->W; a.F = s->Y; a.pad = s->pad;
  a.Rs = s->Rank;
  a.X = X; a.dU = dU; a.K0 = K0; a.K1 = K1; a.KH = KH; a.KW = KW; a.dK = dK_packed;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  if (bwd_filter_by_planes(s, flags)) {
    // rank planes by two plane-only convolutions in one launch (they read X and dU once), then the gradient band
    // kernel of the training step; taken where the workspace has room for the planes and both kernels take the shape
    const size_t plane = bwd_filter_plane_bytes(s);
    const size_t gws = cp4_grad_band_workspace(*s);
    a.r0 = 0;
    a.R = (int)s->Rank;
    if (gws > 0 && workspace_bytes >= 2 * plane + gws && cp4_grad_band_supported(a)) {
      float* P = static_cast<float*>(workspace);
      float* Q = reinterpret_cast<float*>(static_cast<char*>(workspace) + plane);
      cudaStream_t st = static_cast<cudaStream_t>(stream);
      Cp4Args cv[2] = {conv_args(s, X, K0, K1, KH, KW, nullptr, false, nullptr, P),
                       conv_args(s, dU, K0, K1, KH, KW, nullptr, true, nullptr, Q)};
      bool both = false;
      if (int rc = cp4_stream_launch(cv, 2, st, &both)) return rc;
      if (both) {
        Cp4BwdFilterArgs b = a;
        b.ws = static_cast<char*>(workspace) + 2 * plane;
        b.ws_bytes = workspace_bytes - 2 * plane;
        bool done = false;
        if (int rc = cp4_grad_band_launch(b, P, Q, st, &done, /*after_own_kernel=*/true)) return rc;
        if (done) return B200CP_OK;
      }
    }
  }
  for (unsigned r0 = 0; r0 < s->Rank; r0 += 64) {
    a.r0 = r0;
    a.R = std::min(64u, s->Rank - r0);
    // measured: with at most 8 ranks and at most 128 channels the CUDA-core kernel is the faster one
    const bool small = padded_rank(a.R) <= 8 && std::max(a.C, a.T) <= 128;
    const bool mma = (path == B200CP_PATH_MMA || (path == B200CP_PATH_AUTO && g_auto_mma && !small)) &&
                     cp4_bwd_filter_mma_supported(a);
    if (int rc = mma ? cp4_bwd_filter_mma_launch(a, static_cast<cudaStream_t>(stream))
                     : cp4_bwd_filter_simt_launch(a, static_cast<cudaStream_t>(stream)))
      return rc;
  }
  return B200CP_OK;
}

// ---- three-factor CP conv ---------------------------------------------------------
int b200cp_cp3_fwd(const b200cp_tensor_shape* s, const float* X, const float* KT, const float* KCin, const float* KC,
                   float* U, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp3_fwd")) return rc;
  if (int rc = check_ptrs("b200cp_cp3_fwd", {X, KT, KCin, KC, U})) return rc;
  return run_conv(s, X, KT, KCin, nullptr, nullptr, U, static_cast<cudaStream_t>(stream), flags, false, KC);
}

int b200cp_cp3_bwd_data(const b200cp_tensor_shape* s, const float* dU, const float* KT, const float* KCin,
                        const float* KC, float* dX, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp3_bwd_data")) return rc;
  if (int rc = check_ptrs("b200cp_cp3_bwd_data", {dU, KT, KCin, KC, dX})) return rc;
  return run_conv(s, dU, KT, KCin, nullptr, nullptr, dX, static_cast<cudaStream_t>(stream), flags, true, KC);
}

size_t b200cp_cp3_bwd_filter_workspace_bytes(const b200cp_tensor_shape* s, int flags) {
  (void)flags;
  if (check_shape(s, "b200cp_cp3_bwd_filter_workspace_bytes")) return 0;
  return cp4_bwd_filter_mma_workspace(*s);
}

int b200cp_cp3_bwd_filter(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* KT,
                          const float* KCin, const float* KC, float* dK_packed, void* workspace,
                          size_t workspace_bytes, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp3_bwd_filter")) return rc;
  if (int rc = check_ptrs("b200cp_cp3_bwd_filter", {X, dU, KT, KCin, KC, dK_packed})) return rc;
  if (s->Y != 3 || s->X != 3 || s->pad != 1)
    return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp3_bwd_filter: 3x3 filters with pad 1 only (Y=%u X=%u pad=%u)", s->Y, s->X,
                s->pad);
  const int path = path_of(flags);
  if (path != B200CP_PATH_AUTO && path != B200CP_PATH_MMA)
    return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp3_bwd_filter: runs on the mma path only (flags AUTO or MMA)");
  if (!workspace) return fail(B200CP_ERR_WORKSPACE, "b200cp_cp3_bwd_filter: workspace is null");
  Cp4BwdFilterArgs a{};
  a.N = s->N; a.C = s->C; a.T = s->T; a.H = s->H; a.W = s->W; a.F = 3; a.pad = 1;
  a.Rs = s->Rank;
  a.X = X; a.dU = dU; a.K0 = KT; a.K1 = KCin; a.KC = KC; a.dK = dK_packed;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  for (unsigned r0 = 0; r0 < s->Rank; r0 += 64) {
    a.r0 = r0;
    a.R = std::min(64u, s->Rank - r0);
    if (int rc = cp4_bwd_filter_mma_launch(a, static_cast<cudaStream_t>(stream))) return rc;
  }
  return B200CP_OK;
}

int b200cp_cp4_bwd_filter_noalloc(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                                  const float* K1, const float* KH, const float* KW, float* dK_packed, void* stream) {
  if (int rc = check_shape(s, "b200cp_cp4_bwd_filter_noalloc")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_bwd_filter_noalloc", {X, dU, K0, K1, KH, KW, dK_packed})) return rc;
  if (s->Y != s->X || (s->Y & 1) == 0 || s->pad != (s->Y - 1) / 2)
    return fail(B200CP_ERR_UNSUPPORTED,
                "b200cp_cp4_bwd_filter_noalloc: needs Y == X odd and pad == (Y-1)/2 (Y=%u X=%u pad=%u)", s->Y, s->X, s->pad);
  const size_t need = cp4_bwd_filter_simt_workspace(*s), cap = cp4_bwd_filter_static_scratch_bytes();
  if (need > cap)
    return fail(B200CP_ERR_UNSUPPORTED,
                "b200cp_cp4_bwd_filter_noalloc: this shape needs %zu bytes of scratch, the built-in array holds %zu; "
                "use b200cp_cp4_bwd_filter with a caller-provided workspace", need, cap);
  Cp4BwdFilterArgs a{};
  a.N = s->N; a.C = s->C; a.T = s->T; a.H = s->H; a.W = s->W; a.F = s->Y; a.pad = s->pad;
  a.Rs = s->Rank;
  a.X = X; a.dU = dU; a.K0 = K0; a.K1 = K1; a.KH = KH; a.KW = KW; a.dK = dK_packed;
  for (unsigned r0 = 0; r0 < s->Rank; r0 += 64) {
    a.r0 = r0;
    a.R = std::min(64u, s->Rank - r0);
    if (int rc = cp4_bwd_filter_static_launch(a, static_cast<cudaStream_t>(stream))) return rc;
  }
  return B200CP_OK;
}

int b200cp_cp4_bwd_filter_full(const b200cp_tensor_shape* s, const float* X, const float* dU, float* dK,
                               void* stream) {
  if (int rc = check_shape(s, "b200cp_cp4_bwd_filter_full")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_bwd_filter_full", {X, dU, dK})) return rc;
  if ((size_t)s->T * s->C > 0x7fffffffu) return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_bwd_filter_full: T*C too large");
  return cp4_bwd_filter_full_launch(*s, X, dU, dK, static_cast<cudaStream_t>(stream));
}

int b200cp_cp4_recompose(const b200cp_tensor_shape* s, const float* K0, const float* K1, const float* KH,
                         const float* KW, float* K, void* stream) {
  if (int rc = check_shape(s, "b200cp_cp4_recompose")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_recompose", {K0, K1, KH, KW, K})) return rc;
  return cp4_recompose_launch(*s, K0, K1, KH, KW, K, static_cast<cudaStream_t>(stream));
}

// The reference's AllClose (Cuda_kernels/Utils.cu:159-180): the count of elements out of tolerance, computed on the
// device; the one word comes back through a pinned-free synchronous copy (this is a test helper, not a hot call).
int b200cp_allclose_count(const float* A, const float* B, size_t n, float tolerance, unsigned long long* exceeds,
                          void* stream) {
  if (!exceeds) return fail(B200CP_ERR_INVALID_ARG, "b200cp_allclose_count: exceeds is null");
  if (n)
    if (int rc = check_ptrs("b200cp_allclose_count", {A, B})) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  unsigned long long* d = nullptr;
  B200CP_CUDA_OK(cudaMalloc(&d, sizeof(unsigned long long)));
  int rc = allclose_count_launch(A, B, n, tolerance, d, st);
  cudaError_t e = cudaSuccess;
  if (!rc) e = cudaMemcpyAsync(exceeds, d, sizeof(unsigned long long), cudaMemcpyDeviceToHost, st);
  if (!rc && e == cudaSuccess) e = cudaStreamSynchronize(st);
  cudaFree(d);
  if (rc) return rc;
  if (e != cudaSuccess) return fail(B200CP_ERR_CUDA, "b200cp_allclose_count: %s", cudaGetErrorString(e));
  return B200CP_OK;
}

// One training step on device buffers: forward, backward-data and backward-filter.  With 3x3 filters (pad 1) on the
// default path the two convolutions also write their rank planes P = K1^T X and Q = K0^T dU into the workspace and
// the factor gradients are computed from those, without contracting the channels a second time.
// (the two switches are read once, when the library is loaded)
static const bool g_step_no_share = getenv("B200CP_STEP_NO_SHARE") != nullptr;
static const bool g_step_no_slices = getenv("B200CP_STEP_NO_SLICES") != nullptr;   // ranks > 16: the tile gradient kernels
static const bool g_step_no_fork = getenv("B200CP_STEP_NO_FORK") != nullptr;
static bool step_shares_planes(const b200cp_tensor_shape* s, int flags) {
  const int path = path_of(flags);
  return s->Y == 3 && s->X == 3 && s->pad == 1 && (path == B200CP_PATH_MMA || (path == B200CP_PATH_AUTO && g_auto_mma)) &&
         !g_step_no_share;
}

int b200cp_cp4_shares_planes(const b200cp_tensor_shape* s, int flags) {
  if (check_shape(s, "b200cp_cp4_shares_planes")) return 0;
  return step_shares_planes(s, flags) ? 1 : 0;
}

// a second stream and two events per device: forward and backward-data of a step are independent and run side by
// side (the tail of one kernel's last wave overlaps the other kernel), joined again before the factor gradients
struct StepFork {
  cudaStream_t side = nullptr;
  cudaEvent_t fork = nullptr, join = nullptr, fwd_done = nullptr;
};
static StepFork g_step_fork[64];
static std::mutex g_step_mu;
static int step_fork(int dev, StepFork** out) {   // caller holds g_step_mu
  StepFork& f = g_step_fork[dev];
  if (!f.side) {
    B200CP_CUDA_OK(cudaStreamCreateWithFlags(&f.side, cudaStreamNonBlocking));
    B200CP_CUDA_OK(cudaEventCreateWithFlags(&f.fork, cudaEventDisableTiming));
    B200CP_CUDA_OK(cudaEventCreateWithFlags(&f.join, cudaEventDisableTiming));
    B200CP_CUDA_OK(cudaEventCreateWithFlags(&f.fwd_done, cudaEventDisableTiming));
  }
  *out = &f;
  return B200CP_OK;
}

size_t b200cp_cp4_step_workspace_bytes(const b200cp_tensor_shape* s, int flags) {
  if (check_shape(s, "b200cp_cp4_step_workspace_bytes")) return 0;
  const size_t plain = b200cp_cp4_bwd_filter_workspace_bytes(s, flags);
  if (!step_shares_planes(s, flags)) return plain;
  const size_t plane = align_up((size_t)s->N * s->Rank * s->H * s->W * sizeof(float), 256);
  return 2 * plane + std::max(std::max(plain, cp4_bwd_filter_saved_workspace(*s)), cp4_grad_band_workspace(*s));
}

// The step.  `exchange` (may be null): the peer-memory exchange to run as the tail of the gradient reduction;
// *exchanged tells the caller whether that happened (only the fused kernel chain can do it).
static int cp4_step_impl(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0, const float* K1,
                         const float* KH, const float* KW, float* U, float* dX, float* dK_packed, void* workspace,
                         size_t workspace_bytes, void* stream, int flags, const ExchangeArgs* exchange,
                         bool* exchanged) {
  *exchanged = false;
  if (int rc = check_shape(s, "b200cp_cp4_step")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_step", {X, dU, K0, K1, KH, KW, U, dX, dK_packed})) return rc;
  const size_t need = b200cp_cp4_step_workspace_bytes(s, flags);
  if (!workspace || workspace_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "b200cp_cp4_step: workspace of %zu bytes needed, %zu given", need, workspace_bytes);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (!step_shares_planes(s, flags)) {
    const int pf = path_of(flags);
    const int fflags = (pf == B200CP_PATH_TC3X || pf == B200CP_PATH_TC1X) ? (flags & ~B200CP_PATH_MASK) : flags;
    if (int rc = b200cp_cp4_fwd(s, X, K0, K1, KH, KW, U, stream, flags)) return rc;
    if (int rc = b200cp_cp4_bwd_data(s, dU, K0, K1, KH, KW, dX, stream, flags)) return rc;
    return b200cp_cp4_bwd_filter(s, X, dU, K0, K1, KH, KW, dK_packed, workspace, workspace_bytes, stream, fflags);
  }
  const size_t plane = align_up((size_t)s->N * s->Rank * s->H * s->W * sizeof(float), 256);
  float* P = static_cast<float*>(workspace);
  float* Q = reinterpret_cast<float*>(static_cast<char*>(workspace) + plane);
  void* part = static_cast<char*>(workspace) + 2 * plane;
  int dev = 0;
  B200CP_CUDA_OK(cudaGetDevice(&dev));
  StepFork* fk = nullptr;
  const bool may_fork = dev >= 0 && dev < 64 && !g_step_no_fork;
  // the fork / join pairs of two host threads must not interleave on the shared side stream
  std::unique_lock<std::mutex> lk(g_step_mu, std::defer_lock);
  // Whatever way this call ends, the side stream is joined back into the caller's stream: an error return must not
  // leave a stream capture of the caller with an unjoined branch.
  struct Rejoin {
    StepFork* fk = nullptr;
    cudaStream_t st = nullptr;
    bool joined = false;
    void join() {
      if (fk && !joined) {
        joined = true;
        cudaEventRecord(fk->join, fk->side);
        cudaStreamWaitEvent(st, fk->join, 0);
      }
    }
    ~Rejoin() { join(); }
  } rejoin;
  // forward and backward-data: one launch of the band kernel carries both where the shape allows it; otherwise
  // two launches side by side
  bool both = false;
  if (s->Rank <= 32) {
    Cp4Args cv[2] = {conv_args(s, X, K0, K1, KH, KW, U, false, nullptr, P), conv_args(s, dU, K0, K1, KH, KW, dX, true, nullptr, Q)};
    if (int rc = cp4_stream_launch(cv, 2, st, &both)) return rc;
    if (!both)
      if (int rc = cp4_band_launch(cv, 2, st, &both)) return rc;
  }
  // The fused path (both convolutions in one launch, then the gradient band kernel) is a plain chain of kernels on
  // the caller's stream; everything else runs two branches side by side.
  const bool fork = may_fork && !(both && s->Rank <= 16);
  if (fork) {
    lk.lock();
    if (int rc = step_fork(dev, &fk)) return rc;
    B200CP_CUDA_OK(cudaEventRecord(fk->fork, st));
    B200CP_CUDA_OK(cudaStreamWaitEvent(fk->side, fk->fork, 0));
    rejoin.fk = fk;
    rejoin.st = st;
  }
  if (!both) {
    if (int rc = run_conv(s, X, K0, K1, KH, KW, U, st, flags, false, nullptr, P)) return rc;
    if (int rc = run_conv(s, dU, K0, K1, KH, KW, dX, fork ? fk->side : st, flags, true, nullptr, Q)) return rc;
  }
  Cp4BwdFilterArgs a{};
  a.N = s->N; a.C = s->C; a.T = s->T; a.H = s->H; a.W = s->W; a.F = 3; a.pad = 1;
  a.Rs = s->Rank;
  a.X = X; a.dU = dU; a.K0 = K0; a.K1 = K1; a.KH = KH; a.KW = KW; a.dK = dK_packed;
  a.ws = part; a.ws_bytes = workspace_bytes - 2 * plane;
  if (both && s->Rank <= 16) {
    // one more launch: both halves of the factor gradients over the same row bands, then the sum of the bands
    a.r0 = 0;
    a.R = (int)s->Rank;
    bool done = false;
    rejoin.join();   // nothing ran on the side stream
    if (int rc = cp4_grad_band_launch(a, P, Q, st, &done, /*after_own_kernel=*/true, exchange)) return rc;
    if (done) {
      *exchanged = exchange != nullptr;
      return B200CP_OK;
    }
  }
  if (s->Rank > 16 && exchange == nullptr && !g_step_no_slices) {
    // larger ranks: the gradient band kernel once per slice of 16 ranks (each slice streams X and dU again, which
    // still beats the tile kernels that contract the planes' ranks in one pass)
    Cp4BwdFilterArgs b = a;
    b.r0 = 0;
    b.R = 16;
    if (cp4_grad_band_supported(b) && a.ws_bytes >= cp4_grad_band_workspace(*s)) {
      rejoin.join();   // both rank planes are complete before the first slice
      bool taken = true;
      for (unsigned r0 = 0; r0 < s->Rank && taken; r0 += 16) {
        b.r0 = (int)r0;
        b.R = (int)std::min(16u, s->Rank - r0);
        bool done = false;
        if (int rc = cp4_grad_band_launch(b, P, Q, st, &done, /*after_own_kernel=*/r0 > 0, nullptr)) return rc;
        if (!done && r0 > 0) return fail(B200CP_ERR_UNSUPPORTED, "cp4 step: the gradient kernel took rank slice 0 but not %u", r0);
        taken = done;
      }
      if (taken) return B200CP_OK;
      if (fork) {   // not a shape for the band kernel after all: fork again for the two-branch path below
        B200CP_CUDA_OK(cudaEventRecord(fk->fork, st));
        B200CP_CUDA_OK(cudaStreamWaitEvent(fk->side, fk->fork, 0));
        rejoin.joined = false;
      }
    }
  }
  if (fork && s->Rank <= 64) {
    // the gradient kernel in two halves, also side by side: the dK0 half follows the forward on the caller's
    // stream, the dK1 / spatial half follows backward-data on the side stream once the forward's plane is there
    a.r0 = 0;
    a.R = (int)s->Rank;
    B200CP_CUDA_OK(cudaEventRecord(fk->fwd_done, st));
    if (int rc = cp4_bwd_filter_saved_launch(a, P, Q, st, 1)) return rc;
    B200CP_CUDA_OK(cudaStreamWaitEvent(fk->side, fk->fwd_done, 0));
    if (int rc = cp4_bwd_filter_saved_launch(a, P, Q, fk->side, 2)) return rc;
    rejoin.join();
    return cp4_bwd_filter_saved_launch(a, P, Q, st, 3);
  }
  rejoin.join();
  for (unsigned r0 = 0; r0 < s->Rank; r0 += 64) {
    a.r0 = r0;
    a.R = std::min(64u, s->Rank - r0);
    if (int rc = cp4_bwd_filter_saved_launch(a, P, Q, st)) return rc;
  }
  return B200CP_OK;
}

int b200cp_cp4_step(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0, const float* K1,
                    const float* KH, const float* KW, float* U, float* dX, float* dK_packed, void* workspace,
                    size_t workspace_bytes, void* stream, int flags) {
  bool exchanged = false;
  return cp4_step_impl(s, X, dU, K0, K1, KH, KW, U, dX, dK_packed, workspace, workspace_bytes, stream, flags, nullptr,
                       &exchanged);
}

int b200cp_cp4_step_allreduce(void* p2p_ctx, const b200cp_tensor_shape* s, const float* X, const float* dU,
                              const float* K0, const float* K1, const float* KH, const float* KW, float* U, float* dX,
                              float* dK_packed, void* workspace, size_t workspace_bytes, void* stream, int flags) {
  if (!p2p_ctx) return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_allreduce: null exchange context");
  if (int rc = check_shape(s, "b200cp_cp4_step_allreduce")) return rc;
  const size_t n = ((size_t)s->T + s->C + s->Y + s->X) * s->Rank;
  ExchangeArgs ex{};
  if (int rc = p2p_fused_args(p2p_ctx, n, 0, nullptr, &ex)) return rc;
  bool exchanged = false;
  if (int rc = cp4_step_impl(s, X, dU, K0, K1, KH, KW, U, dX, dK_packed, workspace, workspace_bytes, stream, flags, &ex,
                             &exchanged))
    return rc;
  // a shape outside the fused kernel chain: the stand-alone exchange kernel on the finished gradients
  return exchanged ? B200CP_OK : b200cp_p2p_allreduce(p2p_ctx, dK_packed, dK_packed, n, stream);
}

int b200cp_cp4_step_allreduce_pipelined(void* p2p_ctx, const b200cp_tensor_shape* s, const float* X, const float* dU,
                                        const float* K0, const float* K1, const float* KH, const float* KW, float* U,
                                        float* dX, float* dK_scratch, float* dK_prev, void* workspace,
                                        size_t workspace_bytes, void* stream, int flags) {
  if (!p2p_ctx) return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_allreduce_pipelined: null exchange context");
  if (int rc = check_shape(s, "b200cp_cp4_step_allreduce_pipelined")) return rc;
  if (!dK_scratch) return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_allreduce_pipelined: null scratch");
  const size_t n = ((size_t)s->T + s->C + s->Y + s->X) * s->Rank;
  ExchangeArgs ex{};
  if (int rc = p2p_fused_args(p2p_ctx, n, 1, dK_prev, &ex)) return rc;
  bool exchanged = false;
  if (int rc = cp4_step_impl(s, X, dU, K0, K1, KH, KW, U, dX, dK_scratch, workspace, workspace_bytes, stream, flags, &ex,
                             &exchanged))
    return rc;
  if (!exchanged) {
    // a shape outside the fused kernel chain: this rank's gradients are in the scratch vector; the reduction kernel,
    // run over that one "partial", posts them and completes the previous exchange
    if (int rc = cp4_reduce_partials_launch(dK_scratch, 1, (int)n, (int)s->Rank, (int)s->Rank, 0, dK_scratch,
                                            static_cast<cudaStream_t>(stream), true, &ex))
      return rc;
  }
  p2p_fused_set_pending(p2p_ctx, n, (int)s->Rank, (int)s->Rank);
  return B200CP_OK;
}

// The pieces of the step, for callers that run forward and backward at different times (autograd): the convolutions
// with their rank plane written out, and the factor gradients from the two planes.
int b200cp_cp4_fwd_save(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1, const float* KH,
                        const float* KW, float* U, float* P, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_fwd_save")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_fwd_save", {X, K0, K1, KH, KW, U, P})) return rc;
  if (!step_shares_planes(s, flags))
    return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_fwd_save: 3x3 filters with pad 1 on the default (mma) path only");
  return run_conv(s, X, K0, K1, KH, KW, U, static_cast<cudaStream_t>(stream), flags, false, nullptr, P);
}

int b200cp_cp4_bwd_data_save(const b200cp_tensor_shape* s, const float* dU, const float* K0, const float* K1,
                             const float* KH, const float* KW, float* dX, float* Q, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_bwd_data_save")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_bwd_data_save", {dU, K0, K1, KH, KW, dX, Q})) return rc;
  if (!step_shares_planes(s, flags))
    return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_bwd_data_save: 3x3 filters with pad 1 on the default (mma) path only");
  return run_conv(s, dU, K0, K1, KH, KW, dX, static_cast<cudaStream_t>(stream), flags, true, nullptr, Q);
}

// Forward of X and backward-data of dU in one call -- the two convolutions of a training step of a layer whose
// factors are frozen, and the first launch of b200cp_cp4_step: where the row stream or the row bands take the shape,
// one launch carries both (its CTAs share the factor planes and no SM idles between the two).  P / Q (both or
// neither) receive the rank planes.
int b200cp_cp4_fwd_bwd_data(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                            const float* K1, const float* KH, const float* KW, float* U, float* dX, float* P, float* Q,
                            void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_fwd_bwd_data")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_fwd_bwd_data", {X, dU, K0, K1, KH, KW, U, dX})) return rc;
  if ((P == nullptr) != (Q == nullptr))
    return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_fwd_bwd_data: P and Q go together");
  if (P != nullptr) {
    if (int rc = check_ptrs("b200cp_cp4_fwd_bwd_data", {P, Q})) return rc;
    if (!step_shares_planes(s, flags))
      return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_fwd_bwd_data: rank planes for 3x3 filters with pad 1 on the default (mma) path only");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int path = path_of(flags);
  if (s->Y == 3 && s->X == 3 && s->pad == 1 && s->Rank <= 32 &&
      (path == B200CP_PATH_MMA || (path == B200CP_PATH_AUTO && g_auto_mma))) {
    Cp4Args cv[2] = {conv_args(s, X, K0, K1, KH, KW, U, false, nullptr, P), conv_args(s, dU, K0, K1, KH, KW, dX, true, nullptr, Q)};
    bool both = false;
    if (int rc = cp4_stream_launch(cv, 2, st, &both)) return rc;
    if (!both)
      if (int rc = cp4_band_launch(cv, 2, st, &both)) return rc;
    if (both) return B200CP_OK;
  }
  if (int rc = run_conv(s, X, K0, K1, KH, KW, U, st, flags, false, nullptr, P)) return rc;
  return run_conv(s, dU, K0, K1, KH, KW, dX, st, flags, true, nullptr, Q);
}

size_t b200cp_cp4_bwd_filter_saved_workspace_bytes(const b200cp_tensor_shape* s, int flags) {
  (void)flags;
  if (check_shape(s, "b200cp_cp4_bwd_filter_saved_workspace_bytes")) return 0;
  return std::max(cp4_bwd_filter_saved_workspace(*s), cp4_grad_band_workspace(*s));
}

int b200cp_cp4_bwd_filter_saved(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* P,
                                const float* Q, const float* KH, const float* KW, float* dK_packed, void* workspace,
                                size_t workspace_bytes, void* stream, int flags) {
  if (int rc = check_shape(s, "b200cp_cp4_bwd_filter_saved")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_bwd_filter_saved", {X, dU, P, Q, KH, KW, dK_packed})) return rc;
  if (!step_shares_planes(s, flags))
    return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_bwd_filter_saved: 3x3 filters with pad 1 on the default (mma) path only");
  if (!workspace) return fail(B200CP_ERR_WORKSPACE, "b200cp_cp4_bwd_filter_saved: workspace is null");
  Cp4BwdFilterArgs a{};
  a.N = s->N; a.C = s->C; a.T = s->T; a.H = s->H; a.W = s->W; a.F = 3; a.pad = 1;
  a.Rs = s->Rank;
  a.X = X; a.dU = dU; a.KH = KH; a.KW = KW; a.dK = dK_packed;
  a.ws = workspace; a.ws_bytes = workspace_bytes;
  if (s->Rank <= 16 || !g_step_no_slices) {
    // the gradient band kernel, in slices of 16 ranks where there are more
    bool taken = true;
    for (unsigned r0 = 0; r0 < s->Rank && taken; r0 += 16) {
      a.r0 = (int)r0;
      a.R = (int)std::min(16u, s->Rank - r0);
      bool done = false;
      if (int rc = cp4_grad_band_launch(a, P, Q, static_cast<cudaStream_t>(stream), &done, /*after_own_kernel=*/r0 > 0)) return rc;
      if (!done && r0 > 0)
        return fail(B200CP_ERR_UNSUPPORTED, "b200cp_cp4_bwd_filter_saved: the gradient kernel took rank slice 0 but not %u", r0);
      taken = done;
    }
    if (taken) return B200CP_OK;
  }
  for (unsigned r0 = 0; r0 < s->Rank; r0 += 64) {
    a.r0 = r0;
    a.R = std::min(64u, s->Rank - r0);
    if (int rc = cp4_bwd_filter_saved_launch(a, P, Q, static_cast<cudaStream_t>(stream))) return rc;
  }
  return B200CP_OK;
}

static int host_ctx_ready(HostCtx& c) {
  if (c.s_in) return B200CP_OK;
  B200CP_CUDA_OK(cudaStreamCreateWithFlags(&c.s_in, cudaStreamNonBlocking));
  B200CP_CUDA_OK(cudaStreamCreateWithFlags(&c.s_cmp, cudaStreamNonBlocking));
  B200CP_CUDA_OK(cudaStreamCreateWithFlags(&c.s_out, cudaStreamNonBlocking));
  for (int sl = 0; sl < kHostSlots; ++sl)
    for (int e = 0; e < 6; ++e) B200CP_CUDA_OK(cudaEventCreateWithFlags(&c.ev[sl][e], cudaEventDisableTiming));
  return B200CP_OK;
}

int b200cp_cp4_step_host_submit(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                                const float* K1, const float* KH, const float* KW, float* U, float* dX,
                                float* dK_packed, int flags, int slot) {
  if (int rc = check_shape(s, "b200cp_cp4_step_host_submit")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_step_host_submit", {X, K0, K1, KH, KW})) return rc;
  if (slot < 0 || slot >= kHostSlots)
    return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_host_submit: slot must be 0 .. %d", kHostSlots - 1);
  const bool bwd = dU != nullptr;
  if (!U && !bwd) return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_host_submit: nothing to compute");
  if (bwd && (!dX || !dK_packed))
    return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_host_submit: dX and dK_packed required with dU");
  int dev = 0;
  B200CP_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200CP_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_host_mu);
  HostCtx& c = g_host_ctx[dev];
  if (int rc = host_ctx_ready(c)) return rc;
  if (c.pending[slot]) {  // the slot's buffers are still in use by its previous submission
    B200CP_CUDA_OK(cudaEventSynchronize(c.ev[slot][5]));
    c.pending[slot] = false;
  }
  const size_t HW = (size_t)s->H * s->W, R = s->Rank;
  const size_t nX = (size_t)s->N * s->C * HW, nU = (size_t)s->N * s->T * HW;
  const size_t nK0 = s->T * R, nK1 = s->C * R, nKH = s->Y * R, nKW = s->X * R, nK = nK0 + nK1 + nKH + nKW;
  float *dXin, *dUout, *dF, *ddU = nullptr, *ddX = nullptr, *ddK = nullptr, *ws = nullptr;
  const size_t b0 = (size_t)slot * 8;
  constexpr int kWsIndex = 8 * kHostSlots;
  size_t wsb = 0;
  if (bwd) wsb = b200cp_cp4_step_workspace_bytes(s, flags);
  // a (re)allocation frees a buffer the other slot's queued work may still use: drain first
  {
    const size_t want[7] = {nX * 4, nU * 4, nK * 4, bwd ? nU * 4 : 0, bwd ? nX * 4 : 0, bwd ? nK * 4 : 0, 0};
    bool grow = c.bufs.size() <= (size_t)kWsIndex || c.sizes[kWsIndex] < wsb;
    for (int k = 0; k < 7 && !grow; ++k) grow = c.sizes[b0 + k] < want[k];
    for (int o = 0; o < kHostSlots && grow; ++o)
      if (o != slot && c.pending[o]) {
        B200CP_CUDA_OK(cudaEventSynchronize(c.ev[o][5]));
        c.pending[o] = false;
      }
  }
  if (int rc = host_buffer(c, b0 + 0, nX * 4, &dXin)) return rc;
  if (int rc = host_buffer(c, b0 + 1, nU * 4, &dUout)) return rc;
  if (int rc = host_buffer(c, b0 + 2, nK * 4, &dF)) return rc;
  if (bwd) {
    if (int rc = host_buffer(c, b0 + 3, nU * 4, &ddU)) return rc;
    if (int rc = host_buffer(c, b0 + 4, nX * 4, &ddX)) return rc;
    if (int rc = host_buffer(c, b0 + 5, nK * 4, &ddK)) return rc;
    if (int rc = host_buffer(c, kWsIndex, wsb, &ws)) return rc;  // one workspace: the compute stream is serial
  }
  cudaEvent_t* ev = c.ev[slot];
  float *dK0 = dF, *dK1 = dK0 + nK0, *dKH = dK1 + nK1, *dKW = dKH + nKH;
  if (c.stage_bytes[slot] < nK * 4) {
    if (c.stage[slot]) B200CP_CUDA_OK(cudaFreeHost(c.stage[slot]));
    c.stage[slot] = nullptr;
    c.stage_bytes[slot] = 0;
    B200CP_CUDA_OK(cudaHostAlloc(reinterpret_cast<void**>(&c.stage[slot]), nK * 4, cudaHostAllocDefault));
    c.stage_bytes[slot] = nK * 4;
  }
  // (the slot's previous copy out of the staging buffer is complete: its step was waited for above)
  memcpy(c.stage[slot], K0, nK0 * 4);
  memcpy(c.stage[slot] + nK0, K1, nK1 * 4);
  memcpy(c.stage[slot] + nK0 + nK1, KH, nKH * 4);
  memcpy(c.stage[slot] + nK0 + nK1 + nKH, KW, nKW * 4);
  B200CP_CUDA_OK(cudaMemcpyAsync(dF, c.stage[slot], nK * 4, cudaMemcpyHostToDevice, c.s_in));
  B200CP_CUDA_OK(cudaMemcpyAsync(dXin, X, nX * 4, cudaMemcpyHostToDevice, c.s_in));
  B200CP_CUDA_OK(cudaEventRecord(ev[0], c.s_in));
  if (bwd) {
    B200CP_CUDA_OK(cudaMemcpyAsync(ddU, dU, nU * 4, cudaMemcpyHostToDevice, c.s_in));
    B200CP_CUDA_OK(cudaEventRecord(ev[1], c.s_in));
  }
  B200CP_CUDA_OK(cudaStreamWaitEvent(c.s_cmp, ev[0], 0));
  if (!bwd) {
    if (int rc = b200cp_cp4_fwd(s, dXin, dK0, dK1, dKH, dKW, dUout, c.s_cmp, flags)) return rc;
    B200CP_CUDA_OK(cudaEventRecord(ev[2], c.s_cmp));
    B200CP_CUDA_OK(cudaStreamWaitEvent(c.s_out, ev[2], 0));
    B200CP_CUDA_OK(cudaMemcpyAsync(U, dUout, nU * 4, cudaMemcpyDeviceToHost, c.s_out));
  } else {
    // the whole step in one call: the convolutions share their rank planes with the factor gradients
    B200CP_CUDA_OK(cudaStreamWaitEvent(c.s_cmp, ev[1], 0));
    // the factor gradients have no tcgen05 kernel: a forced tcgen05 path applies to the two convolutions only
    if (int rc = b200cp_cp4_step(s, dXin, ddU, dK0, dK1, dKH, dKW, dUout, ddX, ddK, ws, wsb, c.s_cmp, flags)) return rc;
    B200CP_CUDA_OK(cudaEventRecord(ev[4], c.s_cmp));
    B200CP_CUDA_OK(cudaStreamWaitEvent(c.s_out, ev[4], 0));
    if (U) B200CP_CUDA_OK(cudaMemcpyAsync(U, dUout, nU * 4, cudaMemcpyDeviceToHost, c.s_out));
    B200CP_CUDA_OK(cudaMemcpyAsync(dX, ddX, nX * 4, cudaMemcpyDeviceToHost, c.s_out));
    B200CP_CUDA_OK(cudaMemcpyAsync(dK_packed, ddK, nK * 4, cudaMemcpyDeviceToHost, c.s_out));
  }
  B200CP_CUDA_OK(cudaEventRecord(ev[5], c.s_out));
  c.pending[slot] = true;
  return B200CP_OK;
}

int b200cp_cp4_step_host_wait(int slot) {
  if (slot < 0 || slot >= kHostSlots)
    return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_step_host_wait: slot must be 0 .. %d", kHostSlots - 1);
  int dev = 0;
  B200CP_CUDA_OK(cudaGetDevice(&dev));
  if (dev < 0 || dev >= 64) return fail(B200CP_ERR_NO_DEVICE, "device ordinal %d out of range", dev);
  std::lock_guard<std::mutex> lk(g_host_mu);
  HostCtx& c = g_host_ctx[dev];
  if (!c.s_in || !c.pending[slot]) return B200CP_OK;
  B200CP_CUDA_OK(cudaEventSynchronize(c.ev[slot][5]));
  c.pending[slot] = false;
  return B200CP_OK;
}

int b200cp_cp4_step_host(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                         const float* K1, const float* KH, const float* KW, float* U, float* dX, float* dK_packed,
                         int flags) {
  if (int rc = b200cp_cp4_step_host_submit(s, X, dU, K0, K1, KH, KW, U, dX, dK_packed, flags, 0)) return rc;
  return b200cp_cp4_step_host_wait(0);
}

int b200cp_cp4_fwd_host(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1,
                        const float* KH, const float* KW, float* U, int flags) {
  if (!U) return fail(B200CP_ERR_INVALID_ARG, "b200cp_cp4_fwd_host: U is null");
  return b200cp_cp4_step_host(s, X, nullptr, K0, K1, KH, KW, U, nullptr, nullptr, flags);
}

// ---- rCP -------------------------------------------------------------------
static int check_modes(const char* who, int order, const int* a, const int* b, const float* const* F) {
  if (order < 1 || order > 4) return fail(B200CP_ERR_UNSUPPORTED, "%s: order %d not in 1..4", who, order);
  if (!a || !b || !F) return fail(B200CP_ERR_INVALID_ARG, "%s: null mode-size or factor array", who);
  for (int k = 0; k < order; ++k)
    if (!F[k]) return fail(B200CP_ERR_INVALID_ARG, "%s: factor %d is null", who, k);
  return B200CP_OK;
}

int b200cp_rcp_fwd(int N, int H, int W, int order, const int* cdims, const int* tdims, int R, int FH, int FW,
                   const float* X, const float* const* A, const float* S, float* V, void* stream, int flags) {
  (void)flags;
  if (int rc = check_modes("b200cp_rcp_fwd", order, cdims, tdims, A)) return rc;
  if (int rc = check_ptrs("b200cp_rcp_fwd", {X, S, V})) return rc;
  return rcp_chain_launch(N, H, W, order, cdims, tdims, R, FH, FW, X, A, S, V, false,
                          static_cast<cudaStream_t>(stream));
}

size_t b200cp_rcp_bwd_workspace_bytes(int N, int H, int W, int order, const int* cdims, const int* tdims, int R,
                                      int FH, int FW, int flags) {
  (void)R; (void)flags;
  if (order < 1 || order > 4 || !cdims || !tdims || FH < 1 || FW < 1) return 0;
  size_t C = 1, T = 1;
  for (int k = 0; k < order; ++k) { C *= (size_t)cdims[k]; T *= (size_t)tdims[k]; }
  // G itself, then the split-K partial tiles of the GEMM that produces it
  const size_t gemm = dense_grad_scratch_floats(N, (int)T, (int)C, H, W, FH, FW);
  const size_t contr = contract_scratch_floats(order, cdims, tdims, R, FH * FW, true);
  return (T * C * FH * FW + std::max(gemm, contr)) * sizeof(float);
}

int b200cp_rcp_bwd(int N, int H, int W, int order, const int* cdims, const int* tdims, int R, int FH, int FW,
                   const float* X, const float* dV, const float* const* A, const float* S, float* dX,
                   float* const* dA, float* dS, void* workspace, size_t workspace_bytes, void* stream, int flags) {
  if (int rc = check_modes("b200cp_rcp_bwd", order, cdims, tdims, A)) return rc;
  if (int rc = check_ptrs("b200cp_rcp_bwd", {dV, S})) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dX) {
    if (int rc = rcp_chain_launch(N, H, W, order, cdims, tdims, R, FH, FW, dV, A, S, dX, true, st)) return rc;
  }
  if (dA || dS) {
    if (!dA || !dS || !X) return fail(B200CP_ERR_INVALID_ARG, "b200cp_rcp_bwd: dA, dS and X go together");
    for (int k = 0; k < order; ++k)
      if (!dA[k]) return fail(B200CP_ERR_INVALID_ARG, "b200cp_rcp_bwd: dA[%d] is null", k);
    const size_t need = b200cp_rcp_bwd_workspace_bytes(N, H, W, order, cdims, tdims, R, FH, FW, flags);
    if (!workspace || workspace_bytes < need)
      return fail(B200CP_ERR_WORKSPACE, "b200cp_rcp_bwd: workspace of %zu bytes needed, %zu given", need,
                  workspace_bytes);
    int C = 1, T = 1;
    for (int k = 0; k < order; ++k) { C *= cdims[k]; T *= tdims[k]; }
    float* G = static_cast<float*>(workspace);
    if (int rc = dense_grad_launch(N, T, C, H, W, FH, FW, dV, X, G, G + (size_t)T * C * FH * FW, st)) return rc;
    if (int rc = contract_factors_launch(order, cdims, tdims, R, FH * FW, A, S, G, dA, dS, G + (size_t)T * C * FH * FW, st))
      return rc;
  }
  return B200CP_OK;
}

// ---- dense-CP -----------------------------------------------------------------
// ---- the reference's "rebuild" variants: the undecomposed layer with the recomposed weight ------------------------
static int dense_conv_shape(const b200cp_tensor_shape* s, const char* who, b200cp_tensor_shape* q) {
  if (!s) return fail(B200CP_ERR_INVALID_ARG, "%s: shape is null", who);
  *q = *s;
  q->Rank = 1;  // not used by the dense convolution
  return check_shape(q, who);
}

size_t b200cp_conv2d_dense_fwd_workspace_bytes(const b200cp_tensor_shape* s) {
  b200cp_tensor_shape q;
  if (!s || !s->T || !s->C || !s->Y || !s->X || !s->W) return 0;
  q = *s;
  return align_up(conv_dense_scratch_floats(q) * sizeof(float), 256);
}

int b200cp_conv2d_dense_fwd(const b200cp_tensor_shape* s, const float* X, const float* K, float* U, void* workspace,
                            size_t workspace_bytes, void* stream) {
  b200cp_tensor_shape q;
  if (int rc = dense_conv_shape(s, "b200cp_conv2d_dense_fwd", &q)) return rc;
  if (int rc = check_ptrs("b200cp_conv2d_dense_fwd", {X, K, U})) return rc;
  const size_t need = b200cp_conv2d_dense_fwd_workspace_bytes(&q);
  if (!workspace || workspace_bytes < need)
    return fail(B200CP_ERR_WORKSPACE, "b200cp_conv2d_dense_fwd: workspace of %zu bytes needed, %zu given", need,
                workspace ? workspace_bytes : (size_t)0);
  return conv_dense_launch(q, X, K, U, static_cast<float*>(workspace), static_cast<cudaStream_t>(stream));
}

size_t b200cp_cp4_rebuild_fwd_workspace_bytes(const b200cp_tensor_shape* s) {
  if (!s) return 0;
  return align_up((size_t)s->T * s->C * s->Y * s->X * sizeof(float), 256) + b200cp_conv2d_dense_fwd_workspace_bytes(s);
}

int b200cp_cp4_rebuild_fwd(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1,
                           const float* KH, const float* KW, float* U, void* workspace, size_t workspace_bytes,
                           void* stream) {
  if (int rc = check_shape(s, "b200cp_cp4_rebuild_fwd")) return rc;
  if (int rc = check_ptrs("b200cp_cp4_rebuild_fwd", {X, K0, K1, KH, KW, U})) return rc;
  if (!workspace || workspace_bytes < b200cp_cp4_rebuild_fwd_workspace_bytes(s) ||
      (reinterpret_cast<uintptr_t>(workspace) & 15))
    return fail(B200CP_ERR_WORKSPACE, "b200cp_cp4_rebuild_fwd: a 16-byte aligned workspace of %zu bytes is needed, %zu given",
                b200cp_cp4_rebuild_fwd_workspace_bytes(s), workspace ? workspace_bytes : (size_t)0);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  float* K = static_cast<float*>(workspace);
  float* scratch = K + align_up((size_t)s->T * s->C * s->Y * s->X * sizeof(float), 256) / sizeof(float);
  if (int rc = cp4_recompose_launch(*s, K0, K1, KH, KW, K, st)) return rc;
  return conv_dense_launch(*s, X, K, U, scratch, st);
}

int b200cp_rcp_recompose(int order, const int* cdims, const int* tdims, int R, int FH, int FW, const float* const* A,
                         const float* S, float* K, void* stream) {
  if (int rc = check_modes("b200cp_rcp_recompose", order, cdims, tdims, A)) return rc;
  if (int rc = check_ptrs("b200cp_rcp_recompose", {S, K})) return rc;
  if (FH < 1 || FW < 1) return fail(B200CP_ERR_INVALID_ARG, "b200cp_rcp_recompose: filter %d x %d", FH, FW);
  return kron_recompose_launch(order, cdims, tdims, R, A, S, FH * FW, K, static_cast<cudaStream_t>(stream));
}

size_t b200cp_dense_recompose_workspace_bytes(int order, const int* idims, const int* odims, int R) {
  if (order < 1 || order > 4 || !idims || !odims || R < 1) return 0;
  return dense_recompose_scratch_floats(order, idims, odims, R) * sizeof(float);
}

int b200cp_dense_recompose(int order, const int* idims, const int* odims, int R, const float* const* F, float* M,
                           void* workspace, size_t workspace_bytes, void* stream) {
  if (int rc = check_modes("b200cp_dense_recompose", order, idims, odims, F)) return rc;
  if (int rc = check_ptrs("b200cp_dense_recompose", {M})) return rc;
  // without the workspace (or with one that is too small) the direct kernel runs: every element from all factors
  const size_t need = b200cp_dense_recompose_workspace_bytes(order, idims, odims, R);
  const bool two_stage = need && workspace && workspace_bytes >= need && !(reinterpret_cast<uintptr_t>(workspace) & 15);
  return dense_recompose_launch(order, idims, odims, R, F, M, two_stage ? static_cast<float*>(workspace) : nullptr,
                                static_cast<cudaStream_t>(stream));
}

size_t b200cp_dense_matmul_workspace_bytes(int B, int I, int O) {
  if (B < 1 || I < 1 || O < 1) return 0;
  return dense_matmul_scratch_floats(B, I, O) * sizeof(float);
}

int b200cp_dense_matmul(int B, int I, int O, const float* X, const float* M, float* Y, void* workspace,
                        size_t workspace_bytes, void* stream) {
  if (B < 1 || I < 1 || O < 1) return fail(B200CP_ERR_INVALID_ARG, "b200cp_dense_matmul: B=%d I=%d O=%d", B, I, O);
  if (int rc = check_ptrs("b200cp_dense_matmul", {X, M, Y})) return rc;
  const size_t need = b200cp_dense_matmul_workspace_bytes(B, I, O);
  if (!workspace || workspace_bytes < need || (reinterpret_cast<uintptr_t>(workspace) & 255))
    return fail(B200CP_ERR_WORKSPACE, "b200cp_dense_matmul: a 256-byte aligned workspace of %zu bytes is needed", need);
  return dense_matmul_launch(B, I, O, X, M, Y, static_cast<float*>(workspace), static_cast<cudaStream_t>(stream));
}

int b200cp_dense_fwd(int B, int order, const int* idims, const int* odims, int R, const float* X,
                     const float* const* F, float* Y, void* stream, int flags) {
  (void)flags;
  if (int rc = check_modes("b200cp_dense_fwd", order, idims, odims, F)) return rc;
  if (int rc = check_ptrs("b200cp_dense_fwd", {X, Y})) return rc;
  return dense_chain_launch(B, order, idims, odims, R, X, F, Y, false, static_cast<cudaStream_t>(stream));
}

size_t b200cp_dense_bwd_workspace_bytes(int B, int order, const int* idims, const int* odims, int R, int flags) {
  (void)R; (void)flags;
  if (order < 1 || order > 4 || !idims || !odims) return 0;
  size_t I = 1, O = 1;
  for (int k = 0; k < order; ++k) { I *= (size_t)idims[k]; O *= (size_t)odims[k]; }
  const size_t gemm = dense_grad_scratch_floats(B, (int)O, (int)I, 1, 1, 1, 1);
  const size_t contr = contract_scratch_floats(order, idims, odims, R, 1, false);
  return (I * O + std::max(gemm, contr)) * sizeof(float);
}

int b200cp_dense_bwd(int B, int order, const int* idims, const int* odims, int R, const float* X, const float* dY,
                     const float* const* F, float* dX, float* const* dF, void* workspace, size_t workspace_bytes,
                     void* stream, int flags) {
  if (int rc = check_modes("b200cp_dense_bwd", order, idims, odims, F)) return rc;
  if (int rc = check_ptrs("b200cp_dense_bwd", {dY})) return rc;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (dX) {
    if (int rc = dense_chain_launch(B, order, idims, odims, R, dY, F, dX, true, st)) return rc;
  }
  if (dF) {
    if (!X) return fail(B200CP_ERR_INVALID_ARG, "b200cp_dense_bwd: X is needed for dF");
    for (int k = 0; k < order; ++k)
      if (!dF[k]) return fail(B200CP_ERR_INVALID_ARG, "b200cp_dense_bwd: dF[%d] is null", k);
    const size_t need = b200cp_dense_bwd_workspace_bytes(B, order, idims, odims, R, flags);
    if (!workspace || workspace_bytes < need)
      return fail(B200CP_ERR_WORKSPACE, "b200cp_dense_bwd: workspace of %zu bytes needed, %zu given", need,
                  workspace_bytes);
    int I = 1, O = 1;
    for (int k = 0; k < order; ++k) { I *= idims[k]; O *= odims[k]; }
    float* G = static_cast<float*>(workspace);  // G[o][i] = sum_b dY[b,o] X[b,i]
    if (int rc = dense_grad_launch(B, O, I, 1, 1, 1, 1, dY, X, G, G + (size_t)I * O, st)) return rc;
    if (int rc = contract_factors_launch(order, idims, odims, R, 1, F, nullptr, G, dF, nullptr, G + (size_t)I * O, st))
      return rc;
  }
  return B200CP_OK;
}

int b200cp_device_status(void) {
  int v = 0;
  if (int rc = tc_device_status(&v)) return rc;
  if (v) return fail(B200CP_ERR_TIMEOUT, "a bounded wait ran out in block %d (code %d)", v & 0xffff, v >> 16);
  if (int rc = gemm_tc_status(&v)) return rc;
  if (v) return fail(B200CP_ERR_TIMEOUT, "gradient GEMM: a bounded wait ran out in block %d", v & 0xffff);
  if (int rc = band_device_status(&v)) return rc;
  if (v) return fail(B200CP_ERR_TIMEOUT, "cp4 band kernel: a bounded wait ran out in block %d", v & 0xffff);
  if (int rc = stream_device_status(&v)) return rc;
  if (v) return fail(B200CP_ERR_TIMEOUT, "cp4 row-stream kernel: a bounded wait ran out in block %d", v & 0xffff);
  if (int rc = grad_band_device_status(&v)) return rc;
  if (v) return fail(B200CP_ERR_TIMEOUT, "cp4 gradient band kernel: a bounded wait ran out in block %d", v & 0xffff);
  return B200CP_OK;
}

int b200cp_debug_cp4_tc(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1,
                        const float* KH, const float* KW, float* U, float* P_block0, int terms, void* stream) {
  if (int rc = check_shape(s, "b200cp_debug_cp4_tc")) return rc;
  if (int rc = check_ptrs("b200cp_debug_cp4_tc", {X, K0, K1, KH, KW, U})) return rc;
  Cp4Args a{};
  a.N = s->N; a.H = s->H; a.W = s->W; a.Y = s->Y; a.X = s->X; a.pad = s->pad; a.Cin = s->C; a.Cout = s->T;
  a.Fin = K1; a.Fout = K0; a.KH = KH; a.KW = KW; a.in = X; a.out = U; a.Rs = s->Rank; a.R = s->Rank;
  return cp4_tc_launch(a, terms == 1 ? 1 : 3, P_block0, static_cast<cudaStream_t>(stream));
}

int b200cp_debug_tc_selftest(int mode, const float* A, const float* B, float* D, int* status, void* stream) {
  if (int rc = check_ptrs("b200cp_debug_tc_selftest", {A, B, D, status})) return rc;
  if (mode != 0 && mode != 1) return fail(B200CP_ERR_INVALID_ARG, "b200cp_debug_tc_selftest: mode must be 0 or 1");
  DeviceInfo di;
  if (int rc = device_info(&di)) return rc;
  return tc_selftest_launch(mode, A, B, D, status, static_cast<cudaStream_t>(stream));
}

const char* b200cp_last_error_string(void) { return last_error_buffer(); }

const char* b200cp_status_string(int status) {
  switch (status) {
    case B200CP_OK: return "ok";
    case B200CP_ERR_INVALID_ARG: return "invalid argument";
    case B200CP_ERR_UNSUPPORTED: return "unsupported shape or path";
    case B200CP_ERR_WORKSPACE: return "workspace missing or too small";
    case B200CP_ERR_CUDA: return "CUDA runtime error";
    case B200CP_ERR_TIMEOUT: return "device-side wait timed out";
    case B200CP_ERR_NO_DEVICE: return "no usable sm_100 device";
    default: return "unknown status";
  }
}

unsigned long long b200cp_launch_count(void) { return g_launches.load(); }
int b200cp_version(void) { return 100; }

}  // extern "C"
