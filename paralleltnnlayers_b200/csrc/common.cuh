// Shared host/device helpers of the b200cp library (internal).
#pragma once

#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "b200cp.h"

namespace b200cp {

// ---- error reporting ------------------------------------------------------
char* last_error_buffer();  // thread-local, 512 bytes
int fail(int status, const char* fmt, ...);
extern std::atomic<unsigned long long> g_launches;

inline void count_launch(unsigned n = 1) { g_launches.fetch_add(n, std::memory_order_relaxed); }

#define B200CP_CUDA_OK(expr)                                                                        \
  do {                                                                                              \
    cudaError_t err__ = (expr);                                                                     \
    if (err__ != cudaSuccess)                                                                       \
      return ::b200cp::fail(B200CP_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(err__));    \
  } while (0)

#define B200CP_LAUNCH_OK(name)                                                                      \
  do {                                                                                              \
    cudaError_t err__ = cudaPeekAtLastError();                                                      \
    if (err__ != cudaSuccess)                                                                       \
      return ::b200cp::fail(B200CP_ERR_CUDA, "launch of %s failed: %s", name,                       \
                            cudaGetErrorString(cudaGetLastError()));                                \
    ::b200cp::count_launch();                                                                       \
  } while (0)

// ---- device properties (cached per device) --------------------------------
struct DeviceInfo {
  int sm_count = 0;
  int smem_optin = 0;  // max dynamic shared memory per block (opt-in), bytes
  int cc_major = 0;
};
int device_info(DeviceInfo* out);  // status

// cudaFuncSetAttribute(MaxDynamicSharedMemorySize) once per kernel, device and size instead of once per launch:
// `slot` is a function-local static array of 64 zero-initialised atomics, one per device ordinal.
inline cudaError_t ensure_dynamic_smem(const void* kernel, std::atomic<int>* slot, int bytes) {
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  if (dev < 0 || dev >= 64) return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (slot[dev].load(std::memory_order_relaxed) >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) slot[dev].store(bytes, std::memory_order_relaxed);
  return e;
}

__host__ __device__ inline int ceil_div(int a, int b) { return (a + b - 1) / b; }
inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// padded rank used by the SIMT kernels' register tiles
inline int padded_rank(int r) { return r <= 4 ? 4 : r <= 8 ? 8 : r <= 16 ? 16 : r <= 32 ? 32 : 64; }

// ---- launch entry points implemented in the .cu files ---------------------
struct Cp4Args {
  int N, Cin, Cout, H, W, Y, X, pad;
  int R;        // ranks handled by this launch (<= 64)
  int Rs;       // row stride of the factor matrices (total rank)
  int r0;       // first rank of this launch
  int flip;     // 1: use KH[Y-1-y], KW[X-1-x]
  int accumulate;
  const float *in, *Fin, *Fout, *KH, *KW;
  float* out;
  const float* KC = nullptr;  // free [Y][X][Rs] spatial core (three-factor CP conv) instead of KH x KW; mma path only
  float* save = nullptr;      // [N][Rs][H][W]: the rank plane sum_ch Fin[ch][r] in[ch][px] is also written here (mma, 3x3)
};
// Programmatic dependent launch.  A kernel launched with `programmatic` may be scheduled while the previous kernel on
// the stream drains: it executes grid_dependency_wait() before its first global read, which returns when that kernel
// has completed and its writes are visible.  (Without the attribute the wait returns at once.)  B200CP_PDL=0 keeps
// every launch a plain one.
#ifdef __CUDACC__
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Lets a programmatically dependent kernel be scheduled once every CTA of this grid has got here (or has exited): its
// CTAs take the SMs this grid leaves and wait in grid_dependency_wait() for the grid's completion.
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, bool programmatic,
                          Args&&... args) {
  static const bool off = [] {
    const char* e = getenv("B200CP_PDL");
    return e && e[0] == '0';
  }();
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute at[1];
  at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  at[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = at;
  cfg.numAttrs = (programmatic && !off) ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<KArgs>(args)...);
}
#endif

int cp4_simt_launch(const Cp4Args& a, cudaStream_t st);
// same arguments; channel contractions on the warp-level tensor path (mma.sync, three tf32 terms)
int cp4_mma_launch(const Cp4Args& a, cudaStream_t st);

// Full-width row bands, TMA loads (3x3 filters, pad 1, W a multiple of 4, at most 32 ranks per launch): one or two
// convolutions of the same image size in one launch.  *done = false: not a shape this kernel takes.
int cp4_band_launch(const Cp4Args* convs, int nconv, cudaStream_t st, bool* done);
int band_device_status(int* out);
// Row stream (one persistent CTA per SM; 3x3, pad 1, W a multiple of 8 that is 8 or 24 modulo 32, at most 16 ranks,
// input channels a multiple of 8, at most 256): the same contract as cp4_band_launch.
int cp4_stream_launch(const Cp4Args* convs, int nconv, cudaStream_t st, bool* done);
int stream_device_status(int* out);
long long* band_trace_buffer();   // diagnostics buffer set by b200cp_test_set_band_trace (null: off)

struct Cp4BwdFilterArgs {
  int N, C, T, H, W, F, pad;
  int R, Rs, r0;
  const float *X, *dU, *K0, *K1, *KH, *KW;
  const float* KC = nullptr;  // free [3][3][Rs] core: dK is then packed [T*Rs | C*Rs | 9*Rs]; mma path only
  float* dK;  // packed [T*Rs | C*Rs | F*Rs | F*Rs]
  void* ws;
  size_t ws_bytes;
};
size_t cp4_bwd_filter_simt_workspace(const b200cp_tensor_shape& s);
int cp4_bwd_filter_simt_launch(const Cp4BwdFilterArgs& a, cudaStream_t st);
// warp-level tensor path (mma.sync, three tf32 terms); 3x3 filters with pad 1
bool cp4_bwd_filter_mma_supported(const Cp4BwdFilterArgs& a);
size_t cp4_bwd_filter_mma_workspace(const b200cp_tensor_shape& s);
int cp4_bwd_filter_mma_launch(const Cp4BwdFilterArgs& a, cudaStream_t st);
// the same gradients from the rank planes P = K1^T X, Q = K0^T dU ([N][Rs][H][W]) saved by the convolutions
size_t cp4_bwd_filter_saved_workspace(const b200cp_tensor_shape& s);
// part 0: everything and the sum of the per-CTA partials; 1: the dK0 half (needs P only); 2: the dK1 / spatial half;
// 3: the sum of the partials only (after halves 1 and 2, which may run on different streams)
int cp4_bwd_filter_saved_launch(const Cp4BwdFilterArgs& a, const float* P, const float* Q, cudaStream_t st, int part = 0);
// dK[row*Rs + r0 + r] = sum over parts of partial[part][row*R + r], in a fixed order
// The peer-memory exchange of a data-parallel step, as the tail of the kernel that sums the partial gradients: every
// CTA of that kernel owns 32 gradient entries, stores each of its sums together with the exchange's sequence number
// as one 8-byte word into every rank's exchange region (plain peer stores), then reads the words of all ranks from
// its own region, spinning (bounded) on a word until it carries the sequence number, and adds them in rank order.
// An aligned 8-byte store is one transaction, so the value and its "arrived" mark cannot be seen apart: no fence and
// no separate flag.  Filled by p2p_fused_args() from a context of b200cp_p2p_init.
struct ExchangeArgs {
  unsigned long long* const* data;   // [world] every rank's region: [2 slots][world][row] words {value, sequence}
  unsigned* seqs;          // [ctas] sequence number of this rank's last exchange, per CTA
  int* status;
  int rank, world, ctas;
  size_t row;
  long long wait_cycles;
  int mode;                // 0: post and complete in the same kernel; 1: post, and complete the previous exchange
  float* prev_out;         // mode 1: where the previous exchange's sums go (null: nothing is pending)
};
// one word of an exchange region
__device__ __forceinline__ void exchange_store(unsigned long long* p, float v, unsigned seq) {
  asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(__float_as_uint(v)), "r"(seq) : "memory");
}
__device__ __forceinline__ bool exchange_load(const unsigned long long* p, unsigned seq, float* v) {
  unsigned a, b;
  asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(a), "=r"(b) : "l"(p) : "memory");
  *v = __uint_as_float(a);
  return b == seq;
}
// mode 1 keeps the posted exchange pending in the context until the next mode-1 call or p2p_fused_flush completes it
int p2p_fused_args(void* ctx, size_t n, int mode, float* prev_out, ExchangeArgs* out);
void p2p_fused_set_pending(void* ctx, size_t n, int R, int Rs);
int exchange_finish_launch(const ExchangeArgs& ex, int nparam, int R, int Rs, int r0, float* dK, cudaStream_t st);
// split > 0: entries below `split` are summed over the first nparts_low partial vectors, the others over nparts
int cp4_reduce_partials_launch(const float* partial, int nparts, int nparam, int R, int Rs, int r0, float* dK,
                               cudaStream_t st, bool after_own_kernel = false, const ExchangeArgs* exchange = nullptr,
                               int split = 0, int nparts_low = 0);
// the same gradients over full-width row bands (bulk / tensor-map loads, 3x3, W % 4 == 0, at most 16 ranks);
// *done = false: not a shape this kernel takes
bool cp4_grad_band_supported(const Cp4BwdFilterArgs& a);
size_t cp4_grad_band_workspace(const b200cp_tensor_shape& s);
// after_own_kernel: the previous launch on the stream is one of this library's kernels (the convolutions that wrote P
// and Q); the launch then overlaps that kernel's completion (programmatic dependent launch)
int cp4_grad_band_launch(const Cp4BwdFilterArgs& a, const float* P, const float* Q, cudaStream_t st, bool* done,
                         bool after_own_kernel = false, const ExchangeArgs* exchange = nullptr);
int grad_band_device_status(int* out);
size_t cp4_bwd_filter_static_scratch_bytes();
int cp4_bwd_filter_static_launch(const Cp4BwdFilterArgs& a, cudaStream_t st);
int cp4_bwd_filter_full_launch(const b200cp_tensor_shape& s, const float* X, const float* dU, float* dK,
                               cudaStream_t st);
int cp4_recompose_launch(const b200cp_tensor_shape& s, const float* K0, const float* K1, const float* KH,
                         const float* KW, float* K, cudaStream_t st);


// *count_dev = number of elements whose relative difference exceeds tol (Cuda_kernels/Utils.cu:143-156)
int allclose_count_launch(const float* A, const float* B, size_t n, float tol, unsigned long long* count_dev,
                          cudaStream_t st);

struct TcPlan {
  int TH = 0, RP = 0;
};
bool cp4_tc_supported(const Cp4Args& a, const DeviceInfo& di, TcPlan* plan);
// terms: 3 = hi/lo split (fp32-grade accuracy), 1 = single tf32 pass.  dbgP (nullable): CTA 0 dumps its P tile.
int cp4_tc_launch(const Cp4Args& a, int terms, float* dbgP, cudaStream_t st);
int tc_device_status(int* out);
int tc_selftest_launch(int mode, const float* A, const float* B, float* D, int* status, cudaStream_t st);

int rcp_chain_launch(int N, int H, int W, int order, const int* cdims, const int* tdims, int R, int FH, int FW,
                     const float* X, const float* const* A, const float* S, float* V, bool transposed,
                     cudaStream_t st);
// register-tiled kernel for the shapes it is compiled for; *done = false means "not this shape, use the chain kernel"
int rcp_fast_launch(int N, int H, int W, int order, const int* din, const int* dout, const int* fsi, const int* fso,
                    int R, int FH, int FW, const float* X, const float* const* A, const float* S, float* V, bool flip,
                    cudaStream_t st, bool* done);
int dense_fast_launch(int B, int order, const int* din, const int* dout, const int* fsi, const int* fso, int R,
                      const float* X, const float* const* F, float* Y, cudaStream_t st, bool* done);
int dense_chain_launch(int B, int order, const int* idims, const int* odims, int R, const float* X,
                       const float* const* F, float* Y, bool transposed, cudaStream_t st);
// G[tap][t][c] = sum_{n,h,w} dV[n,t,h,w] * Xpad[n,c,h+y,w+x]; scratch holds dense_grad_scratch_floats() floats
size_t dense_grad_scratch_floats(int N, int T, int C, int H, int W, int FH, int FW);
int dense_grad_launch(int N, int T, int C, int H, int W, int FH, int FW, const float* dV, const float* X, float* G,
                      float* scratch, cudaStream_t st);
// tcgen05 form of the flat gradient GEMM (G[M][N] = A^T B, A [K][M], B [K][N]); three-term tf32 split, fp32-grade
bool gemm_tc_supported(int K, int M, int N);
size_t gemm_tc_scratch_floats(int K, int M, int N);
int gemm_tc_launch(int K, int M, int N, const float* A, const float* B, float* G, float* scratch, cudaStream_t st);
int gemm_tc_status(int* out);
// conv form of the same kernel: G[tap][T][C] from NCHW operands (padded, transposed hi / lo planes in the scratch)
bool conv_gemm_tc_supported(int N, int T, int C, int H, int W, int FH, int FW);
size_t conv_gemm_tc_scratch_floats(int N, int T, int C, int H, int W, int FH, int FW);
int conv_gemm_tc_launch(int N, int T, int C, int H, int W, int FH, int FW, const float* dV, const float* X, float* G,
                        float* scratch, cudaStream_t st);
// the reference's "rebuild" variants: dense conv2d forward with an undecomposed filter K [T][C][FH][FW]; recomposed
// weights of the dense ([I][O]) and reshaped-CP ([T][C][FH][FW], S != nullptr) layers; Y = X M for the dense layer
bool conv_dense_supported(const b200cp_tensor_shape& s);
size_t conv_dense_scratch_floats(const b200cp_tensor_shape& s);
int conv_dense_launch(const b200cp_tensor_shape& s, const float* X, const float* K, float* U, float* scratch,
                      cudaStream_t st);
int kron_recompose_launch(int order, const int* a, const int* b, int R, const float* const* F, const float* S, int taps,
                          float* Wout, cudaStream_t st);
size_t dense_recompose_scratch_floats(int order, const int* a, const int* b, int R);
int dense_recompose_launch(int order, const int* a, const int* b, int R, const float* const* F, float* M, float* scratch,
                           cudaStream_t st);
size_t dense_matmul_scratch_floats(int B, int I, int O);
int dense_matmul_launch(int B, int I, int O, const float* X, const float* M, float* Y, float* scratch, cudaStream_t st);
// G[e] = sum over splits of P[split][e], in split order
void sum_splits_launch(const float* P, float* G, size_t n, int splits, cudaStream_t st);
size_t contract_scratch_floats(int order, const int* cdims, const int* tdims, int R, int taps, bool has_s);
int contract_factors_launch(int order, const int* cdims, const int* tdims, int R, int taps, const float* const* A,
                            const float* S, const float* G, float* const* dA, float* dS, float* scratch,
                            cudaStream_t st);

}  // namespace b200cp
