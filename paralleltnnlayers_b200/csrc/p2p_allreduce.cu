// One-shot allreduce of the packed factor gradients over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The buffer is a few KB ((T + C + FH + FW) * R floats), so the collective is pure latency.  Every rank owns an
// exchange region [2 slots][world][max floats] plus flags [2 slots][world] in its own memory, exported to the peers
// through CUDA IPC.  One launch per step:
//   1. the rank stores its vector into slot s, row `rank`, of EVERY rank's region (plain peer stores),
//   2. fences and raises flag (s, rank) in every region to the step's sequence number,
//   3. waits until all `world` flags of slot s in its OWN region carry that number (a bounded wait: about half a
//      second, then a status word is set, the result is filled with NaN -- a missed exchange cannot pass for a sum --
//      and the kernel leaves; b200cp_p2p_status reports it),
//   4. adds the `world` rows of its own region in rank order, so every rank gets bitwise the same sums.
// Flags are written with st.release.sys after a system-scope fence and polled with ld.acquire.sys.
// Two slots alternate.  A rank that writes slot s for step q has finished step q - 1, for which it needed every
// peer's flag of step q - 1; a peer raises that flag in its launch q - 1, which runs after its launch q - 2 has read
// slot s.  So a slot is never overwritten while a peer still reads it.  The sequence number lives in device memory and is advanced by the kernel, so a captured CUDA graph can
// be replayed.  No NCCL kernel, no multicast, no peer loads: a CTA of 256 threads that fits next to the compute kernels.
#include <atomic>
#include <cstring>

#include "common.cuh"
#include "b200cp_test.h"

namespace b200cp {

namespace {

constexpr int kMaxWorld = 16;
constexpr int kP2PThreads = 256;
constexpr int kP2PCtas = 4;   // CTAs of one exchange; each moves a quarter of the vector and has its own flags
constexpr long long kDefaultWaitCycles = 1000000000ll;   // about half a second
std::atomic<long long> g_wait_cycles{kDefaultWaitCycles};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

struct P2PCtx {
  int rank, world, device;
  size_t max_floats, row;     // row = floats per (slot, rank) row
  void* base;                 // own allocation
  void* peer[kMaxWorld];      // mapped allocations (peer[rank] == base)
  bool opened[kMaxWorld];
  // device-side table
  float** d_data;             // [world] data pointers
  unsigned** d_flags;         // [world] flag pointers
  unsigned* d_seq;            // [kP2PCtas] next sequence number per CTA
  int* d_status;
  size_t bytes;
};

__host__ __device__ inline size_t flags_offset(size_t row, int world) { return 2 * (size_t)world * row * sizeof(float); }

__global__ void __launch_bounds__(kP2PThreads) p2p_allreduce_kernel(float* const* __restrict__ data,
                                                                    unsigned* const* __restrict__ flags, unsigned* seqs,
                                                                    int* status, int rank, int world, size_t row,
                                                                    const float* src, float* dst, size_t n,
                                                                    long long wait_cycles) {
  // (src and dst may be the same buffer: a CTA reads and writes only its own part of the vector)
  const int cta = blockIdx.x, tid = threadIdx.x;
  __shared__ unsigned s_seq;
  __shared__ int s_missed;
  if (tid == 0) {
    s_seq = seqs[cta] + 1;
    s_missed = 0;
  }
  __syncthreads();
  const unsigned seq = s_seq;
  const int slot = seq & 1;
  // this CTA's part of the vector
  const size_t per = (n + kP2PCtas - 1) / kP2PCtas;
  const size_t lo = min(n, (size_t)cta * per), hi = min(n, lo + per);
  // 1. the own part into every rank's region
  for (int p = 0; p < world; ++p) {
    float* d = data[p] + ((size_t)slot * world + rank) * row;
    for (size_t i = lo + tid; i < hi; i += kP2PThreads) d[i] = src[i];
  }
  __threadfence_system();
  __syncthreads();
  // 2. flag (slot, cta, rank) of every region: the CTA's stores were fenced above by the threads that made them;
  //    the flag-writing thread fences again after the barrier and stores with release semantics
  if (tid < world) {
    __threadfence_system();
    st_release_sys(flags[tid] + ((size_t)slot * kP2PCtas + cta) * kMaxWorld + rank, seq);
  }
  // 3. all flags of the own region
  if (tid < world) {
    const unsigned* f = flags[rank] + ((size_t)slot * kP2PCtas + cta) * kMaxWorld + tid;
    const long long t0 = clock64();
    while ((int)(ld_acquire_sys(f) - seq) < 0) {
      if (clock64() - t0 > wait_cycles) {   // give up, never hang
        s_missed = 1;
        atomicExch(status, 1 + rank);
        break;
      }
      __nanosleep(64);
    }
  }
  __threadfence_system();
  __syncthreads();
  // 4. the rows of the own region, in rank order; NaN where a peer's part never arrived
  const bool missed = s_missed != 0;
  const float* own = data[rank] + (size_t)slot * world * row;
  for (size_t i = lo + tid; i < hi; i += kP2PThreads) {
    float s = 0.f;
    for (int p = 0; p < world; ++p) s += __ldcg(own + (size_t)p * row + i);
    dst[i] = missed ? __int_as_float(0x7fc00000) : s;
  }
  if (tid == 0) seqs[cta] = seq;   // the sequence advances either way: the next exchange lines up with the peers' again
}

}  // namespace

}  // namespace b200cp

using namespace b200cp;

extern "C" {

int b200cp_p2p_destroy(void* ctx);

int b200cp_p2p_init(int rank, int world, size_t max_floats, unsigned char* handle_out, void** ctx_out) {
  if (!handle_out || !ctx_out) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_init: null argument");
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world || max_floats == 0)
    return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_init: rank %d of %d ranks (at most %d), %zu floats", rank, world,
                kMaxWorld, max_floats);
  P2PCtx* c = new P2PCtx();
  c->rank = rank; c->world = world; c->max_floats = max_floats;
  c->row = (max_floats + 3) / 4 * 4;
  c->base = nullptr; c->d_data = nullptr; c->d_flags = nullptr; c->d_seq = nullptr; c->d_status = nullptr;
  for (int p = 0; p < kMaxWorld; ++p) { c->peer[p] = nullptr; c->opened[p] = false; }
  c->bytes = flags_offset(c->row, world) + 2 * (size_t)kP2PCtas * kMaxWorld * sizeof(unsigned);
  cudaIpcMemHandle_t h;
  memset(&h, 0, sizeof(h));
  static_assert(sizeof(cudaIpcMemHandle_t) == B200CP_P2P_HANDLE_BYTES, "IPC handle size");
  // every allocation of the context, or none: a failure frees what exists and reports the CUDA error
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc(&c->base, c->bytes);
  if (e == cudaSuccess) e = cudaMemset(c->base, 0, c->bytes);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_data, sizeof(float*) * kMaxWorld);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_flags, sizeof(unsigned*) * kMaxWorld);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_seq, sizeof(unsigned) * kP2PCtas);
  if (e == cudaSuccess) e = cudaMemset(c->d_seq, 0, sizeof(unsigned) * kP2PCtas);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_status, sizeof(int));
  if (e == cudaSuccess) e = cudaMemset(c->d_status, 0, sizeof(int));
  if (e == cudaSuccess && world > 1) e = cudaIpcGetMemHandle(&h, c->base);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e != cudaSuccess) {
    b200cp_p2p_destroy(c);
    return fail(B200CP_ERR_CUDA, "b200cp_p2p_init: %s", cudaGetErrorString(e));
  }
  c->peer[rank] = c->base;
  memcpy(handle_out, &h, sizeof(h));
  *ctx_out = c;
  return B200CP_OK;
}

int b200cp_p2p_connect(void* ctx, const unsigned char* handles) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c || (!handles && c->world > 1)) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_connect: null argument");
  for (int p = 0; p < c->world; ++p) {
    if (p == c->rank || c->opened[p]) continue;
    cudaIpcMemHandle_t h;
    memcpy(&h, handles + (size_t)p * B200CP_P2P_HANDLE_BYTES, sizeof(h));
    B200CP_CUDA_OK(cudaIpcOpenMemHandle(&c->peer[p], h, cudaIpcMemLazyEnablePeerAccess));
    c->opened[p] = true;
  }
  float* data[kMaxWorld] = {};
  unsigned* flags[kMaxWorld] = {};
  for (int p = 0; p < c->world; ++p) {
    data[p] = static_cast<float*>(c->peer[p]);
    flags[p] = reinterpret_cast<unsigned*>(static_cast<char*>(c->peer[p]) + flags_offset(c->row, c->world));
  }
  B200CP_CUDA_OK(cudaMemcpy(c->d_data, data, sizeof(data), cudaMemcpyHostToDevice));
  B200CP_CUDA_OK(cudaMemcpy(c->d_flags, flags, sizeof(flags), cudaMemcpyHostToDevice));
  return B200CP_OK;
}

int b200cp_p2p_allreduce(void* ctx, const float* src, float* dst, size_t n, void* stream) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c || !src || !dst) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_allreduce: null argument");
  if (n > c->max_floats) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_allreduce: %zu floats, room for %zu", n, c->max_floats);
  p2p_allreduce_kernel<<<kP2PCtas, kP2PThreads, 0, static_cast<cudaStream_t>(stream)>>>(
      c->d_data, c->d_flags, c->d_seq, c->d_status, c->rank, c->world, c->row, src, dst, n, g_wait_cycles.load());
  B200CP_LAUNCH_OK("p2p_allreduce_kernel");
  return B200CP_OK;
}

void b200cp_test_set_p2p_wait_cycles(long long cycles) { g_wait_cycles.store(cycles > 0 ? cycles : kDefaultWaitCycles); }

// Test hook: the ranks of a single-process world (contexts made by b200cp_p2p_init in this process, in rank order)
// map each other's regions directly instead of through CUDA IPC.
int b200cp_test_p2p_connect_local(void* ctx, void* const* all_ctx) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c || !all_ctx) return fail(B200CP_ERR_INVALID_ARG, "b200cp_test_p2p_connect_local: null argument");
  float* data[kMaxWorld] = {};
  unsigned* flags[kMaxWorld] = {};
  for (int p = 0; p < c->world; ++p) {
    P2PCtx* o = static_cast<P2PCtx*>(all_ctx[p]);
    if (!o || o->world != c->world || o->row != c->row || o->rank != p)
      return fail(B200CP_ERR_INVALID_ARG, "b200cp_test_p2p_connect_local: context %d does not belong to this world", p);
    c->peer[p] = o->base;
    data[p] = static_cast<float*>(o->base);
    flags[p] = reinterpret_cast<unsigned*>(static_cast<char*>(o->base) + flags_offset(c->row, c->world));
  }
  B200CP_CUDA_OK(cudaMemcpy(c->d_data, data, sizeof(data), cudaMemcpyHostToDevice));
  B200CP_CUDA_OK(cudaMemcpy(c->d_flags, flags, sizeof(flags), cudaMemcpyHostToDevice));
  return B200CP_OK;
}

// 0 when no wait has run out; synchronises the device
int b200cp_p2p_status(void* ctx) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_status: null argument");
  int v = 0, zero = 0;
  B200CP_CUDA_OK(cudaDeviceSynchronize());
  B200CP_CUDA_OK(cudaMemcpy(&v, c->d_status, sizeof(int), cudaMemcpyDeviceToHost));
  if (v) {
    B200CP_CUDA_OK(cudaMemcpy(c->d_status, &zero, sizeof(int), cudaMemcpyHostToDevice));
    return fail(B200CP_ERR_TIMEOUT, "p2p allreduce: rank %d waited in vain for a peer's flag", v - 1);
  }
  return B200CP_OK;
}

int b200cp_p2p_destroy(void* ctx) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c) return B200CP_OK;
  cudaDeviceSynchronize();
  for (int p = 0; p < c->world; ++p)
    if (c->opened[p]) cudaIpcCloseMemHandle(c->peer[p]);
  cudaFree(c->base);
  cudaFree(c->d_data);
  cudaFree(c->d_flags);
  cudaFree(c->d_seq);
  cudaFree(c->d_status);
  delete c;
  return B200CP_OK;
}

}  // extern "C"
