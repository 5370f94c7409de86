// One-shot allreduce of the packed factor gradients over peer memory (NVLink / NVSwitch), one process per GPU.
//
// The buffer is a few KB ((T + C + FH + FW) * R floats), so the collective is pure latency.  Every rank owns an
// exchange region [2 slots][world][max floats] of 8-byte words in its own memory, exported to the peers through CUDA
// IPC.  A word holds a value and the sequence number of the exchange it belongs to; it is written with one aligned
// 8-byte store, which is one transaction, so a reader sees either the old word or the new one, never a new value
// without its number.  One launch per step:
//   1. the rank stores its vector, every value with the step's sequence number, into slot s, row `rank`, of EVERY
//      rank's region (plain peer stores; no fence, no flag),
//   2. reads the `world` rows of its OWN region, spinning on a word until it carries the number (a bounded wait: about
//      half a second, then a status word is set, the result is filled with NaN -- a missed exchange cannot pass for
//      a sum -- and the kernel leaves; b200cp_p2p_status reports it), and adds them in rank order, so every rank
//      gets bitwise the same sums.
// (An earlier form wrote the data, then a system-scope fence and a release store of a flag; on one GPU exchanging
// with itself the fence alone cost 9 us per step.)
// Two slots alternate.  A rank that writes slot s for step q has finished step q - 1, for which it needed every
// peer's words of step q - 1; a peer writes those in its launch q - 1, which runs after its launch q - 2 has read
// slot s.  So a slot is never overwritten while a peer still reads it.  The sequence number lives in device memory
// and is advanced by the kernel, so a captured CUDA graph can be replayed.  No NCCL kernel, no multicast, no peer
// loads.  The same exchange also exists as the tail of the kernel that adds the partial factor gradients of a
// training step (cp4_reduce_partials_kernel<true>), with a region and sequence numbers of its own.
#include <atomic>
#include <cstring>

#include "common.cuh"
#include "b200cp_test.h"

namespace b200cp {

namespace {

constexpr int kMaxWorld = 16;
// 128 threads of at most 32 registers: 4096 registers, which is what a 480-thread row-stream CTA (or two gradient band
// CTAs) leaves free on an SM -- the exchange has to become resident next to the next step's kernels to overlap them.
constexpr int kP2PThreads = 128;
constexpr int kP2PCtas = 4;   // CTAs of one exchange; each moves a quarter of the vector
constexpr long long kDefaultWaitCycles = 1000000000ll;   // about half a second
std::atomic<long long> g_wait_cycles{kDefaultWaitCycles};

struct P2PCtx {
  int rank, world, device;
  size_t max_floats, row;     // row = floats per (slot, rank) row
  void* base;                 // own allocation
  void* peer[kMaxWorld];      // mapped allocations (peer[rank] == base)
  bool opened[kMaxWorld];
  // device-side table
  unsigned long long** d_data;   // [world] region pointers of the stand-alone exchange kernel
  unsigned* d_seq;            // [kP2PCtas] next sequence number per CTA
  int* d_status;
  size_t bytes;
  // the exchange fused into the gradient reduction (cp4_reduce_partials_kernel<true>) has its own region and
  // sequence numbers behind the stand-alone kernel's, so the two kinds of exchange can be mixed on one context
  int fctas;                  // CTAs of 32 entries
  size_t off_data2;
  unsigned long long** d_data2;   // [world]
  unsigned* d_seq2;           // [fctas]
  size_t pending_n;           // floats of a posted, not yet completed pipelined exchange (0: none)
  int pending_R, pending_Rs;
};

// bytes of one exchange region: [2 slots][world][row] words of 8 bytes {value, sequence number}
inline size_t region_bytes(size_t row, int world) { return 2 * (size_t)world * row * sizeof(unsigned long long); }

// Every value travels with the exchange's sequence number in one aligned 8-byte word (one transaction: the value and
// its "arrived" mark cannot be seen apart), so the exchange needs no fence and no separate flag: a rank stores its
// words into every rank's region and spins, bounded, on the words of its own region until they carry the number.
__global__ void __maxnreg__(32) p2p_allreduce_kernel(unsigned long long* const* __restrict__ data, unsigned* seqs,
                                                     int* status, int rank, int world, size_t row, const float* src,
                                                     float* dst, size_t n, long long wait_cycles) {
  // (src and dst may be the same buffer: a thread reads the entries it later writes)
  const int cta = blockIdx.x, tid = threadIdx.x;
  __shared__ unsigned s_seq;
  __shared__ int s_missed;
  grid_dependency_wait();   // launched as a programmatic dependent: src is the previous kernel's output
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
  for (size_t i = lo + tid; i < hi; i += kP2PThreads) {
    const float v = src[i];
    for (int p = 0; p < world; ++p) exchange_store(data[p] + ((size_t)slot * world + rank) * row + i, v, seq);
  }
  // 2. the words of the own region, added in rank order
  const unsigned long long* own = data[rank] + (size_t)slot * world * row;
  const long long t0 = clock64();
  volatile int* missed = &s_missed;
  for (size_t i = lo + tid; i < hi; i += kP2PThreads) {
    float s = 0.f;
    for (int p = 0; p < world; ++p) {
      float v = 0.f;
      while (!*missed && !exchange_load(own + (size_t)p * row + i, seq, &v)) {
        if (clock64() - t0 > wait_cycles) {   // give up, never hang
          *missed = 1;
          atomicExch(status, 1 + rank);
          break;
        }
        __nanosleep(20);
      }
      s += v;
    }
    dst[i] = s;
  }
  __syncthreads();
  // a missed exchange cannot pass for a sum: NaN for the CTA's whole part
  if (s_missed)
    for (size_t i = lo + tid; i < hi; i += kP2PThreads) dst[i] = __int_as_float(0x7fc00000);
  if (tid == 0) seqs[cta] = seq;   // the sequence advances either way: the next exchange lines up with the peers' again
}

}  // namespace

namespace {
// device-side pointer tables of both kinds of exchange from the mapped peer allocations
int upload_tables(P2PCtx* c) {
  unsigned long long* data[kMaxWorld] = {};
  unsigned long long* data2[kMaxWorld] = {};
  for (int p = 0; p < c->world; ++p) {
    char* b = static_cast<char*>(c->peer[p]);
    data[p] = reinterpret_cast<unsigned long long*>(b);
    data2[p] = reinterpret_cast<unsigned long long*>(b + c->off_data2);
  }
  B200CP_CUDA_OK(cudaMemcpy(c->d_data, data, sizeof(data), cudaMemcpyHostToDevice));
  B200CP_CUDA_OK(cudaMemcpy(c->d_data2, data2, sizeof(data2), cudaMemcpyHostToDevice));
  return B200CP_OK;
}
}  // namespace

// The arguments of the exchange fused into the gradient reduction, for a vector of n floats.
int p2p_fused_args(void* ctx, size_t n, int mode, float* prev_out, ExchangeArgs* out) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c || !out) return fail(B200CP_ERR_INVALID_ARG, "fused exchange: null context");
  if (n > c->max_floats) return fail(B200CP_ERR_INVALID_ARG, "fused exchange: %zu floats, room for %zu", n, c->max_floats);
  if (c->pending_n != 0) {
    if (mode != 1) return fail(B200CP_ERR_INVALID_ARG, "fused exchange: a pipelined exchange is pending; complete it with b200cp_p2p_flush");
    if (!prev_out) return fail(B200CP_ERR_INVALID_ARG, "pipelined exchange: the previous step's gradients need a destination");
    if (c->pending_n != n) return fail(B200CP_ERR_INVALID_ARG, "pipelined exchange: %zu floats after %zu", n, c->pending_n);
  }
  out->data = c->d_data2;
  out->seqs = c->d_seq2;
  out->status = c->d_status;
  out->rank = c->rank;
  out->world = c->world;
  out->ctas = c->fctas;
  out->row = c->row;
  out->wait_cycles = g_wait_cycles.load();
  out->mode = mode;
  out->prev_out = c->pending_n != 0 ? prev_out : nullptr;
  return B200CP_OK;
}

void p2p_fused_set_pending(void* ctx, size_t n, int R, int Rs) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  c->pending_n = n; c->pending_R = R; c->pending_Rs = Rs;
}

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
  c->base = nullptr; c->d_data = nullptr; c->d_seq = nullptr; c->d_status = nullptr;
  for (int p = 0; p < kMaxWorld; ++p) { c->peer[p] = nullptr; c->opened[p] = false; }
  c->fctas = (int)((c->row + 31) / 32);
  c->off_data2 = (region_bytes(c->row, world) + 255) / 256 * 256;
  c->bytes = c->off_data2 + region_bytes(c->row, world);
  c->d_data2 = nullptr; c->d_seq2 = nullptr;
  c->pending_n = 0; c->pending_R = c->pending_Rs = 0;
  cudaIpcMemHandle_t h;
  memset(&h, 0, sizeof(h));
  static_assert(sizeof(cudaIpcMemHandle_t) == B200CP_P2P_HANDLE_BYTES, "IPC handle size");
  // every allocation of the context, or none: a failure frees what exists and reports the CUDA error
  cudaError_t e = cudaGetDevice(&c->device);
  if (e == cudaSuccess) e = cudaMalloc(&c->base, c->bytes);
  if (e == cudaSuccess) e = cudaMemset(c->base, 0, c->bytes);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_data, sizeof(unsigned long long*) * kMaxWorld);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_seq, sizeof(unsigned) * kP2PCtas);
  if (e == cudaSuccess) e = cudaMemset(c->d_seq, 0, sizeof(unsigned) * kP2PCtas);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_data2, sizeof(unsigned long long*) * kMaxWorld);
  if (e == cudaSuccess) e = cudaMalloc(&c->d_seq2, sizeof(unsigned) * c->fctas);
  if (e == cudaSuccess) e = cudaMemset(c->d_seq2, 0, sizeof(unsigned) * c->fctas);
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
  return upload_tables(c);
}

int b200cp_p2p_allreduce(void* ctx, const float* src, float* dst, size_t n, void* stream) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c || !src || !dst) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_allreduce: null argument");
  if (n > c->max_floats) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_allreduce: %zu floats, room for %zu", n, c->max_floats);
  B200CP_CUDA_OK(launch_kernel(p2p_allreduce_kernel, dim3(kP2PCtas), dim3(kP2PThreads), 0, static_cast<cudaStream_t>(stream),
                               /*programmatic=*/true, c->d_data, c->d_seq, c->d_status, c->rank, c->world, c->row, src, dst, n,
                               g_wait_cycles.load()));
  B200CP_LAUNCH_OK("p2p_allreduce_kernel");
  return B200CP_OK;
}

int b200cp_p2p_flush(void* ctx, float* dK_last, void* stream) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_flush: null context");
  if (c->pending_n == 0) return B200CP_OK;
  if (!dK_last) return fail(B200CP_ERR_INVALID_ARG, "b200cp_p2p_flush: the pending gradients need a destination");
  ExchangeArgs ex{};
  ex.data = c->d_data2; ex.seqs = c->d_seq2; ex.status = c->d_status;
  ex.rank = c->rank; ex.world = c->world; ex.ctas = c->fctas; ex.row = c->row; ex.wait_cycles = g_wait_cycles.load();
  const int n = (int)c->pending_n, R = c->pending_R, Rs = c->pending_Rs;
  c->pending_n = 0;
  return exchange_finish_launch(ex, n, R, Rs, 0, dK_last, static_cast<cudaStream_t>(stream));
}

void b200cp_test_set_p2p_wait_cycles(long long cycles) { g_wait_cycles.store(cycles > 0 ? cycles : kDefaultWaitCycles); }

// Test hook: the ranks of a single-process world (contexts made by b200cp_p2p_init in this process, in rank order)
// map each other's regions directly instead of through CUDA IPC.
int b200cp_test_p2p_connect_local(void* ctx, void* const* all_ctx) {
  P2PCtx* c = static_cast<P2PCtx*>(ctx);
  if (!c || !all_ctx) return fail(B200CP_ERR_INVALID_ARG, "b200cp_test_p2p_connect_local: null argument");
  for (int p = 0; p < c->world; ++p) {
    P2PCtx* o = static_cast<P2PCtx*>(all_ctx[p]);
    if (!o || o->world != c->world || o->row != c->row || o->rank != p)
      return fail(B200CP_ERR_INVALID_ARG, "b200cp_test_p2p_connect_local: context %d does not belong to this world", p);
    c->peer[p] = o->base;
  }
  return upload_tables(c);
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
  cudaFree(c->d_seq);
  cudaFree(c->d_data2);
  cudaFree(c->d_seq2);
  cudaFree(c->d_status);
  delete c;
  return B200CP_OK;
}

}  // extern "C"
