/* b200cp -- C ABI of the B200 (sm_100a) fused CP-decomposed layer kernels.
 *
 * Plain C: pointers, sizes, an opaque stream handle.  Every pointer named
 * "device" must be device memory of the current CUDA device; the *_host entry
 * points take ordinary host memory and do the transfers themselves.  All
 * tensors are fp32, row-major, last index fastest:
 *
 *   X  [N, C, H, W]   U, dU [N, T, H, W]
 *   K0 [T, R]  K1 [C, R]  KH [Y, R]  KW [X, R]      (the reference's FT, FC, FY, FX)
 *
 * Every function returns a b200cp_status (0 = ok, negative = error, nothing
 * was launched unless stated).  Calls are asynchronous on `stream` (a
 * cudaStream_t passed as void*; NULL = the default stream) and re-entrant
 * across streams and devices; no function allocates device memory except the
 * *_host helpers and those that say so.
 */
#ifndef B200CP_H
#define B200CP_H

#include <stddef.h>

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Same field order and types as the reference's `struct tensor_shape`
 * (Cuda_kernels/Tensor.cuh:10-19): N H W pad T C Y X Rank. */
typedef struct b200cp_tensor_shape {
  unsigned N, H, W, pad, T, C, Y, X, Rank;
} b200cp_tensor_shape;

typedef enum b200cp_status {
  B200CP_OK = 0,
  B200CP_ERR_INVALID_ARG = -1,  /* null pointer, zero dimension, misaligned buffer */
  B200CP_ERR_UNSUPPORTED = -2,  /* shape outside what the kernels implement       */
  B200CP_ERR_WORKSPACE = -3,    /* workspace missing or too small                  */
  B200CP_ERR_CUDA = -4,         /* a CUDA runtime call failed                      */
  B200CP_ERR_TIMEOUT = -5,      /* a bounded device-side wait ran out              */
  B200CP_ERR_NO_DEVICE = -6     /* no sm_100 device / driver entry point missing   */
} b200cp_status;

/* flags: which arithmetic path runs the two channel contractions. */
enum {
  B200CP_PATH_AUTO = 0,   /* the fastest fp32-grade path for the shape (mma.sync today)  */
  B200CP_PATH_SIMT = 1,   /* exact fp32 FFMA                                        */
  B200CP_PATH_TC3X = 2,   /* tcgen05 kind::tf32, 3-term split (fp32-grade accuracy) */
  B200CP_PATH_TC1X = 3,   /* tcgen05 kind::tf32, single pass (about 1e-3 relative)  */
  B200CP_PATH_MMA = 4,    /* warp-level mma.sync tf32, 3-term split (fp32-grade)    */
  B200CP_PATH_MASK = 7
};

/* ---- CP4 conv2d ------------------------------------------------------- */

/* U[n,t,h,w] = sum_r K0[t,r] sum_c K1[c,r] sum_{y,x} KH[y,r] KW[x,r] X[n,c,h+y-pad,w+x-pad].
 * Replaces cp4_conv2d_forward_gpu (Cuda_kernels/cp4Conv2dForward.cuh:7-14,
 * body cp4Conv2dForward.cu:187-328) and, with K0..KW permuted, the TF launcher
 * Cp4Conv2dFusedNchwKernelLauncher (Kernels/cp4_conv_nchw.cc:34). */
int b200cp_cp4_fwd(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1, const float* KH,
                   const float* KW, float* U, void* stream, int flags);

/* dX[n,c,h,w] = sum_r K1[c,r] sum_t K0[t,r] sum_{y,x} KH[Y-1-y,r] KW[X-1-x,r] dU[n,t,h+y-pad,w+x-pad].
 * Replaces cp4_conv2d_backward_data_gpu (Cuda_kernels/cp4Conv2dBackwardData.cuh:7-14,
 * body cp4Conv2dBackwardData.cu:112-282). */
int b200cp_cp4_bwd_data(const b200cp_tensor_shape* s, const float* dU, const float* K0, const float* K1,
                        const float* KH, const float* KW, float* dX, void* stream, int flags);

/* Bytes of device scratch b200cp_cp4_bwd_filter needs for this shape (0 on error). */
size_t b200cp_cp4_bwd_filter_workspace_bytes(const b200cp_tensor_shape* s, int flags);

/* All four factor gradients in one pass over X and dU, written back-to-back:
 *   dK_packed = [ dK0 (T*R) | dK1 (C*R) | dKH (Y*R) | dKW (X*R) ]
 * Replaces cp4_conv2d_backward_filter_{t,c,y,x}_gpu
 * (Cuda_kernels/cp4Conv2dBackwardFilter.cuh:13-47, bodies
 * cp4Conv2dBackwardFilter.cu:64-257), which are host loops in the reference.
 * The gradients are overwritten, not accumulated; the sum over tiles is done
 * in a fixed order (bitwise reproducible).  Requires Y == X odd, pad = (Y-1)/2. */
int b200cp_cp4_bwd_filter(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                          const float* K1, const float* KH, const float* KW, float* dK_packed, void* workspace,
                          size_t workspace_bytes, void* stream, int flags);

/* The same four factor gradients for callers that must not allocate device memory and have no
 * workspace to hand over: code running inside another framework's stream-ordered section, a
 * real-time loop, or a plugin whose host forbids cudaMalloc after initialisation.  It has no
 * counterpart in the reference.  It runs the CUDA-core kernels (bit-identical to b200cp_cp4_bwd_filter with
 * B200CP_PATH_SIMT).  The per-tile partial sums go to a fixed 8 MiB array inside the
 * library's device image (every GPU that loads the library holds it until the process exits), so
 *   - shapes whose partial sums need more than 8 MiB are refused with B200CP_ERR_UNSUPPORTED
 *     (b200cp_cp4_bwd_filter_workspace_bytes with B200CP_PATH_SIMT tells the need; e.g. N=32, C=T=64, 56x56, R=16 needs 5.5 MB);
 *   - the call itself performs no cudaMalloc / cudaFree and calls no allocating library routine;
 *   - the first call on each device looks up the array's device address (cudaGetSymbolAddress);
 *     make that first call before any stream capture begins on that device;
 *   - all calls on a device share the one array: two calls that may overlap on the GPU (different
 *     streams, no dependency between them) race and give wrong gradients.  Nothing in the array has to
 *     be cleared between calls: every launch overwrites all the partial sums it later reads. */
int b200cp_cp4_bwd_filter_noalloc(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                                  const float* K1, const float* KH, const float* KW, float* dK_packed, void* stream);

/* *exceeds = number of elements with max(|a-b|/|a|, |a-b|/|b|) > tolerance (|a-b| where a or b is zero), counted on
 * the device; A and B are device (or managed) arrays of n floats.  Synchronises `stream`.  Replaces the count kernel
 * behind AllClose (Cuda_kernels/Utils.cu:143-180): AllClose(A, B, tol) == (*exceeds == 0). */
int b200cp_allclose_count(const float* A, const float* B, size_t n, float tolerance, unsigned long long* exceeds,
                          void* stream);

/* Dense filter gradient dK[t,c,y,x] = sum_{n,h,w} dU[n,t,h,w] Xpad[n,c,h+y,w+x].
 * Replaces cp4_conv2d_backward_filter_full_gpu (Cuda_kernels/cp4Conv2dBackwardFilter.cuh:7-11). */
int b200cp_cp4_bwd_filter_full(const b200cp_tensor_shape* s, const float* X, const float* dU, float* dK, void* stream);

/* K[t,c,y,x] = sum_r K0[t,r] K1[c,r] KH[y,r] KW[x,r]  (the reference's cp4recom,
 * Cuda_kernels/Utils.cu:36-98). */
int b200cp_cp4_recompose(const b200cp_tensor_shape* s, const float* K0, const float* K1, const float* KH,
                         const float* KW, float* K, void* stream);

/* 1 when b200cp_cp4_step / _fwd_save / _bwd_data_save / _bwd_filter_saved share the rank planes for this shape and
 * flags (3x3 filter, pad 1, default or mma path, not switched off by B200CP_STEP_NO_SHARE / B200CP_AUTO_MMA=0), else
 * 0: the one rule callers such as an autograd function should ask instead of restating it.  No counterpart in the
 * reference, which has no backward-filter kernel (Cuda_kernels/cp4Conv2dBackwardFilter.cu:64-257 are host loops). */
int b200cp_cp4_shares_planes(const b200cp_tensor_shape* s, int flags);

/* One training step on device buffers: U = forward(X), dX = backward-data(dU) and the packed factor gradients,
 * the three results of b200cp_cp4_fwd, _bwd_data and _bwd_filter on the same inputs.  Inside one call the work
 * the three have in common is done once: with 3x3 filters (pad 1) on the default path the two convolutions leave
 * their rank-R planes K1^T X and K0^T dU ([N,R,H,W] each) in the workspace and the factor gradients start from
 * those instead of contracting the channels again.  No counterpart in the reference, whose three entry points
 * (Cuda_kernels/cp4Conv2d.cuh:8-28) are called one after the other by its callers. */
size_t b200cp_cp4_step_workspace_bytes(const b200cp_tensor_shape* s, int flags);
int b200cp_cp4_step(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0, const float* K1,
                    const float* KH, const float* KW, float* U, float* dX, float* dK_packed, void* workspace,
                    size_t workspace_bytes, void* stream, int flags);

/* Forward of X and backward-data of dU in one call: the convolutions of a training step of a layer whose factors are
 * frozen (cp4_conv2d_forward_gpu + cp4_conv2d_backward_data_gpu of the reference, one after the other), and the first
 * launch of b200cp_cp4_step.  Where the shape allows it one launch carries both.  P and Q (both or neither, [N,R,H,W]
 * each; 3x3 / pad 1 / AUTO or MMA only) receive the rank planes for b200cp_cp4_bwd_filter_saved. */
int b200cp_cp4_fwd_bwd_data(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                            const float* K1, const float* KH, const float* KW, float* U, float* dX, float* P, float* Q,
                            void* stream, int flags);

/* The pieces of b200cp_cp4_step for callers that run the forward and the backward pass at different times
 * (an autograd function): the two convolutions that also write their rank plane (P = K1^T X from the forward,
 * Q = K0^T dU from backward-data; [N,R,H,W] fp32 each, caller-owned), and the factor gradients from the two
 * planes.  3x3 filters with pad 1, flags AUTO or MMA.  No counterpart in the reference. */
int b200cp_cp4_fwd_save(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1, const float* KH,
                        const float* KW, float* U, float* P, void* stream, int flags);
int b200cp_cp4_bwd_data_save(const b200cp_tensor_shape* s, const float* dU, const float* K0, const float* K1,
                             const float* KH, const float* KW, float* dX, float* Q, void* stream, int flags);
size_t b200cp_cp4_bwd_filter_saved_workspace_bytes(const b200cp_tensor_shape* s, int flags);
int b200cp_cp4_bwd_filter_saved(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* P,
                                const float* Q, const float* KH, const float* KW, float* dK_packed, void* workspace,
                                size_t workspace_bytes, void* stream, int flags);

/* ---- three-factor CP conv2d ------------------------------------------------ */

/* U[n,t,h,w] = sum_r KT[t,r] sum_{y,x} KC[y,x,r] sum_c KCin[c,r] X[n,c,h+y-pad,w+x-pad]: the layer
 * `conv2d_cp` defines (test/layers.py:265-283: 1x1 conv C->R, depthwise YxX conv, 1x1 conv R->T) and
 * Conv2dCpFusedNchwKernelLauncher(U, K0, K1, K2, V) fuses (Kernels/cp_fused_nchw.cc, .cu).  Factors are
 * [dim, R] like everywhere in this header: KCin[C,R] is the op's kernel0, KC[Y,X,R] its kernel1 and
 * KT[T,R] its kernel2[R,T] transposed.  Runs on the mma.sync path (flags AUTO or MMA).
 * The factor gradients come packed as [dKT (T*R) | dKCin (C*R) | dKC (Y*X*R)]; 3x3 filters with pad 1 only. */
int b200cp_cp3_fwd(const b200cp_tensor_shape* s, const float* X, const float* KT, const float* KCin, const float* KC,
                   float* U, void* stream, int flags);
int b200cp_cp3_bwd_data(const b200cp_tensor_shape* s, const float* dU, const float* KT, const float* KCin,
                        const float* KC, float* dX, void* stream, int flags);
size_t b200cp_cp3_bwd_filter_workspace_bytes(const b200cp_tensor_shape* s, int flags);
int b200cp_cp3_bwd_filter(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* KT,
                          const float* KCin, const float* KC, float* dK_packed, void* workspace,
                          size_t workspace_bytes, void* stream, int flags);

/* Host-memory variants: copy in, run, copy out, synchronise.  They allocate
 * (and cache per device) their own device buffers.  `dK_packed` may be NULL in
 * the step call to skip nothing -- all three results are always produced. */
int b200cp_cp4_fwd_host(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1,
                        const float* KH, const float* KW, float* U, int flags);
int b200cp_cp4_step_host(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                         const float* K1, const float* KH, const float* KW, float* U, float* dX, float* dK_packed,
                         int flags);

/* The same step, queued: `submit` returns once the copies and kernels of one step are on the library's
 * copy-in, compute and copy-out streams; `wait` blocks until that slot's results are in U / dX / dK_packed.
 * Four slots (0 .. 3) with their own device buffers let a caller submit the next steps while step i drains, so the
 * host-to-device copy of one step, the kernels of another and the device-to-host copy of a third overlap; with three
 * or four steps in flight neither direction of the host link waits for a kernel.
 * Host buffers should be pinned and must stay untouched until `wait` returns.  Submitting to a slot that is
 * still pending waits for it first.  No counterpart in the reference (its launchers synchronise the device). */
int b200cp_cp4_step_host_submit(const b200cp_tensor_shape* s, const float* X, const float* dU, const float* K0,
                                const float* K1, const float* KH, const float* KW, float* U, float* dX,
                                float* dK_packed, int flags, int slot);
int b200cp_cp4_step_host_wait(int slot);

/* ---- reshaped-CP (rCP) conv2d, order m (1..4) ------------------------- */

/* V[n,t,h,w] = sum_r sum_{i,j} S[i,j,r] sum_c (prod_k A_k[c_k,t_k,r]) X[n,c,h+i-p,w+j-p],
 * c = (c_1,..,c_m) and t = (t_1,..,t_m) flattened first mode slowest, p = (FH-1)/2.
 * A[k] is [c_k, t_k, R], S is [FH, FW, R]: the operand order of
 * Conv2dRcpFusedNchwKernelLauncher(U, K0, K1, KC, V) (Kernels/rcp_fused_nchw.cc:33,
 * kernel Kernels/rcp_fused_nchw.cu:4-89), generalised from its one compiled shape. */
int b200cp_rcp_fwd(int N, int H, int W, int order, const int* cdims, const int* tdims, int R, int FH, int FW,
                   const float* X, const float* const* A, const float* S, float* V, void* stream, int flags);

size_t b200cp_rcp_bwd_workspace_bytes(int N, int H, int W, int order, const int* cdims, const int* tdims, int R,
                                      int FH, int FW, int flags);

/* Gradients of b200cp_rcp_fwd: dX [N,C,H,W], dA[k] [c_k,t_k,R], dS [FH,FW,R]
 * (any of dX / dA / dS may be NULL to skip it; dA and dS are skipped together).
 * The reference has no rCP backward. */
int b200cp_rcp_bwd(int N, int H, int W, int order, const int* cdims, const int* tdims, int R, int FH, int FW,
                   const float* X, const float* dV, const float* const* A, const float* S, float* dX,
                   float* const* dA, float* dS, void* workspace, size_t workspace_bytes, void* stream, int flags);

/* ---- the reference's "rebuild" variants ------------------------------------
 * Its benchmarks time, beside each fused layer, the undecomposed layer run with the recomposed weight
 * (test/benchmark_conv2d_cp4.py:35-42: cp4recom + conv2d; test/benchmark_dense_cp.py:43-49: einsum of the factors +
 * matmul).  These entry points give that line without cuDNN / cuBLAS. */

/* U[n,t,h,w] = sum_{c,y,x} K[t,c,y,x] X[n,c,h+y-pad,w+x-pad], zero outside the image, H x W output; K is
 * [T,C,Y,X] as b200cp_cp4_recompose / b200cp_rcp_recompose write it.  s->Rank is not used.  The 16-byte aligned
 * workspace takes the filter re-laid as tf32 hi / lo planes. */
size_t b200cp_conv2d_dense_fwd_workspace_bytes(const b200cp_tensor_shape* s);
int b200cp_conv2d_dense_fwd(const b200cp_tensor_shape* s, const float* X, const float* K, float* U, void* workspace,
                            size_t workspace_bytes, void* stream);

/* b200cp_cp4_recompose into the workspace, then b200cp_conv2d_dense_fwd. */
size_t b200cp_cp4_rebuild_fwd_workspace_bytes(const b200cp_tensor_shape* s);
int b200cp_cp4_rebuild_fwd(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1,
                           const float* KH, const float* KW, float* U, void* workspace, size_t workspace_bytes,
                           void* stream);

/* K[t,c,y,x] = sum_r S[y,x,r] prod_k A_k[c_k,t_k,r], c and t flattened first-mode-slowest: the filter of the
 * reshaped-CP conv (einsum of test/test_conv2d_rcp.py:41-42 in [T,C,FH,FW] order). */
int b200cp_rcp_recompose(int order, const int* cdims, const int* tdims, int R, int FH, int FW, const float* const* A,
                         const float* S, float* K, void* stream);

/* M[i,o] = sum_r prod_k F_k[i_k,o_k,r], i and o flattened first-mode-slowest (test/benchmark_dense_cp.py:43-44).
 * With the workspace the two halves of the modes are multiplied out first and M is their rank-wise outer product;
 * without one (NULL) every element is formed from all factors, which is several times slower for large M. */
size_t b200cp_dense_recompose_workspace_bytes(int order, const int* idims, const int* odims, int R);
int b200cp_dense_recompose(int order, const int* idims, const int* odims, int R, const float* const* F, float* M,
                           void* workspace, size_t workspace_bytes, void* stream);

/* Y[b,o] = sum_i X[b,i] M[i,o] (test/benchmark_dense_cp.py:45-48) with fp32-grade results: tcgen05 with three tf32
 * terms where B, I, O fill its tiles, CUDA cores otherwise. */
size_t b200cp_dense_matmul_workspace_bytes(int B, int I, int O);
int b200cp_dense_matmul(int B, int I, int O, const float* X, const float* M, float* Y, void* workspace,
                        size_t workspace_bytes, void* stream);

/* ---- CP dense layer, order m (1..4) ------------------------------------ */

/* Y[b,o] = sum_r sum_i X[b,i] prod_k F_k[i_k,o_k,r]; F[k] is [i_k, o_k, R]: the
 * operand order of DenseCpKernelLauncher(U, K0, K1, K2, V) (Kernels/dense_cp.cc:33,
 * kernel Kernels/dense_cp.cu:4-57), generalised from its one compiled shape. */
int b200cp_dense_fwd(int B, int order, const int* idims, const int* odims, int R, const float* X,
                     const float* const* F, float* Y, void* stream, int flags);

size_t b200cp_dense_bwd_workspace_bytes(int B, int order, const int* idims, const int* odims, int R, int flags);

/* Gradients of b200cp_dense_fwd: dX [B,I], dF[k] [i_k,o_k,R] (dX or dF may be NULL).
 * The reference has no dense-CP backward. */
int b200cp_dense_bwd(int B, int order, const int* idims, const int* odims, int R, const float* X, const float* dY,
                     const float* const* F, float* dX, float* const* dF, void* workspace, size_t workspace_bytes,
                     void* stream, int flags);

/* ---- gradient allreduce over peer memory ---------------------------------
 * The reference is single-GPU (cudaSetDevice, Cuda_kernels/cp4Conv2d.cu:210,221); data parallelism sums the packed
 * factor gradients of b200cp_cp4_bwd_filter / _step over the ranks.  These calls do that sum with one small kernel
 * per step over NVLink peer memory, one process per GPU, in place of a library allreduce: every rank stores its
 * vector into every rank's exchange region, raises a flag, waits (bounded) for the other ranks' flags and adds the
 * rows in rank order, so all ranks hold bitwise the same result.
 *
 *   b200cp_p2p_init      allocates this rank's exchange region (set-up time, not in the hot path) for vectors of up
 *                        to max_floats floats and writes its 64-byte CUDA IPC handle to handle_out;
 *   b200cp_p2p_connect   takes all ranks' handles (world * 64 bytes, in rank order; the host exchanges them, e.g.
 *                        with an all-gather) and maps the peers' regions; all ranks must have returned from it
 *                        (a host barrier) before the first allreduce;
 *   b200cp_p2p_allreduce dst[i] = sum over ranks of src[i], asynchronous on `stream`, capturable in a CUDA graph;
 *                        every rank must issue the same sequence of calls; src and dst may be the same buffer;
 *   b200cp_p2p_status    synchronises the device; B200CP_ERR_TIMEOUT if a wait for a peer ran out (about 0.5 s);
 *   b200cp_p2p_destroy   unmaps and frees.
 * world = 1 is allowed (no IPC, a copy). */
#define B200CP_P2P_HANDLE_BYTES 64
int b200cp_p2p_init(int rank, int world, size_t max_floats, unsigned char* handle_out, void** ctx_out);
int b200cp_p2p_connect(void* ctx, const unsigned char* handles);
int b200cp_p2p_allreduce(void* ctx, const float* src, float* dst, size_t n, void* stream);
int b200cp_p2p_status(void* ctx);
int b200cp_p2p_destroy(void* ctx);

/* A data-parallel training step: b200cp_cp4_step on this rank's shard with dK_packed summed over the ranks of the
 * exchange context (b200cp_p2p_init / _connect, made for at least (T+C+Y+X)*Rank floats).  Where the step runs as its
 * fused kernel chain, the exchange is the tail of the kernel that adds the per-band partial gradients: every CTA of
 * that kernel stores its 32 sums into every rank's region over NVLink, raises its flag, waits (bounded) for the
 * peers' flags and adds the rows in rank order -- no separate collective launch.  Other shapes run the step and then
 * b200cp_p2p_allreduce.  Every rank must make the same sequence of calls on its context.  The reference has no
 * counterpart (it is single-GPU: Cuda_kernels/cp4Conv2d.cu:210,221). */
int b200cp_cp4_step_allreduce(void* p2p_ctx, const b200cp_tensor_shape* s, const float* X, const float* dU,
                              const float* K0, const float* K1, const float* KH, const float* KW, float* U, float* dX,
                              float* dK_packed, void* workspace, size_t workspace_bytes, void* stream, int flags);

/* The same step with the exchange pipelined over consecutive steps: the call only posts this step's gradient sums to
 * the peers (the tail of its reduction kernel) and completes the exchange of the *previous* pipelined call, whose
 * flags arrived a whole step ago, writing those summed gradients to dK_prev (ignored when nothing is pending).  The
 * exchange latency then costs the step nothing and no second kernel runs beside the step's.  dK_scratch:
 * (T+C+Y+X)*Rank floats the call may use.  b200cp_p2p_flush completes the last posted exchange into dK_last (a no-op
 * when nothing is pending); until then no other exchange may use the context.  Consecutive pipelined calls must have
 * the same shape.  Every rank makes the same sequence of calls.  No counterpart in the reference. */
int b200cp_cp4_step_allreduce_pipelined(void* p2p_ctx, const b200cp_tensor_shape* s, const float* X, const float* dU,
                                        const float* K0, const float* K1, const float* KH, const float* KW, float* U,
                                        float* dX, float* dK_scratch, float* dK_prev, void* workspace,
                                        size_t workspace_bytes, void* stream, int flags);
int b200cp_p2p_flush(void* ctx, float* dK_last, void* stream);

/* ---- misc --------------------------------------------------------------- */

/* Synchronises the device and reports whether any tensor-path kernel gave up a bounded wait since
 * the last call (B200CP_ERR_TIMEOUT), clearing the record.  B200CP_OK otherwise. */
int b200cp_device_status(void);

/* Text of the last error raised on the calling thread ("" if none). */
const char* b200cp_last_error_string(void);
const char* b200cp_status_string(int status);
/* Number of kernel launches issued by this library since load (all threads). */
unsigned long long b200cp_launch_count(void);
int b200cp_version(void);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* B200CP_H */
