/* Test and diagnostic entry points of libb200cp.so.  Not part of the product interface (include/b200cp.h): they
 * exist for the test-suite and for profiling experiments, and may change without notice. */
#ifndef B200CP_TEST_H
#define B200CP_TEST_H

#include "b200cp.h"

#ifdef __cplusplus
extern "C" {
#endif
#if defined(__GNUC__)
#pragma GCC visibility push(default)
#endif

/* Diagnostic: the tensor-path forward with the first CTA's rank-R intermediate P copied out
 * (P_block0: [RP][Mmax] floats, may be NULL).  terms = 3 (split) or 1 (single tf32 pass). */
int b200cp_debug_cp4_tc(const b200cp_tensor_shape* s, const float* X, const float* K0, const float* K1,
                        const float* KH, const float* KW, float* U, float* P_block0, int terms, void* stream);

/* Diagnostic: one tcgen05.mma, D[128x16] = A[128x8] * B[16x8]^T (all device pointers, row-major).
 * mode 0: A staged K-major without swizzle; mode 1: A staged MN-major with the 128-byte swizzle.
 * *status (device int) is 0 on success, 1 if the bounded wait for the MMA ran out. */
int b200cp_debug_tc_selftest(int mode, const float* A, const float* B, float* D, int* status, void* stream);

/* Forces the band height (image rows per CTA) of the row-band CP4 kernel; 0 gives the choice back to the planner.
 * Heights the kernel cannot take for a shape are skipped as usual.  Process-wide. */
void b200cp_test_set_band_rows(int rows);

/* Input loads of the row-band kernel: 1 = one 4-D tensor-map box per pipeline stage (cp.async.bulk.tensor),
 * 0 = one 1-D bulk copy per channel (cp.async.bulk; the default).  Process-wide. */
void b200cp_test_set_band_tensor_loads(int on);

/* Largest rank the row-band kernel takes (1 .. 32; the default, 16, leaves ranks 17 .. 32 to the tile kernel, which
 * measures faster there).  Process-wide. */
void b200cp_test_set_band_max_rank(int rank);

/* Output contraction of the row-band kernel: 1 = tcgen05.mma with the accumulators in tensor memory where the shape
 * allows it, 0 = mma.sync with the output staged in shared memory (the default: it measures faster).  Process-wide. */
void b200cp_test_set_band_tcgen05(int on);

/* The row-stream convolution kernel (tried before the row bands): 0 = off, 1 = on, -1 = what the environment
 * variable B200CP_STREAM says (on unless it is 0).  Process-wide. */
void b200cp_test_set_stream(int on);

/* Number of launches of the row-stream kernel by this process so far: a test that means to exercise that kernel
 * checks that the count moved. */
long long b200cp_test_stream_launches(void);

/* Diagnostics: the row-band kernel writes 64 cycle stamps (long long) per CTA for its first 512 CTAs into this
 * device buffer (512 * 64 * 8 bytes); NULL switches it off.  Process-wide. */
void b200cp_test_set_band_trace(void* device_buffer);

/* Wait limit (in SM clock cycles) of the peer-memory allreduce's flag wait for launches issued after the call;
 * 0 restores the default (about half a second).  Lets a test make a wait run out without hanging anything. */
void b200cp_test_set_p2p_wait_cycles(long long cycles);

/* The ranks of a single-process world (contexts from b200cp_p2p_init in this process, `all_ctx` in rank order) map
 * each other's exchange regions directly, without CUDA IPC: a test can then drive the ranks one after the other. */
int b200cp_test_p2p_connect_local(void* ctx, void* const* all_ctx);

#if defined(__GNUC__)
#pragma GCC visibility pop
#endif
#ifdef __cplusplus
}
#endif
#endif /* B200CP_TEST_H */
