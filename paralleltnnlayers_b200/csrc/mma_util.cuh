// Warp-level tensor-core helpers (mma.sync m16n8k8, tf32 operands, fp32 accumulation) and cp.async wrappers.
//
// Fragment layout of mma.sync.aligned.m16n8k8.row.col (g = lane / 4, t = lane % 4):
//   A (16 x 8): a0 = (row g, col t), a1 = (row g+8, col t), a2 = (row g, col t+4), a3 = (row g+8, col t+4)
//   B ( 8 x 8): b0 = (row t, col g), b1 = (row t+4, col g)
//   D (16 x 8): d0 = (row g, col 2t), d1 = (row g, col 2t+1), d2 = (row g+8, col 2t), d3 = (row g+8, col 2t+1)
#pragma once

#include <cuda_runtime.h>

#include <cstdint>

namespace b200cp {
namespace mma {

// x rounded to tf32, round to nearest with ties away from zero -- what cvt.rna.tf32.f32 returns for every finite
// x below the overflow threshold: half an ulp of the 10-bit mantissa is added to the magnitude bits and the low 13
// bits are cut.  Two integer instructions; the cvt itself expands to about five on this target.  (A NaN whose
// payload overflows into the sign comes out as -0 here, and the lo part x - hi is then NaN, so NaNs still propagate.)
__device__ __forceinline__ uint32_t tf32_rna_bits(uint32_t x) { return (x + 0x1000u) & 0xffffe000u; }
__device__ __forceinline__ float tf32_round(float x) { return __uint_as_float(tf32_rna_bits(__float_as_uint(x))); }
// hi = x rounded to tf32; lo = x - hi (exact in fp32; the tensor core reads its upper 19 bits)
__device__ __forceinline__ void split_tf32(float x, uint32_t& hi, uint32_t& lo) {
  hi = tf32_rna_bits(__float_as_uint(x));
  lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  // not volatile: the instruction only touches its register operands, so the compiler may interleave
  // independent accumulator chains
  asm("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
      : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// The same instruction kept in program order: the issue order of independent accumulator chains is part of the
// design (consecutive mma on one accumulator must be far enough apart to hide its latency).
__device__ __forceinline__ void mma_tf32_ordered(float (&d)[4], const uint32_t (&a)[4], const uint32_t (&b)[2]) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b[0]), "r"(b[1]));
}

// Four 8 x 4 tiles of 32-bit values (ldmatrix on 8 x 8 b16 tiles): lane l gives the address of row l%8 of tile l/8
// (16-byte aligned); every thread receives element (row lane/4, column lane%4) of each tile -- the layout of the
// tf32 A fragment rows and of a "col" B fragment whose K index is contiguous in shared memory.
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const float* row_ptr) {
  const unsigned a = (unsigned)__cvta_generic_to_shared(row_ptr);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
               : "r"(a));
}
__device__ __forceinline__ void split_tf32_bits(uint32_t x, uint32_t& hi, uint32_t& lo) {
  hi = tf32_rna_bits(x);
  lo = __float_as_uint(__uint_as_float(x) - __uint_as_float(hi));
}

__device__ __forceinline__ void cp_async4(float* smem_dst, const float* gsrc, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
  const int sz = valid ? 4 : 0;  // src-size 0: the destination is zero-filled, nothing is read
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gsrc), "r"(sz) : "memory");
}
// same with the destination given as a shared-memory address and the source size (4, or 0 = zero fill)
__device__ __forceinline__ void cp_async4_s(unsigned smem_dst, const float* gsrc, int src_size) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_size) : "memory");
}
__device__ __forceinline__ void cp_async16_s(unsigned smem_dst, const float* gsrc, int src_size) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gsrc), "r"(src_size) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// the same with a count that is known after unrolling (at most 3 groups may stay pending)
__device__ __forceinline__ void cp_async_wait_upto(int pending) {
  switch (pending) {
    case 3: cp_async_wait<3>(); break;
    case 2: cp_async_wait<2>(); break;
    case 1: cp_async_wait<1>(); break;
    default: cp_async_wait<0>(); break;
  }
}

}  // namespace mma
}  // namespace b200cp
