// Pieces shared by the two attention kernels (attn.cu: two softmax groups over 128-key tiles; attn4.cu: three groups
// over 64-key chunks): the kernel arguments and a few instruction wrappers.
#pragma once

#include <cuda.h>

#include "common.cuh"
#include "rope.cuh"
#include "sm100.cuh"

namespace qb {

struct AttnArgs {
  const uint16_t* qkv;
  const int32_t* segments;
  const int32_t* n_segments;
  const int32_t* frame_t;
  uint16_t* out;
  uint8_t* out_q;  // optional e4m3 copy of the output
  const float* rope_xy;
  const float* k_scale;
  const float* v_scale;
  unsigned int* status;
  int tpf, n_q_heads, gqa, capacity, max_segments;
  // Q of token t, head h starts at qkv + t * q_row + h * q_head (16-bit words), its output row at out + t * o_row +
  // h * o_head: the packed projection has q_row = qkv_dim, q_head = 64, o_row = Hq * 64, o_head = 64; the head-major
  // layout [Hq * tpf, 64] of Q and of the output has 64 and tpf * 64 for both
  int q_row, q_head, o_row, o_head;
  // Key splits (gridDim.z > 1): CTA z walks its share of the key tiles and leaves (m, row sum, 64 outputs)
  // per query row in `partials`; the CTA that draws the last ticket of a (query tile, head) sums the
  // shares in order of z and writes the output.
  float* partials;  // [heads][query tiles][splits][66][128]
  int* tickets;     // [heads][query tiles], zero between launches
};

#ifndef QB_EX2_VOLATILE
#define QB_EX2_VOLATILE 0
#endif
__device__ __forceinline__ float ex2_approx(float x) {
  float y;
#if QB_EX2_VOLATILE
  asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
#else
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
#endif
  return y;
}
// One arrival for the whole warp: an mbarrier arrival is an atomic on shared memory.  __syncwarp orders the
// lanes' earlier writes (and fences) before lane 0's arrival, which releases them to the waiting thread.
__device__ __forceinline__ void warp_arrive(uint32_t bar, int lane) {
  __syncwarp();
  if (lane == 0) mbar_arrive(bar);
}
__device__ __forceinline__ float max3f(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
// UMMA descriptor for a K-major tile with 64-byte rows and the 64-byte swizzle (fp8, head_dim 64).
__device__ __forceinline__ uint64_t umma_desc_k_sw64(uint32_t smem_addr) {
  uint64_t d = 0;
  d |= static_cast<uint64_t>((smem_addr & 0x3FFFF) >> 4);
  d |= static_cast<uint64_t>(1) << 16;
  d |= static_cast<uint64_t>(512 >> 4) << 32;  // 8 rows x 64 B
  d |= static_cast<uint64_t>(1) << 46;
  d |= static_cast<uint64_t>(4) << 61;         // SWIZZLE_64B
  return d;
}

}  // namespace qb
