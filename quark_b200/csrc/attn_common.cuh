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

// 2^x for an e4m3 probability without the special-function unit, in three instructions of the FMA / integer pipes:
// the caller adds 1.5 * 2^15 to x inside the multiply-add that forms x (so v = x rounded to 8 fractional bits, sitting in
// the low mantissa bits of v), and the float whose exponent field is floor(x) + 127 and whose mantissa is the fraction
// is v's bit pattern times 2^15 plus a constant: 2^floor(x) * (1 + frac(x) - 0.052), the chord of 2^x lowered by 0.052 so
// that its mean error over the fraction is near zero (-5.2 % .. +2.3 %; an e4m3 code is 6.25 % wide; in a simulation of
// 8192-key rows the output's 1 - cosine against exact arithmetic goes from 3.6e-4 to 4.3e-4 at worst).  x is clamped at -120 (the result then
// narrows to zero).  Every second probability of a row is built this way in the kLin instantiations of the e4m3 kernel
// (the default; qb_set_attn_exact_exp(1) or QB_ATTN_EXACT_EXP=1 selects the instantiations that use the special-function
// unit for every element): the exponentials no longer queue behind one another there, at the same number of
// instructions issued.  Measured at 720p, 8320 keys, us per launch: 52.0 exact; 49.5 with the turn passing at chunk 2 as
// in the exact kernel; 46.5 with the turn passing before chunk 0 (the groups then overlap almost fully, which the exact
// kernel cannot afford: 62.6); 47.9 without turns; 3 / 5 of every 8 elements instead of 4: 51.6 / 47.2; all: 56.0.
constexpr float kLinMagic = 49152.0f;  // 1.5 * 2^15: floats in [2^15, 2^16) have an ulp of 2^-8
// (The clamp is a maximum on the ALU pipe, the busiest one of the kernel at 58 %; moving it to the FMA pipe as a
// saturating multiply-add followed by a second multiply-add costs one instruction more and measured 49.5 against 46.5 us:
// what counts is the number of instructions issued.)
__device__ __forceinline__ float ex2_lin_from_biased(float v) {
  v = fmaxf(v, kLinMagic - 120.0f);
  constexpr uint32_t kC = 0x3F800000u - 0x47400000u * 32768u - 436208u;  // 0x47400000 = bits of 49152.0f; 436208 = 0.052 * 2^23
  return __uint_as_float(__float_as_uint(v) * 32768u + kC);
}

}  // namespace qb
