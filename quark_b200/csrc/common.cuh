// Shared host/device helpers of the kernel library: error reporting, dtype sizes, bf16 / e4m3
// conversions that match the rounding rules the parity tests expect.
#pragma once

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cuda_bf16.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>

#include "../../include/quark_b200.h"

namespace qb {

// Thread-local message behind qb_last_error_string().
char* error_buffer();
int32_t fail(int32_t code, const char* fmt, ...);
// Device address of the status word kernels raise bits in (see qb_device_status).
unsigned int* status_word();

#define QB_CUDA_OK(expr)                                                                         \
  do {                                                                                           \
    cudaError_t _e = (expr);                                                                     \
    if (_e != cudaSuccess) return qb::fail(QB_ERR_CUDA, "%s: %s", #expr, cudaGetErrorString(_e)); \
  } while (0)

#define QB_REQUIRE(cond, code, ...)                  \
  do {                                               \
    if (!(cond)) return qb::fail(code, __VA_ARGS__); \
  } while (0)

// Kernels launched by this library since it was loaded (qb_kernel_launch_count).
extern unsigned long long g_launch_count;

inline int32_t check_launch(const char* what) {
  ++g_launch_count;
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return fail(QB_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return QB_OK;
}

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline size_t dtype_size(int32_t dt) { return dt == QB_BF16 ? 2 : dt == QB_E4M3 ? 1 : 4; }
inline size_t round_up(size_t x, size_t a) { return (x + a - 1) / a * a; }

// ---------------------------------------------------------------- device conversions
__device__ __forceinline__ float bf16_bits_to_f32(uint16_t b) { return __uint_as_float(static_cast<uint32_t>(b) << 16); }
__device__ __forceinline__ float bf16lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16hi(uint32_t w) { return __uint_as_float(w & 0xFFFF0000u); }

// Two f32 -> packed bf16x2 (round to nearest even); `lo` lands in the low half.
__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}

// Two f32 -> packed e4m3x2 (RN-even, saturate to +-448, NaN -> 0x7F); `lo` in the low byte.
__device__ __forceinline__ uint16_t pack_e4m3x2(float lo, float hi) {
  uint16_t r;
  asm("cvt.rn.satfinite.e4m3x2.f32 %0, %1, %2;" : "=h"(r) : "f"(hi), "f"(lo));
  return r;
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  return static_cast<uint32_t>(pack_e4m3x2(a, b)) | (static_cast<uint32_t>(pack_e4m3x2(c, d)) << 16);
}

// x * sigmoid(x) with the exact exponential (the reference oracle uses exp, not an approximation).
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// The same with the hardware approximations (2^x and 1/x, ~2^-22 relative error each), which is what
// the reference's GEMM epilogue uses (ref: src/quark/lang/epilogue.py:43-69): a handful of
// instructions instead of ~50, for epilogues that sit on the critical path of a tensor-core kernel.
__device__ __forceinline__ float silu_fast(float x) {
  float e, r;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(x * -1.4426950408889634f));
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
  return x * r;
}

}  // namespace qb
