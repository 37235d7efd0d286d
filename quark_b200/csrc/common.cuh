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

// Programmatic dependent launch: a kernel launched through launch_dep() may start while the kernel
// before it in the stream is still running, so that its set-up (barrier init, TMEM allocation,
// descriptor and weight prefetch) overlaps that kernel's tail.  Every such kernel executes
// grid_dep_wait() before it reads anything an earlier kernel wrote and before it writes global
// memory; the wait returns when all earlier kernels have completed and their writes are visible.
// qb_set_dependent_launch(0) (or QB_DEPENDENT_LAUNCH=0 in the environment) turns the attribute off;
// the device-side calls are then no-ops.
extern int g_dependent_launch;

template <typename... KArgs, typename... Args>
inline int32_t launch_dep(const char* what, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_dependent_launch ? 1 : 0;
  ++g_launch_count;
  cudaError_t e = cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
  if (e != cudaSuccess) return fail(QB_ERR_LAUNCH, "%s: %s", what, cudaGetErrorString(e));
  return QB_OK;
}

__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// What an earlier kernel of the stream may have written is read with ordinary loads through a pointer that has passed
// through after_wait(): a read-only load (ld.global.nc: __ldg, or what the compiler makes of a const __restrict__
// parameter) counts as invariant for the whole kernel, so the compiler may issue it before griddepcontrol.wait, i.e.
// while the earlier kernel is still writing.  __ldg stays for tables nothing on the device ever writes (RoPE table,
// weights and their scales).
template <class T>
__device__ __forceinline__ T* after_wait(T* p) {
  asm volatile("" : "+l"(p)::"memory");
  return p;
}
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

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
// Joining the halves with a register-pair move inside one asm block (mov.b32 {lo, hi}) instead of the shift and OR
// below was measured on the attention kernel: 52.2 -> 58.4 us (the instruction schedule the compiler finds for the
// softmax loop changes for the worse), so the plain form stays.
// Every e4m3 value is a bf16 value (3 mantissa bits, exponents -9 .. 8), so the widening is exact; NaN stays NaN.
__device__ __forceinline__ uint32_t e4m3x2_to_bf16x2(uint16_t v) {
  uint32_t h2;
  asm("cvt.rn.f16x2.e4m3x2 %0, %1;" : "=r"(h2) : "h"(v));
  const __half2 h = *reinterpret_cast<const __half2*>(&h2);
  const __nv_bfloat162 b = __floats2bfloat162_rn(__low2float(h), __high2float(h));
  return *reinterpret_cast<const uint32_t*>(&b);
}
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
  return static_cast<uint32_t>(pack_e4m3x2(a, b)) | (static_cast<uint32_t>(pack_e4m3x2(c, d)) << 16);
}

// x * sigmoid(x) with the exact exponential (the reference oracle uses exp, not an approximation).
__device__ __forceinline__ float silu_f(float x) { return x / (1.0f + expf(-x)); }

// The same with a hardware approximation (tanh.approx.f32, 2^-11 relative error: a quarter of a bf16
// ulp) for epilogues on the critical path of a tensor-core kernel, where the special-function unit is
// the bound: 3 instructions, one of them on that unit.  The reference's GEMM epilogue uses approximate
// exp2 and reciprocal for the same reason (ref: src/quark/lang/epilogue.py:43-69).
__device__ __forceinline__ float silu_fast(float x) {
  // x * sigmoid(x) = h + h * tanh(h) with h = x / 2: one special-function instruction per element
  const float h = 0.5f * x;
  float t;
  asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
  return fmaf(h, t, h);
}

// 32-byte global stores (one full sector per thread); the address must be 32-byte aligned.
__device__ __forceinline__ void st_global_v8(void* p, const uint32_t (&w)[8]) {
  asm volatile("st.global.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(w[0]), "r"(w[1]), "r"(w[2]), "r"(w[3]),
               "r"(w[4]), "r"(w[5]), "r"(w[6]), "r"(w[7])
               : "memory");
}

}  // namespace qb
