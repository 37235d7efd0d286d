// HBM-bound norm / elementwise kernels that chain the GEMMs and the attention into a block:
// AdaRMSNorm, per-head RMSNorm, value residual, gate + residual, SiLU, Euler step, e4m3 narrowing,
// patchify / unpatchify and the frame counter.  bf16 in and out, f32 arithmetic written as
// separate multiplies and adds where the CPU oracle does so, 16-byte accesses throughout.
#include <cuda_fp16.h>

#include "common.cuh"

namespace qb {

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16lo(u.x); f[1] = bf16hi(u.x); f[2] = bf16lo(u.y); f[3] = bf16hi(u.y);
  f[4] = bf16lo(u.z); f[5] = bf16hi(u.z); f[6] = bf16lo(u.w); f[7] = bf16hi(u.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 o;
  o.x = pack_bf16x2(f[0], f[1]); o.y = pack_bf16x2(f[2], f[3]);
  o.z = pack_bf16x2(f[4], f[5]); o.w = pack_bf16x2(f[6], f[7]);
  return o;
}
__device__ __forceinline__ uint2 pack8_e4m3(const float (&f)[8]) {
  uint2 o;
  o.x = pack_e4m3x4(f[0], f[1], f[2], f[3]);
  o.y = pack_e4m3x4(f[4], f[5], f[6], f[7]);
  return o;
}
// The e4m3 side output is narrowed from the bf16-rounded value, i.e. it equals what a separate
// bf16 -> e4m3 cast of the main output would give.
__device__ __forceinline__ void round_through_bf16(float (&f)[8]) {
#pragma unroll
  for (int j = 0; j < 8; ++j) f[j] = __bfloat162float(__float2bfloat16_rn(f[j]));
}

// ---------------------------------------------------------------- AdaRMSNorm
// One CTA per row; each thread owns D / (8 * blockDim) groups of 8 consecutive elements.
// kMaxVec: 16-byte vectors of the row per thread (D <= 8 * kThreads * kMaxVec); the narrow instantiation keeps four CTAs
// on an SM, so that the 512 rows of a 720p frame are all resident at once instead of running as two waves.
template <int kThreads, int kMaxVec>
__global__ void __launch_bounds__(kThreads, kMaxVec == 1 ? 4 : 2) ada_rmsnorm_kernel(const uint16_t* X, const uint16_t* scale,
                                                                const uint16_t* bias, uint16_t* out,
                                                                uint8_t* out_q, int D, int rows_per_group, float eps,
                                                                int activation) {
  grid_dep_wait();    // inputs come from the kernels before this one
  grid_dep_launch();  // the next kernel may begin its set-up (triggering before the wait measured the same: 80.5 / 80.6 FPS)
  const int row = blockIdx.x;
  const uint16_t* x = X + static_cast<size_t>(row) * D;
  const size_t goff = static_cast<size_t>(row / rows_per_group) * D;
  uint4 xv[kMaxVec], sv[kMaxVec], bv[kMaxVec];  // scale and bias are fetched with the row, not after the reduction
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
    if (c < D) {
      xv[i] = *reinterpret_cast<const uint4*>(x + c);
      sv[i] = *reinterpret_cast<const uint4*>(scale + goff + c);
      bv[i] = *reinterpret_cast<const uint4*>(bias + goff + c);
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  __shared__ float red[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) tot += red[w];
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(D) + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
    if (c < D) {
      float f[8], s[8], b[8];
      unpack8(xv[i], f);
      unpack8(sv[i], s);
      unpack8(bv[i], b);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float y = __fmul_rn(f[j], inv);
        y = __fadd_rn(__fmul_rn(y, __fadd_rn(1.0f, s[j])), b[j]);
        f[j] = activation == 1 ? silu_f(y) : y;
      }
      if (out != nullptr) *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * D + c) = pack8(f);
      if (out_q != nullptr) {
        round_through_bf16(f);
        *reinterpret_cast<uint2*>(out_q + static_cast<size_t>(row) * D + c) = pack8_e4m3(f);
      }
    }
  }
}

// ---------------------------------------------------------------- per-head RMSNorm on packed qkv
// 8 threads per (row, head): 8 x 8 = 64 elements; heads >= n_norm_heads (the V heads) are copied.
__global__ void __launch_bounds__(256) head_rmsnorm_kernel(const uint16_t* X, uint16_t* out, int rows,
                                                            int heads_total, int n_norm_heads, float eps) {
  const size_t gid = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  const size_t item = gid >> 3;  // (row, head)
  const int sub = gid & 7;
  const bool active = item < static_cast<size_t>(rows) * heads_total;
  const int head = active ? static_cast<int>(item % heads_total) : 0;
  const size_t off = (active ? item : 0) * 64 + sub * 8;
  float f[8];
  uint4 v = make_uint4(0, 0, 0, 0);
  if (active) v = *reinterpret_cast<const uint4*>(X + off);
  unpack8(v, f);
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  ss += __shfl_xor_sync(0xffffffffu, ss, 4);
  if (!active) return;
  if (head < n_norm_heads) {
    const float inv = 1.0f / sqrtf(ss * (1.0f / 64.0f) + eps);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(f[j], inv);
    v = pack8(f);
  }
  *reinterpret_cast<uint4*>(out + off) = v;
}

// ---------------------------------------------------------------- value residual on the V columns
__global__ void __launch_bounds__(256) value_residual_kernel(const uint16_t* cur, const uint16_t* first,
                                                              const float* lamb, uint16_t* out, int rows,
                                                              int D_full, int v_off, int v_width) {
  const size_t i8 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  if (i8 >= static_cast<size_t>(rows) * D_full) return;
  const int col = static_cast<int>(i8 % D_full);
  uint4 c = *reinterpret_cast<const uint4*>(cur + i8);
  if (col >= v_off && col < v_off + v_width) {
    const float lam = *lamb;
    float a[8], b[8];
    unpack8(c, a);
    unpack8(*reinterpret_cast<const uint4*>(first + i8), b);
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = __fadd_rn(a[j], __fmul_rn(lam, __fsub_rn(b[j], a[j])));
    c = pack8(a);
  }
  *reinterpret_cast<uint4*>(out + i8) = c;
}

// ---------------------------------------------------------------- x + gate * y
__global__ void __launch_bounds__(256) gate_residual_kernel(const uint16_t* X, const uint16_t* Y,
                                                             const uint16_t* gate, uint16_t* out, int rows,
                                                             int D, int rows_per_group) {
  const size_t i8 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  if (i8 >= static_cast<size_t>(rows) * D) return;
  const int row = static_cast<int>(i8 / D), col = static_cast<int>(i8 % D);
  float x[8], y[8], g[8];
  unpack8(*reinterpret_cast<const uint4*>(X + i8), x);
  unpack8(*reinterpret_cast<const uint4*>(Y + i8), y);
  unpack8(*reinterpret_cast<const uint4*>(gate + static_cast<size_t>(row / rows_per_group) * D + col), g);
#pragma unroll
  for (int j = 0; j < 8; ++j) x[j] = __fadd_rn(x[j], __fmul_rn(g[j], y[j]));
  *reinterpret_cast<uint4*>(out + i8) = pack8(x);
}

// ---------------------------------------------------------------- SiLU / Euler / quantise
__global__ void __launch_bounds__(256) silu_kernel(const uint16_t* X, uint16_t* out, uint8_t* out_q,
                                                    size_t n) {
  const size_t i8 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  if (i8 + 8 <= n) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(X + i8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = silu_f(f[j]);
    if (out != nullptr) *reinterpret_cast<uint4*>(out + i8) = pack8(f);
    if (out_q != nullptr) {
      round_through_bf16(f);
      *reinterpret_cast<uint2*>(out_q + i8) = pack8_e4m3(f);
    }
  } else {
    for (size_t i = i8; i < n; ++i) {
      const float y = silu_f(bf16_bits_to_f32(X[i]));
      const __nv_bfloat16 yb = __float2bfloat16_rn(y);
      if (out != nullptr) out[i] = *reinterpret_cast<const uint16_t*>(&yb);
      if (out_q != nullptr) out_q[i] = static_cast<uint8_t>(pack_e4m3x2(__bfloat162float(yb), 0.f) & 0xFF);
    }
  }
}

// ---------------------------------------------------------------- plain RMSNorm and elementwise add
// (the controller-conditioning path: src/quark/kernels/rmsnorm/reference.py:10-22, elementwise add)
// One CTA per row, like ada_rmsnorm without the affine step.
template <int kThreads>
__global__ void __launch_bounds__(kThreads) rmsnorm_kernel(const uint16_t* X, uint16_t* out, int D, float eps) {
  grid_dep_wait();
  grid_dep_launch();
  const int row = blockIdx.x;
  const uint16_t* x = X + static_cast<size_t>(row) * D;
  constexpr int kMaxVec = 4;  // D <= 8 * kThreads * kMaxVec
  uint4 xv[kMaxVec];
  float ss = 0.f;
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
    if (c < D) {
      xv[i] = *reinterpret_cast<const uint4*>(x + c);
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
    }
  }
  __shared__ float red[kThreads / 32];
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
#pragma unroll
  for (int w = 0; w < kThreads / 32; ++w) tot += red[w];
  const float inv = 1.0f / sqrtf(tot / static_cast<float>(D) + eps);
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kThreads + threadIdx.x) * 8;
    if (c < D) {
      float f[8];
      unpack8(xv[i], f);
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(f[j], inv);
      *reinterpret_cast<uint4*>(out + static_cast<size_t>(row) * D + c) = pack8(f);
    }
  }
}

__global__ void __launch_bounds__(256) add_kernel(const uint16_t* X, const uint16_t* Y, uint16_t* out,
                                                   size_t n) {
  grid_dep_wait();
  grid_dep_launch();
  const size_t i8 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  if (i8 + 8 <= n) {
    float x[8], y[8];
    unpack8(*reinterpret_cast<const uint4*>(X + i8), x);
    unpack8(*reinterpret_cast<const uint4*>(Y + i8), y);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = __fadd_rn(x[j], y[j]);
    *reinterpret_cast<uint4*>(out + i8) = pack8(x);
  } else {
    for (size_t i = i8; i < n; ++i) {
      const __nv_bfloat16 r = __float2bfloat16_rn(__fadd_rn(bf16_bits_to_f32(X[i]), bf16_bits_to_f32(Y[i])));
      out[i] = *reinterpret_cast<const uint16_t*>(&r);
    }
  }
}

__global__ void __launch_bounds__(256) euler_kernel(const uint16_t* X, const uint16_t* V,
                                                     const float* dsig, uint16_t* out, size_t n) {
  grid_dep_wait();    // inputs come from the kernels before this one
  grid_dep_launch();  // the next kernel may begin its set-up
  const size_t i8 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  const float d = *dsig;
  if (i8 + 8 <= n) {
    float x[8], v[8];
    unpack8(*reinterpret_cast<const uint4*>(X + i8), x);
    unpack8(*reinterpret_cast<const uint4*>(V + i8), v);
#pragma unroll
    for (int j = 0; j < 8; ++j) x[j] = __fadd_rn(x[j], __fmul_rn(d, v[j]));
    *reinterpret_cast<uint4*>(out + i8) = pack8(x);
  } else {
    for (size_t i = i8; i < n; ++i) {
      const __nv_bfloat16 y = __float2bfloat16_rn(__fadd_rn(bf16_bits_to_f32(X[i]), __fmul_rn(d, bf16_bits_to_f32(V[i]))));
      out[i] = *reinterpret_cast<const uint16_t*>(&y);
    }
  }
}

template <bool kFromF32>
__global__ void __launch_bounds__(256) quantize_kernel(const void* X, uint8_t* out, size_t n) {
  const size_t i8 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 8;
  if (i8 + 8 <= n) {
    float f[8];
    if (kFromF32) {
      const float4 a = reinterpret_cast<const float4*>(X)[i8 / 4], b = reinterpret_cast<const float4*>(X)[i8 / 4 + 1];
      f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
    } else {
      unpack8(*reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(X) + i8), f);
    }
    *reinterpret_cast<uint2*>(out + i8) = pack8_e4m3(f);
  } else {
    for (size_t i = i8; i < n; ++i) {
      const float v = kFromF32 ? static_cast<const float*>(X)[i] : bf16_bits_to_f32(static_cast<const uint16_t*>(X)[i]);
      out[i] = static_cast<uint8_t>(pack_e4m3x2(v, 0.f) & 0xFF);
    }
  }
}

// One CTA per row: row maximum of |x| (a maximum does not depend on the order it is taken in), scale = amax / 448,
// out = e4m3(x * (1 / scale)).  Weights are narrowed once, at load time: nothing here is tuned.
__global__ void __launch_bounds__(256) quantize_rows_kernel(const uint16_t* X, uint8_t* out,
                                                            float* scale_out, int cols) {
  __shared__ float red[8];
  const uint16_t* x = X + static_cast<size_t>(blockIdx.x) * cols;
  float m = 0.f;
  for (int i8 = threadIdx.x * 8; i8 < cols; i8 += 256 * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + i8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) m = fmaxf(m, fabsf(f[j]));
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = red[0];
#pragma unroll
  for (int w = 1; w < 8; ++w) m = fmaxf(m, red[w]);
  const float scale = m > 0.f ? __fdiv_rn(m, 448.0f) : 1.0f;
  const float inv = __fdiv_rn(1.0f, scale);
  if (threadIdx.x == 0) scale_out[blockIdx.x] = scale;
  uint8_t* o = out + static_cast<size_t>(blockIdx.x) * cols;
  for (int i8 = threadIdx.x * 8; i8 < cols; i8 += 256 * 8) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(x + i8), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = __fmul_rn(f[j], inv);
    *reinterpret_cast<uint2*>(o + i8) = pack8_e4m3(f);
  }
}

__global__ void increment_kernel(int32_t* c) {
  grid_dep_wait();    // inputs come from the kernels before this one
  grid_dep_launch();  // the next kernel may begin its set-up
  c[0] += 1;
}

// ---------------------------------------------------------------- e4m3 -> bf16
// (e4m3x2_to_bf16x2 in common.cuh: the widening is exact)

__global__ void __launch_bounds__(256) dequantize_kernel(const uint8_t* X, uint16_t* out, size_t n) {
  grid_dep_wait();
  grid_dep_launch();
  const size_t i16 = (blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x) * 16;
  if (i16 + 16 <= n) {
    const uint4 v = *reinterpret_cast<const uint4*>(X + i16);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = e4m3x2_to_bf16x2(static_cast<uint16_t>(w[j] & 0xFFFF));
      o[2 * j + 1] = e4m3x2_to_bf16x2(static_cast<uint16_t>(w[j] >> 16));
    }
    *reinterpret_cast<uint4*>(out + i16) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(out + i16 + 8) = make_uint4(o[4], o[5], o[6], o[7]);
  } else {
    for (size_t i = i16; i < n; ++i) out[i] = static_cast<uint16_t>(e4m3x2_to_bf16x2(X[i]) & 0xFFFF);
  }
}

// ---------------------------------------------------------------- mixture of experts: routing weights, combination
// Per token: the top_k experts by logit (ties to the lower index, like a stable descending sort), a softmax over
// those top_k logits, written as a dense [E][M] f32 table that is zero for the experts a token does not use
// (ref: src/quark/kernels/moe_router_correct/reference.py:38-49, the "correct" routing).
constexpr int kMoeMaxExperts = 32;

__global__ void __launch_bounds__(128) moe_route_kernel(const uint16_t* logits, float* weights, int M, int E,
                                                         int top_k) {
  grid_dep_wait();
  grid_dep_launch();
  const int m = blockIdx.x * blockDim.x + threadIdx.x;
  if (m >= M) return;
  float l[kMoeMaxExperts];
  float w[kMoeMaxExperts];
  for (int e = 0; e < E; ++e) {
    l[e] = bf16_bits_to_f32(logits[static_cast<size_t>(m) * E + e]);
    w[e] = 0.f;
  }
  unsigned taken = 0;
  float top = 0.f, sum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    int best = -1;
    for (int e = 0; e < E; ++e)
      if (!((taken >> e) & 1u) && (best < 0 || l[e] > l[best])) best = e;
    taken |= 1u << best;
    if (k == 0) top = l[best];
    w[best] = expf(l[best] - top);
    sum += w[best];
  }
  for (int e = 0; e < E; ++e) weights[static_cast<size_t>(e) * M + m] = w[e] / sum;
}

// out[m, :] = bf16( sum over the experts e with weights[e][m] != 0, in order of e, of weights[e][m] * partials[e][m][:] ),
// the sum in f32 and one narrowing at the end (ref: src/quark/kernels/moe_reduce/reference.py:16-33).
__global__ void __launch_bounds__(256) moe_combine_kernel(const float* partials, const float* weights,
                                                           uint16_t* out, int M, int D, int E) {
  grid_dep_wait();
  grid_dep_launch();
  const int m = blockIdx.x;
  for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int e = 0; e < E; ++e) {
      const float w = weights[static_cast<size_t>(e) * M + m];
      if (w == 0.f) continue;  // an expert the token does not use: its partial is never read
      const float4 y = *reinterpret_cast<const float4*>(partials + (static_cast<size_t>(e) * M + m) * D + d);
      acc[0] = fmaf(w, y.x, acc[0]); acc[1] = fmaf(w, y.y, acc[1]); acc[2] = fmaf(w, y.z, acc[2]); acc[3] = fmaf(w, y.w, acc[3]);
    }
    const uint2 o = make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]));
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(m) * D + d) = o;
  }
}

// ---------------------------------------------------------------- mixture of experts: slot-sorted schedule
// The routing of moe_route_kernel laid out as slots sorted by expert, every expert's run padded to whole 128-row
// tiles (the row tile of the GEMM kernel), so that the expert projections are two grouped GEMMs over
// M * top_k (+ padding) rows instead of E dense GEMMs over M rows each (ref: the slot tables of
// src/quark/kernels/moe_router_correct/reference.py:51-120, whose tile is 32 rows).  One CTA: the tables are tiny.
//   slot_token[s]   token whose row occupies slot s, -1 for padding
//   slot_weight[s]  its routing weight (0 for padding)
//   tile_expert[i]  expert of rows [128 i, 128 i + 128), -1 past the last used tile
//   token_slot[m,k] slot of token m's k-th choice (k in order of decreasing logit)
// Within an expert the slots follow (token, k) order, whatever order the threads run in.
constexpr int kMoeTile = 128;
constexpr int kMoeRouteThreads = 1024;

__device__ __forceinline__ void moe_topk(const uint16_t* row, int E, int top_k, int (&ex)[kMoeMaxExperts], float (&wt)[kMoeMaxExperts]) {
  float l[kMoeMaxExperts];
  for (int e = 0; e < E; ++e) l[e] = bf16_bits_to_f32(row[e]);
  unsigned taken = 0;
  float top = 0.f, sum = 0.f;
  for (int k = 0; k < top_k; ++k) {
    int best = -1;
    for (int e = 0; e < E; ++e)
      if (!((taken >> e) & 1u) && (best < 0 || l[e] > l[best])) best = e;
    taken |= 1u << best;
    if (k == 0) top = l[best];
    ex[k] = best;
    wt[k] = expf(l[best] - top);
    sum += wt[k];
  }
  for (int k = 0; k < top_k; ++k) wt[k] = wt[k] / sum;
}

__global__ void __launch_bounds__(kMoeRouteThreads) moe_route_slots_kernel(const uint16_t* logits, int* slot_token,
                                                                            float* slot_weight, int* tile_expert,
                                                                            int* token_slot, int* counts_out, int M, int E,
                                                                            int top_k, int n_slots) {
  grid_dep_wait();
  grid_dep_launch();
  __shared__ int count[kMoeMaxExperts], offset[kMoeMaxExperts + 1], base[kMoeMaxExperts];
  __shared__ int warp_tot[kMoeMaxExperts][kMoeRouteThreads / 32];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  if (tid < kMoeMaxExperts) count[tid] = 0;
  __syncthreads();
  int ex[kMoeMaxExperts];
  float wt[kMoeMaxExperts];
  // pass 1: how many tokens each expert receives
  for (int t = tid; t < M; t += kMoeRouteThreads) {
    moe_topk(logits + static_cast<size_t>(t) * E, E, top_k, ex, wt);
    for (int k = 0; k < top_k; ++k) atomicAdd(&count[ex[k]], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int cum = 0;
    for (int e = 0; e < E; ++e) {
      offset[e] = cum;
      base[e] = 0;
      cum += (count[e] + kMoeTile - 1) / kMoeTile * kMoeTile;
      if (counts_out != nullptr) counts_out[e] = count[e];
    }
    offset[E] = cum;
  }
  __syncthreads();
  // pass 2: tokens in chunks of one per thread, in order; a choice's rank among its expert's = choices of earlier chunks
  // + of earlier warps of this chunk + of earlier lanes of this warp
  for (int t0 = 0; t0 < M; t0 += kMoeRouteThreads) {
    const int t = t0 + tid;
    const bool live = t < M;
    if (live) moe_topk(logits + static_cast<size_t>(t) * E, E, top_k, ex, wt);
    unsigned mine = 0;
    if (live)
      for (int k = 0; k < top_k; ++k) mine |= 1u << ex[k];
    unsigned before[kMoeMaxExperts];  // lanes of this warp that chose expert e, below this lane
    for (int e = 0; e < E; ++e) {
      const unsigned b = __ballot_sync(0xffffffffu, (mine >> e) & 1u);
      before[e] = __popc(b & ((1u << lane) - 1u));
      if (lane == 0) warp_tot[e][warp] = __popc(b);
    }
    __syncthreads();
    if (live) {
      for (int k = 0; k < top_k; ++k) {
        const int e = ex[k];
        int rank = base[e] + static_cast<int>(before[e]);
        for (int w = 0; w < warp; ++w) rank += warp_tot[e][w];
        const int slot = offset[e] + rank;
        slot_token[slot] = t;
        slot_weight[slot] = wt[k];
        token_slot[static_cast<size_t>(t) * top_k + k] = slot;
      }
    }
    __syncthreads();
    if (tid < E) {
      int tot = 0;
      for (int w = 0; w < kMoeRouteThreads / 32; ++w) tot += warp_tot[tid][w];
      base[tid] += tot;
    }
    __syncthreads();
  }
  // padding slots and the tile table
  for (int e = 0; e < E; ++e)
    for (int s = offset[e] + count[e] + tid; s < offset[e + 1]; s += kMoeRouteThreads) {
      slot_token[s] = -1;
      slot_weight[s] = 0.f;
    }
  for (int s = offset[E] + tid; s < n_slots; s += kMoeRouteThreads) {
    slot_token[s] = -1;
    slot_weight[s] = 0.f;
  }
  for (int i = tid; i < n_slots / kMoeTile; i += kMoeRouteThreads) {
    const int s = i * kMoeTile;
    int e = -1;
    for (int q = 0; q < E; ++q)
      if (s >= offset[q] && s < offset[q + 1]) e = q;
    tile_expert[i] = e;
  }
}

// out[s, :] = X[slot_token[s], :] (rows of `row_bytes` bytes, a multiple of 16), zeros for padding slots
__global__ void __launch_bounds__(256) moe_gather_kernel(const uint8_t* X, const int* slot_token, uint8_t* out,
                                                          int row_bytes) {
  grid_dep_wait();
  grid_dep_launch();
  const int s = blockIdx.x;
  const int t = slot_token[s];
  for (int b = threadIdx.x * 16; b < row_bytes; b += blockDim.x * 16) {
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (t >= 0) v = *reinterpret_cast<const uint4*>(X + static_cast<size_t>(t) * row_bytes + b);
    *reinterpret_cast<uint4*>(out + static_cast<size_t>(s) * row_bytes + b) = v;
  }
}

// out[m, :] = bf16( sum over the token's top_k slots of slot_weight[slot] * partials[slot][:] ), the sum in f32 (fused
// multiply-adds) in order of increasing slot, i.e. of increasing expert index - the order of the dense schedule's
// moe_combine_kernel, so that both schedules give the same bits - and one narrowing at the end
// (ref: src/quark/kernels/moe_reduce/reference.py:16-33)
__global__ void __launch_bounds__(256) moe_reduce_kernel(const float* partials, const float* slot_weight,
                                                          const int* token_slot, uint16_t* out, int D, int top_k) {
  grid_dep_wait();
  grid_dep_launch();
  const int m = blockIdx.x;
  int slots[kMoeMaxExperts];
  for (int k = 0; k < top_k; ++k) {  // insertion sort: top_k is small
    const int s = token_slot[static_cast<size_t>(m) * top_k + k];
    int j = k;
    while (j > 0 && slots[j - 1] > s) {
      slots[j] = slots[j - 1];
      --j;
    }
    slots[j] = s;
  }
  for (int d = threadIdx.x * 4; d < D; d += blockDim.x * 4) {
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k = 0; k < top_k; ++k) {
      const int slot = slots[k];
      const float w = slot_weight[slot];
      const float4 y = *reinterpret_cast<const float4*>(partials + static_cast<size_t>(slot) * D + d);
      acc[0] = fmaf(w, y.x, acc[0]); acc[1] = fmaf(w, y.y, acc[1]); acc[2] = fmaf(w, y.z, acc[2]); acc[3] = fmaf(w, y.w, acc[3]);
    }
    *reinterpret_cast<uint2*>(out + static_cast<size_t>(m) * D + d) = make_uint2(pack_bf16x2(acc[0], acc[1]), pack_bf16x2(acc[2], acc[3]));
  }
}

// ---------------------------------------------------------------- randn
// Standard normals from a counter: Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3")
// on the counter (group, 0, seed0, seed1) with the key (seed0, seed1), the four words turned into uniforms
// (top 24 bits) * 2^-24 + 2^-25 and pairwise into normals by Box-Muller.  A block of 128 threads fills 2048
// consecutive outputs: thread t, pass g (0..3) draws group block * 512 + g * 128 + t + offset and writes its four
// normals to positions block * 2048 + (4 g + k) * 128 + t, k = 0..3, so that every store is coalesced.  This
// is the layout of the reference's kernel at its default tile (src/quark/kernels/randn/kernel.py:200-254,
// config.py:11-20), which has no oracle of its own (reference.py: "statistical, not bitwise").
constexpr int kRandnThreads = 128;
constexpr int kRandnPerBlock = 2048;

__device__ __forceinline__ void philox4x32_10(uint32_t (&c)[4], uint32_t k0, uint32_t k1) {
#pragma unroll
  for (int r = 0; r < 10; ++r) {
    const uint32_t hi0 = __umulhi(0xD2511F53u, c[0]), lo0 = 0xD2511F53u * c[0];
    const uint32_t hi1 = __umulhi(0xCD9E8D57u, c[2]), lo1 = 0xCD9E8D57u * c[2];
    c[0] = hi1 ^ c[1] ^ k0;
    c[1] = lo1;
    c[2] = hi0 ^ c[3] ^ k1;
    c[3] = lo0;
    k0 += 0x9E3779B9u;
    k1 += 0xBB67AE85u;
  }
}

__device__ __forceinline__ float randn_uniform(uint32_t x) { return fmaf(static_cast<float>(x >> 8), 5.9604644775390625e-8f, 2.98023223876953125e-8f); }

template <typename Out>
__global__ void __launch_bounds__(kRandnThreads) randn_kernel(const uint32_t* counter, Out* out, size_t n,
                                                              uint32_t stride, uint32_t seed0, uint32_t seed1) {
  grid_dep_wait();
  grid_dep_launch();
  const uint32_t offset = counter[0] * stride;
  const size_t base = static_cast<size_t>(blockIdx.x) * kRandnPerBlock;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint32_t c[4] = {static_cast<uint32_t>(blockIdx.x) * (kRandnPerBlock / 4) + g * kRandnThreads + threadIdx.x + offset, 0u, seed0, seed1};
    philox4x32_10(c, seed0, seed1);
    float z[4];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
      const float u1 = randn_uniform(c[2 * h]), u2 = randn_uniform(c[2 * h + 1]);
      const float r = sqrtf(-1.3862943611198906f * log2f(u1));  // sqrt(-2 ln u1)
      float sn, cs;
      sincosf(6.283185307179586f * u2, &sn, &cs);
      z[2 * h] = r * cs;
      z[2 * h + 1] = r * sn;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      const size_t i = base + (4 * g + k) * kRandnThreads + threadIdx.x;
      if (i < n) {
        if constexpr (sizeof(Out) == 4) {
          out[i] = z[k];
        } else {
          const __nv_bfloat16 b = __float2bfloat16_rn(z[k]);
          out[i] = *reinterpret_cast<const uint16_t*>(&b);
        }
      }
    }
  }
}

// ---------------------------------------------------------------- patchify / unpatchify
// Both are thin GEMMs (K = C*ph*pw = 128 in, N = 128 out for the model) run once per NFE.
// A CTA stages kTok token rows in shared memory as f32; each thread owns one output feature and
// reads its weight row once for all staged tokens.
constexpr int kPatchTok = 8;

__global__ void __launch_bounds__(256) patchify_kernel(const uint16_t* X, const uint16_t* W,
                                                        uint16_t* out, int C, int H, int Wd, int ph, int pw, int d_model,
                                                        int tokens) {
  extern __shared__ float patch[];  // [kPatchTok][K]
  const int K = C * ph * pw;
  const int Wp = Wd / pw;
  const int t0 = blockIdx.x * kPatchTok;
  for (int i = threadIdx.x; i < kPatchTok * K; i += blockDim.x) {
    const int tt = i / K, k = i % K;
    const int tok = t0 + tt;
    float v = 0.f;
    if (tok < tokens) {
      const int c = k / (ph * pw), r = (k / pw) % ph, q = k % pw;
      const int hp = tok / Wp, wp = tok % Wp;
      v = bf16_bits_to_f32(X[static_cast<size_t>(c) * H * Wd + static_cast<size_t>(hp * ph + r) * Wd + wp * pw + q]);
    }
    patch[i] = v;
  }
  __syncthreads();
  const int d = blockIdx.y * blockDim.x + threadIdx.x;
  if (d >= d_model) return;
  float acc[kPatchTok];
#pragma unroll
  for (int t = 0; t < kPatchTok; ++t) acc[t] = 0.f;
  const uint16_t* w = W + static_cast<size_t>(d) * K;
  for (int k = 0; k < K; k += 8) {
    float wf[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(w + k)), wf);
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int t = 0; t < kPatchTok; ++t) acc[t] = fmaf(patch[t * K + k + j], wf[j], acc[t]);
  }
  for (int t = 0; t < kPatchTok; ++t) {
    if (t0 + t < tokens) {
      const __nv_bfloat16 y = __float2bfloat16_rn(acc[t]);
      out[static_cast<size_t>(t0 + t) * d_model + d] = *reinterpret_cast<const uint16_t*>(&y);
    }
  }
}

__global__ void __launch_bounds__(128) unpatchify_kernel(const uint16_t* X, const uint16_t* W,
                                                          const uint16_t* bias, uint16_t* out, int C, int H,
                                                          int Wd, int ph, int pw, int d_model, int tokens) {
  extern __shared__ float xs[];  // [kPatchTok][d_model]
  const int Nout = C * ph * pw;
  const int Wp = Wd / pw;
  const int t0 = blockIdx.x * kPatchTok;
  for (int i = threadIdx.x * 8; i < kPatchTok * d_model; i += blockDim.x * 8) {
    const int tt = i / d_model, k = i % d_model;
    float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (t0 + tt < tokens) unpack8(*reinterpret_cast<const uint4*>(X + static_cast<size_t>(t0 + tt) * d_model + k), f);
#pragma unroll
    for (int j = 0; j < 8; ++j) xs[i + j] = f[j];
  }
  __syncthreads();
  const int o = blockIdx.y * blockDim.x + threadIdx.x;
  if (o >= Nout) return;
  float acc[kPatchTok];
#pragma unroll
  for (int t = 0; t < kPatchTok; ++t) acc[t] = 0.f;
  const uint16_t* w = W + static_cast<size_t>(o) * d_model;
  for (int k = 0; k < d_model; k += 8) {
    float wf[8];
    unpack8(__ldg(reinterpret_cast<const uint4*>(w + k)), wf);
#pragma unroll
    for (int j = 0; j < 8; ++j)
#pragma unroll
      for (int t = 0; t < kPatchTok; ++t) acc[t] = fmaf(xs[t * d_model + k + j], wf[j], acc[t]);
  }
  const float b = bias != nullptr ? bf16_bits_to_f32(bias[o]) : 0.f;
  const int c = o / (ph * pw), r = (o / pw) % ph, q = o % pw;
  for (int t = 0; t < kPatchTok; ++t) {
    const int tok = t0 + t;
    if (tok < tokens) {
      const int hp = tok / Wp, wp = tok % Wp;
      const __nv_bfloat16 y = __float2bfloat16_rn(acc[t] + b);
      out[static_cast<size_t>(c) * H * Wd + static_cast<size_t>(hp * ph + r) * Wd + wp * pw + q] = *reinterpret_cast<const uint16_t*>(&y);
    }
  }
}

// Pure data movement between the latent layout [C, H, W] and the token layout [tokens, C*ph*pw]
// (token = patch (hp, wp), feature k = c*ph*pw + r*pw + q), so that patchify / unpatchify can run
// their contraction on the tensor-core GEMM.  kToTokens: latent -> tokens, else tokens -> latent.
template <bool kToTokens>
__global__ void __launch_bounds__(256) patch_move_kernel(const uint16_t* src, uint16_t* dst, int C, int H, int Wd,
                                                          int ph, int pw, int tokens) {
  grid_dep_wait();    // inputs come from the kernels before this one
  grid_dep_launch();  // the next kernel may begin its set-up
  const int K = C * ph * pw;
  const size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x;
  if (i >= static_cast<size_t>(tokens) * K) return;
  const int tok = static_cast<int>(i / K), k = static_cast<int>(i % K);
  const int Wp = Wd / pw;
  const int c = k / (ph * pw), r = (k / pw) % ph, q = k % pw;
  const int hp = tok / Wp, wp = tok % Wp;
  const size_t lat = static_cast<size_t>(c) * H * Wd + static_cast<size_t>(hp * ph + r) * Wd + wp * pw + q;
  if (kToTokens)
    dst[i] = src[lat];
  else
    dst[lat] = src[i];
}

int32_t quantize_e4m3_launch(const void* X, void* out, size_t n, int32_t src_dtype, cudaStream_t st) {
  if (n == 0) return QB_OK;
  const unsigned blocks = static_cast<unsigned>((n + 2047) / 2048);
  if (src_dtype == QB_F32)
    quantize_kernel<true><<<blocks, 256, 0, st>>>(X, static_cast<uint8_t*>(out), n);
  else
    quantize_kernel<false><<<blocks, 256, 0, st>>>(X, static_cast<uint8_t*>(out), n);
  return check_launch("quantize_e4m3");
}

}  // namespace qb

using namespace qb;

static inline unsigned blocks_for(size_t n_elems) { return static_cast<unsigned>((n_elems + 2047) / 2048); }

extern "C" {

int32_t qb_quantize_e4m3(const void* X, void* out, size_t n, int32_t src_dtype, void* stream) {
  QB_REQUIRE(src_dtype == QB_BF16 || src_dtype == QB_F32, QB_ERR_INVALID_ARG, "quantize_e4m3: src_dtype %d", src_dtype);
  QB_REQUIRE(n == 0 || (X && out), QB_ERR_INVALID_ARG, "quantize_e4m3: NULL pointer");
  QB_REQUIRE(aligned16(X) && aligned16(out), QB_ERR_ALIGN, "quantize_e4m3: pointers must be 16-byte aligned");
  return quantize_e4m3_launch(X, out, n, src_dtype, static_cast<cudaStream_t>(stream));
}

int32_t qb_quantize_e4m3_rows(const void* X, void* out, float* scale_out, int32_t rows, int32_t cols, void* stream) {
  QB_REQUIRE(X && out && scale_out, QB_ERR_INVALID_ARG, "quantize_e4m3_rows: NULL pointer");
  QB_REQUIRE(rows > 0 && cols > 0 && cols % 8 == 0, QB_ERR_INVALID_ARG, "quantize_e4m3_rows: [%d, %d] (cols must be a positive multiple of 8)", rows, cols);
  QB_REQUIRE(aligned16(X) && (reinterpret_cast<uintptr_t>(out) & 7u) == 0, QB_ERR_ALIGN, "quantize_e4m3_rows: X must be 16-byte and out 8-byte aligned");
  quantize_rows_kernel<<<rows, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint16_t*>(X), static_cast<uint8_t*>(out), scale_out, cols);
  return check_launch("quantize_e4m3_rows");
}

int32_t qb_ada_rmsnorm(const void* X, const void* scale, const void* bias, void* out, void* out_q, int32_t rows, int32_t D,
                       int32_t groups, float eps, int32_t activation, void* stream) {
  QB_REQUIRE(X && scale && bias && (out || out_q), QB_ERR_INVALID_ARG, "ada_rmsnorm: NULL pointer (out may be NULL only when out_q is given)");
  QB_REQUIRE(rows > 0 && D > 0 && groups > 0 && rows % groups == 0, QB_ERR_INVALID_ARG, "ada_rmsnorm: rows %d, D %d, groups %d", rows, D,
             groups);
  QB_REQUIRE(D % 8 == 0 && D <= 8192, QB_ERR_UNSUPPORTED, "ada_rmsnorm: D = %d must be a multiple of 8 and at most 8192", D);
  QB_REQUIRE(activation == 0 || activation == 1, QB_ERR_INVALID_ARG, "ada_rmsnorm: activation %d", activation);
  QB_REQUIRE(aligned16(X) && aligned16(scale) && aligned16(bias) && aligned16(out) && aligned16(out_q), QB_ERR_ALIGN,
             "ada_rmsnorm: pointers must be 16-byte aligned");
  auto kernel = D <= 2048 ? ada_rmsnorm_kernel<256, 1> : D <= 4096 ? ada_rmsnorm_kernel<256, 2> : ada_rmsnorm_kernel<256, 4>;
  return launch_dep("ada_rmsnorm", kernel, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(X), static_cast<const uint16_t*>(scale), static_cast<const uint16_t*>(bias),
                    static_cast<uint16_t*>(out), static_cast<uint8_t*>(out_q), D, rows / groups, eps, activation);
}

int32_t qb_head_rmsnorm(const void* X, void* out, int32_t rows, int32_t n_q_heads, int32_t n_kv_heads, int32_t Dh, float eps,
                        void* stream) {
  QB_REQUIRE(X && out, QB_ERR_INVALID_ARG, "head_rmsnorm: NULL pointer");
  QB_REQUIRE(Dh == 64, QB_ERR_UNSUPPORTED, "head_rmsnorm: head_dim %d (only 64)", Dh);
  QB_REQUIRE(rows > 0 && n_q_heads >= 0 && n_kv_heads >= 0 && n_q_heads + n_kv_heads > 0, QB_ERR_INVALID_ARG, "head_rmsnorm: bad sizes");
  QB_REQUIRE(aligned16(X) && aligned16(out), QB_ERR_ALIGN, "head_rmsnorm: pointers must be 16-byte aligned");
  const int heads_total = n_q_heads + 2 * n_kv_heads;
  const size_t threads = static_cast<size_t>(rows) * heads_total * 8;
  head_rmsnorm_kernel<<<static_cast<unsigned>((threads + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(X), static_cast<uint16_t*>(out), rows, heads_total, n_q_heads + n_kv_heads, eps);
  return check_launch("head_rmsnorm");
}

int32_t qb_value_residual_packed(const void* cur, const void* first, const float* lamb, void* out, int32_t rows, int32_t D_full,
                                 int32_t v_col_offset, int32_t v_width, void* stream) {
  QB_REQUIRE(cur && first && lamb && out, QB_ERR_INVALID_ARG, "value_residual_packed: NULL pointer");
  QB_REQUIRE(rows > 0 && D_full > 0 && v_col_offset >= 0 && v_width >= 0 && v_col_offset + v_width <= D_full, QB_ERR_INVALID_ARG,
             "value_residual_packed: bad sizes");
  QB_REQUIRE(D_full % 8 == 0 && v_col_offset % 8 == 0 && v_width % 8 == 0, QB_ERR_ALIGN, "value_residual_packed: columns must be multiples of 8");
  QB_REQUIRE(aligned16(cur) && aligned16(first) && aligned16(out), QB_ERR_ALIGN, "value_residual_packed: pointers must be 16-byte aligned");
  value_residual_kernel<<<blocks_for(static_cast<size_t>(rows) * D_full), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(cur), static_cast<const uint16_t*>(first), lamb, static_cast<uint16_t*>(out), rows, D_full,
      v_col_offset, v_width);
  return check_launch("value_residual_packed");
}

int32_t qb_ada_gate_residual(const void* X, const void* Y, const void* gate, void* out, int32_t rows, int32_t D, int32_t groups,
                             void* stream) {
  QB_REQUIRE(X && Y && gate && out, QB_ERR_INVALID_ARG, "ada_gate_residual: NULL pointer");
  QB_REQUIRE(rows > 0 && D > 0 && groups > 0 && rows % groups == 0, QB_ERR_INVALID_ARG, "ada_gate_residual: bad sizes");
  QB_REQUIRE(D % 8 == 0, QB_ERR_ALIGN, "ada_gate_residual: D must be a multiple of 8");
  QB_REQUIRE(aligned16(X) && aligned16(Y) && aligned16(gate) && aligned16(out), QB_ERR_ALIGN, "ada_gate_residual: pointers must be 16-byte aligned");
  gate_residual_kernel<<<blocks_for(static_cast<size_t>(rows) * D), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint16_t*>(X), static_cast<const uint16_t*>(Y), static_cast<const uint16_t*>(gate), static_cast<uint16_t*>(out),
      rows, D, rows / groups);
  return check_launch("ada_gate_residual");
}

int32_t qb_silu(const void* X, void* out, void* out_q, size_t n, void* stream) {
  QB_REQUIRE(X && (out || out_q), QB_ERR_INVALID_ARG, "silu: NULL pointer");
  QB_REQUIRE(aligned16(X) && aligned16(out) && aligned16(out_q), QB_ERR_ALIGN, "silu: pointers must be 16-byte aligned");
  if (n == 0) return QB_OK;
  silu_kernel<<<blocks_for(n), 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint16_t*>(X), static_cast<uint16_t*>(out),
                                                                            static_cast<uint8_t*>(out_q), n);
  return check_launch("silu");
}

int32_t qb_rmsnorm(const void* X, void* out, int32_t rows, int32_t D, float eps, void* stream) {
  QB_REQUIRE(X && out, QB_ERR_INVALID_ARG, "rmsnorm: NULL pointer");
  QB_REQUIRE(rows > 0 && D > 0, QB_ERR_INVALID_ARG, "rmsnorm: rows %d, D %d", rows, D);
  QB_REQUIRE(D % 8 == 0 && D <= 8192, QB_ERR_UNSUPPORTED, "rmsnorm: D = %d must be a multiple of 8 and at most 8192", D);
  QB_REQUIRE(eps > 0.f, QB_ERR_INVALID_ARG, "rmsnorm: eps must be positive");
  QB_REQUIRE(aligned16(X) && aligned16(out), QB_ERR_ALIGN, "rmsnorm: pointers must be 16-byte aligned");
  return launch_dep("rmsnorm", rmsnorm_kernel<256>, dim3(rows), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(X), static_cast<uint16_t*>(out), D, eps);
}

int32_t qb_add(const void* X, const void* Y, void* out, size_t n, void* stream) {
  QB_REQUIRE(X && Y && out, QB_ERR_INVALID_ARG, "add: NULL pointer");
  QB_REQUIRE(aligned16(X) && aligned16(Y) && aligned16(out), QB_ERR_ALIGN, "add: pointers must be 16-byte aligned");
  if (n == 0) return QB_OK;
  return launch_dep("add", add_kernel, dim3(blocks_for(n)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(X), static_cast<const uint16_t*>(Y), static_cast<uint16_t*>(out), n);
}

int32_t qb_euler_step(const void* X, const void* V, const float* dsig, void* out, size_t n, void* stream) {
  QB_REQUIRE(X && V && dsig && out, QB_ERR_INVALID_ARG, "euler_step: NULL pointer");
  QB_REQUIRE(aligned16(X) && aligned16(V) && aligned16(out), QB_ERR_ALIGN, "euler_step: pointers must be 16-byte aligned");
  if (n == 0) return QB_OK;
  return launch_dep("euler_step", euler_kernel, dim3(blocks_for(n)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(X), static_cast<const uint16_t*>(V), dsig, static_cast<uint16_t*>(out), n);
}

int32_t qb_dequantize_e4m3(const void* X, void* out, size_t n, void* stream) {
  QB_REQUIRE(n == 0 || (X && out), QB_ERR_INVALID_ARG, "dequantize_e4m3: NULL pointer");
  QB_REQUIRE(aligned16(X) && aligned16(out), QB_ERR_ALIGN, "dequantize_e4m3: pointers must be 16-byte aligned");
  if (n == 0) return QB_OK;
  const size_t blocks = (n + 256 * 16 - 1) / (256 * 16);
  return launch_dep("dequantize_e4m3", dequantize_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint8_t*>(X), static_cast<uint16_t*>(out), n);
}

int32_t qb_moe_route(const void* logits, float* weights, int32_t M, int32_t E, int32_t top_k, void* stream) {
  QB_REQUIRE(logits && weights, QB_ERR_INVALID_ARG, "moe_route: NULL pointer");
  QB_REQUIRE(M > 0 && E > 0 && E <= kMoeMaxExperts && top_k > 0 && top_k <= E, QB_ERR_INVALID_ARG, "moe_route: M %d, E %d (at most %d), top_k %d", M, E,
             kMoeMaxExperts, top_k);
  return launch_dep("moe_route", moe_route_kernel, dim3((M + 127) / 128), dim3(128), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(logits), weights, M, E, top_k);
}

int32_t qb_moe_combine(const float* partials, const float* weights, void* out, int32_t M, int32_t D, int32_t E, void* stream) {
  QB_REQUIRE(partials && weights && out, QB_ERR_INVALID_ARG, "moe_combine: NULL pointer");
  QB_REQUIRE(M > 0 && D > 0 && D % 4 == 0 && E > 0, QB_ERR_INVALID_ARG, "moe_combine: M %d, D %d (a multiple of 4), E %d", M, D, E);
  QB_REQUIRE(aligned16(partials) && aligned16(out), QB_ERR_ALIGN, "moe_combine: pointers must be 16-byte aligned");
  return launch_dep("moe_combine", moe_combine_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), partials, weights,
                    static_cast<uint16_t*>(out), M, D, E);
}

size_t qb_moe_slots(int32_t M, int32_t E, int32_t top_k) {
  if (M <= 0 || E <= 0 || top_k <= 0 || top_k > E) return 0;
  // every expert's run is padded to whole tiles: at most E * (tile - 1) padding rows
  const size_t worst = static_cast<size_t>(M) * top_k + static_cast<size_t>(E) * (kMoeTile - 1);
  return (worst + kMoeTile - 1) / kMoeTile * kMoeTile;
}

int32_t qb_moe_route_slots(const void* logits, int32_t* slot_token, float* slot_weight, int32_t* tile_expert, int32_t* token_slot,
                           int32_t* counts, int32_t M, int32_t E, int32_t top_k, void* stream) {
  QB_REQUIRE(logits && slot_token && slot_weight && tile_expert && token_slot, QB_ERR_INVALID_ARG, "moe_route_slots: NULL pointer");
  QB_REQUIRE(M > 0 && E > 0 && E <= kMoeMaxExperts && top_k > 0 && top_k <= E, QB_ERR_INVALID_ARG, "moe_route_slots: M %d, E %d (at most %d), top_k %d", M, E,
             kMoeMaxExperts, top_k);
  const int n_slots = static_cast<int>(qb_moe_slots(M, E, top_k));
  return launch_dep("moe_route_slots", moe_route_slots_kernel, dim3(1), dim3(kMoeRouteThreads), 0, static_cast<cudaStream_t>(stream),
                    static_cast<const uint16_t*>(logits), slot_token, slot_weight, tile_expert, token_slot, counts, M, E, top_k, n_slots);
}

int32_t qb_moe_gather(const void* X, const int32_t* slot_token, void* out, int32_t n_slots, int32_t row_bytes, void* stream) {
  QB_REQUIRE(X && slot_token && out, QB_ERR_INVALID_ARG, "moe_gather: NULL pointer");
  QB_REQUIRE(n_slots > 0 && row_bytes > 0 && row_bytes % 16 == 0, QB_ERR_INVALID_ARG, "moe_gather: %d slots of %d bytes (a multiple of 16)", n_slots, row_bytes);
  QB_REQUIRE(aligned16(X) && aligned16(out), QB_ERR_ALIGN, "moe_gather: pointers must be 16-byte aligned");
  return launch_dep("moe_gather", moe_gather_kernel, dim3(n_slots), dim3(256), 0, static_cast<cudaStream_t>(stream), static_cast<const uint8_t*>(X),
                    slot_token, static_cast<uint8_t*>(out), row_bytes);
}

int32_t qb_moe_reduce(const float* partials, const float* slot_weight, const int32_t* token_slot, void* out, int32_t M, int32_t D, int32_t top_k,
                      void* stream) {
  QB_REQUIRE(partials && slot_weight && token_slot && out, QB_ERR_INVALID_ARG, "moe_reduce: NULL pointer");
  QB_REQUIRE(M > 0 && D > 0 && D % 4 == 0 && top_k > 0 && top_k <= kMoeMaxExperts, QB_ERR_INVALID_ARG,
             "moe_reduce: M %d, D %d (a multiple of 4), top_k %d (at most %d)", M, D, top_k, kMoeMaxExperts);
  QB_REQUIRE(aligned16(partials) && aligned16(out), QB_ERR_ALIGN, "moe_reduce: pointers must be 16-byte aligned");
  return launch_dep("moe_reduce", moe_reduce_kernel, dim3(M), dim3(256), 0, static_cast<cudaStream_t>(stream), partials, slot_weight, token_slot,
                    static_cast<uint16_t*>(out), D, top_k);
}

int32_t qb_randn(const uint32_t* counter, void* out, size_t n, int32_t out_dtype, uint32_t counter_stride, uint32_t seed0, uint32_t seed1,
                 void* stream) {
  QB_REQUIRE(counter && out, QB_ERR_INVALID_ARG, "randn: NULL pointer");
  QB_REQUIRE(out_dtype == QB_BF16 || out_dtype == QB_F32, QB_ERR_INVALID_ARG, "randn: out_dtype %d (bf16 or f32)", out_dtype);
  QB_REQUIRE(n <= (static_cast<size_t>(1) << 33), QB_ERR_INVALID_ARG, "randn: %zu samples exceed one 32-bit counter range", n);
  if (n == 0) return QB_OK;
  const dim3 grid(static_cast<unsigned>((n + kRandnPerBlock - 1) / kRandnPerBlock));
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (out_dtype == QB_F32)
    return launch_dep("randn", randn_kernel<float>, grid, dim3(kRandnThreads), 0, st, counter, static_cast<float*>(out), n, counter_stride, seed0, seed1);
  return launch_dep("randn", randn_kernel<uint16_t>, grid, dim3(kRandnThreads), 0, st, counter, static_cast<uint16_t*>(out), n, counter_stride, seed0,
                    seed1);
}

int32_t qb_increment(int32_t* counter, void* stream) {
  QB_REQUIRE(counter != nullptr, QB_ERR_INVALID_ARG, "increment: NULL pointer");
  return launch_dep("increment", increment_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream), counter);
}

static int32_t check_patch_geometry(const char* who, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw, int32_t d_model) {
  QB_REQUIRE(C > 0 && H > 0 && Wd > 0 && ph > 0 && pw > 0 && d_model > 0, QB_ERR_INVALID_ARG, "%s: sizes must be positive", who);
  QB_REQUIRE(H % ph == 0 && Wd % pw == 0, QB_ERR_INVALID_ARG, "%s: H=%d W=%d not divisible by patch (%d,%d)", who, H, Wd, ph, pw);
  QB_REQUIRE((C * ph * pw) % 8 == 0 && d_model % 8 == 0, QB_ERR_ALIGN, "%s: C*ph*pw and d_model must be multiples of 8", who);
  return QB_OK;
}

int32_t qb_patchify(const void* X, const void* W, void* out, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw,
                    int32_t d_model, void* stream) {
  QB_REQUIRE(X && W && out, QB_ERR_INVALID_ARG, "patchify: NULL pointer");
  int32_t rc = check_patch_geometry("patchify", C, H, Wd, ph, pw, d_model);
  if (rc != QB_OK) return rc;
  QB_REQUIRE(aligned16(W), QB_ERR_ALIGN, "patchify: W must be 16-byte aligned");
  const int tokens = (H / ph) * (Wd / pw);
  const int K = C * ph * pw;
  const size_t smem = static_cast<size_t>(kPatchTok) * K * sizeof(float);
  QB_REQUIRE(smem <= 48 * 1024, QB_ERR_UNSUPPORTED, "patchify: C*ph*pw = %d too large", K);
  dim3 grid((tokens + kPatchTok - 1) / kPatchTok, (d_model + 255) / 256);
  patchify_kernel<<<grid, 256, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint16_t*>(X), static_cast<const uint16_t*>(W),
                                                                           static_cast<uint16_t*>(out), C, H, Wd, ph, pw, d_model, tokens);
  return check_launch("patchify");
}

int32_t qb_patch_gather(const void* latent, void* tokens_out, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw, void* stream) {
  QB_REQUIRE(latent && tokens_out, QB_ERR_INVALID_ARG, "patch_gather: NULL pointer");
  QB_REQUIRE(C > 0 && H > 0 && Wd > 0 && ph > 0 && pw > 0 && H % ph == 0 && Wd % pw == 0, QB_ERR_INVALID_ARG, "patch_gather: bad geometry");
  const int tokens = (H / ph) * (Wd / pw);
  const size_t n = static_cast<size_t>(tokens) * C * ph * pw;
  return launch_dep("patch_gather", patch_move_kernel<true>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(latent), static_cast<uint16_t*>(tokens_out), C, H, Wd, ph,
                    pw, tokens);
}

int32_t qb_patch_scatter(const void* tokens_in, void* latent_out, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw, void* stream) {
  QB_REQUIRE(tokens_in && latent_out, QB_ERR_INVALID_ARG, "patch_scatter: NULL pointer");
  QB_REQUIRE(C > 0 && H > 0 && Wd > 0 && ph > 0 && pw > 0 && H % ph == 0 && Wd % pw == 0, QB_ERR_INVALID_ARG, "patch_scatter: bad geometry");
  const int tokens = (H / ph) * (Wd / pw);
  const size_t n = static_cast<size_t>(tokens) * C * ph * pw;
  return launch_dep("patch_scatter", patch_move_kernel<false>, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0,
                    static_cast<cudaStream_t>(stream), static_cast<const uint16_t*>(tokens_in), static_cast<uint16_t*>(latent_out), C, H, Wd,
                    ph, pw, tokens);
}

int32_t qb_unpatchify(const void* X, const void* W, const void* bias, void* out, int32_t C, int32_t H, int32_t Wd, int32_t ph,
                      int32_t pw, int32_t d_model, void* stream) {
  QB_REQUIRE(X && W && out, QB_ERR_INVALID_ARG, "unpatchify: NULL pointer");
  int32_t rc = check_patch_geometry("unpatchify", C, H, Wd, ph, pw, d_model);
  if (rc != QB_OK) return rc;
  QB_REQUIRE(aligned16(X) && aligned16(W), QB_ERR_ALIGN, "unpatchify: X and W must be 16-byte aligned");
  const int tokens = (H / ph) * (Wd / pw);
  const int Nout = C * ph * pw;
  const size_t smem = static_cast<size_t>(kPatchTok) * d_model * sizeof(float);
  QB_REQUIRE(smem <= 96 * 1024, QB_ERR_UNSUPPORTED, "unpatchify: d_model = %d too large", d_model);
  QB_CUDA_OK(cudaFuncSetAttribute(unpatchify_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
  dim3 grid((tokens + kPatchTok - 1) / kPatchTok, (Nout + 127) / 128);
  unpatchify_kernel<<<grid, 128, smem, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint16_t*>(X), static_cast<const uint16_t*>(W),
                                                                             static_cast<const uint16_t*>(bias), static_cast<uint16_t*>(out),
                                                                             C, H, Wd, ph, pw, d_model, tokens);
  return check_launch("unpatchify");
}

}  // extern "C"
