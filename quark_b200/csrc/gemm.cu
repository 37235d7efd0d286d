// C[M,N] = epilogue(A[M,K] . B[N,K]^T) on the sm_100a tensor cores.
//
// One CTA computes one 128 x BN output tile over one K slice.  Warp 0 feeds a ring of
// shared-memory stages with TMA (128-byte swizzle), one thread of warp 1 issues
// tcgen05.mma into a TMEM accumulator, warps 2-9 read the accumulator back (one row per thread, two
// warps per TMEM lane quarter sharing each row's columns) and run the epilogue: 320 threads per CTA.  bf16 operands use kind::f16 (K = 16 per instruction), e4m3
// operands kind::f8f6f4 (K = 32); both move 128 bytes of K per stage row, so the two paths share
// every address computation.
//
// K can be split over `splits` CTAs per tile: each writes its f32 partial tile to the
// workspace, takes a ticket on the tile's counter, and the CTA that draws the last ticket adds
// the partials in slice order (so the sum does not depend on which CTA came last), applies the
// epilogue and stores.  No CTA ever waits for another.
#include <atomic>

#include <cuda.h>

#include "common.cuh"
#include "rope.cuh"
#include "sm100.cuh"

namespace qb {

constexpr int kBM = 128;          // rows of A per tile = TMEM lanes
constexpr int kRowBytes = 128;    // bytes of K per stage row = one swizzle atom
constexpr int kGemmThreads = 320; // 10 warps: TMA, MMA, 2 x 4 epilogue (two warps per TMEM lane quarter)
constexpr int kSmemBudget = 200 * 1024;

#ifdef QB_GEMM_TRACE
__device__ long long g_gemm_trace[148 * 4][8];  // [CTA][point]: globaltimer ns
__device__ __forceinline__ long long gtime() { long long t; asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t)); return t; }
#define QB_GT(pt) do { const int cta_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x; if (cta_ < 148 * 4) g_gemm_trace[cta_][pt] = gtime(); } while (0)
#else
#define QB_GT(pt) do { } while (0)
#endif

// What the QKV projection's fused epilogue needs beyond the GEMM: per-head RMS norm of Q and K, value
// residual on V, RoPE(K) and the KV-cache append happen on the accumulator tile, before anything is
// written (the stand-alone kernels are in qkv_post.cu and kv.cu; results are bit-identical to them).
struct QkvTail {
  const uint16_t* qkv_first;  // may be null: no value residual
  const float* lamb;
  const int32_t* frame_t;
  const int32_t* frozen;
  void* K_cache;
  void* Vt_cache;
  int32_t* segments;
  int32_t* n_segments;
  const float* rope_xy;
  const float* k_scale;  // optional per-KV-head cache scales (see qb_kv_params)
  const float* v_scale;
  int n_q_heads, n_kv_heads, tpf, nb, pd, max_segments, kv_fp8;
  // Quilt: the cache keeps tokens qoff, qoff + quilt, ... of the frame (tpf / quilt of them); slots, capacity and the
  // segment table are those of a frame of tpf / quilt tokens (src/quark/kernels/kv_cache_update/reference.py:201-207)
  int quilt, qoff;
  float eps;
};

struct GemmArgs {
  int M, N, K;
  int kb_total, kb_per_split, splits;
  int cluster;  // K slices are the CTAs of one thread-block cluster and are summed through distributed shared memory
  int b_const;  // no kernel still in flight writes B (weights): its first tiles are fetched ahead of the grid dependency
  int c_dtype, activation, rows_per_gate;
  const float* a_scale;
  const float* w_scale;
  const uint16_t* bias;
  const uint16_t* gate;
  const uint16_t* residual;
  void* C;
  float* partials;
  int* counters;
  unsigned int* status;
  int qkv_mode;  // the fused QKV epilogue below replaces the plain one (128-column tiles only)
  QkvTail qkv;
  // Row-parallel GEMM of a tensor-parallel rank: row m of the bf16 partial goes to the rank that owns that row in the
  // cross-GPU reduction (m / tp_rpo), into that rank's staging area for partials from this rank (peer-mapped memory,
  // plain stores over NVLink): tp_dst[owner] + (m % tp_rpo) * N.  tp_world == 0: the ordinary output C.
  int tp_world, tp_rpo;
  uint16_t* tp_dst[8];
  // Grouped GEMM (mixture of experts): the 128-row tile i of A belongs to expert tile_expert[i] and is multiplied with
  // rows [expert * N, expert * N + N) of B; a tile with expert -1 is skipped.  NULL: the ordinary GEMM.
  const int* tile_expert;
};

template <int BN>
struct GemmSmem {
  static constexpr int kStageBytes = kBM * kRowBytes + BN * kRowBytes;
  static constexpr int kStages = (kSmemBudget / kStageBytes) > 8 ? 8 : (kSmemBudget / kStageBytes);
  static constexpr int kBarOffset = kStages * kStageBytes;
  static constexpr int kColOffset = kBarOffset + 256;            // per-column scale, bias, gate of this tile as f32
  static constexpr int kTotal = kColOffset + 3 * BN * 4 + 1024;  // + alignment slack
};

// Applies the epilogue to 8 consecutive columns of one row and stores them.
__device__ __forceinline__ void epilogue_store8(const GemmArgs& g, float (&v)[8], int m, int n) {
  if (g.a_scale != nullptr || g.w_scale != nullptr) {
    const float sa = g.a_scale ? *g.a_scale : 1.0f;
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] *= g.w_scale ? sa * __ldg(g.w_scale + n + j) : sa;
  }
  if (g.bias != nullptr) {
    const uint4 b = *reinterpret_cast<const uint4*>(g.bias + n);  // may be the output of the kernel before (MLPFusion)
    const uint32_t w[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] += bf16lo(w[j]);
      v[2 * j + 1] += bf16hi(w[j]);
    }
  }
  if (g.activation == 1) {
#pragma unroll
    for (int j = 0; j < 8; ++j) v[j] = silu_fast(v[j]);
  }
  if (g.gate != nullptr) {
    const size_t grow = static_cast<size_t>(m / g.rows_per_gate) * g.N;
    const uint4 gt = *reinterpret_cast<const uint4*>(g.gate + grow + n);
    const uint4 rs = *reinterpret_cast<const uint4*>(g.residual + static_cast<size_t>(m) * g.N + n);
    const uint32_t gw[4] = {gt.x, gt.y, gt.z, gt.w};
    const uint32_t rw[4] = {rs.x, rs.y, rs.z, rs.w};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      v[2 * j] = __fadd_rn(bf16lo(rw[j]), __fmul_rn(bf16lo(gw[j]), v[2 * j]));
      v[2 * j + 1] = __fadd_rn(bf16hi(rw[j]), __fmul_rn(bf16hi(gw[j]), v[2 * j + 1]));
    }
  }
  const size_t off = static_cast<size_t>(m) * g.N + n;
  if (g.c_dtype == QB_BF16) {
    uint4 o;
    o.x = pack_bf16x2(v[0], v[1]);
    o.y = pack_bf16x2(v[2], v[3]);
    o.z = pack_bf16x2(v[4], v[5]);
    o.w = pack_bf16x2(v[6], v[7]);
    *reinterpret_cast<uint4*>(static_cast<uint16_t*>(g.C) + off) = o;
  } else if (g.c_dtype == QB_E4M3) {
    uint2 o;
    o.x = pack_e4m3x4(v[0], v[1], v[2], v[3]);
    o.y = pack_e4m3x4(v[4], v[5], v[6], v[7]);
    *reinterpret_cast<uint2*>(static_cast<uint8_t*>(g.C) + off) = o;
  } else {
    float4* dst = reinterpret_cast<float4*>(static_cast<float*>(g.C) + off);
    dst[0] = make_float4(v[0], v[1], v[2], v[3]);
    dst[1] = make_float4(v[4], v[5], v[6], v[7]);
  }
}

// Thread-block cluster helpers: hardware barrier over all threads of the cluster, and loads from
// the shared memory of another CTA of the cluster.
__device__ __forceinline__ void cluster_sync() {
  asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t map_to_cta(uint32_t smem_addr, int cta_rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(cta_rank));
  return r;
}
__device__ __forceinline__ float4 ld_dsmem_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}

// ---------------------------------------------------------------- fused epilogue of the QKV projection
// Tile = 128 tokens x 2 heads (128 columns).  Epilogue warp w owns the 32 tokens of TMEM lane quarter
// w % 4 and head (w - 2) / 4 of the tile, so every thread holds one whole head of one token: the head's
// RMS norm, the value residual and the K rotation need no exchange between threads.  Arithmetic, rounding
// points and summation order are those of qkv_post.cu (and through it of head_rmsnorm, value_residual_packed
// and kv_cache_update), so the bytes written are the same.  V is transposed through the idle stage memory.
constexpr int kQkvVPitch = 72;  // 16-bit words per token row of the V staging tile

template <bool kCacheFp8>
__device__ __forceinline__ void qkv_tail_epilogue(const GemmArgs& g, uint8_t* smem, float* tm, uint64_t* acc_bar, volatile int* abort_flag,
                                                  uint32_t tmem_base, int warp, int lane, int m0, int n0) {
  constexpr int kEs = kCacheFp8 ? 1 : 2;
  const QkvTail& q = g.qkv;
  const int half = (warp - 2) >> 2, lane_grp = warp & 3;
  const int row = lane_grp * 32 + lane;
  const int t = m0 + row;  // token
  const bool valid = t < g.M;
  const int et = threadIdx.x - 64;  // 0 .. 255
  const int col0 = n0 + half * 64;  // first column of this thread's head
  const int k_off = q.n_q_heads * 64, v_off = (q.n_q_heads + q.n_kv_heads) * 64;
  const int kind = col0 < k_off ? 0 : col0 < v_off ? 1 : 2;  // Q, K or V head (uniform over the warp)
  const bool in_n = col0 < g.N;
  const int ft = *after_wait(q.frame_t);  // written on the device: ordinary loads, after the grid dependency
  const int frozen = *after_wait(q.frozen);
  const int tpf_c = q.tpf / q.quilt;  // tokens of a frame that the cache keeps
  const int L = q.nb * tpf_c;
  const int cap = L + tpf_c;
  // this thread's token in the cache: kept iff it is one of the quilt's residue class
  const bool kept = (t - q.qoff) >= 0 && (t - q.qoff) % q.quilt == 0;
  const int tc = (t - q.qoff) / q.quilt;
  const int bucket = (ft + q.pd - 1) / q.pd;
  const int slot = bucket % q.nb;
  const bool is_write = (ft % q.pd) == 0;
  const bool ring = is_write && frozen == 0;

  if (et < 8) temporal_cos_sin(ft, et, tm);
  if (blockIdx.x == 0 && blockIdx.y == 0 && et == 32) {  // segment table: one thread of the grid
    int sg[6] = {0, 0, 0, 0, 0, 0};
    int n;
    if (is_write && bucket >= q.nb) {
      sg[1] = slot * tpf_c;
      sg[2] = (slot + 1) * tpf_c;
      sg[3] = (q.nb - slot - 1) * tpf_c;
      sg[4] = L;
      sg[5] = tpf_c;
      n = 3;
    } else {
      sg[1] = min(bucket, q.nb) * tpf_c;
      sg[2] = L;
      sg[3] = tpf_c;
      n = 2;
    }
#pragma unroll
    for (int i = 0; i < 6; ++i)
      if (i < 2 * q.max_segments) q.segments[i] = sg[i];
    for (int i = 6; i < 2 * q.max_segments; ++i) q.segments[i] = 0;
    q.n_segments[0] = n;
  }
  // while the main loop runs: what this thread's head needs from global memory
  float xy[16];
  uint32_t vf[32];
  const bool mix = kind == 2 && q.qkv_first != nullptr;
  const float lam = mix ? *q.lamb : 0.f;
  if (kind == 1 && valid && in_n) {
    const float4* rp = reinterpret_cast<const float4*>(q.rope_xy + static_cast<size_t>(t) * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(rp + i);
      xy[4 * i] = v.x; xy[4 * i + 1] = v.y; xy[4 * i + 2] = v.z; xy[4 * i + 3] = v.w;
    }
  }
  if (mix && valid && in_n) {
    const uint4* fp = reinterpret_cast<const uint4*>(q.qkv_first + static_cast<size_t>(t) * g.N + col0);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const uint4 v = fp[i];  // the first block's QKV, written earlier in this pass
      vf[4 * i] = v.x; vf[4 * i + 1] = v.y; vf[4 * i + 2] = v.z; vf[4 * i + 3] = v.w;
    }
  }
  asm volatile("bar.sync 2, 256;" ::: "memory");  // temporal cos / sin visible

  const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc_bar), 0, abort_flag, g.status, QB_DEV_WAIT_TIMEOUT_GEMM));
  tc_fence_after();
  uint16_t* vt = reinterpret_cast<uint16_t*>(smem);  // [2 heads][128 tokens][kQkvVPitch], over the stage memory (idle now)
  if (ok) {
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16) + half * 64;
    uint32_t r0[32], r1[32];
    tmem_ld32(taddr, r0);
    tmem_ld32(taddr + 32, r1);
    tmem_wait_ld_into(r0);
    tmem_loaded(r1);
    // the projection's output as the unfused path would store and re-read it: scaled (acc * (a_scale * w_scale[n]),
    // as the plain epilogue does) and rounded to bf16
    float f[64];
    if (g.a_scale != nullptr || g.w_scale != nullptr) {
      const float sa = g.a_scale ? *g.a_scale : 1.0f;
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float c0 = (g.w_scale && in_n) ? sa * __ldg(g.w_scale + col0 + j) : sa;
        const float c1 = (g.w_scale && in_n) ? sa * __ldg(g.w_scale + col0 + 32 + j) : sa;
        r0[j] = __float_as_uint(__uint_as_float(r0[j]) * c0);
        r1[j] = __float_as_uint(__uint_as_float(r1[j]) * c1);
      }
    }
#pragma unroll
    for (int j = 0; j < 32; ++j) {
      f[j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r0[j])));
      f[32 + j] = __bfloat162float(__float2bfloat16_rn(__uint_as_float(r1[j])));
    }
    uint32_t o[32];  // the head as it goes to qkv_out: 64 bf16
    if (kind < 2) {
      // sum of squares in the order of the 4-lanes-per-head kernel: per 16 elements 8 + 8, then pairs of sixteenths
      float sq[4];
#pragma unroll
      for (int l = 0; l < 4; ++l) {
        float sa = 0.f, sb = 0.f;
#pragma unroll
        for (int j = 0; j < 8; ++j) sa += f[16 * l + j] * f[16 * l + j];
#pragma unroll
        for (int j = 8; j < 16; ++j) sb += f[16 * l + j] * f[16 * l + j];
        sq[l] = sa + sb;
      }
      const float ss = (sq[0] + sq[1]) + (sq[2] + sq[3]);
      const float inv = 1.0f / sqrtf(ss * (1.0f / 64.0f) + q.eps);
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = pack_bf16x2(__fmul_rn(f[2 * j], inv), __fmul_rn(f[2 * j + 1], inv));
    } else if (mix) {
#pragma unroll
      for (int j = 0; j < 32; ++j) {
        const float c0 = f[2 * j], c1 = f[2 * j + 1];
        o[j] = pack_bf16x2(__fadd_rn(c0, __fmul_rn(lam, __fsub_rn(bf16lo(vf[j]), c0))),
                           __fadd_rn(c1, __fmul_rn(lam, __fsub_rn(bf16hi(vf[j]), c1))));
      }
    } else {
#pragma unroll
      for (int j = 0; j < 32; ++j) o[j] = pack_bf16x2(f[2 * j], f[2 * j + 1]);
    }
    if (valid && in_n) {
      uint16_t* dst = static_cast<uint16_t*>(g.C) + static_cast<size_t>(t) * g.N + col0;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        const uint32_t w[8] = {o[8 * h], o[8 * h + 1], o[8 * h + 2], o[8 * h + 3], o[8 * h + 4], o[8 * h + 5], o[8 * h + 6], o[8 * h + 7]};
        st_global_v8(dst + 16 * h, w);
      }
    }
    if (kind == 1 && valid && in_n && kept) {
      // rotate what the stand-alone append would read back (the bf16-rounded normalised K): y0 = pairs' first
      // outputs, y1 = their second outputs; a cache row is y0[0..31] followed by y1[0..31]
      const int head = (col0 - k_off) >> 6;
      const float inv_k = q.k_scale != nullptr ? __fdiv_rn(1.0f, __ldg(q.k_scale + head)) : 1.0f;  // * 1 changes no bit
      float y0[32], y1[32];
#pragma unroll
      for (int pr = 0; pr < 32; ++pr) {
        float c, sn;
        pair_cos_sin(pr, xy, tm, c, sn);
        const float x0 = bf16lo(o[pr]), x1 = bf16hi(o[pr]);
        y0[pr] = __fmul_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn)), inv_k);
        y1[pr] = __fmul_rn(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, sn)), inv_k);
      }
      uint8_t* kc = static_cast<uint8_t*>(q.K_cache);
      const size_t row_bytes = 64 * kEs;
      uint8_t* tail = kc + (static_cast<size_t>(head) * cap + L + tc) * row_bytes;
      uint8_t* rr = kc + (static_cast<size_t>(head) * cap + static_cast<size_t>(slot) * tpf_c + tc) * row_bytes;
      if (kCacheFp8) {
        uint32_t w0[8], w1[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          w0[j] = pack_e4m3x4(y0[4 * j], y0[4 * j + 1], y0[4 * j + 2], y0[4 * j + 3]);
          w1[j] = pack_e4m3x4(y1[4 * j], y1[4 * j + 1], y1[4 * j + 2], y1[4 * j + 3]);
        }
        st_global_v8(tail, w0);
        st_global_v8(tail + 32, w1);
        if (ring) {
          st_global_v8(rr, w0);
          st_global_v8(rr + 32, w1);
        }
      } else {
#pragma unroll
        for (int h = 0; h < 4; ++h) {
          uint32_t w[8];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const int e = 16 * (h & 1) + 2 * j;  // 16 values per 32-byte store; h < 2: y0, h >= 2: y1
            w[j] = h < 2 ? pack_bf16x2(y0[e], y0[e + 1]) : pack_bf16x2(y1[e], y1[e + 1]);
          }
          st_global_v8(tail + 32 * h, w);
          if (ring) st_global_v8(rr + 32 * h, w);
        }
      }
    }
    if (kind == 2) {  // the mixed V head of this token into the staging tile, 16-byte rows of 8 channels
      uint16_t* vrow = vt + (half * 128 + row) * kQkvVPitch;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        *reinterpret_cast<uint4*>(vrow + c8 * 8) = make_uint4(o[4 * c8], o[4 * c8 + 1], o[4 * c8 + 2], o[4 * c8 + 3]);
    }
  }
  asm volatile("bar.sync 2, 256;" ::: "memory");  // V staging complete
  if (ok) {
    // transposed 16-byte stores: one channel x (8 | 16) consecutive cached tokens each, for the V heads of this tile.
    // The tile's cached tokens are its rows qoff, qoff + quilt, ... (m0 is a multiple of the quilt factor).
    constexpr int kTokPerVec = 16 / kEs;
    const int cached_rows = 128 / q.quilt;
    const int vec_per_ch = cached_rows / kTokPerVec;
    uint8_t* vc = static_cast<uint8_t*>(q.Vt_cache);
#pragma unroll 1
    for (int hh = 0; hh < 2; ++hh) {
      const int hcol = n0 + hh * 64;
      if (hcol < v_off || hcol >= g.N) continue;
      const int head = (hcol - v_off) >> 6;
      const float inv_v = q.v_scale != nullptr ? __fdiv_rn(1.0f, __ldg(q.v_scale + head)) : 1.0f;
      const uint16_t* src = vt + hh * 128 * kQkvVPitch;
      for (int v = et; v < 64 * vec_per_ch; v += 256) {
        const int d = v / vec_per_ch, j = v % vec_per_ch;
        const int c1 = j * kTokPerVec;                  // first cached token of the vector, inside the tile
        const int c_abs = m0 / q.quilt + c1;            // ... and inside the frame's cached tokens
        if (c_abs + kTokPerVec > tpf_c) continue;
        auto sv = [&](int i) { return src[(q.qoff + (c1 + i) * q.quilt) * kQkvVPitch + d]; };
        uint32_t w[4];
        if (kCacheFp8) {
#pragma unroll
          for (int i = 0; i < 4; ++i)
            w[i] = pack_e4m3x4(__fmul_rn(bf16_bits_to_f32(sv(4 * i)), inv_v), __fmul_rn(bf16_bits_to_f32(sv(4 * i + 1)), inv_v),
                               __fmul_rn(bf16_bits_to_f32(sv(4 * i + 2)), inv_v), __fmul_rn(bf16_bits_to_f32(sv(4 * i + 3)), inv_v));
        } else {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint16_t lo = sv(2 * i), hi = sv(2 * i + 1);
            w[i] = q.v_scale != nullptr ? pack_bf16x2(__fmul_rn(bf16_bits_to_f32(lo), inv_v), __fmul_rn(bf16_bits_to_f32(hi), inv_v))
                                        : static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
          }
        }
        const uint4 ov = make_uint4(w[0], w[1], w[2], w[3]);
        const size_t ch = (static_cast<size_t>(head) * 64 + d) * cap;
        *reinterpret_cast<uint4*>(vc + (ch + L + c_abs) * kEs) = ov;
        if (ring) *reinterpret_cast<uint4*>(vc + (ch + static_cast<size_t>(slot) * tpf_c + c_abs) * kEs) = ov;
      }
    }
  }
}

template <int BN, bool FP8>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, const GemmArgs g) {
  using L = GemmSmem<BN>;
  constexpr int kStages = L::kStages;
  constexpr int kKElems = FP8 ? 128 : 64;  // elements of K per stage
  constexpr uint32_t kTmemCols = BN < 32 ? 32 : BN;
  constexpr uint32_t kIdesc = FP8 ? umma_idesc(0, 0, kBM, BN) : umma_idesc(1, 1, kBM, BN);
  constexpr int kStgPitch = BN + 4;  // f32 words per staged row: the pad spreads a column of rows over the banks
  static_assert(kBM * kStgPitch * 4 <= L::kStages * L::kStageBytes, "staging tile must fit in the stage memory");

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOffset);
  uint64_t* full_bar = bars;
  uint64_t* empty_bar = bars + kStages;
  uint64_t* acc_bar = bars + 2 * kStages;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * kStages + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* last_flag = abort_flag + 1;
  volatile int* drain_flag = abort_flag + 2;  // never set: lets the drain waits below run their own limit

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) QB_GT(0);
  int b_row0 = 0;  // first row of this tile's expert in B
  if (g.tile_expert != nullptr) {
    grid_dep_wait();  // the table is written by the routing kernel just before
    const int expert = g.tile_expert[blockIdx.y];
    if (expert < 0) return;  // a padding tile: nothing allocated yet, the whole CTA leaves
    b_row0 = expert * g.N;
  }
  const int n0 = blockIdx.x * BN;
  const int m0 = blockIdx.y * kBM;
  const int split = blockIdx.z;
  const int kb0 = split * g.kb_per_split;
  const int kb1 = min(kb0 + g.kb_per_split, g.kb_total);
  const int n_iter = kb1 - kb0;
  const bool clustered = g.cluster != 0 && g.splits > 1;
  const bool use_staging = clustered;  // a single slice goes straight from TMEM to global memory (measured faster)

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&full_bar[s]), 1);
      mbar_init(smem_u32(&empty_bar[s]), 1);
    }
    mbar_init(smem_u32(acc_bar), 1);
    *abort_flag = 0;
    *last_flag = 0;
    *drain_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  grid_dep_launch();  // set-up is done: the next kernel in the stream may begin its own
  if (threadIdx.x == 0) QB_GT(1);

  if (warp == 0) {
    // ---------------- TMA producer
    if (elect_one()) {
      // The weight tiles of the first stages do not depend on the kernels before this one, so they are
      // already on their way while those kernels finish; A follows once they have.
      const int ahead = g.b_const ? min(kStages, n_iter) : 0;
      for (int it = 0; it < ahead; ++it) {
        const uint32_t fb = smem_u32(&full_bar[it]);
        mbar_arrive_expect_tx(fb, L::kStageBytes);
        tma_load_2d(smem_u32(smem + it * L::kStageBytes + kBM * kRowBytes), &tmB, fb, (kb0 + it) * kKElems, b_row0 + n0);
      }
      grid_dep_wait();
      QB_GT(2);
      for (int it = 0; it < ahead; ++it)
        tma_load_2d(smem_u32(smem + it * L::kStageBytes), &tmA, smem_u32(&full_bar[it]), (kb0 + it) * kKElems, m0);
      int issued = ahead;
      for (int it = ahead; it < n_iter; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        if (!mbar_wait(smem_u32(&empty_bar[s]), ph ^ 1, abort_flag, g.status, QB_DEV_WAIT_TIMEOUT_GEMM)) break;
        const uint32_t fb = smem_u32(&full_bar[s]);
        mbar_arrive_expect_tx(fb, L::kStageBytes);
        uint8_t* a_s = smem + s * L::kStageBytes;
        tma_load_2d(smem_u32(a_s), &tmA, fb, (kb0 + it) * kKElems, m0);
        tma_load_2d(smem_u32(a_s + kBM * kRowBytes), &tmB, fb, (kb0 + it) * kKElems, b_row0 + n0);
        issued = it + 1;
      }
      if (*abort_flag) {
        // Giving up: let the copies already in flight land before this CTA's memory goes away.
        for (int it = max(0, issued - kStages); it < issued; ++it)
          mbar_wait(smem_u32(&full_bar[it % kStages]), (it / kStages) & 1, drain_flag, g.status, QB_DEV_WAIT_TIMEOUT_GEMM);
      } else {
        // Tail: the MMA warp's last stage releases arrive on barriers in this CTA's shared memory;
        // see them land before the CTA can exit.
        for (int it = max(0, n_iter - kStages); it < n_iter; ++it)
          if (!mbar_wait(smem_u32(&empty_bar[it % kStages]), (it / kStages) & 1, abort_flag, g.status, QB_DEV_WAIT_TIMEOUT_GEMM)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (elect_one()) {
      bool ok = true;
      for (int it = 0; it < n_iter && ok; ++it) {
        const int s = it % kStages;
        const uint32_t ph = (it / kStages) & 1;
        ok = mbar_wait(smem_u32(&full_bar[s]), ph, abort_flag, g.status, QB_DEV_WAIT_TIMEOUT_GEMM);
        if (!ok) break;
        if (it == 0) QB_GT(3);
        tc_fence_after();
        const uint32_t a_addr = smem_u32(smem + s * L::kStageBytes);
        const uint64_t a_desc = umma_desc_k_sw128(a_addr);
        const uint64_t b_desc = umma_desc_k_sw128(a_addr + kBM * kRowBytes);
#pragma unroll
        for (int k = 0; k < 4; ++k) {  // 4 x 32 bytes of K per stage row
          const uint32_t acc = (it > 0 || k > 0) ? 1u : 0u;
          if (FP8)
            umma_f8(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kIdesc, acc);
          else
            umma_f16(tmem_base, a_desc + 2 * k, b_desc + 2 * k, kIdesc, acc);
        }
        umma_commit(smem_u32(&empty_bar[s]));
      }
      umma_commit(smem_u32(acc_bar));
      QB_GT(4);
    }
  } else {
    // ---------------- epilogue, part 1: warp w may touch TMEM lanes 32 * (w % 4) .. + 31
    const int lane_grp = warp & 3;
    const int row = lane_grp * 32 + lane;
    const int m = m0 + row;
    grid_dep_wait();  // bias / gate / residual are read and C is written only after the earlier kernels are done
    bool qkv_done = false;
    if constexpr (BN == 128) {
      if (g.qkv_mode) {
        float* tm = reinterpret_cast<float*>(smem + L::kColOffset);
        if (g.qkv.kv_fp8)
          qkv_tail_epilogue<true>(g, smem, tm, acc_bar, abort_flag, tmem_base, warp, lane, m0, n0);
        else
          qkv_tail_epilogue<false>(g, smem, tm, acc_bar, abort_flag, tmem_base, warp, lane, m0, n0);
        qkv_done = true;
      }
    }
    // The fast epilogue needs whole 32-column chunks inside N, 32-byte aligned rows of C, and one gate row
    // for the whole tile; anything else takes the general path below.
    const int m_last = min(m0 + kBM, g.M) - 1;
    const bool fast = !qkv_done && g.splits == 1 && g.N % 32 == 0 && (reinterpret_cast<uintptr_t>(g.C) & 31u) == 0 &&
                      (g.gate == nullptr || m0 / g.rows_per_gate == m_last / g.rows_per_gate);
    // Two warps share each TMEM lane quarter (w and w + 4 see the same 32 rows): in the fast epilogue the
    // first takes the even 32-column chunks of the row, the second the odd ones.  The other epilogue paths
    // are run by the first four warps alone.
    const int half = (warp - 2) >> 2;
    constexpr int kMyChunks = BN / 64;  // 32-column chunks per warp
    constexpr int kResInRegs = BN <= 128 ? 1 : 0;
    uint32_t res[kResInRegs ? kMyChunks * 16 : 1];
    if (fast) {
      // while the main loop runs: per-column vectors of this tile to shared memory, this row's residual to registers
      float* col = reinterpret_cast<float*>(smem + L::kColOffset);
      const int et = threadIdx.x - 64;  // 0 .. 255
      const float sa = g.a_scale ? *g.a_scale : 1.0f;
      const size_t grow = g.gate ? static_cast<size_t>(m0 / g.rows_per_gate) * g.N : 0;
      for (int j = et; j < BN; j += 256) {
        const int n = n0 + j;
        const bool in = n < g.N;
        col[j] = (in && g.w_scale) ? sa * __ldg(g.w_scale + n) : sa;
        col[BN + j] = (in && g.bias) ? bf16_bits_to_f32(g.bias[n]) : 0.f;
        col[2 * BN + j] = (in && g.gate) ? bf16_bits_to_f32(g.gate[grow + n]) : 0.f;
      }
      if (kResInRegs && g.gate != nullptr && m < g.M) {
#pragma unroll
        for (int q = 0; q < kMyChunks * 4; ++q) {
          const int n = n0 + (2 * (q >> 2) + half) * 32 + (q & 3) * 8;  // chunk 2 * (q / 4) + half, 8 columns at a time
          uint4 x = make_uint4(0u, 0u, 0u, 0u);
          if (n < g.N) x = *reinterpret_cast<const uint4*>(g.residual + static_cast<size_t>(m) * g.N + n);
          res[(kResInRegs ? q : 0) * 4 + 0] = x.x;
          res[(kResInRegs ? q : 0) * 4 + 1] = x.y;
          res[(kResInRegs ? q : 0) * 4 + 2] = x.z;
          res[(kResInRegs ? q : 0) * 4 + 3] = x.w;
        }
      }
      asm volatile("bar.sync 2, 256;" ::: "memory");
    }
    const bool ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(acc_bar), 0, abort_flag, g.status, QB_DEV_WAIT_TIMEOUT_GEMM));
    if (threadIdx.x == 64) QB_GT(5);
    tc_fence_after();
    const uint32_t taddr = tmem_base + (static_cast<uint32_t>(lane_grp * 32) << 16);
    if (ok && fast) {
      // One accumulator row per thread, 32 columns at a time.  Per-column vectors come from shared
      // memory and the residual row from registers, both fetched during the main loop, so no global
      // load sits between the accumulator and the stores; every store writes whole 32-byte sectors.
      const float* col = reinterpret_cast<const float*>(smem + L::kColOffset);
      const bool has_gate = g.gate != nullptr;
      const bool has_scale = g.a_scale != nullptr || g.w_scale != nullptr;
      const bool has_bias = g.bias != nullptr;
      uint32_t rbuf[2][32];  // this warp's next chunk is on its way from TMEM while the current one is processed
      tmem_ld32(taddr + half * 32, rbuf[0]);
#pragma unroll
      for (int lc = 0; lc < kMyChunks; ++lc) {
        const int c = 2 * lc + half;
        tmem_wait_ld_into(rbuf[lc & 1]);
        if (lc + 1 < kMyChunks) tmem_ld32(taddr + (c + 2) * 32, rbuf[(lc + 1) & 1]);
        const uint32_t(&r)[32] = rbuf[lc & 1];
        const int n = n0 + c * 32;
        if (m < g.M && n < g.N) {
          float v[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) v[j] = __uint_as_float(r[j]);
          if (has_scale) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] *= col[c * 32 + j];
          }
          if (has_bias) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] += col[BN + c * 32 + j];
          }
          if (g.activation == 1) {
#pragma unroll
            for (int j = 0; j < 32; ++j) v[j] = silu_fast(v[j]);
          }
          if (has_gate) {
            uint32_t rw[16];
            if (kResInRegs) {
#pragma unroll
              for (int j = 0; j < 16; ++j) rw[j] = res[kResInRegs ? lc * 16 + j : 0];
            } else {  // 256-column tiles: the row does not fit in registers beside the accumulator chunk
              const uint4* rp = reinterpret_cast<const uint4*>(g.residual + static_cast<size_t>(m) * g.N + n);
#pragma unroll
              for (int q = 0; q < 4; ++q) {
                const uint4 x = rp[q];
                rw[4 * q] = x.x; rw[4 * q + 1] = x.y; rw[4 * q + 2] = x.z; rw[4 * q + 3] = x.w;
              }
            }
#pragma unroll
            for (int j = 0; j < 16; ++j) {
              v[2 * j] = __fadd_rn(bf16lo(rw[j]), __fmul_rn(col[2 * BN + c * 32 + 2 * j], v[2 * j]));
              v[2 * j + 1] = __fadd_rn(bf16hi(rw[j]), __fmul_rn(col[2 * BN + c * 32 + 2 * j + 1], v[2 * j + 1]));
            }
          }
          const size_t off = static_cast<size_t>(m) * g.N + n;
          if (g.c_dtype == QB_BF16) {
            uint16_t* dst = static_cast<uint16_t*>(g.C) + off;
            if (g.tp_world != 0) {
              const int owner = m / g.tp_rpo;
              dst = g.tp_dst[owner] + static_cast<size_t>(m - owner * g.tp_rpo) * g.N + n;
            }
#pragma unroll
            for (int h = 0; h < 2; ++h) {
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(v[16 * h + 2 * j], v[16 * h + 2 * j + 1]);
              st_global_v8(dst + 16 * h, w);
            }
          } else if (g.c_dtype == QB_E4M3) {
            uint32_t w[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) w[j] = pack_e4m3x4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            st_global_v8(static_cast<uint8_t*>(g.C) + off, w);
          } else {
#pragma unroll
            for (int h = 0; h < 4; ++h) {
              uint32_t w[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) w[j] = __float_as_uint(v[8 * h + j]);
              st_global_v8(static_cast<float*>(g.C) + off + 8 * h, w);
            }
          }
        }
      }
    } else if (half == 1 || qkv_done) {
      // the general paths below are written for the first four epilogue warps
    } else if (ok && g.splits == 1) {
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_wait_ld_into(r);
        if (m < g.M) {
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int n = n0 + c * 32 + q * 8;
            if (n < g.N) {
              float v[8];
#pragma unroll
              for (int j = 0; j < 8; ++j) v[j] = __uint_as_float(r[q * 8 + j]);
              epilogue_store8(g, v, m, n);
            }
          }
        }
      }
    } else if (ok && use_staging) {
      // accumulator row -> staging tile in the (now idle) stage memory, f32, padded pitch: one row per thread
      float* dst = reinterpret_cast<float*>(smem) + static_cast<size_t>(row) * kStgPitch;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_wait_ld_into(r);
#pragma unroll
        for (int q = 0; q < 8; ++q)
          *reinterpret_cast<float4*>(dst + c * 32 + q * 4) = make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]),
                                                                        __uint_as_float(r[q * 4 + 2]), __uint_as_float(r[q * 4 + 3]));
      }
    } else if (ok) {
      // K slices through the global workspace: partial tile out, ticket, last CTA adds the slices in order
      float* part = g.partials + static_cast<size_t>(split) * g.M * g.N;
#pragma unroll 1
      for (int c = 0; c < BN / 32; ++c) {
        uint32_t r[32];
        tmem_ld32(taddr + c * 32, r);
        tmem_wait_ld_into(r);
        if (m < g.M) {
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            const int n = n0 + c * 32 + q * 4;
            if (n < g.N)
              __stcg(reinterpret_cast<float4*>(part + static_cast<size_t>(m) * g.N + n),
                     make_float4(__uint_as_float(r[q * 4]), __uint_as_float(r[q * 4 + 1]), __uint_as_float(r[q * 4 + 2]),
                                 __uint_as_float(r[q * 4 + 3])));
          }
        }
      }
      __threadfence();
      asm volatile("bar.sync 1, 128;" ::: "memory");
      int* counter = g.counters + blockIdx.y * gridDim.x + blockIdx.x;
      if (threadIdx.x == 64) {
        const int ticket = atomicAdd(counter, 1);
        *last_flag = (ticket == g.splits - 1) ? 1 : 0;
        __threadfence();
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      if (*last_flag) {
        const int et = threadIdx.x - 64;  // 0..127
#pragma unroll 1
        for (int i8 = et; i8 < kBM * (BN / 8); i8 += 128) {
          const int mm = m0 + i8 / (BN / 8);
          const int n = n0 + (i8 % (BN / 8)) * 8;
          if (mm >= g.M || n >= g.N) continue;
          float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
          for (int s = 0; s < g.splits; ++s) {
            const float4* src = reinterpret_cast<const float4*>(g.partials + (static_cast<size_t>(s) * g.M + mm) * g.N + n);
            const float4 x = __ldcg(src), y = __ldcg(src + 1);
            v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
            v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
          }
          epilogue_store8(g, v, mm, n);
        }
        if (threadIdx.x == 64) *counter = 0;  // ready for the next launch
      }
    }
  }

  // ---------------- epilogue, part 2: every staged tile of the cluster is complete after this barrier
  tc_fence_before();
  if (clustered) {
    cluster_sync();
  } else {
    __syncthreads();
  }
  if (use_staging && warp >= 2 && warp < 6 && *abort_flag == 0) {
    // Rows are dealt out to the CTAs of the cluster; each sums its rows over all slices, in slice order,
    // reading the peers' staging tiles through distributed shared memory.  Consecutive threads take
    // consecutive groups of 8 columns, so global loads and stores are coalesced.
    const int n_slices = clustered ? g.splits : 1;
    const int rows_per_cta = kBM / n_slices;
    const int row_begin = clustered ? split * rows_per_cta : 0;
    const uint32_t stg_base = smem_u32(smem);
    const int et = threadIdx.x - 64;  // 0..127
#pragma unroll 1
    for (int i8 = et; i8 < rows_per_cta * (BN / 8); i8 += 128) {
      const int rr = row_begin + i8 / (BN / 8);
      const int c8 = (i8 % (BN / 8)) * 8;
      const int mm = m0 + rr, n = n0 + c8;
      if (mm >= g.M || n >= g.N) continue;
      const uint32_t local = stg_base + (static_cast<uint32_t>(rr) * kStgPitch + c8) * 4u;
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (clustered) {
        for (int s = 0; s < n_slices; ++s) {
          const uint32_t remote = map_to_cta(local, s);
          const float4 x = ld_dsmem_f4(remote), y = ld_dsmem_f4(remote + 16);
          v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
          v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
        }
      } else {
        const float4* src = reinterpret_cast<const float4*>(reinterpret_cast<const float*>(smem) + static_cast<size_t>(rr) * kStgPitch + c8);
        const float4 x = src[0], y = src[1];
        v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
        v[4] = y.x; v[5] = y.y; v[6] = y.z; v[7] = y.w;
      }
      epilogue_store8(g, v, mm, n);
    }
  }
  if (clustered) cluster_sync();  // nobody leaves while a peer may still read its staging tile

  __syncthreads();
  if (threadIdx.x == 0) QB_GT(6);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

// ---------------------------------------------------------------- host side
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_tiled_fn() {
  static EncodeTiledFn fn = nullptr;
  if (fn == nullptr) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess)
      fn = reinterpret_cast<EncodeTiledFn>(p);
  }
  return fn;
}

// Tensor map of a contiguous row-major tensor [rows, cols] of 1- or 2-byte elements with a box of
// [box_rows, box_cols] elements; box_cols * elem_bytes must equal the swizzle span (64 or 128).
// Out-of-range parts of a box are filled with zeros.
int32_t make_tmap_2d_sw(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols, int swizzle_bytes) {
  EncodeTiledFn enc = encode_tiled_fn();
  QB_REQUIRE(enc != nullptr, QB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
  QB_REQUIRE((cols * elem_bytes) % 16 == 0, QB_ERR_ALIGN, "tensor map: row pitch of %llu bytes is not a multiple of 16",
             static_cast<unsigned long long>(cols * elem_bytes));
  const cuuint64_t dims[2] = {cols, rows};
  const cuuint64_t strides[1] = {cols * elem_bytes};
  const cuuint32_t box[2] = {box_cols, box_rows};
  const cuuint32_t estr[2] = {1, 1};
  const CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  const CUtensorMapSwizzle sw = swizzle_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B;
  CUresult r = enc(tm, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, sw,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  QB_REQUIRE(r == CUDA_SUCCESS, QB_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
  return QB_OK;
}

static int32_t make_tmap_2d(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows) {
  return make_tmap_2d_sw(tm, base, elem_bytes, rows, cols, box_rows, static_cast<uint32_t>(kRowBytes / elem_bytes), 128);
}

// Tile counters of the workspace K slices live in a fixed area at the start of the workspace, so that calls of
// different shapes that share one workspace agree on where the counters end and the data begins (a
// shape-dependent area would let one call's e4m3 copy of A or partial sums land on counters that a later
// call with more tiles expects to find zero).
constexpr size_t kCounterBytes = 64u << 10;  // 16384 tiles

struct GemmPlan {
  int bn, splits, kb_total, kb_per_split;
  int cluster;  // slices summed inside a thread-block cluster (2, 4 or 8 slices) instead of through the workspace
  size_t counters_bytes, aq_bytes, partial_bytes;
};

static int num_sms() {
  static int n = 0;
  if (n == 0) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

// Picks the tile width and the number of K slices from a small cost model (cycles per CTA:
// the slower of tensor-core issue and operand delivery per 128 bytes of K, plus fixed costs),
// so that every call with the same shape makes the same choice.
static GemmPlan plan_gemm(const qb_gemm_params& p) {
  const bool fp8 = p.compute_dtype == QB_E4M3;
  const int k_elems = fp8 ? 128 : 64;
  GemmPlan best{};
  double best_cost = 1e30;
  const int sms = num_sms();
  const int kb_total = (p.K + k_elems - 1) / k_elems;
  const int bns[3] = {256, 128, 64};
  const int ss[10] = {1, 2, 3, 4, 5, 6, 8, 10, 12, 16};
  for (int bn : bns) {
    if (p.tile_n != 0 && p.tile_n != bn) continue;
    if (p.tile_n == 0 && bn > 64 && bn / 2 >= p.N) continue;  // tile mostly empty
    const int tiles = ((p.M + kBM - 1) / kBM) * ((p.N + bn - 1) / bn);
    for (int s : ss) {
      if (p.split_k != 0 && p.split_k != s) continue;
      if (s > kb_total) continue;
      const int kbps = (kb_total + s - 1) / s;
      const int s_eff = (kb_total + kbps - 1) / kbps;
      if (s_eff != s) continue;
      const long ctas = static_cast<long>(tiles) * s;
      const long waves = (ctas + sms - 1) / sms;
      // Cycles per 128 bytes of K: the slower of what one SM can take in (150 + 2.3 BN, fitted at M = 128 where
      // few CTAs run) and its share of the L2's aggregate delivery when a whole wave pulls at once (about
      // 9000 bytes per clock over the chip: 19 TB/s measured at M = 512).  Fixed cost: launch, set-up, first
      // tile, epilogue (2.8 us at BN = 64).  K slices add the staging, the cluster barrier and the reduction
      // through distributed shared memory (3.5 - 5.7 us measured for 2 - 4 slices), or the far slower trip
      // through the workspace (12 - 14 us), so slices pay only when they multiply the number of busy SMs or
      // K is long.  Measured at M = 128, bf16, 2048 x 8192: 22 us in one slice, 12 us in 4 cluster slices.
      const long in_wave = ctas < sms ? ctas : sms;
      const double stage_bytes = 128.0 * (kBM + bn);
      const double per_sm = 150.0 + 2.3 * bn, shared = in_wave * stage_bytes / 9000.0;
      const double per_kb = per_sm > shared ? per_sm : shared;
      double cta = kbps * per_kb + 5000.0 + bn * 12.0;
      const bool cl = (p.reserved & 1) == 0 && (s == 2 || s == 4 || s == 8);
      if (s > 1 && !cl && static_cast<size_t>(tiles) * sizeof(int) > kCounterBytes) continue;  // more tiles than counters
      if (s > 1) cta += cl ? 7500.0 + bn * 20.0 + s * bn * 4.0 : 26000.0;
      const double cost = waves * cta;
      if (cost < best_cost) {
        best_cost = cost;
        best.bn = bn;
        best.splits = s;
        best.kb_total = kb_total;
        best.kb_per_split = kbps;
        best.cluster = (s > 1 && cl) ? 1 : 0;
      }
    }
  }
  if (best.bn == 0) {  // forced values that fit nothing: fall back to the plain configuration
    best.bn = p.tile_n ? p.tile_n : 128;
    best.splits = 1;
    best.kb_total = kb_total;
    best.kb_per_split = kb_total;
  }
  best.counters_bytes = kCounterBytes;
  best.aq_bytes = (fp8 && p.a_dtype == QB_BF16) ? round_up(static_cast<size_t>(p.M) * p.K, 1024) : 0;
  best.partial_bytes = (best.splits > 1 && !best.cluster) ? static_cast<size_t>(best.splits) * p.M * p.N * sizeof(float) : 0;
  return best;
}

static int32_t validate_gemm(const qb_gemm_params* p) {
  QB_REQUIRE(p != nullptr, QB_ERR_INVALID_ARG, "gemm params are NULL");
  QB_REQUIRE(p->M > 0 && p->N > 0 && p->K > 0, QB_ERR_INVALID_ARG, "gemm: M, N, K must be positive (got %d, %d, %d)", p->M, p->N, p->K);
  QB_REQUIRE(p->compute_dtype == QB_BF16 || p->compute_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "gemm: compute_dtype %d", p->compute_dtype);
  if (p->compute_dtype == QB_BF16) {
    QB_REQUIRE(p->a_dtype == QB_BF16 && p->b_dtype == QB_BF16, QB_ERR_INVALID_ARG, "gemm: bf16 compute needs bf16 A and B");
  } else {
    QB_REQUIRE(p->b_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "gemm: e4m3 compute needs an e4m3 B (weights are quantised ahead of time)");
    QB_REQUIRE(p->a_dtype == QB_E4M3 || p->a_dtype == QB_BF16, QB_ERR_INVALID_ARG, "gemm: A must be bf16 or e4m3");
  }
  QB_REQUIRE(p->c_dtype == QB_BF16 || p->c_dtype == QB_F32 || p->c_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "gemm: c_dtype %d", p->c_dtype);
  QB_REQUIRE(p->K % 16 == 0, QB_ERR_ALIGN, "gemm: K = %d must be a multiple of 16", p->K);
  QB_REQUIRE(p->N % 8 == 0, QB_ERR_ALIGN, "gemm: N = %d must be a multiple of 8", p->N);
  QB_REQUIRE(p->activation == 0 || p->activation == 1, QB_ERR_INVALID_ARG, "gemm: activation %d", p->activation);
  QB_REQUIRE(p->tile_n == 0 || p->tile_n == 64 || p->tile_n == 128 || p->tile_n == 256, QB_ERR_INVALID_ARG, "gemm: tile_n %d", p->tile_n);
  QB_REQUIRE(p->split_k >= 0 && p->split_k <= 16, QB_ERR_INVALID_ARG, "gemm: split_k %d", p->split_k);
  QB_REQUIRE(p->reserved >= 0 && p->reserved <= 3, QB_ERR_INVALID_ARG, "gemm: flags %d", p->reserved);
  return QB_OK;
}

template <int BN, bool FP8>
static int32_t launch_gemm(const CUtensorMap& tmA, const CUtensorMap& tmB, const GemmArgs& args, dim3 grid, cudaStream_t st) {
  using L = GemmSmem<BN>;
  QB_CUDA_OK(cudaFuncSetAttribute(gemm_kernel<BN, FP8>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::kTotal));
  if (args.cluster && args.splits > 1) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = L::kTotal;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = static_cast<unsigned>(args.splits);
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_dependent_launch ? 2 : 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, gemm_kernel<BN, FP8>, tmA, tmB, args);
    ++g_launch_count;
    if (e != cudaSuccess) return fail(QB_ERR_LAUNCH, "gemm kernel (cluster of %d): %s", args.splits, cudaGetErrorString(e));
    return QB_OK;
  }
  return launch_dep("gemm kernel", gemm_kernel<BN, FP8>, grid, dim3(kGemmThreads), L::kTotal, st, tmA, tmB, args);
}

int32_t quantize_e4m3_launch(const void* X, void* out, size_t n, int32_t src_dtype, cudaStream_t st);

}  // namespace qb

using namespace qb;

#ifdef QB_GEMM_TRACE
extern "C" int32_t qb_debug_gemm_trace(void* host_out) {
  return cudaMemcpyFromSymbol(host_out, qb::g_gemm_trace, sizeof(qb::g_gemm_trace)) == cudaSuccess ? 0 : -1;
}
#endif

extern "C" size_t qb_gemm_workspace_bytes(const qb_gemm_params* p) {
  if (validate_gemm(p) != QB_OK) return 0;
  const GemmPlan pl = plan_gemm(*p);
  if (pl.aq_bytes == 0 && pl.partial_bytes == 0) return 0;  // no scratch memory is touched
  return pl.counters_bytes + pl.aq_bytes + pl.partial_bytes;
}

// clear_counters: the workspace may hold anything (the built-in scratch array keeps the last call's contents), so the
// tile counters are zeroed on the stream first, after every check has passed and only if this plan reads them.
struct TpDest {
  int world, rpo;
  uint16_t* dst[8];
};

static int32_t gemm_run(const void* A, const void* B, void* C, const void* bias, const void* gate, const void* residual,
                        const qb_gemm_params* p, void* workspace, size_t workspace_bytes, void* stream, const QkvTail* tail,
                        bool clear_counters = false, const TpDest* tp = nullptr, const int* tile_expert = nullptr, int n_experts = 1) {
  int32_t rc = validate_gemm(p);
  if (rc != QB_OK) return rc;
  QB_REQUIRE(A && B && C, QB_ERR_INVALID_ARG, "gemm: A, B and C must not be NULL");
  QB_REQUIRE((gate == nullptr) == (residual == nullptr), QB_ERR_INVALID_ARG, "gemm: gate and residual come together");
  QB_REQUIRE(aligned16(A) && aligned16(B) && aligned16(C) && aligned16(bias) && aligned16(gate) && aligned16(residual), QB_ERR_ALIGN,
             "gemm: every pointer must be 16-byte aligned");
  int rows_per_gate = p->M;
  if (gate != nullptr) {
    QB_REQUIRE(p->gate_groups >= 1 && p->M % p->gate_groups == 0, QB_ERR_INVALID_ARG, "gemm: gate_groups %d does not divide M = %d",
               p->gate_groups, p->M);
    rows_per_gate = p->M / p->gate_groups;
  }
  const GemmPlan pl = plan_gemm(*p);
  const size_t need = pl.counters_bytes + pl.aq_bytes + pl.partial_bytes;
  const bool uses_ws = pl.aq_bytes > 0 || pl.partial_bytes > 0;
  if (uses_ws) {
    QB_REQUIRE(workspace != nullptr && workspace_bytes >= need, QB_ERR_WORKSPACE, "gemm: workspace of %zu bytes needed, %zu given", need,
               workspace_bytes);
    QB_REQUIRE(aligned16(workspace), QB_ERR_ALIGN, "gemm: workspace must be 16-byte aligned");
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const bool fp8 = p->compute_dtype == QB_E4M3;
  uint8_t* ws = static_cast<uint8_t*>(workspace);
  unsigned int* status = status_word();
  QB_REQUIRE(status != nullptr, QB_ERR_CUDA, "gemm: device status word unavailable");
  if (tail != nullptr) QB_REQUIRE(pl.bn == 128 && pl.splits == 1, QB_ERR_INVALID_ARG, "gemm_qkv_post: needs 128-column tiles and one K slice");
  if (clear_counters && pl.partial_bytes > 0) QB_CUDA_OK(cudaMemsetAsync(ws, 0, pl.counters_bytes, st));
  const void* a_ptr = A;
  if (pl.aq_bytes > 0) {
    uint8_t* aq = ws + pl.counters_bytes;
    rc = quantize_e4m3_launch(A, aq, static_cast<size_t>(p->M) * p->K, QB_BF16, st);
    if (rc != QB_OK) return rc;
    a_ptr = aq;
  }
  CUtensorMap tmA, tmB;
  const int es = fp8 ? 1 : 2;
  rc = make_tmap_2d(&tmA, a_ptr, es, p->M, p->K, kBM);
  if (rc != QB_OK) return rc;
  rc = make_tmap_2d(&tmB, B, es, static_cast<uint64_t>(p->N) * n_experts, p->K, pl.bn);
  if (rc != QB_OK) return rc;

  GemmArgs g{};
  g.M = p->M; g.N = p->N; g.K = p->K;
  g.kb_total = pl.kb_total; g.kb_per_split = pl.kb_per_split; g.splits = pl.splits;
  g.cluster = pl.cluster;
  g.b_const = (p->reserved & 2) != 0;
  g.c_dtype = p->c_dtype; g.activation = p->activation; g.rows_per_gate = rows_per_gate;
  g.a_scale = p->a_scale; g.w_scale = p->w_scale;
  g.bias = static_cast<const uint16_t*>(bias);
  g.gate = static_cast<const uint16_t*>(gate);
  g.residual = static_cast<const uint16_t*>(residual);
  g.C = C;
  g.counters = reinterpret_cast<int*>(ws);
  g.partials = pl.partial_bytes ? reinterpret_cast<float*>(ws + pl.counters_bytes + pl.aq_bytes) : nullptr;
  g.status = status;
  if (tp != nullptr) {
    // the per-row destinations exist in the one-slice fast epilogue only: whole 32-column chunks, bf16, no gate
    QB_REQUIRE(pl.splits == 1 && p->N % 32 == 0 && p->c_dtype == QB_BF16 && gate == nullptr && tail == nullptr, QB_ERR_UNSUPPORTED,
               "gemm_tp: needs one K slice, N a multiple of 32, bf16 output, no gate");
    g.tp_world = tp->world;
    g.tp_rpo = tp->rpo;
    for (int r = 0; r < tp->world; ++r) g.tp_dst[r] = tp->dst[r];
  }
  if (tail != nullptr) {
    g.qkv_mode = 1;
    g.qkv = *tail;
  }
  if (tile_expert != nullptr) {
    // per-column vectors would have to be per expert
    // (a B tile that runs past the expert's last row only feeds columns >= N, which no epilogue stores)
    QB_REQUIRE(pl.splits == 1 && p->M % kBM == 0, QB_ERR_UNSUPPORTED, "gemm_grouped: needs one K slice and M = %d a multiple of 128", p->M);
    QB_REQUIRE(tail == nullptr && tp == nullptr && bias == nullptr && gate == nullptr && p->w_scale == nullptr,
               QB_ERR_UNSUPPORTED, "gemm_grouped: takes the plain or the SiLU epilogue only");
    g.tile_expert = tile_expert;
  }

  dim3 grid((p->N + pl.bn - 1) / pl.bn, (p->M + kBM - 1) / kBM, pl.splits);
  if (fp8) {
    if (pl.bn == 256) return launch_gemm<256, true>(tmA, tmB, g, grid, st);
    if (pl.bn == 128) return launch_gemm<128, true>(tmA, tmB, g, grid, st);
    return launch_gemm<64, true>(tmA, tmB, g, grid, st);
  }
  if (pl.bn == 256) return launch_gemm<256, false>(tmA, tmB, g, grid, st);
  if (pl.bn == 128) return launch_gemm<128, false>(tmA, tmB, g, grid, st);
  return launch_gemm<64, false>(tmA, tmB, g, grid, st);
}

extern "C" int32_t qb_gemm(const void* A, const void* B, void* C, const void* bias, const void* gate, const void* residual,
                           const qb_gemm_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  return gemm_run(A, B, C, bias, gate, residual, p, workspace, workspace_bytes, stream, nullptr);
}

extern "C" int32_t qb_gemm_qkv_post(const void* A, const void* B, void* qkv_out, const void* qkv_first, const float* lamb,
                                    const int32_t* frame_t, const int32_t* frozen, void* K_cache, void* Vt_cache, int32_t* segments,
                                    int32_t* n_segments, const float* rope_xy, const qb_gemm_params* gp, const qb_kv_params* kp, float eps,
                                    void* workspace, size_t workspace_bytes, void* stream) {
  QB_REQUIRE(gp != nullptr && kp != nullptr, QB_ERR_INVALID_ARG, "gemm_qkv_post: params are NULL");
  QB_REQUIRE(qkv_out && frame_t && frozen && K_cache && Vt_cache && segments && n_segments && rope_xy, QB_ERR_INVALID_ARG,
             "gemm_qkv_post: NULL pointer");
  QB_REQUIRE((qkv_first == nullptr) == (lamb == nullptr), QB_ERR_INVALID_ARG, "gemm_qkv_post: qkv_first and lamb come together");
  QB_REQUIRE(kp->packed_qkv == 1, QB_ERR_UNSUPPORTED, "gemm_qkv_post: the packed QKV layout only");
  // a 128-token tile must hold whole 16-byte vectors of cached V tokens (8 bf16 / 16 e4m3 per vector)
  QB_REQUIRE(kp->quilt_factor >= 1 && (kp->quilt_factor & (kp->quilt_factor - 1)) == 0 &&
                 kp->quilt_factor * (kp->kv_dtype == QB_E4M3 ? 16 : 8) <= 128,
             QB_ERR_UNSUPPORTED, "gemm_qkv_post: quilt_factor %d (a power of two, at most %d for this cache dtype)", kp->quilt_factor,
             kp->kv_dtype == QB_E4M3 ? 8 : 16);
  QB_REQUIRE(kp->quilt_offset >= 0 && kp->quilt_offset < kp->quilt_factor, QB_ERR_INVALID_ARG, "gemm_qkv_post: quilt_offset %d", kp->quilt_offset);
  QB_REQUIRE(kp->n_kv_heads > 0 && kp->n_q_heads > 0 && kp->n_q_heads % kp->n_kv_heads == 0, QB_ERR_INVALID_ARG,
             "gemm_qkv_post: %d Q heads over %d KV heads", kp->n_q_heads, kp->n_kv_heads);
  QB_REQUIRE(kp->H_spatial > 0 && kp->W_spatial > 0 && kp->num_buckets > 0 && kp->pinned_dilation > 0, QB_ERR_INVALID_ARG,
             "gemm_qkv_post: sizes must be positive");
  QB_REQUIRE(kp->kv_dtype == QB_BF16 || kp->kv_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "gemm_qkv_post: kv_dtype %d", kp->kv_dtype);
  QB_REQUIRE(kp->max_segments >= 3, QB_ERR_INVALID_ARG, "gemm_qkv_post: max_segments %d < 3", kp->max_segments);
  const int tpf = kp->H_spatial * kp->W_spatial;
  QB_REQUIRE(gp->M == tpf && gp->N == (kp->n_q_heads + 2 * kp->n_kv_heads) * 64, QB_ERR_INVALID_ARG,
             "gemm_qkv_post: the projection is [%d, %d] but the geometry needs [%d, %d]", gp->M, gp->N, tpf,
             (kp->n_q_heads + 2 * kp->n_kv_heads) * 64);
  QB_REQUIRE((tpf / kp->quilt_factor) % 16 == 0 && tpf % kp->quilt_factor == 0, QB_ERR_UNSUPPORTED,
             "gemm_qkv_post: H*W / quilt_factor = %d / %d must be a multiple of 16", tpf, kp->quilt_factor);
  QB_REQUIRE(gp->c_dtype == QB_BF16 && gp->activation == 0, QB_ERR_INVALID_ARG, "gemm_qkv_post: bf16 output without activation");
  QB_REQUIRE((reinterpret_cast<uintptr_t>(qkv_out) & 31u) == 0 && (reinterpret_cast<uintptr_t>(K_cache) & 31u) == 0 && aligned16(Vt_cache) &&
                 aligned16(qkv_first) && aligned16(rope_xy),
             QB_ERR_ALIGN, "gemm_qkv_post: qkv_out and K_cache must be 32-byte aligned, the other pointers 16-byte aligned");
  qb_gemm_params p = *gp;
  p.tile_n = 128;
  p.split_k = 1;
  QkvTail t{};
  t.qkv_first = static_cast<const uint16_t*>(qkv_first);
  t.lamb = lamb; t.frame_t = frame_t; t.frozen = frozen;
  t.K_cache = K_cache; t.Vt_cache = Vt_cache; t.segments = segments; t.n_segments = n_segments; t.rope_xy = rope_xy;
  t.n_q_heads = kp->n_q_heads; t.n_kv_heads = kp->n_kv_heads; t.tpf = tpf; t.nb = kp->num_buckets; t.pd = kp->pinned_dilation;
  t.max_segments = kp->max_segments; t.kv_fp8 = kp->kv_dtype == QB_E4M3; t.eps = eps;
  t.k_scale = kp->k_scale; t.v_scale = kp->v_scale;
  t.quilt = kp->quilt_factor; t.qoff = kp->quilt_offset;
  return gemm_run(A, B, qkv_out, nullptr, nullptr, nullptr, &p, workspace, workspace_bytes, stream, &t);
}

extern "C" int32_t qb_gemm_tp(const void* A, const void* B, const qb_gemm_params* p, const qb_tp_params* tp, void* workspace,
                              size_t workspace_bytes, void* stream) {
  QB_REQUIRE(p != nullptr && tp != nullptr, QB_ERR_INVALID_ARG, "gemm_tp: params are NULL");
  QB_REQUIRE(tp->world >= 1 && tp->world <= 8 && tp->rank >= 0 && tp->rank < tp->world, QB_ERR_INVALID_ARG, "gemm_tp: rank %d of %d", tp->rank,
             tp->world);
  QB_REQUIRE(tp->rows == p->M && tp->D == p->N && p->M % tp->world == 0, QB_ERR_INVALID_ARG,
             "gemm_tp: the partial is [%d, %d] but the arenas are laid out for [%d, %d] over %d ranks", p->M, p->N, tp->rows, tp->D, tp->world);
  qb_gemm_params q = *p;
  q.split_k = 1;  // the partial must leave the kernel in one piece
  TpDest d{};
  d.world = tp->world;
  d.rpo = p->M / tp->world;
  size_t off[6];
  int32_t rc = qb_tp_arena_offsets(tp->rows, tp->D, off);
  if (rc != QB_OK) return rc;
  for (int r = 0; r < tp->world; ++r) {
    QB_REQUIRE(tp->arena[r] != nullptr, QB_ERR_INVALID_ARG, "gemm_tp: arena %d is NULL", r);
    // rank r's staging area (its y slot 0) holds one block of rows per source rank: [source][rows / world][D]
    d.dst[r] = reinterpret_cast<uint16_t*>(static_cast<uint8_t*>(tp->arena[r]) + off[0]) + static_cast<size_t>(tp->rank) * d.rpo * p->N;
  }
  // C is unused (every row has a destination of its own); the rank's own staging block stands in for the pointer checks
  return gemm_run(A, B, d.dst[tp->rank], nullptr, nullptr, nullptr, &q, workspace, workspace_bytes, stream, nullptr, false, &d);
}

extern "C" size_t qb_gemm_grouped_workspace_bytes(const qb_gemm_params* p) {
  if (validate_gemm(p) != QB_OK) return 0;
  qb_gemm_params q = *p;
  q.split_k = 1;
  return qb_gemm_workspace_bytes(&q);
}

extern "C" int32_t qb_gemm_grouped(const void* A, const void* B, void* C, const int32_t* tile_expert, int32_t n_experts, const qb_gemm_params* p,
                                   void* workspace, size_t workspace_bytes, void* stream) {
  QB_REQUIRE(p != nullptr && tile_expert != nullptr, QB_ERR_INVALID_ARG, "gemm_grouped: params or tile table are NULL");
  QB_REQUIRE(n_experts >= 1 && static_cast<long long>(n_experts) * p->N < (1ll << 31), QB_ERR_INVALID_ARG, "gemm_grouped: %d experts", n_experts);
  qb_gemm_params q = *p;
  q.split_k = 1;  // a padding tile leaves before any K slice could wait for it
  return gemm_run(A, B, C, nullptr, nullptr, nullptr, &q, workspace, workspace_bytes, stream, nullptr, false, nullptr, tile_expert, n_experts);
}

// ---------------------------------------------------------------- GEMM on built-in scratch memory
// Scratch for qb_gemm_static_scratch: lives in the library image, so every GPU that loads the library
// holds these 8 MiB until the process exits.  In host code the name below is only a handle for
// cudaGetSymbolAddress; the device address it yields is what the kernels receive.
namespace qb {
constexpr size_t kStaticScratchBytes = 8u << 20;
static __device__ __align__(256) unsigned char g_gemm_static_scratch[kStaticScratchBytes];

// Device address of the scratch array on the calling thread's current device (the device the stream must belong
// to), looked up once per device and published with a release store, so that two host threads that make their
// first calls at the same time both end up with the same, fully written entry.  cudaDeviceReset invalidates
// the entry of that device; a process that resets a device must not call this entry point on it afterwards.
static int32_t static_scratch_ptr(void** out) {
  static std::atomic<void*> cache[64];
  int dev = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  QB_REQUIRE(dev >= 0 && dev < 64, QB_ERR_DEVICE, "gemm_static_scratch: device ordinal %d out of range", dev);
  void* p = cache[dev].load(std::memory_order_acquire);
  if (p == nullptr) {
    QB_CUDA_OK(cudaGetSymbolAddress(&p, g_gemm_static_scratch));
    QB_REQUIRE(p != nullptr, QB_ERR_CUDA, "gemm_static_scratch: cudaGetSymbolAddress returned a null address");
    cache[dev].store(p, std::memory_order_release);
  }
  *out = p;
  return QB_OK;
}
}  // namespace qb

extern "C" size_t qb_gemm_static_scratch_capacity(void) { return qb::kStaticScratchBytes; }

extern "C" int32_t qb_gemm_static_scratch(const void* A, const void* B, void* C, const void* bias, const void* gate,
                                          const void* residual, const qb_gemm_params* p, void* stream) {
  int32_t rc = validate_gemm(p);
  if (rc != QB_OK) return rc;
  const GemmPlan pl = plan_gemm(*p);
  const size_t need = pl.counters_bytes + pl.aq_bytes + pl.partial_bytes;
  QB_REQUIRE(need <= kStaticScratchBytes, QB_ERR_WORKSPACE,
             "gemm_static_scratch: this GEMM needs %zu bytes of scratch but the built-in scratch holds %zu; "
             "use qb_gemm with a caller-provided workspace, or force a smaller split_k",
             need, static_cast<size_t>(kStaticScratchBytes));
  void* scratch = nullptr;
  rc = static_scratch_ptr(&scratch);
  if (rc != QB_OK) return rc;
  // The array keeps whatever the previous call left.  Only the tile counters must start at zero (the e4m3 copy of
  // A and the K-slice partials are fully written before they are read); gemm_run clears them on the stream once all
  // of its own checks have passed, and only when this plan sums K slices through the scratch memory.
  return gemm_run(A, B, C, bias, gate, residual, p, scratch, kStaticScratchBytes, stream, nullptr, true);
}
