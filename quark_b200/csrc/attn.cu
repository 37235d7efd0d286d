// owl_attn: segment-sparse GQA flash attention with inline ortho-RoPE on Q, head_dim 64.
//
// One CTA owns 128 query tokens of one Q head and walks the valid keys in tiles of 128:
//   warp 0      TMA producer: K tile [128 keys x 64] and V^T tile [64 x 128 keys] per stage
//   warp 1      one thread issues tcgen05.mma:  S = Q K^T  (TMEM, double buffered)  and
//               PV = P V (TMEM), operands straight from the swizzled shared-memory tiles
//   warps 2-5   one query row per thread: rotate Q (RoPE) into shared memory once, then per tile
//               read S from TMEM, online softmax (exp2 with the 1/sqrt(Dh) scale folded in),
//               write P to shared memory in the layout the MMA wants, and fold PV into the
//               f32 output row kept in registers.
// Masked buckets cost nothing: the key tiles are enumerated from the (start, length) segment
// table, so a tile outside every segment is never loaded.  bf16 path: kind::f16 MMAs, P rounded
// to bf16.  fp8 path: Q (after RoPE), K, V and P are e4m3, kind::f8f6f4 MMAs, f32 accumulation;
// P is stored scaled by 2^8 so that small probabilities keep mantissa bits (the factor cancels
// in the final division by the row sum).
#include <cuda.h>

#include "common.cuh"
#include "rope.cuh"
#include "sm100.cuh"

namespace qb {

int32_t make_tmap_2d_sw(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols, int swizzle_bytes);

constexpr int kAttnThreads = 192;
constexpr int kQTile = 128;
constexpr int kKeyTile = 128;
constexpr int kStagesAttn = 3;

struct AttnArgs {
  const uint16_t* qkv;
  const int32_t* segments;
  const int32_t* n_segments;
  const int32_t* frame_t;
  uint16_t* out;
  const float* rope_xy;
  const float* k_scale;
  const float* v_scale;
  unsigned int* status;
  int tpf, qkv_dim, n_q_heads, gqa, capacity, max_segments;
};

template <bool kFp8>
struct AttnSmem {
  static constexpr int kEs = kFp8 ? 1 : 2;
  static constexpr int kQBytes = kQTile * 64 * kEs;          // 16 KB | 8 KB
  static constexpr int kKBytes = kKeyTile * 64 * kEs;        // 16 KB | 8 KB
  static constexpr int kVBytes = 64 * kKeyTile * kEs;        // 16 KB | 8 KB
  static constexpr int kPBytes = kQTile * kKeyTile * kEs;    // 32 KB | 16 KB
  static constexpr int kStageBytes = kKBytes + kVBytes;
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kQOff + kQBytes;
  static constexpr int kStageOff = kPOff + kPBytes;
  static constexpr int kBarOff = kStageOff + kStagesAttn * kStageBytes;
  static constexpr int kTotal = kBarOff + 256 + 1024;
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

// Which 128-key tile is the j-th valid one?  Returns its first cache row and how many of its
// keys are valid.  Segments are (start, length) pairs; zero-length entries are legal.
__device__ __forceinline__ void locate_tile(const int (&seg)[6], int nseg, int j, int& row, int& valid) {
  row = 0;
  valid = 0;
  for (int i = 0; i < nseg; ++i) {
    const int nt = (seg[2 * i + 1] + kKeyTile - 1) / kKeyTile;
    if (j < nt) {
      row = seg[2 * i] + j * kKeyTile;
      valid = min(kKeyTile, seg[2 * i + 1] - j * kKeyTile);
      return;
    }
    j -= nt;
  }
}

template <bool kFp8>
__global__ void __launch_bounds__(kAttnThreads, 1)
owl_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using L = AttnSmem<kFp8>;
  constexpr int kEs = L::kEs;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescS = kFp8 ? umma_idesc(0, 0, 128, 128) : umma_idesc(1, 1, 128, 128);
  constexpr uint32_t kIdescPV = kFp8 ? umma_idesc(0, 0, 128, 64) : umma_idesc(1, 1, 128, 64);
  constexpr float kPShift = kFp8 ? 8.0f : 0.0f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem + L::kQOff;
  uint8_t* p_s = smem + L::kPOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;                       // [stages]
  uint64_t* kv_empty = bars + kStagesAttn;        // [stages]
  uint64_t* s_full = bars + 2 * kStagesAttn;      // [2]
  uint64_t* s_free = s_full + 2;                  // [2]
  uint64_t* p_full = s_free + 2;
  uint64_t* pv_full = p_full + 1;
  uint64_t* q_ready = pv_full + 1;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* drain_flag = abort_flag + 1;
  float* tm = reinterpret_cast<float*>(const_cast<int*>(abort_flag + 2));  // 16 floats

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * kQTile;
  const int qh = blockIdx.y;
  const int kvh = qh / a.gqa;

  // segment table -> number of key tiles (same in every thread)
  int seg[6] = {0, 0, 0, 0, 0, 0};
  int nseg = min(__ldg(a.n_segments), min(a.max_segments, 3));
  bool seg_ok = true;
  int n_tiles = 0;
  for (int i = 0; i < nseg; ++i) {
    seg[2 * i] = __ldg(a.segments + 2 * i);
    seg[2 * i + 1] = __ldg(a.segments + 2 * i + 1);
    if (seg[2 * i] < 0 || seg[2 * i + 1] < 0 || (seg[2 * i] & 15) != 0 || seg[2 * i] + seg[2 * i + 1] > a.capacity) seg_ok = false;
    n_tiles += (seg[2 * i + 1] + kKeyTile - 1) / kKeyTile;
  }
  if (!seg_ok) {  // malformed table: report and attend to nothing (output rows become 0)
    n_tiles = 0;
    if (threadIdx.x == 0) atomicOr(a.status, QB_DEV_BAD_SEGMENT);
  }

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    for (int s = 0; s < kStagesAttn; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_full[b]), 1);
      mbar_init(smem_u32(&s_free[b]), 128);
    }
    mbar_init(smem_u32(p_full), 128);
    mbar_init(smem_u32(pv_full), 1);
    mbar_init(smem_u32(q_ready), 128);
    *abort_flag = 0;
    *drain_flag = 0;
    fence_barrier_init();
  }
  if (threadIdx.x >= 64 && threadIdx.x < 72) temporal_cos_sin(__ldg(a.frame_t), threadIdx.x - 64, tm);
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const uint32_t tmem_s[2] = {tmem_base, tmem_base + 128};
  const uint32_t tmem_pv = tmem_base + 256;

  if (warp == 0) {
    // ---------------- TMA producer
    if (elect_one()) {
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStagesAttn;
        const uint32_t ph = (j / kStagesAttn) & 1;
        if (!mbar_wait(smem_u32(&kv_empty[s]), ph ^ 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
        int row, valid;
        locate_tile(seg, nseg, j, row, valid);
        const uint32_t fb = smem_u32(&kv_full[s]);
        mbar_arrive_expect_tx(fb, L::kStageBytes);
        uint8_t* st = smem + L::kStageOff + s * L::kStageBytes;
        tma_load_2d(smem_u32(st), &tmK, fb, 0, kvh * a.capacity + row);
        if (kFp8) {
          tma_load_2d(smem_u32(st + L::kKBytes), &tmV, fb, row, kvh * 64);
        } else {
          tma_load_2d(smem_u32(st + L::kKBytes), &tmV, fb, row, kvh * 64);
          tma_load_2d(smem_u32(st + L::kKBytes + L::kVBytes / 2), &tmV, fb, row + 64, kvh * 64);
        }
        issued = j + 1;
      }
      if (*abort_flag) {
        // Giving up: let the copies already in flight land before this CTA's memory goes away.
        for (int j = max(0, issued - kStagesAttn); j < issued; ++j)
          mbar_wait(smem_u32(&kv_full[j % kStagesAttn]), (j / kStagesAttn) & 1, drain_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
      } else {
        // Tail: see the last stage releases land before the CTA can exit.
        for (int j = max(0, n_tiles - kStagesAttn); j < n_tiles; ++j)
          if (!mbar_wait(smem_u32(&kv_empty[j % kStagesAttn]), (j / kStagesAttn) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer
    if (elect_one() && n_tiles > 0) {
      const uint32_t q_addr = smem_u32(q_s), p_addr = smem_u32(p_s);
      auto issue_s = [&](int j) {
        const uint32_t k_addr = smem_u32(smem + L::kStageOff + (j % kStagesAttn) * L::kStageBytes);
        if (kFp8) {
          const uint64_t qd = umma_desc_k_sw64(q_addr), kd = umma_desc_k_sw64(k_addr);
#pragma unroll
          for (int k = 0; k < 2; ++k) umma_f8(tmem_s[j & 1], qd + 2 * k, kd + 2 * k, kIdescS, k > 0);
        } else {
          const uint64_t qd = umma_desc_k_sw128(q_addr), kd = umma_desc_k_sw128(k_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem_s[j & 1], qd + 2 * k, kd + 2 * k, kIdescS, k > 0);
        }
        umma_commit(smem_u32(&s_full[j & 1]));
      };
      bool ok = mbar_wait(smem_u32(q_ready), 0, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
      ok = ok && mbar_wait(smem_u32(&kv_full[0]), 0, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int j = 0; j < n_tiles && ok; ++j) {
        if (j + 1 < n_tiles) {
          const int jn = j + 1;
          ok = mbar_wait(smem_u32(&kv_full[jn % kStagesAttn]), (jn / kStagesAttn) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
          const int use = jn >> 1;
          if (ok && use > 0) ok = mbar_wait(smem_u32(&s_free[jn & 1]), (use - 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
          if (!ok) break;
          tc_fence_after();
          issue_s(jn);
        }
        ok = mbar_wait(smem_u32(p_full), j & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = smem_u32(smem + L::kStageOff + (j % kStagesAttn) * L::kStageBytes + L::kKBytes);
        if (kFp8) {
          const uint64_t pd = umma_desc_k_sw128(p_addr), vd = umma_desc_k_sw128(v_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(tmem_pv, pd + 2 * k, vd + 2 * k, kIdescPV, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t pd = umma_desc_k_sw128(p_addr + (k >> 2) * (L::kPBytes / 2));
            const uint64_t vd = umma_desc_k_sw128(v_addr + (k >> 2) * (L::kVBytes / 2));
            umma_f16(tmem_pv, pd + 2 * (k & 3), vd + 2 * (k & 3), kIdescPV, k > 0);
          }
        }
        umma_commit(smem_u32(pv_full));
        umma_commit(smem_u32(&kv_empty[j % kStagesAttn]));
      }
    }
  } else {
    // ---------------- softmax / output: one query row per thread
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int t = q0 + r;
    const bool row_ok = t < a.tpf;
    const uint32_t lane_addr = static_cast<uint32_t>(lane_grp * 32) << 16;

    // Q row -> RoPE -> shared memory (K-major, swizzled like a TMA tile)
    {
      float xy[16];
      float y0[32], y1[32];
      if (row_ok) {
        const float4* rp = reinterpret_cast<const float4*>(a.rope_xy + static_cast<size_t>(t) * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float4 v = __ldg(rp + i);
          xy[4 * i] = v.x; xy[4 * i + 1] = v.y; xy[4 * i + 2] = v.z; xy[4 * i + 3] = v.w;
        }
        const uint4* src = reinterpret_cast<const uint4*>(a.qkv + static_cast<size_t>(t) * a.qkv_dim + qh * 64);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          const uint4 x = __ldg(src + v);
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int p = v * 4 + j;
            float c, s;
            pair_cos_sin(p, xy, tm, c, s);
            const float x0 = bf16lo(w[j]), x1 = bf16hi(w[j]);
            y0[p] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            y1[p] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
          }
        }
      } else {
#pragma unroll
        for (int p = 0; p < 32; ++p) y0[p] = y1[p] = 0.f;
      }
      if (kFp8) {
        // 64-byte rows, 16-byte chunk index XOR ((row >> 1) & 3)
        uint8_t* rowp = q_s + r * 64;
        const int sw = (r >> 1) & 3;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          *reinterpret_cast<uint4*>(rowp + ((c ^ sw) << 4)) =
              make_uint4(pack_e4m3x4(y0[16 * c], y0[16 * c + 1], y0[16 * c + 2], y0[16 * c + 3]),
                         pack_e4m3x4(y0[16 * c + 4], y0[16 * c + 5], y0[16 * c + 6], y0[16 * c + 7]),
                         pack_e4m3x4(y0[16 * c + 8], y0[16 * c + 9], y0[16 * c + 10], y0[16 * c + 11]),
                         pack_e4m3x4(y0[16 * c + 12], y0[16 * c + 13], y0[16 * c + 14], y0[16 * c + 15]));
          *reinterpret_cast<uint4*>(rowp + (((c + 2) ^ sw) << 4)) =
              make_uint4(pack_e4m3x4(y1[16 * c], y1[16 * c + 1], y1[16 * c + 2], y1[16 * c + 3]),
                         pack_e4m3x4(y1[16 * c + 4], y1[16 * c + 5], y1[16 * c + 6], y1[16 * c + 7]),
                         pack_e4m3x4(y1[16 * c + 8], y1[16 * c + 9], y1[16 * c + 10], y1[16 * c + 11]),
                         pack_e4m3x4(y1[16 * c + 12], y1[16 * c + 13], y1[16 * c + 14], y1[16 * c + 15]));
        }
      } else {
        uint8_t* rowp = q_s + r * 128;
        const int sw = r & 7;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          *reinterpret_cast<uint4*>(rowp + ((c ^ sw) << 4)) =
              make_uint4(pack_bf16x2(y0[8 * c], y0[8 * c + 1]), pack_bf16x2(y0[8 * c + 2], y0[8 * c + 3]),
                         pack_bf16x2(y0[8 * c + 4], y0[8 * c + 5]), pack_bf16x2(y0[8 * c + 6], y0[8 * c + 7]));
          *reinterpret_cast<uint4*>(rowp + (((c + 4) ^ sw) << 4)) =
              make_uint4(pack_bf16x2(y1[8 * c], y1[8 * c + 1]), pack_bf16x2(y1[8 * c + 2], y1[8 * c + 3]),
                         pack_bf16x2(y1[8 * c + 4], y1[8 * c + 5]), pack_bf16x2(y1[8 * c + 6], y1[8 * c + 7]));
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(q_ready));
    }

    const float ks = a.k_scale ? __ldg(a.k_scale + kvh) : 1.0f;
    const float sl2 = ks * 0.125f * 1.4426950408889634f;  // scores -> log2 domain, 1/sqrt(64) folded in
    float m_run = -1.0e30f, l_run = 0.f, alpha_prev = 0.f;
    float o[64];
#pragma unroll
    for (int d = 0; d < 64; ++d) o[d] = 0.f;
    bool ok = true;

    auto fold_pv = [&](int j) {  // o = o * alpha + PV(j)
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(pv_full), j & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (!ok) return;
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rr[32];
        tmem_ld32(tmem_pv + lane_addr + c * 32, rr);
        tmem_wait_ld();
#pragma unroll
        for (int i = 0; i < 32; ++i) o[c * 32 + i] = fmaf(o[c * 32 + i], alpha_prev, __uint_as_float(rr[i]));
      }
    };

    for (int j = 0; j < n_tiles && ok; ++j) {
      int row, valid;
      locate_tile(seg, nseg, j, row, valid);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[j & 1]), (j >> 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (!ok) break;
      tc_fence_after();
      const uint32_t s_addr = tmem_s[j & 1] + lane_addr;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t rr[32];
        tmem_ld32(s_addr + c * 32, rr);
        tmem_wait_ld();
        if (valid == kKeyTile) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(rr[i]));
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i)
            if (c * 32 + i < valid) mx = fmaxf(mx, __uint_as_float(rr[i]));
        }
      }
      const float m_new = fmaxf(m_run, mx * sl2);
      const float alpha = ex2_approx(m_run - m_new);
      if (j > 0) {
        fold_pv(j - 1);
        if (!ok) break;
      }
      // pass 2: probabilities -> shared memory
      const float mshift = m_new - kPShift;
      float lsum = 0.f;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t rr[32];
        tmem_ld32(s_addr + c * 32, rr);
        tmem_wait_ld();
        float p[32];
#pragma unroll
        for (int i = 0; i < 32; ++i) {
          float e = ex2_approx(fmaf(__uint_as_float(rr[i]), sl2, -mshift));
          if (valid != kKeyTile && c * 32 + i >= valid) e = 0.f;
          p[i] = e;
          lsum += e;
        }
        if (kFp8) {
          uint8_t* rowp = p_s + r * 128;
          const int sw = r & 7;
#pragma unroll
          for (int h = 0; h < 2; ++h) {
            const int chunk = c * 2 + h;
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ sw) << 4)) =
                make_uint4(pack_e4m3x4(p[16 * h], p[16 * h + 1], p[16 * h + 2], p[16 * h + 3]),
                           pack_e4m3x4(p[16 * h + 4], p[16 * h + 5], p[16 * h + 6], p[16 * h + 7]),
                           pack_e4m3x4(p[16 * h + 8], p[16 * h + 9], p[16 * h + 10], p[16 * h + 11]),
                           pack_e4m3x4(p[16 * h + 12], p[16 * h + 13], p[16 * h + 14], p[16 * h + 15]));
          }
        } else {
          // keys 0..63 in the first 16 KB half, 64..127 in the second; 128-byte rows
          uint8_t* rowp = p_s + (c >> 1) * (L::kPBytes / 2) + r * 128;
          const int sw = r & 7;
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            const int chunk = (c & 1) * 4 + h;
            *reinterpret_cast<uint4*>(rowp + ((chunk ^ sw) << 4)) =
                make_uint4(pack_bf16x2(p[8 * h], p[8 * h + 1]), pack_bf16x2(p[8 * h + 2], p[8 * h + 3]),
                           pack_bf16x2(p[8 * h + 4], p[8 * h + 5]), pack_bf16x2(p[8 * h + 6], p[8 * h + 7]));
          }
        }
      }
      l_run = fmaf(l_run, alpha, lsum);
      m_run = m_new;
      alpha_prev = alpha;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(p_full));
      mbar_arrive(smem_u32(&s_free[j & 1]));
    }
    if (ok && n_tiles > 0) fold_pv(n_tiles - 1);

    if (ok && row_ok) {
      const float vs = a.v_scale ? __ldg(a.v_scale + kvh) : 1.0f;
      const float inv = l_run > 0.f ? vs / l_run : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * (a.n_q_heads * 64) + qh * 64);
#pragma unroll
      for (int v = 0; v < 8; ++v)
        dst[v] = make_uint4(pack_bf16x2(o[8 * v] * inv, o[8 * v + 1] * inv), pack_bf16x2(o[8 * v + 2] * inv, o[8 * v + 3] * inv),
                            pack_bf16x2(o[8 * v + 4] * inv, o[8 * v + 5] * inv), pack_bf16x2(o[8 * v + 6] * inv, o[8 * v + 7] * inv));
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace qb

using namespace qb;

extern "C" size_t qb_owl_attn_workspace_bytes(const qb_attn_params* p) {
  (void)p;
  return 0;
}

extern "C" int32_t qb_owl_attn(const void* qkv, const void* K_cache, const void* Vt_cache, const int32_t* segments,
                               const int32_t* n_segments, const int32_t* frame_t, void* out, const float* rope_xy,
                               const qb_attn_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  (void)workspace;
  (void)workspace_bytes;
  QB_REQUIRE(p != nullptr, QB_ERR_INVALID_ARG, "owl_attn: params are NULL");
  QB_REQUIRE(qkv && K_cache && Vt_cache && segments && n_segments && frame_t && out && rope_xy, QB_ERR_INVALID_ARG,
             "owl_attn: NULL pointer");
  QB_REQUIRE(p->quilt_factor == 1, QB_ERR_UNSUPPORTED, "owl_attn: quilt_factor %d is not supported (only 1)", p->quilt_factor);
  QB_REQUIRE(p->packed_qkv == 1, QB_ERR_UNSUPPORTED, "owl_attn: only the packed-QKV layout is supported");
  QB_REQUIRE(p->n_kv_heads > 0 && p->gqa_ratio > 0 && p->H_spatial > 0 && p->W_spatial > 0 && p->num_buckets > 0,
             QB_ERR_INVALID_ARG, "owl_attn: sizes must be positive");
  QB_REQUIRE(p->kv_dtype == QB_BF16 || p->kv_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "owl_attn: kv_dtype %d", p->kv_dtype);
  QB_REQUIRE(p->compute_dtype == p->kv_dtype, QB_ERR_UNSUPPORTED,
             "owl_attn: compute_dtype must equal kv_dtype (bf16 cache + bf16 MMAs, or e4m3 cache + e4m3 MMAs)");
  QB_REQUIRE(p->max_segments >= 1, QB_ERR_INVALID_ARG, "owl_attn: max_segments %d", p->max_segments);
  const int tpf = p->H_spatial * p->W_spatial;
  const int cap = (p->num_buckets + 1) * tpf;
  QB_REQUIRE(cap % 16 == 0, QB_ERR_UNSUPPORTED, "owl_attn: capacity %d must be a multiple of 16", cap);
  QB_REQUIRE(aligned16(qkv) && aligned16(K_cache) && aligned16(Vt_cache) && aligned16(out) && aligned16(rope_xy), QB_ERR_ALIGN,
             "owl_attn: pointers must be 16-byte aligned");
  const bool fp8 = p->kv_dtype == QB_E4M3;
  const int es = fp8 ? 1 : 2;
  const int Hq = p->n_kv_heads * p->gqa_ratio;
  CUtensorMap tmK, tmV;
  int32_t rc = make_tmap_2d_sw(&tmK, K_cache, es, static_cast<uint64_t>(p->n_kv_heads) * cap, 64, kKeyTile, 64, fp8 ? 64 : 128);
  if (rc != QB_OK) return rc;
  rc = make_tmap_2d_sw(&tmV, Vt_cache, es, static_cast<uint64_t>(p->n_kv_heads) * 64, cap, 64, fp8 ? 128 : 64, 128);
  if (rc != QB_OK) return rc;

  AttnArgs a{};
  a.qkv = static_cast<const uint16_t*>(qkv);
  a.segments = segments; a.n_segments = n_segments; a.frame_t = frame_t;
  a.out = static_cast<uint16_t*>(out);
  a.rope_xy = rope_xy;
  a.k_scale = p->k_scale; a.v_scale = p->v_scale;
  a.status = status_word();
  QB_REQUIRE(a.status != nullptr, QB_ERR_CUDA, "owl_attn: device status word unavailable");
  a.tpf = tpf;
  a.qkv_dim = (Hq + 2 * p->n_kv_heads) * 64;
  a.n_q_heads = Hq; a.gqa = p->gqa_ratio; a.capacity = cap; a.max_segments = p->max_segments;

  dim3 grid((tpf + kQTile - 1) / kQTile, Hq);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (fp8) {
    QB_CUDA_OK(cudaFuncSetAttribute(owl_attn_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<true>::kTotal));
    owl_attn_kernel<true><<<grid, kAttnThreads, AttnSmem<true>::kTotal, st>>>(tmK, tmV, a);
  } else {
    QB_CUDA_OK(cudaFuncSetAttribute(owl_attn_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem<false>::kTotal));
    owl_attn_kernel<false><<<grid, kAttnThreads, AttnSmem<false>::kTotal, st>>>(tmK, tmV, a);
  }
  return check_launch("owl_attn kernel");
}
