// owl_attn: segment-sparse GQA flash attention with inline ortho-RoPE on Q, head_dim 64.
//
// One CTA owns 128 query tokens of one Q head and walks the valid keys in tiles of 128, enumerated
// from the (start, length) segment table, so a masked bucket is never loaded.  384 threads:
//   warp 0        TMA producer: K tile [128 keys x 64] and V^T tile [64 x 128 keys] per stage
//   warps 1, 2    one thread each issues tcgen05.mma for softmax group 0 / 1: S = Q K^T and PV = P V
//   warp 3        idle (keeps the softmax warps aligned to the TMEM lane quarters)
//   warps 4-7     softmax group 0: even key tiles        warps 8-11  softmax group 1: odd key tiles
// Each softmax group runs its own online softmax over its half of the tiles, one query row per
// thread, with two S buffers in TMEM (S(i+1) is computed while the group works on S(i)), its own P
// buffer in shared memory, and PV(i) written over the TMEM columns of the S(i) it came from.  The two
// partial results (row max, row sum, 64 outputs) are merged once at the end.  Two independent groups
// give every SM sub-partition two warps of exp / FMA work to interleave; a single group (one warp
// per sub-partition) is latency bound.
//
// The row sum of P comes out of the tensor core: 16 rows of ones follow the 64 V^T rows of every
// stage, so PV has 80 columns and column 64 is sum_k P[q, k] of exactly the rounded P that is
// multiplied with V.  bf16 path: kind::f16 MMAs, P rounded to bf16.  fp8 path: Q (after RoPE), K, V
// and P are e4m3 (kind::f8f6f4); P is scaled by 2^8 so small probabilities keep mantissa bits (the
// factor cancels in the division by the row sum).  exp2 is ex2.approx.f32 in both paths: measured on
// B200, ex2.approx.f16x2 issues at half the rate of the f32 form (no gain per element) and the
// f16x2 -> e4m3x2 conversion is four times slower than f32 -> e4m3x2.
#include <cuda.h>

#include "common.cuh"
#include "rope.cuh"
#include "sm100.cuh"

namespace qb {

int32_t make_tmap_2d_sw(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols, int swizzle_bytes);

constexpr int kAttnThreads = 384;
constexpr int kQTile = 128;
constexpr int kKeyTile = 128;
constexpr int kVRows = 80;  // 64 channels + 16 rows of ones (row sum of P)

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
  int tpf, qkv_dim, n_q_heads, gqa, capacity, max_segments;
};

template <bool kFp8>
struct AttnSmem {
  static constexpr int kEs = kFp8 ? 1 : 2;
  static constexpr int kStages = kFp8 ? 4 : 3;
  static constexpr int kQBytes = kQTile * 64 * kEs;          // 16 KB | 8 KB
  static constexpr int kKBytes = kKeyTile * 64 * kEs;        // 16 KB | 8 KB
  static constexpr int kVTile = kVRows * 128;                // one 128-byte-wide V^T tile incl. ones rows: 10 KB
  static constexpr int kVBytes = kVTile * kEs;               // bf16: two tiles (keys 0-63, 64-127)
  static constexpr int kPBytes = kQTile * kKeyTile * kEs;    // 32 KB | 16 KB, per softmax group
  static constexpr int kStageBytes = kKBytes + kVBytes;
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kQOff + kQBytes;
  static constexpr int kStageOff = kPOff + 2 * kPBytes;
  static constexpr int kBarOff = kStageOff + kStages * kStageBytes;
  static constexpr int kTotal = kBarOff + 512 + 1024;
  static_assert(kStages * kStageBytes >= 66 * 128 * 4, "merge buffer aliases the stage area");
};

__device__ __forceinline__ float ex2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
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

// 32 columns of one score row -> probabilities -> the P tile in shared memory (layout of a TMA tile).
template <bool kFp8, bool kMasked>
__device__ __forceinline__ void p_chunk(uint32_t tmem_s, int c, int valid, float sl2, float nshift, uint8_t* p_s, int r) {
  uint32_t rr[32];
  tmem_ld32(tmem_s + c * 32, rr);
  tmem_wait_ld();
  float e[32];
#pragma unroll
  for (int q = 0; q < 32; ++q) {
    float x = fmaf(__uint_as_float(rr[q]), sl2, nshift);
    if (kMasked && c * 32 + q >= valid) x = -INFINITY;
    e[q] = ex2_approx(x);
  }
  const int sw = r & 7;
  if (kFp8) {
    uint32_t w[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) w[q] = pack_e4m3x4(e[4 * q], e[4 * q + 1], e[4 * q + 2], e[4 * q + 3]);
    uint8_t* rowp = p_s + r * 128;
    *reinterpret_cast<uint4*>(rowp + (((2 * c) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(rowp + (((2 * c + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    // keys 0..63 in the first half of the P buffer, 64..127 in the second; 128-byte rows
    uint32_t w[16];
#pragma unroll
    for (int q = 0; q < 16; ++q) w[q] = pack_bf16x2(e[2 * q], e[2 * q + 1]);
    uint8_t* rowp = p_s + (c >> 1) * (kQTile * kKeyTile) + r * 128;
#pragma unroll
    for (int h = 0; h < 4; ++h)
      *reinterpret_cast<uint4*>(rowp + ((((c & 1) * 4 + h) ^ sw) << 4)) = make_uint4(w[4 * h], w[4 * h + 1], w[4 * h + 2], w[4 * h + 3]);
  }
}

template <bool kFp8>
__global__ void __launch_bounds__(kAttnThreads, 1)
owl_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using L = AttnSmem<kFp8>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescS = kFp8 ? umma_idesc(0, 0, 128, 128) : umma_idesc(1, 1, 128, 128);
  constexpr uint32_t kIdescPV = kFp8 ? umma_idesc(0, 0, 128, kVRows) : umma_idesc(1, 1, 128, kVRows);
  constexpr float kPShift = kFp8 ? 8.0f : 0.0f;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem + L::kQOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;                  // [stages]
  uint64_t* kv_empty = bars + kStages;       // [stages]
  uint64_t* s_full = bars + 2 * kStages;     // [group][buffer]
  uint64_t* s_free = s_full + 4;             // [group][buffer]
  uint64_t* p_full = s_free + 4;             // [group]
  uint64_t* pv_full = p_full + 2;            // [group]
  uint64_t* q_ready = pv_full + 2;
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
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_full[2 * b]), 1);
      mbar_init(smem_u32(&s_full[2 * b + 1]), 1);
      mbar_init(smem_u32(&s_free[2 * b]), 128);
      mbar_init(smem_u32(&s_free[2 * b + 1]), 128);
      mbar_init(smem_u32(&p_full[b]), 128);
      mbar_init(smem_u32(&pv_full[b]), 1);
    }
    mbar_init(smem_u32(q_ready), 256);
    *abort_flag = 0;
    *drain_flag = 0;
    fence_barrier_init();
  }
  if (threadIdx.x >= 96 && threadIdx.x < 104) temporal_cos_sin(__ldg(a.frame_t), threadIdx.x - 96, tm);
  // rows of ones under every V^T tile (16 rows x 128 bytes each): the tensor core then returns the row sum of P
  {
    constexpr uint32_t kOnes = kFp8 ? 0x38383838u : 0x3F803F80u;
    constexpr int kTilesPerStage = kFp8 ? 1 : 2;
    for (int i = threadIdx.x; i < kStages * kTilesPerStage * 128; i += kAttnThreads) {  // 128 x 16 bytes per tile
      const int tile = i >> 7, v = i & 127;
      uint8_t* base = smem + L::kStageOff + (tile / kTilesPerStage) * L::kStageBytes + L::kKBytes + (tile % kTilesPerStage) * L::kVTile;
      *reinterpret_cast<uint4*>(base + 64 * 128 + v * 16) = make_uint4(kOnes, kOnes, kOnes, kOnes);
    }
    fence_proxy_async_smem();
  }
  if (warp == 1) {
    tmem_alloc(smem_u32(tmem_slot), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 0) {
    // ---------------- TMA producer
    if (elect_one()) {
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(smem_u32(&kv_empty[s]), ph ^ 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
        int row, valid;
        locate_tile(seg, nseg, j, row, valid);
        const uint32_t fb = smem_u32(&kv_full[s]);
        mbar_arrive_expect_tx(fb, L::kKBytes + (kFp8 ? 1 : 2) * 64 * 128);
        uint8_t* st = smem + L::kStageOff + s * L::kStageBytes;
        tma_load_2d(smem_u32(st), &tmK, fb, 0, kvh * a.capacity + row);
        tma_load_2d(smem_u32(st + L::kKBytes), &tmV, fb, row, kvh * 64);
        if (!kFp8) tma_load_2d(smem_u32(st + L::kKBytes + L::kVTile), &tmV, fb, row + 64, kvh * 64);
        issued = j + 1;
      }
      if (*abort_flag) {
        // Giving up: let the copies already in flight land before this CTA's memory goes away.
        for (int j = max(0, issued - kStages); j < issued; ++j)
          mbar_wait(smem_u32(&kv_full[j % kStages]), (j / kStages) & 1, drain_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
      } else {
        // Tail: see the last stage releases land before the CTA can exit.
        for (int j = max(0, n_tiles - kStages); j < n_tiles; ++j)
          if (!mbar_wait(smem_u32(&kv_empty[j % kStages]), (j / kStages) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
      }
    }
  } else if (warp == 1 || warp == 2) {
    // ---------------- MMA issuers: warp 1 serves softmax group 0 (even tiles), warp 2 group 1 (odd tiles).
    // Per group: S(i) goes to TMEM buffer i & 1 of the group; once the group has turned S(i) into P(i),
    // PV(i) is written over the first 80 columns of the same buffer; the buffer is free for S(i + 2)
    // when the group has folded PV(i) into its registers.  S(i + 1) is issued ahead of PV(i).
    const int g = warp - 1;
    const int n_g = n_tiles > g ? (n_tiles - g + 1) / 2 : 0;
    if (elect_one() && n_g > 0) {
      const uint32_t q_addr = smem_u32(q_s);
      const uint32_t p_addr = smem_u32(smem + L::kPOff + g * L::kPBytes);
      auto stage_addr = [&](int j) { return smem_u32(smem + L::kStageOff + (j % kStages) * L::kStageBytes); };
      auto issue_s = [&](int i) {
        const uint32_t k_addr = stage_addr(2 * i + g);
        const uint32_t d = tmem_base + g * 256 + (i & 1) * 128;
        if (kFp8) {
          const uint64_t qd = umma_desc_k_sw64(q_addr), kd = umma_desc_k_sw64(k_addr);
#pragma unroll
          for (int k = 0; k < 2; ++k) umma_f8(d, qd + 2 * k, kd + 2 * k, kIdescS, k > 0);
        } else {
          const uint64_t qd = umma_desc_k_sw128(q_addr), kd = umma_desc_k_sw128(k_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(d, qd + 2 * k, kd + 2 * k, kIdescS, k > 0);
        }
        umma_commit(smem_u32(&s_full[2 * g + (i & 1)]));
      };
      auto wait_tile = [&](int j) {
        return mbar_wait(smem_u32(&kv_full[j % kStages]), (j / kStages) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
      };
      bool ok = mbar_wait(smem_u32(q_ready), 0, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
      ok = ok && wait_tile(g);
      if (ok) {
        tc_fence_after();
        issue_s(0);
      }
      for (int i = 0; i < n_g && ok; ++i) {
        if (i + 1 < n_g) {
          const int in = i + 1;
          ok = wait_tile(2 * in + g);
          if (ok && in >= 2)
            ok = mbar_wait(smem_u32(&s_free[2 * g + (in & 1)]), ((in >> 1) - 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
          if (!ok) break;
          tc_fence_after();
          issue_s(in);
        }
        ok = mbar_wait(smem_u32(&p_full[g]), i & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
        if (!ok) break;
        tc_fence_after();
        const uint32_t v_addr = stage_addr(2 * i + g) + L::kKBytes;
        const uint32_t d = tmem_base + g * 256 + (i & 1) * 128;
        if (kFp8) {
          const uint64_t pd = umma_desc_k_sw128(p_addr), vd = umma_desc_k_sw128(v_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(d, pd + 2 * k, vd + 2 * k, kIdescPV, k > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t pd = umma_desc_k_sw128(p_addr + (k >> 2) * (L::kPBytes / 2));
            const uint64_t vd = umma_desc_k_sw128(v_addr + (k >> 2) * L::kVTile);
            umma_f16(d, pd + 2 * (k & 3), vd + 2 * (k & 3), kIdescPV, k > 0);
          }
        }
        umma_commit(smem_u32(&pv_full[g]));
        umma_commit(smem_u32(&kv_empty[(2 * i + g) % kStages]));
      }
    }
  } else if (warp >= 4) {
    // ---------------- softmax groups: one query row per thread, group g takes tiles j = 2 i + g
    const int g = (warp - 4) >> 2;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int t = q0 + r;
    const bool row_ok = t < a.tpf;
    const uint32_t lane_addr = static_cast<uint32_t>(lane_grp * 32) << 16;
    uint8_t* p_s = smem + L::kPOff + g * L::kPBytes;

    // Q row -> RoPE -> shared memory (K-major, swizzled like a TMA tile).  Group 0 rotates pairs
    // 0..15 (spatial angles), group 1 pairs 16..31 (temporal angles).
    {
      float y0[16], y1[16];
      if (row_ok) {
        float xy[16];
        if (g == 0) {
          const float4* rp = reinterpret_cast<const float4*>(a.rope_xy + static_cast<size_t>(t) * 16);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 v = __ldg(rp + i);
            xy[4 * i] = v.x; xy[4 * i + 1] = v.y; xy[4 * i + 2] = v.z; xy[4 * i + 3] = v.w;
          }
        }
        const uint4* src = reinterpret_cast<const uint4*>(a.qkv + static_cast<size_t>(t) * a.qkv_dim + qh * 64 + g * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 x = __ldg(src + v);
          const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int pl = v * 4 + j;
            const int i = pl >> 1;
            const float c = g == 0 ? xy[i] : tm[i];
            const float s = g == 0 ? xy[8 + i] : tm[8 + i];
            const float x0 = bf16lo(w[j]), x1 = bf16hi(w[j]);
            y0[pl] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
            y1[pl] = __fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s));
          }
        }
      } else {
#pragma unroll
        for (int p = 0; p < 16; ++p) y0[p] = y1[p] = 0.f;
      }
      if (kFp8) {
        // 64-byte rows; 16-byte chunk index XOR ((row >> 1) & 3); y0 of this group is chunk g, y1 chunk 2 + g
        uint8_t* rowp = q_s + r * 64;
        const int sw = (r >> 1) & 3;
        *reinterpret_cast<uint4*>(rowp + ((g ^ sw) << 4)) =
            make_uint4(pack_e4m3x4(y0[0], y0[1], y0[2], y0[3]), pack_e4m3x4(y0[4], y0[5], y0[6], y0[7]),
                       pack_e4m3x4(y0[8], y0[9], y0[10], y0[11]), pack_e4m3x4(y0[12], y0[13], y0[14], y0[15]));
        *reinterpret_cast<uint4*>(rowp + (((2 + g) ^ sw) << 4)) =
            make_uint4(pack_e4m3x4(y1[0], y1[1], y1[2], y1[3]), pack_e4m3x4(y1[4], y1[5], y1[6], y1[7]),
                       pack_e4m3x4(y1[8], y1[9], y1[10], y1[11]), pack_e4m3x4(y1[12], y1[13], y1[14], y1[15]));
      } else {
        // 128-byte rows; chunk XOR (row & 7); y0 of this group is chunks 2g, 2g+1, y1 chunks 4+2g, 5+2g
        uint8_t* rowp = q_s + r * 128;
        const int sw = r & 7;
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          *reinterpret_cast<uint4*>(rowp + (((2 * g + c) ^ sw) << 4)) =
              make_uint4(pack_bf16x2(y0[8 * c], y0[8 * c + 1]), pack_bf16x2(y0[8 * c + 2], y0[8 * c + 3]),
                         pack_bf16x2(y0[8 * c + 4], y0[8 * c + 5]), pack_bf16x2(y0[8 * c + 6], y0[8 * c + 7]));
          *reinterpret_cast<uint4*>(rowp + (((4 + 2 * g + c) ^ sw) << 4)) =
              make_uint4(pack_bf16x2(y1[8 * c], y1[8 * c + 1]), pack_bf16x2(y1[8 * c + 2], y1[8 * c + 3]),
                         pack_bf16x2(y1[8 * c + 4], y1[8 * c + 5]), pack_bf16x2(y1[8 * c + 6], y1[8 * c + 7]));
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(smem_u32(q_ready));
    }

    const float ks = a.k_scale ? __ldg(a.k_scale + kvh) : 1.0f;
    const float sl2 = ks * 0.125f * 1.4426950408889634f;  // scores -> log2 domain, 1/sqrt(64) folded in
    const uint32_t tmem_g = tmem_base + g * 256 + lane_addr;  // this group's two S / PV buffers
    float m_run = -1.0e30f, alpha_prev = 0.f, l_run = 0.f;
    float2 o2[32];
#pragma unroll
    for (int d = 0; d < 32; ++d) o2[d] = make_float2(0.f, 0.f);
    bool ok = true;
    const int my_tiles = n_tiles > g ? (n_tiles - g + 1) / 2 : 0;

    auto fold_pv = [&](int i) {  // o = o * alpha + PV(tile i of this group); column 64 carries the row sum
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&pv_full[g]), i & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (!ok) return;
      tc_fence_after();
      const uint32_t tmem_pv = tmem_g + (i & 1) * 128;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t rr[32];
        tmem_ld32(tmem_pv + c * 32, rr);
        tmem_wait_ld();
#pragma unroll
        for (int q = 0; q < 16; ++q)
          {
            o2[c * 16 + q].x = fmaf(o2[c * 16 + q].x, alpha_prev, __uint_as_float(rr[2 * q]));
            o2[c * 16 + q].y = fmaf(o2[c * 16 + q].y, alpha_prev, __uint_as_float(rr[2 * q + 1]));
          }
      }
      uint32_t r16[16];
      tmem_ld16(tmem_pv + 64, r16);
      tmem_wait_ld();
      l_run = fmaf(l_run, alpha_prev, __uint_as_float(r16[0]));
      tc_fence_before();
      mbar_arrive(smem_u32(&s_free[2 * g + (i & 1)]));  // the buffer may take S(i + 2) now
    };

    for (int i = 0; i < my_tiles && ok; ++i) {
      int row, valid;
      locate_tile(seg, nseg, 2 * i + g, row, valid);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[2 * g + (i & 1)]), (i >> 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (!ok) break;
      tc_fence_after();
      const uint32_t tmem_s = tmem_g + (i & 1) * 128;
      // pass 1: row maximum
      float mx = -INFINITY;
#pragma unroll 1
      for (int c = 0; c < 4; ++c) {
        uint32_t rr[32];
        tmem_ld32(tmem_s + c * 32, rr);
        tmem_wait_ld();
        if (valid == kKeyTile) {
          float m0 = mx, m1 = -INFINITY;  // two chains of 3-input max: 16 instructions for 32 values
#pragma unroll
          for (int q = 0; q < 8; ++q) {
            m0 = max3f(m0, __uint_as_float(rr[4 * q]), __uint_as_float(rr[4 * q + 1]));
            m1 = max3f(m1, __uint_as_float(rr[4 * q + 2]), __uint_as_float(rr[4 * q + 3]));
          }
          mx = fmaxf(m0, m1);
        } else {
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (c * 32 + q < valid) mx = fmaxf(mx, __uint_as_float(rr[q]));
        }
      }
      const float m_new = fmaxf(m_run, mx * sl2);
      const float alpha = ex2_approx(m_run - m_new);
      if (i > 0) {
        fold_pv(i - 1);
        if (!ok) break;
      }
      // pass 2: probabilities -> shared memory.  Full tiles (all but the last tile of a segment whose
      // length is not a multiple of 128) take the path without per-element masking.
      const float nshift = kPShift - m_new;
      if (valid == kKeyTile) {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) p_chunk<kFp8, false>(tmem_s, c, valid, sl2, nshift, p_s, r);
      } else {
#pragma unroll 1
        for (int c = 0; c < 4; ++c) p_chunk<kFp8, true>(tmem_s, c, valid, sl2, nshift, p_s, r);
      }
      m_run = m_new;
      alpha_prev = alpha;
      fence_proxy_async_smem();
      tc_fence_before();
      mbar_arrive(smem_u32(&p_full[g]));
    }
    if (ok && my_tiles > 0) fold_pv(my_tiles - 1);

    // ---------------- merge the two groups (tensor work and TMA traffic are finished for both after the barrier)
    asm volatile("bar.sync 2, 256;" ::: "memory");
    float* comb = reinterpret_cast<float*>(smem + L::kStageOff);  // [66][128]
    if (g == 1) {
      comb[0 * 128 + r] = m_run;
      comb[1 * 128 + r] = l_run;
#pragma unroll
      for (int d = 0; d < 32; ++d) {
        comb[(2 + 2 * d) * 128 + r] = o2[d].x;
        comb[(3 + 2 * d) * 128 + r] = o2[d].y;
      }
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (g == 0 && ok && row_ok && *abort_flag == 0) {
      const float m1 = comb[r], l1 = comb[128 + r];
      const float m = fmaxf(m_run, m1);
      const float a0 = ex2_approx(m_run - m), a1 = ex2_approx(m1 - m);
      const float l = l_run * a0 + l1 * a1;
      const float vs = a.v_scale ? __ldg(a.v_scale + kvh) : 1.0f;
      const float inv = l > 0.f ? vs / l : 0.f;
      const float s0 = a0 * inv, s1 = a1 * inv;
      uint4* dst = reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * (a.n_q_heads * 64) + qh * 64);
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          const int d = 4 * v + q;
          const float e0 = o2[d].x * s0 + comb[(2 + 2 * d) * 128 + r] * s1;
          const float e1 = o2[d].y * s0 + comb[(3 + 2 * d) * 128 + r] * s1;
          w[q] = pack_bf16x2(e0, e1);
        }
        dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
        if (a.out_q != nullptr) {  // narrowed from the bf16-rounded values: equals a separate bf16 -> e4m3 cast
          *reinterpret_cast<uint2*>(a.out_q + static_cast<size_t>(t) * (a.n_q_heads * 64) + qh * 64 + v * 8) =
              make_uint2(pack_e4m3x4(bf16lo(w[0]), bf16hi(w[0]), bf16lo(w[1]), bf16hi(w[1])),
                         pack_e4m3x4(bf16lo(w[2]), bf16hi(w[2]), bf16lo(w[3]), bf16hi(w[3])));
        }
      }
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
                               const int32_t* n_segments, const int32_t* frame_t, void* out, void* out_q, const float* rope_xy,
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
  QB_REQUIRE(aligned16(qkv) && aligned16(K_cache) && aligned16(Vt_cache) && aligned16(out) && aligned16(out_q) && aligned16(rope_xy), QB_ERR_ALIGN,
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
  a.out_q = static_cast<uint8_t*>(out_q);
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
