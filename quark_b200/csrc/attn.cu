// owl_attn: segment-sparse GQA flash attention with inline ortho-RoPE on Q, head_dim 64.
//
// One CTA owns 128 query tokens of one Q head and walks the valid keys in tiles of 128, enumerated
// from the (start, length) segment table, so a masked bucket is never loaded.  384 threads:
//   warp 0        TMA producer: K tile [128 keys x 64] and V^T tile [64 x 128 keys] per stage
//   warps 1, 2    one thread each issues tcgen05.mma for softmax group 0 / 1: S = Q K^T and O += P V
//   warp 3        idle (keeps the softmax warps aligned to the TMEM lane quarters)
//   warps 4-7     softmax group 0: even key tiles        warps 8-11  softmax group 1: odd key tiles
// After set-up the control warps hand registers to the softmax warps (setmaxnreg), each of whose
// threads keeps a whole score row of one query (128 values) in registers.
//
// Per group, TMEM holds one S tile (128 columns) and the output accumulator O (80 columns).  A softmax
// thread copies its row of S(i) to registers (S(i + 1) may then be computed), takes the row maximum,
// writes P(i) = 2^(score - m) to shared memory, and the MMA warp accumulates O += P(i) V(i) in TMEM.
// m is the maximum the row was last rescaled to, not the running maximum: O (and the row sum) are
// multiplied by 2^(m - m') only when a tile's maximum exceeds m by more than kSlack, which is rare after
// the first tiles; P then stays below 2^(kPShift + kSlack), inside the range of e4m3 / bf16.  The two
// partial results (m, row sum, 64 outputs) are merged once at the end.
//
// The exponentials bound this kernel (the special-function unit makes 16 per clock and SM; head_dim 64
// gives it only 256 tensor-core flops per exponential to hide behind), so the two groups take turns on
// them: while one group runs its exponentials the other loads its next row, finds the maximum and
// synchronises with the MMA warp.  The turn passes when half of a tile's exponentials are issued, so the
// unit always has two warps per scheduler to draw from.  Measured on B200 (720p, 8320 keys): free-running
// groups fall into lock step and leave the unit idle half of the time (73 us); strict alternation 60 us;
// alternation with the half-tile overlap 54 us.  A polynomial 2^x on the FMA pipe for part of the elements
// (QB_POLY_OF8 > 0) is slower here, because the softmax warps are issue bound as well: 57 / 61 / 63 us for
// 1 / 2 / 3 of every 8 elements.  Also measured and not kept (52 us as it stands): two threads per query row
// (16 softmax warps of 64 keys each, row maxima exchanged through shared memory) 58 us; row maxima taken
// during the exponentials instead of before them, with the rare row that outgrows its maximum written twice,
// 57 us (the instructions moved into the exponential phase lengthen it by what the phase before it saves).
// Every mbarrier wait on a softmax warp's path costs about 100 cycles per tile even when it succeeds at once
// (2 us per launch), which is why each warp arrives once (lane 0, after __syncwarp) and waits as rarely as
// the data flow allows.
//
// The row sum of P comes out of the tensor core: 16 rows of ones follow the 64 V^T rows of every
// stage, so PV has 80 columns and column 64 is sum_k P[q, k] of exactly the rounded P that is
// multiplied with V.  bf16 path: kind::f16 MMAs, P rounded to bf16.  fp8 path: Q (after RoPE), K, V
// and P are e4m3 (kind::f8f6f4); P is scaled by 2^kPShift so small probabilities keep mantissa bits (the
// factor cancels in the division by the row sum), and has two shared-memory tiles per group so that
// writing P(i) never waits for PV(i - 1).  exp2 is ex2.approx.f32 in both paths: measured on B200,
// ex2.approx.f16x2 issues at half the rate of the f32 form (no gain per element) and the f16x2 -> e4m3x2
// conversion is four times slower than f32 -> e4m3x2.
#include <cuda.h>

#include "attn_common.cuh"

namespace qb {

int32_t make_tmap_2d_sw(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols, int swizzle_bytes);

#ifdef QB_ATTN_TRACE
__device__ long long g_attn_trace[5][80][8];  // [role: softmax g0, g1, mma g0, g1][tile][point]
#define QB_TR(role, i, pt)                                                                    \
  do {                                                                                        \
    if (blockIdx.x == 1 && blockIdx.y == 5 && lane == 0 && (i) < 80) g_attn_trace[role][i][pt] = clock64(); \
  } while (0)
#else
#define QB_TR(role, i, pt) do { } while (0)
#endif

constexpr int kAttnThreads = 384;
#ifndef QB_HANDOFF
#define QB_HANDOFF 2
#endif
constexpr int kHandoffChunk = QB_HANDOFF;  // the exponentials' turn passes to the other group before this 32-key chunk
#ifndef QB_POLY_OF8
#define QB_POLY_OF8 0
#endif
constexpr int kPolyOf8 = QB_POLY_OF8;      // exponentials out of every 8 that run as a polynomial on the FMA pipe
constexpr int kCtrlRegs = 64;      // per thread, warps 0-3 (128 x 64 + 256 x 216 <= 64 K registers)
constexpr int kSoftmaxRegs = 216;  // per thread, warps 4-11
constexpr int kQTile = 128;
constexpr int kKeyTile = 128;
constexpr int kVRows = 80;  // 64 channels + 16 rows of ones (row sum of P)

template <bool kFp8>
struct AttnSmem {
  static constexpr int kEs = kFp8 ? 1 : 2;
  static constexpr int kStages = kFp8 ? 4 : 3;
  static constexpr int kQBytes = kQTile * 64 * kEs;          // 16 KB | 8 KB
  static constexpr int kKBytes = kKeyTile * 64 * kEs;        // 16 KB | 8 KB
  static constexpr int kVTile = kVRows * 128;                // one 128-byte-wide V^T tile incl. ones rows: 10 KB
  static constexpr int kVBytes = kVTile * kEs;               // bf16: two tiles (keys 0-63, 64-127)
  static constexpr int kPBytes = kQTile * kKeyTile * kEs;    // 32 KB | 16 KB, one P tile
  static constexpr int kPBufs = kFp8 ? 2 : 1;                // P tiles per softmax group (bf16: no room for two)
  static constexpr int kStageBytes = kKBytes + kVBytes;
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kQOff + kQBytes;
  static constexpr int kStageOff = kPOff + 2 * kPBufs * kPBytes;
  static constexpr int kBarOff = kStageOff + kStages * kStageBytes;
  static constexpr int kTotal = kBarOff + 512 + 1024;
  static_assert(kStages * kStageBytes >= 66 * 128 * 4, "merge buffer aliases the stage area");
};

// 2^x on the FMA and integer pipes, for the share of the exponentials that the special-function unit
// has no time for: x = n + f with n = round(x) taken from the low mantissa bits of x + 1.5 * 2^23, a
// minimax polynomial for 2^f on [-0.5, 0.5] (degree 2: 1.7e-3 relative error, below what an e4m3
// probability resolves; degree 3: 7.5e-5, below a bf16 ulp), n added to the exponent field.
template <int kDegree>
__device__ __forceinline__ float ex2_poly(float x) {
  x = fmaxf(x, -120.0f);
  const float t = x + 12582912.0f;
  const float f = x - (t - 12582912.0f);
  float p;
  if (kDegree == 2) {
    p = fmaf(0.23842892f, f, 0.70344800f);
    p = fmaf(p, f, 1.0004431f);
  } else {
    p = fmaf(0.055171669f, f, 0.24261113f);
    p = fmaf(p, f, 0.69326097f);
    p = fmaf(p, f, 0.99992806f);
  }
  return __uint_as_float(__float_as_uint(p) + (__float_as_uint(t) << 23));
}
// Element q of a chunk goes to the polynomial when (q mod 8) < kPolyOf8.
template <bool kFp8, int kPolyOf8>
__device__ __forceinline__ float p_exp(int q, float x) {
  return (q & 7) < kPolyOf8 ? ex2_poly<kFp8 ? 2 : 3>(x) : ex2_approx(x);
}

// Which 128-key tile is the j-th valid one?  Returns its first cache row and how many of its
// keys are valid.  Segments are (start, length) pairs; zero-length entries are legal.  Fully
// unrolled so the table stays in registers.
__device__ __forceinline__ void locate_tile(const int (&seg)[6], int j, int& row, int& valid) {
  row = 0;
  valid = 0;
  bool found = false;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int nt = (seg[2 * i + 1] + kKeyTile - 1) / kKeyTile;
    if (!found && j < nt) {
      row = seg[2 * i] + j * kKeyTile;
      valid = min(kKeyTile, seg[2 * i + 1] - j * kKeyTile);
      found = true;
    }
    j -= nt;
  }
}

// 32 scores of one row (registers) -> probabilities -> the P tile in shared memory (layout of a TMA tile).
template <bool kFp8, int kPolyOf8, bool kLin>
__device__ __forceinline__ void p_chunk(const uint32_t (&sc)[32], int c, float sl2, float nshift, uint8_t* p_s, int r) {
  const int sw = r & 7;
  const float nshift_lin = nshift + kLinMagic;
  auto pr = [&](int q) {
    if (kFp8 && kLin && (q & 1)) return ex2_lin_from_biased(fmaf(__uint_as_float(sc[q]), sl2, nshift_lin));
    return p_exp<kFp8, kPolyOf8>(q, fmaf(__uint_as_float(sc[q]), sl2, nshift));
  };
  if (kFp8) {
    uint32_t w[8];
#pragma unroll
    for (int q = 0; q < 8; ++q) w[q] = pack_e4m3x4(pr(4 * q), pr(4 * q + 1), pr(4 * q + 2), pr(4 * q + 3));
    uint8_t* rowp = p_s + r * 128;
    *reinterpret_cast<uint4*>(rowp + (((2 * c) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    *reinterpret_cast<uint4*>(rowp + (((2 * c + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
  } else {
    // keys 0..63 in the first half of the P buffer, 64..127 in the second; 128-byte rows
    uint8_t* rowp = p_s + (c >> 1) * (kQTile * kKeyTile) + r * 128;
#pragma unroll
    for (int h = 0; h < 4; ++h) {
      uint32_t w[4];
#pragma unroll
      for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(pr(8 * h + 2 * q), pr(8 * h + 2 * q + 1));
      *reinterpret_cast<uint4*>(rowp + ((((c & 1) * 4 + h) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
    }
  }
}

// kSplit: the keys of a (query tile, head) are shared by gridDim.z CTAs (see AttnArgs::partials).  The
// unsplit kernel is an instantiation of its own so that none of this reaches its instruction stream.
template <bool kFp8, bool kSplit, bool kLin>
__global__ void __launch_bounds__(kAttnThreads, 1)
owl_attn_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using L = AttnSmem<kFp8>;
  constexpr int kStages = L::kStages;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescS = kFp8 ? umma_idesc(0, 0, 128, 128) : umma_idesc(1, 1, 128, 128);
  constexpr uint32_t kIdescPV = kFp8 ? umma_idesc(0, 0, 128, kVRows) : umma_idesc(1, 1, 128, kVRows);
  // P = 2^(kPShift + score - m) with m the row maximum the group last rescaled to; m is raised (and O
  // rescaled) only when a tile's maximum exceeds it by more than kSlack, so P <= 2^(kPShift + kSlack):
  // 256 for e4m3 (largest finite value 448), 256 for bf16.
  constexpr float kPShift = kFp8 ? 5.0f : 0.0f;
  constexpr float kSlack = kFp8 ? 3.0f : 8.0f;
  constexpr uint32_t kGroupCols = 256;  // TMEM columns per softmax group: S at 0..127, O (80 columns) at 128
  constexpr uint32_t kOCol = 128;

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem + L::kQOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;                  // [stages]
  uint64_t* kv_empty = bars + kStages;       // [stages]
  uint64_t* s_full = bars + 2 * kStages;     // [group] S(i) is in TMEM
  uint64_t* s_free = s_full + 2;             // [group] the group holds S(i) in registers
  // p_full counts warps' arrivals, and a warp that had to rescale can be late: were there one barrier per group,
  // an early warp's arrival for tile i + 1 could complete tile i's phase in the late warp's place.  Even and odd
  // tiles therefore have barriers of their own (no warp can be two tiles ahead: S(i + 2) is not computed before
  // all four have copied S(i + 1), which they do after finishing tile i).
  uint64_t* p_full = s_free + 2;             // [group][tile parity] P(i) is in shared memory, O is rescaled
  uint64_t* pv_done = p_full + 4;            // [group] O += P(i) V(i) has finished
  uint64_t* turn = pv_done + 2;              // [group] the other group has issued its exponentials
  uint64_t* o_final = turn + 2;              // [group] every PV of the group has finished
  uint64_t* q_ready = o_final + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* drain_flag = abort_flag + 1;
  float* tm = reinterpret_cast<float*>(const_cast<int*>(abort_flag + 2));  // 16 floats

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  if (warp == 4) QB_TR(4, 0, 0);
  const int q0 = blockIdx.x * kQTile;
  const int qh = blockIdx.y;
  const int kvh = qh / a.gqa;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int b = 0; b < 2; ++b) {
      mbar_init(smem_u32(&s_full[b]), 1);
      mbar_init(smem_u32(&s_free[b]), 4);
      mbar_init(smem_u32(&p_full[2 * b]), 4);
      mbar_init(smem_u32(&p_full[2 * b + 1]), 4);
      mbar_init(smem_u32(&pv_done[b]), 1);
      mbar_init(smem_u32(&turn[b]), 4);
      mbar_init(smem_u32(&o_final[b]), 1);
    }
    mbar_init(smem_u32(q_ready), 8);
    *abort_flag = 0;
    *drain_flag = 0;
    fence_barrier_init();
  }
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
  if (warp == 4) QB_TR(4, 0, 1);

  // Everything above touched only this CTA's shared memory and TMEM, so it may run while the kernels
  // before this one in the stream are still at work; everything below reads what they wrote.
  grid_dep_launch();
  grid_dep_wait();

  // segment table -> number of key tiles (same in every thread)
  int seg[6] = {0, 0, 0, 0, 0, 0};
  int nseg = min(*after_wait(a.n_segments), min(a.max_segments, 3));  // the table is the work of the kernel before: ordinary loads
  bool seg_ok = true;
  int n_tiles = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    if (i < nseg) {
      seg[2 * i] = after_wait(a.segments)[2 * i];
      seg[2 * i + 1] = after_wait(a.segments)[2 * i + 1];
      if (seg[2 * i] < 0 || seg[2 * i + 1] < 0 || (seg[2 * i] & 15) != 0 || seg[2 * i] + seg[2 * i + 1] > a.capacity) seg_ok = false;
      n_tiles += (seg[2 * i + 1] + kKeyTile - 1) / kKeyTile;
    }
  }
  if (!seg_ok) {
#pragma unroll
    for (int i = 0; i < 6; ++i) seg[i] = 0;
  }
  if (!seg_ok) {  // malformed table: report and attend to nothing (output rows become 0)
    n_tiles = 0;
    if (threadIdx.x == 0) atomicOr(a.status, QB_DEV_BAD_SEGMENT);
  }
  // this CTA's share of the key tiles: tiles tile0 .. tile0 + n_tiles - 1 of the list
  const int n_splits = kSplit ? static_cast<int>(gridDim.z) : 1;
  int tile0 = 0;
  if (kSplit) {
    tile0 = static_cast<int>(blockIdx.z) * n_tiles / n_splits;
    n_tiles = static_cast<int>(blockIdx.z + 1) * n_tiles / n_splits - tile0;
  }

  // The softmax threads ask for their half of the query row (and group 0 for the row of the RoPE table) now, so that the
  // loads travel while the frame counter's sines and cosines are worked out and the CTA meets at the barrier below
  // (46.5 -> 46.3 us at 720p).
  uint4 q_pre[4];
  float4 xy_pre[4];
  if (warp >= 4) {
    const int g_ = (warp - 4) >> 2;
    const int t_ = q0 + (warp & 3) * 32 + lane;
    if (t_ < a.tpf) {
      const uint4* src = reinterpret_cast<const uint4*>(after_wait(a.qkv) + static_cast<size_t>(t_) * a.q_row + static_cast<size_t>(qh) * a.q_head + g_ * 32);
#pragma unroll
      for (int v = 0; v < 4; ++v) q_pre[v] = src[v];
      if (g_ == 0) {
        const float4* rp = reinterpret_cast<const float4*>(a.rope_xy + static_cast<size_t>(t_) * 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) xy_pre[i] = __ldg(rp + i);
      }
    }
  }
  if (threadIdx.x >= 96 && threadIdx.x < 104) temporal_cos_sin(*after_wait(a.frame_t), threadIdx.x - 96, tm);
  __syncthreads();


  // Registers move from the four control warps to the softmax warps, which hold a whole score row each.
  if (warp < 4) {
  setmaxnreg_dec<kCtrlRegs>();
  if (warp == 0) {
    // ---------------- TMA producer
    if (elect_one()) {
      int issued = 0;
      for (int j = 0; j < n_tiles; ++j) {
        const int s = j % kStages;
        const uint32_t ph = (j / kStages) & 1;
        if (!mbar_wait(smem_u32(&kv_empty[s]), ph ^ 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
        int row, valid;
        locate_tile(seg, tile0 + j, row, valid);
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
    // Per group: S(i) goes to the group's S columns as soon as the group has copied S(i - 1) into its
    // registers; once the group has written P(i) (and rescaled O if a row maximum jumped), O += P(i) V(i)
    // accumulates in the group's O columns.  S(i + 1) is issued ahead of PV(i).
    const int g = warp - 1;
    const int n_g = n_tiles > g ? (n_tiles - g + 1) / 2 : 0;
    if (elect_one() && n_g > 0) {
      const uint32_t q_addr = smem_u32(q_s);
      const uint32_t p_base = smem_u32(smem + L::kPOff + g * L::kPBufs * L::kPBytes);
      const uint32_t tmem_sg = tmem_base + g * kGroupCols;
      const uint32_t tmem_og = tmem_sg + kOCol;
      auto stage_addr = [&](int j) { return smem_u32(smem + L::kStageOff + (j % kStages) * L::kStageBytes); };
      auto issue_s = [&](int i) {
        const uint32_t k_addr = stage_addr(2 * i + g);
        if (kFp8) {
          const uint64_t qd = umma_desc_k_sw64(q_addr), kd = umma_desc_k_sw64(k_addr);
#pragma unroll
          for (int k = 0; k < 2; ++k) umma_f8(tmem_sg, qd + 2 * k, kd + 2 * k, kIdescS, k > 0);
        } else {
          const uint64_t qd = umma_desc_k_sw128(q_addr), kd = umma_desc_k_sw128(k_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f16(tmem_sg, qd + 2 * k, kd + 2 * k, kIdescS, k > 0);
        }
        umma_commit(smem_u32(&s_full[g]));
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
        QB_TR(2 + g, i, 0);
        if (i + 1 < n_g) {
          ok = wait_tile(2 * (i + 1) + g);
          QB_TR(2 + g, i, 1);
          ok = ok && mbar_wait(smem_u32(&s_free[g]), i & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
          if (!ok) break;
          QB_TR(2 + g, i, 2);
          tc_fence_after();
          issue_s(i + 1);
        }
        QB_TR(2 + g, i, 3);
        ok = mbar_wait(smem_u32(&p_full[2 * g + (i & 1)]), (i >> 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
        if (!ok) break;
        QB_TR(2 + g, i, 4);
        tc_fence_after();
        const uint32_t v_addr = stage_addr(2 * i + g) + L::kKBytes;
        const uint32_t p_addr = p_base + (i % L::kPBufs) * L::kPBytes;
        if (kFp8) {
          const uint64_t pd = umma_desc_k_sw128(p_addr), vd = umma_desc_k_sw128(v_addr);
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_f8(tmem_og, pd + 2 * k, vd + 2 * k, kIdescPV, (i | k) > 0);
        } else {
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            const uint64_t pd = umma_desc_k_sw128(p_addr + (k >> 2) * (L::kPBytes / 2));
            const uint64_t vd = umma_desc_k_sw128(v_addr + (k >> 2) * L::kVTile);
            umma_f16(tmem_og, pd + 2 * (k & 3), vd + 2 * (k & 3), kIdescPV, (i | k) > 0);
          }
        }
        umma_commit(smem_u32(&pv_done[g]));
        umma_commit(smem_u32(&kv_empty[(2 * i + g) % kStages]));
        QB_TR(2 + g, i, 5);
      }
      // pv_done flips once per tile and the fp8 softmax warps rarely look at it, so its parity cannot tell
      // "all finished" from "two still in flight"; the end of the accumulation has a barrier of its own
      if (ok) umma_commit(smem_u32(&o_final[g]));
    }
  }
  } else {
    setmaxnreg_inc<kSoftmaxRegs>();
    // ---------------- softmax groups: one query row per thread, group g takes tiles j = 2 i + g
    const int g = (warp - 4) >> 2;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int t = q0 + r;
    const bool row_ok = t < a.tpf;
    const uint32_t lane_addr = static_cast<uint32_t>(lane_grp * 32) << 16;
    uint8_t* p_g = smem + L::kPOff + g * L::kPBufs * L::kPBytes;

    // Q row -> RoPE -> shared memory (K-major, swizzled like a TMA tile).  Group 0 rotates pairs
    // 0..15 (spatial angles), group 1 pairs 16..31 (temporal angles).
    {
      float y0[16], y1[16];
      if (row_ok) {
        float xy[16];
        if (g == 0) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float4 v = xy_pre[i];
            xy[4 * i] = v.x; xy[4 * i + 1] = v.y; xy[4 * i + 2] = v.z; xy[4 * i + 3] = v.w;
          }
        }
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 x = q_pre[v];
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
      warp_arrive(smem_u32(q_ready), lane);
      if (warp == 4) QB_TR(4, 0, 2);
    }

    const float ks = a.k_scale ? __ldg(a.k_scale + kvh) : 1.0f;
    const float sl2 = ks * 0.125f * 1.4426950408889634f;  // scores -> log2 domain, 1/sqrt(64) folded in
    const uint32_t tmem_s = tmem_base + g * kGroupCols + lane_addr;  // this thread's row of the group's S
    const uint32_t tmem_o = tmem_s + kOCol;                          // ... and of its O accumulator
    float m_run = -1.0e30f;
    bool ok = true;
    const int my_tiles = n_tiles > g ? (n_tiles - g + 1) / 2 : 0;

    for (int i = 0; i < my_tiles && ok; ++i) {
      if (lane_grp == 0) QB_TR(g, i, 0);
      int row, valid;
      locate_tile(seg, tile0 + 2 * i + g, row, valid);
      if (lane_grp == 0) QB_TR(g, i, 1);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[g]), i & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (!ok) break;
      tc_fence_after();
      if (lane_grp == 0) QB_TR(g, i, 2);
      // the whole score row into registers; the S columns are then free for the next tile
      uint32_t sc[4][32];
#pragma unroll
      for (int c = 0; c < 4; ++c) tmem_ld32(tmem_s + c * 32, sc[c]);
      // the wait names the loaded registers, so that nothing the compiler does with them (a move, a spill)
      // can be placed between a load and the wait, where they do not hold the scores yet
      tmem_wait_ld_into(sc[0]);
      tmem_loaded(sc[1]);
      tmem_loaded(sc[2]);
      tmem_loaded(sc[3]);
      if (lane_grp == 0) QB_TR(g, i, 3);
      tc_fence_before();
      warp_arrive(smem_u32(&s_free[g]), lane);
      if (valid != kKeyTile) {  // last tile of a segment whose length is not a multiple of 128
#pragma unroll
        for (int c = 0; c < 4; ++c)
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (c * 32 + q >= valid) sc[c][q] = 0xff800000u;  // -inf
      }
      float mx[4];
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        float m0 = __uint_as_float(sc[c][0]), m1 = __uint_as_float(sc[c][1]);
#pragma unroll
        for (int q = 0; q < 15; ++q) {  // two chains of 3-input max
          if (q & 1) m1 = max3f(m1, __uint_as_float(sc[c][2 + 2 * q]), __uint_as_float(sc[c][3 + 2 * q]));
          else m0 = max3f(m0, __uint_as_float(sc[c][2 + 2 * q]), __uint_as_float(sc[c][3 + 2 * q]));
        }
        mx[c] = fmaxf(m0, m1);
      }
      const float m_tile = max3f(max3f(mx[0], mx[1], mx[2]), mx[3], -1.0e30f) * sl2;
      if (lane_grp == 0) QB_TR(g, i, 4);
      if (i == 0) {
        m_run = m_tile;
      } else {
        const bool jump = m_tile > m_run + kSlack;
        const bool any_jump = __any_sync(0xffffffffu, jump);
        // O may be rescaled only when PV(i - 1) has finished.  The P tile written below was last read
        // by PV(i - 1) when the group has one P tile; with two it was PV(i - 2), which finished before
        // S(i) did (the MMA warp issued it earlier, and s_full covers everything issued before it).
        if (L::kPBufs == 1 || any_jump) {
          ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&pv_done[g]), (i - 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
          if (!ok) break;
        }
        if (any_jump) {
          const float alpha = jump ? ex2_approx(m_run - m_tile) : 1.0f;
          if (jump) m_run = m_tile;
          tc_fence_after();
#pragma unroll 1
          for (int c = 0; c < 2; ++c) {
            uint32_t oo[32];
            tmem_ld32(tmem_o + c * 32, oo);
            tmem_wait_ld_into(oo);
#pragma unroll
            for (int q = 0; q < 32; ++q) oo[q] = __float_as_uint(__uint_as_float(oo[q]) * alpha);
            tmem_st32(tmem_o + c * 32, oo);
          }
          uint32_t lsum = tmem_ld1(tmem_o + 64);
          tmem_wait_ld();
          tmem_loaded(lsum);
          tmem_st1(tmem_o + 64, __float_as_uint(__uint_as_float(lsum) * alpha));
          tmem_wait_st();
        }
      }
      const float nshift = kPShift - m_run;
      if (lane_grp == 0) QB_TR(g, i, 5);
      // The two groups take turns on the exponentials (the special-function unit is the scarcest
      // resource of this kernel): order G0(0) G1(0) G0(1) G1(1) ...  While one group runs its
      // exponentials the other loads its next score row, finds the maximum and talks to the MMA warps.
      if (g == 0 ? i > 0 : true) {
        const uint32_t par = g == 0 ? (i - 1) & 1 : i & 1;
        ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&turn[g]), par, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
        if (!ok) break;
      }
      if (lane_grp == 0) QB_TR(g, i, 6);
      uint8_t* p_s = p_g + (i % L::kPBufs) * L::kPBytes;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        // handed over before the last chunks: the other group needs a while to wake up, and two warps
        // per scheduler keep the special-function unit busier than one
        if (c == (kLin ? 0 : kHandoffChunk) && lane == 0) mbar_arrive(smem_u32(&turn[1 - g]));
        p_chunk<kFp8, kPolyOf8, kLin>(sc[c], c, sl2, nshift, p_s, r);
      }
      fence_proxy_async_smem();
      tc_fence_before();
      warp_arrive(smem_u32(&p_full[2 * g + (i & 1)]), lane);
      if (lane_grp == 0) QB_TR(g, i, 7);
    }
    if (warp == 4) QB_TR(4, 0, 3);
    // the group's result: 64 outputs and the row sum, still scaled by 2^(kPShift - m_run)
    float o[64];
    float l_run = 0.f;
#pragma unroll
    for (int d = 0; d < 64; ++d) o[d] = 0.f;
    if (ok && my_tiles > 0) {
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&o_final[g]), 0, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (ok) {
        tc_fence_after();
        uint32_t oo[2][32];
        tmem_ld32(tmem_o, oo[0]);
        tmem_ld32(tmem_o + 32, oo[1]);
        uint32_t lsum = tmem_ld1(tmem_o + 64);
        tmem_wait_ld_into(oo[0]);
        tmem_loaded(oo[1]);
        tmem_loaded(lsum);
#pragma unroll
        for (int d = 0; d < 64; ++d) o[d] = __uint_as_float(oo[d >> 5][d & 31]);
        l_run = __uint_as_float(lsum);
      }
    }

    if (warp == 4) QB_TR(4, 0, 4);
    // ---------------- merge the two groups (tensor work and TMA traffic are finished for both after the barrier)
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (warp == 4) QB_TR(4, 0, 5);
    float* comb = reinterpret_cast<float*>(smem + L::kStageOff);  // [66][128]
    if (g == 1) {
      comb[0 * 128 + r] = m_run;
      comb[1 * 128 + r] = l_run;
#pragma unroll
      for (int d = 0; d < 64; ++d) comb[(2 + d) * 128 + r] = o[d];
    }
    asm volatile("bar.sync 2, 256;" ::: "memory");
    if (g == 0 && !kSplit) {
      if (ok && row_ok && *abort_flag == 0) {
        const float m1 = comb[r], l1 = comb[128 + r];
        const float m = fmaxf(m_run, m1);
        const float a0 = ex2_approx(m_run - m), a1 = ex2_approx(m1 - m);
        const float l = l_run * a0 + l1 * a1;
        const float vs = a.v_scale ? __ldg(a.v_scale + kvh) : 1.0f;
        const float inv = l > 0.f ? vs / l : 0.f;
        const float s0 = a0 * inv, s1 = a1 * inv;
        uint4* dst = reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * a.o_row + static_cast<size_t>(qh) * a.o_head);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const int d = 4 * v + q;
            const float e0 = o[2 * d] * s0 + comb[(2 + 2 * d) * 128 + r] * s1;
            const float e1 = o[2 * d + 1] * s0 + comb[(3 + 2 * d) * 128 + r] * s1;
            w[q] = pack_bf16x2(e0, e1);
          }
          dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
          if (a.out_q != nullptr) {  // narrowed from the bf16-rounded values: equals a separate bf16 -> e4m3 cast
            *reinterpret_cast<uint2*>(a.out_q + static_cast<size_t>(t) * a.o_row + static_cast<size_t>(qh) * a.o_head + v * 8) =
                make_uint2(pack_e4m3x4(bf16lo(w[0]), bf16hi(w[0]), bf16lo(w[1]), bf16hi(w[1])),
                           pack_e4m3x4(bf16lo(w[2]), bf16hi(w[2]), bf16lo(w[3]), bf16hi(w[3])));
          }
        }
      }
    } else if (kSplit && g == 0) {
      // keys shared with other CTAs.  This CTA's result for the row: both groups brought to a common maximum,
      // not yet divided by the row sum
      const bool good = ok && *abort_flag == 0;
      const float m1 = comb[r], l1 = comb[128 + r];
      float m = fmaxf(m_run, m1);
      const float a0 = ex2_approx(m_run - m), a1 = ex2_approx(m1 - m);
      float l = l_run * a0 + l1 * a1;
      float e[64];
#pragma unroll
      for (int d = 0; d < 64; ++d) e[d] = o[d] * a0 + comb[(2 + d) * 128 + r] * a1;
      bool writer;  // does this CTA write the output rows?
      {
        const int item = qh * gridDim.x + blockIdx.x;  // (head, query tile)
        float* mine = a.partials + (static_cast<size_t>(item) * n_splits + blockIdx.z) * (66 * 128);
        mine[r] = m;
        mine[128 + r] = l;
#pragma unroll
        for (int d = 0; d < 64; ++d) mine[(2 + d) * 128 + r] = e[d];
        __threadfence();
        asm volatile("bar.sync 3, 128;" ::: "memory");
        int* last = reinterpret_cast<int*>(comb);  // the group's exchange buffer is free again
        if (r == 0) *last = atomicAdd(a.tickets + item, 1) == n_splits - 1;
        asm volatile("bar.sync 3, 128;" ::: "memory");
        writer = *last != 0;
        if (writer) {
          __threadfence();
          // sum the shares in order of z: the result does not depend on which CTA came last
          const float* part = a.partials + static_cast<size_t>(item) * n_splits * (66 * 128);
          m = -1.0e30f;
          for (int z = 0; z < n_splits; ++z) m = fmaxf(m, __ldcg(part + z * (66 * 128) + r));
          l = 0.f;
#pragma unroll
          for (int d = 0; d < 64; ++d) e[d] = 0.f;
          for (int z = 0; z < n_splits; ++z) {
            const float* pz = part + z * (66 * 128);
            const float w = ex2_approx(__ldcg(pz + r) - m);
            l = fmaf(w, __ldcg(pz + 128 + r), l);
#pragma unroll
            for (int d = 0; d < 64; ++d) e[d] = fmaf(w, __ldcg(pz + (2 + d) * 128 + r), e[d]);
          }
          if (r == 0) a.tickets[item] = 0;  // ready for the next launch
        }
      }
      if (writer && good && row_ok) {
        const float vs = a.v_scale ? __ldg(a.v_scale + kvh) : 1.0f;
        const float inv = l > 0.f ? vs / l : 0.f;
        uint4* dst = reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * a.o_row + static_cast<size_t>(qh) * a.o_head);
#pragma unroll
        for (int v = 0; v < 8; ++v) {
          uint32_t w[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(e[8 * v + 2 * q] * inv, e[8 * v + 2 * q + 1] * inv);
          dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
          if (a.out_q != nullptr) {  // narrowed from the bf16-rounded values: equals a separate bf16 -> e4m3 cast
            *reinterpret_cast<uint2*>(a.out_q + static_cast<size_t>(t) * a.o_row + static_cast<size_t>(qh) * a.o_head + v * 8) =
                make_uint2(pack_e4m3x4(bf16lo(w[0]), bf16hi(w[0]), bf16lo(w[1]), bf16hi(w[1])),
                           pack_e4m3x4(bf16lo(w[2]), bf16hi(w[2]), bf16lo(w[3]), bf16hi(w[3])));
          }
        }
      }
    }
  }

  if (warp == 4) QB_TR(4, 0, 6);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) QB_TR(4, 0, 7);
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

}  // namespace qb

namespace qb {
int32_t launch_attn4(const void* K_cache, const void* Vt_cache, const AttnArgs& a, int n_kv_heads, bool fp8, cudaStream_t st);
// bf16 calls with one (query tile, head) per CTA go to the three-group kernel of attn4.cu; QB_ATTN4=0 in the environment
// when the library is loaded keeps the two-group kernel of this file for everything (e4m3 and key splits always use it).
// e4m3 probabilities: 0 = every second exponential on the FMA pipe (ex2_lin_from_biased), 1 = all on the special-function unit
static int g_attn_exact_exp = [] {
  const char* e = getenv("QB_ATTN_EXACT_EXP");
  return (e != nullptr && e[0] == '1') ? 1 : 0;
}();
static bool attn4_enabled() {
  static const bool on = [] {
    const char* e = getenv("QB_ATTN4");
    return !(e != nullptr && e[0] == '0');
  }();
  return on;
}
}  // namespace qb

using namespace qb;

extern "C" int32_t qb_set_attn_exact_exp(int32_t on) {
  const int32_t was = g_attn_exact_exp;
  g_attn_exact_exp = on ? 1 : 0;
  return was;
}

#ifdef QB_ATTN_TRACE
extern "C" int32_t qb_debug_attn_trace(void* host_out) {
  return cudaMemcpyFromSymbol(host_out, g_attn_trace, sizeof(g_attn_trace)) == cudaSuccess ? 0 : -1;
}
#endif

// How many CTAs share the keys of one (query tile, head).  One when the grid already fills most of the GPU
// (720p: 4 query tiles x 32 heads); otherwise as many as it takes to reach the SM count, while every
// share keeps a few key tiles (360p: 1 x 32 -> 4 shares; a tensor-parallel rank with 2 KV heads: 8).
static int attn_key_splits(const qb_attn_params* p) {
  if (p->kv_splits > 0) return p->kv_splits;
  const int tpf = p->H_spatial * p->W_spatial;
  const int items = ((tpf + kQTile - 1) / kQTile) * p->n_kv_heads * p->gqa_ratio;
  const int tiles = ((p->num_buckets + 1) * (tpf / (p->quilt_factor > 0 ? p->quilt_factor : 1)) + kKeyTile - 1) / kKeyTile;  // at most
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  int n = sms / (items > 0 ? items : 1);
  if (n > tiles / 3) n = tiles / 3;
  if (n > 8) n = 8;
  return n < 2 ? 1 : n;
}

// The tickets take a fixed area at the start of the workspace (4096 (query tile, head) items; more only for a
// geometry that has more), so that calls of different geometries that share a workspace agree on where the
// tickets end: one call's partial results never land on tickets that another call expects to find zero.
static size_t attn_ticket_bytes(const qb_attn_params* p) {
  const int tpf = p->H_spatial * p->W_spatial;
  const size_t need = round_up(static_cast<size_t>((tpf + kQTile - 1) / kQTile) * p->n_kv_heads * p->gqa_ratio * sizeof(int), 1024);
  return need > (16u << 10) ? need : (16u << 10);
}

extern "C" size_t qb_owl_attn_workspace_bytes(const qb_attn_params* p) {
  if (p == nullptr || p->H_spatial <= 0 || p->W_spatial <= 0 || p->n_kv_heads <= 0 || p->gqa_ratio <= 0 || p->num_buckets <= 0) return 0;
  const int n = attn_key_splits(p);
  if (n <= 1) return 0;
  const int tpf = p->H_spatial * p->W_spatial;
  const size_t items = static_cast<size_t>((tpf + kQTile - 1) / kQTile) * p->n_kv_heads * p->gqa_ratio;
  return attn_ticket_bytes(p) + items * n * (66 * 128) * sizeof(float);
}

extern "C" int32_t qb_owl_attn(const void* qkv, const void* K_cache, const void* Vt_cache, const int32_t* segments,
                               const int32_t* n_segments, const int32_t* frame_t, void* out, void* out_q, const float* rope_xy,
                               const qb_attn_params* p, void* workspace, size_t workspace_bytes, void* stream) {
  QB_REQUIRE(p != nullptr, QB_ERR_INVALID_ARG, "owl_attn: params are NULL");
  QB_REQUIRE(qkv && K_cache && Vt_cache && segments && n_segments && frame_t && out && rope_xy, QB_ERR_INVALID_ARG,
             "owl_attn: NULL pointer");
  QB_REQUIRE(p->quilt_factor >= 1 && (p->H_spatial * p->W_spatial) % p->quilt_factor == 0, QB_ERR_INVALID_ARG,
             "owl_attn: quilt_factor %d does not divide H*W", p->quilt_factor);
  QB_REQUIRE(p->packed_qkv == 0 || p->packed_qkv == 1, QB_ERR_INVALID_ARG, "owl_attn: packed_qkv %d", p->packed_qkv);
  QB_REQUIRE(p->n_kv_heads > 0 && p->gqa_ratio > 0 && p->H_spatial > 0 && p->W_spatial > 0 && p->num_buckets > 0,
             QB_ERR_INVALID_ARG, "owl_attn: sizes must be positive");
  QB_REQUIRE(p->kv_dtype == QB_BF16 || p->kv_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "owl_attn: kv_dtype %d", p->kv_dtype);
  QB_REQUIRE(p->compute_dtype == p->kv_dtype, QB_ERR_UNSUPPORTED,
             "owl_attn: compute_dtype must equal kv_dtype (bf16 cache + bf16 MMAs, or e4m3 cache + e4m3 MMAs)");
  QB_REQUIRE(p->max_segments >= 1, QB_ERR_INVALID_ARG, "owl_attn: max_segments %d", p->max_segments);
  const int tpf = p->H_spatial * p->W_spatial;
  // a quilted cache keeps tpf / quilt_factor tokens per frame (src/quark/kernels/owl_attn/spec.py:79-93); the queries
  // are all tpf tokens either way, and the segment table already counts cached rows
  const int cap = (p->num_buckets + 1) * (tpf / p->quilt_factor);
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
  if (p->packed_qkv) {
    a.q_row = (Hq + 2 * p->n_kv_heads) * 64; a.q_head = 64; a.o_row = Hq * 64; a.o_head = 64;
  } else {
    a.q_row = 64; a.q_head = tpf * 64; a.o_row = 64; a.o_head = tpf * 64;
  }
  a.n_q_heads = Hq; a.gqa = p->gqa_ratio; a.capacity = cap; a.max_segments = p->max_segments;

  QB_REQUIRE(p->kv_splits >= 0 && p->kv_splits <= 16, QB_ERR_INVALID_ARG, "owl_attn: kv_splits %d", p->kv_splits);
  const int splits = attn_key_splits(p);
  if (splits > 1) {
    const size_t need = qb_owl_attn_workspace_bytes(p);
    QB_REQUIRE(workspace != nullptr && workspace_bytes >= need, QB_ERR_WORKSPACE, "owl_attn: %d key splits need a workspace of %zu bytes, %zu given",
               splits, need, workspace_bytes);
    QB_REQUIRE(aligned16(workspace), QB_ERR_ALIGN, "owl_attn: workspace must be 16-byte aligned");
    a.tickets = static_cast<int*>(workspace);
    a.partials = reinterpret_cast<float*>(static_cast<uint8_t*>(workspace) + attn_ticket_bytes(p));
  }
  dim3 grid((tpf + kQTile - 1) / kQTile, Hq, splits);
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  // bf16, one CTA per (query tile, head): the three-group kernel of attn4.cu (66.7 against 70.3 us at 720p).  In the
  // e4m3 path it is the slower one (57.7 against 52.2 us): its per-chunk fixed work outweighs the extra warps.
  if (splits == 1 && !fp8 && attn4_enabled()) return launch_attn4(K_cache, Vt_cache, a, p->n_kv_heads, fp8, st);
  auto launch = [&](auto kernel, int smem_bytes) -> int32_t {
    QB_CUDA_OK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));
    return launch_dep("owl_attn kernel", kernel, grid, dim3(kAttnThreads), smem_bytes, st, tmK, tmV, a);
  };
  if (fp8 && !g_attn_exact_exp)
    return splits > 1 ? launch(owl_attn_kernel<true, true, true>, AttnSmem<true>::kTotal) : launch(owl_attn_kernel<true, false, true>, AttnSmem<true>::kTotal);
  if (fp8) return splits > 1 ? launch(owl_attn_kernel<true, true, false>, AttnSmem<true>::kTotal) : launch(owl_attn_kernel<true, false, false>, AttnSmem<true>::kTotal);
  return splits > 1 ? launch(owl_attn_kernel<false, true, false>, AttnSmem<false>::kTotal) : launch(owl_attn_kernel<false, false, false>, AttnSmem<false>::kTotal);
}
