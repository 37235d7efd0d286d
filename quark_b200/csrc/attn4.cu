// owl_attn with three softmax groups over 64-key chunks (used for bf16 caches, one CTA per (query tile, head)).
//
// attn.cu runs two softmax groups over 128-key tiles, 216 registers per softmax thread.  Here a softmax thread holds 64
// scores instead of 128, which fits three groups (12 softmax warps, three per scheduler) into the register file:
//   warp 0        TMA producer: per stage one K chunk [64 keys x 64] and one V^T chunk [64 x 64 keys] (+ 16 rows of ones)
//   warps 1-3     one thread each issues tcgen05.mma for softmax group 0 / 1 / 2: S = Q K^T and O += P V
//   warps 4-15    softmax groups 0..2 (four warps each, one query row per thread); group g takes chunks g, g + 3, ...
// TMEM: per group one S chunk (64 columns) and the output accumulator O (80 columns: 64 outputs and, from the rows of
// ones under every V^T chunk, the row sum of exactly the rounded P that is multiplied with V).
// As in attn.cu: P = 2^(score - m) with m the maximum the row was last rescaled to (O is rescaled only when a chunk's
// maximum exceeds m by more than kSlack), e4m3 P scaled by 2^5, two P buffers per group in the fp8 path, every wait
// bounded, a malformed segment table reported and treated as empty.  The three partial results are merged at the end.
//
// Measured on B200 at 720p (512 queries x 32 heads x 8320 keys, us per launch; attn.cu in brackets): bf16 66.7 (70.3),
// e4m3 57.7 (52.2).  The extra warp per scheduler pays in the bf16 path, where attn.cu has one P tile per group and three
// stages; in the e4m3 path the fixed work per chunk (barrier waits, TMEM loads, maxima: the same per 64 keys as attn.cu
// spends per 128) outweighs it, so e4m3 calls stay with attn.cu.  A variant with four groups (16 softmax warps, 96
// registers per thread, row sums kept by the threads because four S chunks and four 80-column accumulators exceed the
// 512 TMEM columns) was slower still: 60.7 us e4m3, with 3 % of its instructions spill traffic and 8.9 instructions per
// exponential against 5.4 in attn.cu.  All three kernels issue about one instruction every second cycle per scheduler:
// the softmax loop is bound by instruction issue, not by the special-function unit alone, which is also why computing
// part of the exponentials as a polynomial (more instructions) loses.
#include "attn_common.cuh"

namespace qb {

constexpr int kA4Threads = 512;
constexpr int kA4Groups = 3;
constexpr int kA4VRows = 80;  // 64 channels + 16 rows of ones (row sum of P)
constexpr int kA4Chunk = 64;
// setmaxnreg moves registers inside the pool the CTA was given at launch (512 threads x 128 registers, the most that
// __launch_bounds__(512) allows), not inside the whole register file: an increase waits until other warps of the CTA
// have released enough, so the budget below must close or the softmax warps would wait for ever.
constexpr int kA4LaunchRegs = 128;
constexpr int kA4CtrlRegs = 40;
constexpr int kA4SoftmaxRegs = 152;
static_assert(128 * kA4CtrlRegs + 384 * kA4SoftmaxRegs <= kA4Threads * kA4LaunchRegs, "register budget of the CTA");

template <bool kFp8>
struct A4Smem {
  static constexpr int kEs = kFp8 ? 1 : 2;
  // A group's MMA warp issues S one of its chunks (three chunks overall) ahead of the PV that frees a stage, after the
  // PV of its previous chunk in program order: chunk u + 3 may need the stage of chunk u - 3 at the earliest.
  static constexpr int kStages = 6;
  static constexpr int kRowBytes = 64 * kEs;                 // one row of a K-major tile: 64 | 128 bytes
  static constexpr int kQBytes = 128 * kRowBytes;            // 8 KB | 16 KB
  static constexpr int kKBytes = kA4Chunk * kRowBytes;       // 4 KB | 8 KB: K chunk
  static constexpr int kVBytes = kA4VRows * kRowBytes;       // 5 KB | 10 KB: V^T chunk and the rows of ones
  static constexpr int kPBytes = 128 * kRowBytes;            // 8 KB | 16 KB
  static constexpr int kPBufs = kFp8 ? 2 : 1;
  static constexpr int kStageBytes = kKBytes + kVBytes;      // 9 KB | 18 KB (a multiple of the swizzle atom: 512 | 1024)
  static constexpr int kQOff = 0;
  static constexpr int kPOff = kQOff + kQBytes;
  static constexpr int kStageOff = kPOff + kA4Groups * kPBufs * kPBytes;
  static constexpr int kBarOff = kStageOff + kStages * kStageBytes;
  static constexpr int kTotal = kBarOff + 1024 + 1024;
  static constexpr int kMergeBytes = (kA4Groups - 1) * 66 * 128 * 4;  // groups 1, 2 hand (m, l, 64 outputs) per row to group 0
  static_assert(kBarOff - kPOff >= kMergeBytes, "merge buffer aliases the P and stage areas");
  static_assert(kStageBytes % (kFp8 ? 512 : 1024) == 0, "stages keep the swizzle alignment");
};

// j-th valid 64-key chunk of the segment table: first cache row and number of valid keys.
__device__ __forceinline__ void locate_chunk(const int (&seg)[6], int j, int& row, int& valid) {
  row = 0;
  valid = 0;
  bool found = false;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    const int nt = (seg[2 * i + 1] + kA4Chunk - 1) / kA4Chunk;
    if (!found && j < nt) {
      row = seg[2 * i] + j * kA4Chunk;
      valid = min(kA4Chunk, seg[2 * i + 1] - j * kA4Chunk);
      found = true;
    }
    j -= nt;
  }
}

template <bool kFp8>
__device__ __forceinline__ uint64_t a4_desc(uint32_t addr) {
  return kFp8 ? umma_desc_k_sw64(addr) : umma_desc_k_sw128(addr);
}

template <bool kFp8>
__global__ void __launch_bounds__(kA4Threads, 1)
owl_attn4_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const AttnArgs a) {
  using L = A4Smem<kFp8>;
  constexpr int kStages = L::kStages;
  constexpr int G = kA4Groups;
  constexpr uint32_t kTmemCols = 512;
  constexpr uint32_t kIdescS = kFp8 ? umma_idesc(0, 0, 128, 64) : umma_idesc(1, 1, 128, 64);
  constexpr uint32_t kIdescPV = kFp8 ? umma_idesc(0, 0, 128, kA4VRows) : umma_idesc(1, 1, 128, kA4VRows);
  constexpr int kMmas = kFp8 ? 2 : 4;  // 32 bytes of the contraction per instruction, rows of 64 | 128 bytes
  constexpr float kPShift = kFp8 ? 5.0f : 0.0f;
  constexpr float kSlack = kFp8 ? 3.0f : 8.0f;
  constexpr uint32_t kOCol = 192, kOStride = 96;  // S of group g at columns 64 g, O (80 columns) at 192 + 96 g

  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~static_cast<uintptr_t>(1023));
  uint8_t* q_s = smem + L::kQOff;
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + L::kBarOff);
  uint64_t* kv_full = bars;                 // [stages]
  uint64_t* kv_empty = bars + kStages;      // [stages]
  uint64_t* s_full = bars + 2 * kStages;    // [group] S(i) is in TMEM
  uint64_t* s_free = s_full + G;            // [group] the group holds S(i) in registers
  uint64_t* p_full = s_free + G;            // [group][chunk parity] P(i) is in shared memory, O is rescaled
  uint64_t* pv_done = p_full + 2 * G;       // [group] O += P(i) V(i) has finished
  uint64_t* o_final = pv_done + G;          // [group] every PV of the group has finished
  uint64_t* q_ready = o_final + G;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(q_ready + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  volatile int* drain_flag = abort_flag + 1;
  float* tm = reinterpret_cast<float*>(const_cast<int*>(abort_flag + 2));  // 16 floats

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const int q0 = blockIdx.x * 128;
  const int qh = blockIdx.y;
  const int kvh = qh / a.gqa;

  if (threadIdx.x == 0) {
    tma_prefetch_desc(&tmK);
    tma_prefetch_desc(&tmV);
    for (int s = 0; s < kStages; ++s) {
      mbar_init(smem_u32(&kv_full[s]), 1);
      mbar_init(smem_u32(&kv_empty[s]), 1);
    }
    for (int g = 0; g < G; ++g) {
      mbar_init(smem_u32(&s_full[g]), 1);
      mbar_init(smem_u32(&s_free[g]), 4);
      mbar_init(smem_u32(&p_full[2 * g]), 4);
      mbar_init(smem_u32(&p_full[2 * g + 1]), 4);
      mbar_init(smem_u32(&pv_done[g]), 1);
      mbar_init(smem_u32(&o_final[g]), 1);
    }
    mbar_init(smem_u32(q_ready), 4 * G);
    *abort_flag = 0;
    *drain_flag = 0;
    fence_barrier_init();
  }
  // rows of ones under every V^T chunk (16 rows): the tensor core then returns the row sum of P in column 64 of O
  {
    constexpr uint32_t kOnes = kFp8 ? 0x38383838u : 0x3F803F80u;
    constexpr int kVecPerStage = 16 * L::kRowBytes / 16;  // 16-byte vectors of the ones rows of one stage
    for (int i = threadIdx.x; i < kStages * kVecPerStage; i += kA4Threads) {
      uint8_t* base = smem + L::kStageOff + (i / kVecPerStage) * L::kStageBytes + L::kKBytes + 64 * L::kRowBytes;
      *reinterpret_cast<uint4*>(base + (i % kVecPerStage) * 16) = make_uint4(kOnes, kOnes, kOnes, kOnes);
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

  // Everything above touched only this CTA's shared memory and TMEM; everything below reads what earlier kernels wrote.
  grid_dep_launch();
  grid_dep_wait();

  int seg[6] = {0, 0, 0, 0, 0, 0};
  const int nseg = min(*after_wait(a.n_segments), min(a.max_segments, 3));  // the table is the work of the kernel before: ordinary loads
  bool seg_ok = true;
  int n_chunks = 0;
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    if (i < nseg) {
      seg[2 * i] = after_wait(a.segments)[2 * i];
      seg[2 * i + 1] = after_wait(a.segments)[2 * i + 1];
      if (seg[2 * i] < 0 || seg[2 * i + 1] < 0 || (seg[2 * i] & 15) != 0 || seg[2 * i] + seg[2 * i + 1] > a.capacity) seg_ok = false;
      n_chunks += (seg[2 * i + 1] + kA4Chunk - 1) / kA4Chunk;
    }
  }
  if (!seg_ok) {  // malformed table: report and attend to nothing (output rows become 0)
#pragma unroll
    for (int i = 0; i < 6; ++i) seg[i] = 0;
    n_chunks = 0;
    if (threadIdx.x == 0) atomicOr(a.status, QB_DEV_BAD_SEGMENT);
  }

  if (threadIdx.x < 8) temporal_cos_sin(*after_wait(a.frame_t), threadIdx.x, tm);
  __syncthreads();

  if (warp < 4) {
    setmaxnreg_dec<kA4CtrlRegs>();
    if (warp == 0) {
      // ---------------- TMA producer
      if (elect_one()) {
        int issued = 0;
        for (int u = 0; u < n_chunks; ++u) {
          const int s = u % kStages;
          const uint32_t ph = (u / kStages) & 1;
          if (!mbar_wait(smem_u32(&kv_empty[s]), ph ^ 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
          int row, valid;
          locate_chunk(seg, u, row, valid);
          const uint32_t fb = smem_u32(&kv_full[s]);
          mbar_arrive_expect_tx(fb, L::kKBytes + 64 * L::kRowBytes);
          uint8_t* st = smem + L::kStageOff + s * L::kStageBytes;
          tma_load_2d(smem_u32(st), &tmK, fb, 0, kvh * a.capacity + row);
          tma_load_2d(smem_u32(st + L::kKBytes), &tmV, fb, row, kvh * 64);
          issued = u + 1;
        }
        if (*abort_flag) {
          // Giving up: let the copies already in flight land before this CTA's memory goes away.
          for (int u = max(0, issued - kStages); u < issued; ++u)
            mbar_wait(smem_u32(&kv_full[u % kStages]), (u / kStages) & 1, drain_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
        } else {
          // Tail: see the last stage releases land before the CTA can exit.
          for (int u = max(0, n_chunks - kStages); u < n_chunks; ++u)
            if (!mbar_wait(smem_u32(&kv_empty[u % kStages]), (u / kStages) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN)) break;
        }
      }
    } else {
      // ---------------- MMA issuers: warp 1 + g serves softmax group g, whose i-th chunk is u = g + 3 i.  S(i) goes to the
      // group's S columns as soon as the group has copied S(i - 1) into its registers; once the group has written P(i)
      // (and rescaled O if a row maximum jumped), O += P(i) V(i) accumulates in the group's O columns.  S(i + 1) is issued
      // ahead of PV(i).
      const int g = warp - 1;
      const int n_g = n_chunks > g ? (n_chunks - g + G - 1) / G : 0;
      if (elect_one() && n_g > 0) {
        const uint32_t q_addr = smem_u32(q_s);
        const uint32_t tmem_sg = tmem_base + g * 64;
        const uint32_t tmem_og = tmem_base + kOCol + g * kOStride;
        auto stage_addr = [&](int i) { return smem_u32(smem + L::kStageOff + ((g + G * i) % kStages) * L::kStageBytes); };
        auto wait_chunk = [&](int i) {
          const int u = g + G * i;
          return mbar_wait(smem_u32(&kv_full[u % kStages]), (u / kStages) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
        };
        auto issue_s = [&](int i) {
          const uint64_t qd = a4_desc<kFp8>(q_addr), kd = a4_desc<kFp8>(stage_addr(i));
#pragma unroll
          for (int m = 0; m < kMmas; ++m) {
            if (kFp8) umma_f8(tmem_sg, qd + 2 * m, kd + 2 * m, kIdescS, m > 0);
            else umma_f16(tmem_sg, qd + 2 * m, kd + 2 * m, kIdescS, m > 0);
          }
          umma_commit(smem_u32(&s_full[g]));
        };
        bool ok = mbar_wait(smem_u32(q_ready), 0, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
        ok = ok && wait_chunk(0);
        if (ok) {
          tc_fence_after();
          issue_s(0);
        }
        for (int i = 0; i < n_g && ok; ++i) {
          if (i + 1 < n_g) {
            ok = wait_chunk(i + 1);
            ok = ok && mbar_wait(smem_u32(&s_free[g]), i & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
            if (!ok) break;
            tc_fence_after();
            issue_s(i + 1);
          }
          ok = mbar_wait(smem_u32(&p_full[2 * g + (i & 1)]), (i >> 1) & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN);
          if (!ok) break;
          tc_fence_after();
          const uint32_t p_addr = smem_u32(smem + L::kPOff + (g * L::kPBufs + (i % L::kPBufs)) * L::kPBytes);
          const uint64_t pd = a4_desc<kFp8>(p_addr), vd = a4_desc<kFp8>(stage_addr(i) + L::kKBytes);
#pragma unroll
          for (int m = 0; m < kMmas; ++m) {
            if (kFp8) umma_f8(tmem_og, pd + 2 * m, vd + 2 * m, kIdescPV, (i | m) > 0);
            else umma_f16(tmem_og, pd + 2 * m, vd + 2 * m, kIdescPV, (i | m) > 0);
          }
          umma_commit(smem_u32(&pv_done[g]));
          umma_commit(smem_u32(&kv_empty[(g + G * i) % kStages]));
        }
        if (ok) umma_commit(smem_u32(&o_final[g]));  // the end of the accumulation has a barrier of its own
      }
    }
  } else {
    setmaxnreg_inc<kA4SoftmaxRegs>();
    // ---------------- softmax groups: one query row per thread, group g takes chunks g, g + 3, ...
    const int g = (warp - 4) >> 2;
    const int lane_grp = warp & 3;
    const int r = lane_grp * 32 + lane;
    const int t = q0 + r;
    const bool row_ok = t < a.tpf;
    const uint32_t lane_addr = static_cast<uint32_t>(lane_grp * 32) << 16;
    uint8_t* p_g = smem + L::kPOff + g * L::kPBufs * L::kPBytes;

    // Q row -> RoPE -> shared memory (K-major, swizzled like a TMA tile).  Groups 0 and 1 rotate pairs 0..15 (spatial
    // angles) and 16..31 (temporal angles); group 2 has nothing to do here.
    if (g < 2) {
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
        const uint4* src = reinterpret_cast<const uint4*>(a.qkv + static_cast<size_t>(t) * a.q_row + static_cast<size_t>(qh) * a.q_head + g * 32);
#pragma unroll
        for (int v = 0; v < 4; ++v) {
          const uint4 x = src[v];
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
    }
    warp_arrive(smem_u32(q_ready), lane);

    const float ks = a.k_scale ? __ldg(a.k_scale + kvh) : 1.0f;
    const float sl2 = ks * 0.125f * 1.4426950408889634f;  // scores -> log2 domain, 1/sqrt(64) folded in
    const uint32_t tmem_s = tmem_base + g * 64 + lane_addr;  // this thread's row of the group's S
    const uint32_t tmem_o = tmem_base + kOCol + g * kOStride + lane_addr;
    float m_run = -1.0e30f;
    bool ok = true;
    const int my_chunks = n_chunks > g ? (n_chunks - g + G - 1) / G : 0;

    for (int i = 0; i < my_chunks && ok; ++i) {
      int row, valid;
      locate_chunk(seg, g + G * i, row, valid);
      ok = __all_sync(0xffffffffu, mbar_wait(smem_u32(&s_full[g]), i & 1, abort_flag, a.status, QB_DEV_WAIT_TIMEOUT_ATTN));
      if (!ok) break;
      tc_fence_after();
      uint32_t sc[2][32];
      tmem_ld32(tmem_s, sc[0]);
      tmem_ld32(tmem_s + 32, sc[1]);
      tmem_wait_ld_into(sc[0]);
      tmem_loaded(sc[1]);
      tc_fence_before();
      warp_arrive(smem_u32(&s_free[g]), lane);
      if (valid != kA4Chunk) {  // last chunk of a segment whose length is not a multiple of 64
#pragma unroll
        for (int c = 0; c < 2; ++c)
#pragma unroll
          for (int q = 0; q < 32; ++q)
            if (c * 32 + q >= valid) sc[c][q] = 0xff800000u;  // -inf
      }
      float mx[2];
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        float m0 = __uint_as_float(sc[c][0]), m1 = __uint_as_float(sc[c][1]);
#pragma unroll
        for (int q = 0; q < 15; ++q) {  // two chains of 3-input max
          if (q & 1) m1 = max3f(m1, __uint_as_float(sc[c][2 + 2 * q]), __uint_as_float(sc[c][3 + 2 * q]));
          else m0 = max3f(m0, __uint_as_float(sc[c][2 + 2 * q]), __uint_as_float(sc[c][3 + 2 * q]));
        }
        mx[c] = fmaxf(m0, m1);
      }
      const float m_tile = max3f(mx[0], mx[1], -1.0e30f) * sl2;
      if (i == 0) {
        m_run = m_tile;
      } else {
        const bool jump = m_tile > m_run + kSlack;
        const bool any_jump = __any_sync(0xffffffffu, jump);
        // O may be rescaled only when PV(i - 1) has finished.  With one P buffer the buffer written below was last read
        // by PV(i - 1); with two it was PV(i - 2), which the MMA warp issued before S(i) (whose completion s_full
        // reported, and a commit covers everything issued before it).
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
      uint8_t* p_s = p_g + (i % L::kPBufs) * L::kPBytes;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        auto pr = [&](int q) { return ex2_approx(fmaf(__uint_as_float(sc[c][q]), sl2, nshift)); };
        if (kFp8) {
          uint32_t w[8];
#pragma unroll
          for (int q = 0; q < 8; ++q) w[q] = pack_e4m3x4(pr(4 * q), pr(4 * q + 1), pr(4 * q + 2), pr(4 * q + 3));
          uint8_t* rowp = p_s + r * 64;
          const int sw = (r >> 1) & 3;
          *reinterpret_cast<uint4*>(rowp + (((2 * c) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          *reinterpret_cast<uint4*>(rowp + (((2 * c + 1) ^ sw) << 4)) = make_uint4(w[4], w[5], w[6], w[7]);
        } else {
          uint8_t* rowp = p_s + r * 128;
          const int sw = r & 7;
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            uint32_t w[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(pr(8 * h + 2 * q), pr(8 * h + 2 * q + 1));
            *reinterpret_cast<uint4*>(rowp + (((4 * c + h) ^ sw) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
          }
        }
      }
      fence_proxy_async_smem();
      tc_fence_before();
      warp_arrive(smem_u32(&p_full[2 * g + (i & 1)]), lane);
    }
    // the group's result: 64 outputs and the row sum, still scaled by 2^(kPShift - m_run)
    float o[64];
    float l_run = 0.f;
#pragma unroll
    for (int d = 0; d < 64; ++d) o[d] = 0.f;
    if (ok && my_chunks > 0) {
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

    // ---------------- merge the groups (tensor work and TMA traffic are finished for all after the barrier)
    asm volatile("bar.sync 2, 384;" ::: "memory");
    float* comb = reinterpret_cast<float*>(smem + L::kPOff);  // [2][66][128]
    if (g > 0) {
      float* mine = comb + (g - 1) * 66 * 128;
      mine[r] = m_run;
      mine[128 + r] = l_run;
#pragma unroll
      for (int d = 0; d < 64; ++d) mine[(2 + d) * 128 + r] = o[d];
    }
    asm volatile("bar.sync 2, 384;" ::: "memory");
    if (g == 0 && ok && row_ok && *abort_flag == 0) {
      float m = m_run;
#pragma unroll
      for (int j = 0; j < G - 1; ++j) m = fmaxf(m, comb[j * 66 * 128 + r]);
      const float a0 = ex2_approx(m_run - m);
      float l = l_run * a0;
#pragma unroll
      for (int d = 0; d < 64; ++d) o[d] *= a0;
#pragma unroll 1
      for (int j = 0; j < G - 1; ++j) {
        const float* part = comb + j * 66 * 128;
        const float aj = ex2_approx(part[r] - m);
        l = fmaf(part[128 + r], aj, l);
#pragma unroll
        for (int d = 0; d < 64; ++d) o[d] = fmaf(part[(2 + d) * 128 + r], aj, o[d]);
      }
      const float vs = a.v_scale ? __ldg(a.v_scale + kvh) : 1.0f;
      const float inv = l > 0.f ? vs / l : 0.f;
      uint4* dst = reinterpret_cast<uint4*>(a.out + static_cast<size_t>(t) * a.o_row + static_cast<size_t>(qh) * a.o_head);
#pragma unroll
      for (int v = 0; v < 8; ++v) {
        uint32_t w[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) w[q] = pack_bf16x2(o[8 * v + 2 * q] * inv, o[8 * v + 2 * q + 1] * inv);
        dst[v] = make_uint4(w[0], w[1], w[2], w[3]);
        if (a.out_q != nullptr) {  // narrowed from the bf16-rounded values: equals a separate bf16 -> e4m3 cast
          *reinterpret_cast<uint2*>(a.out_q + static_cast<size_t>(t) * a.o_row + static_cast<size_t>(qh) * a.o_head + v * 8) =
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

int32_t make_tmap_2d_sw(CUtensorMap* tm, const void* base, int elem_bytes, uint64_t rows, uint64_t cols, uint32_t box_rows,
                        uint32_t box_cols, int swizzle_bytes);

// Launches the three-group kernel for one (query tile, head) per CTA (no key splits).
int32_t launch_attn4(const void* K_cache, const void* Vt_cache, const AttnArgs& a, int n_kv_heads, bool fp8, cudaStream_t st) {
  const int es = fp8 ? 1 : 2;
  CUtensorMap tmK, tmV;
  int32_t rc = make_tmap_2d_sw(&tmK, K_cache, es, static_cast<uint64_t>(n_kv_heads) * a.capacity, 64, kA4Chunk, 64, fp8 ? 64 : 128);
  if (rc != QB_OK) return rc;
  rc = make_tmap_2d_sw(&tmV, Vt_cache, es, static_cast<uint64_t>(n_kv_heads) * 64, a.capacity, 64, kA4Chunk, fp8 ? 64 : 128);
  if (rc != QB_OK) return rc;
  dim3 grid((a.tpf + 127) / 128, a.n_q_heads, 1);
  if (fp8) {
    QB_CUDA_OK(cudaFuncSetAttribute(owl_attn4_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, A4Smem<true>::kTotal));
    return launch_dep("owl_attn kernel (three groups)", owl_attn4_kernel<true>, grid, dim3(kA4Threads), A4Smem<true>::kTotal, st, tmK, tmV, a);
  }
  QB_CUDA_OK(cudaFuncSetAttribute(owl_attn4_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, A4Smem<false>::kTotal));
  return launch_dep("owl_attn kernel (three groups)", owl_attn4_kernel<false>, grid, dim3(kA4Threads), A4Smem<false>::kTotal, st, tmK, tmV, a);
}

}  // namespace qb
