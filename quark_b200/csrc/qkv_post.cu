// Fused post-processing of the packed QKV projection: per-head RMS norm of Q and K, value residual
// on V, RoPE(K), and the KV-cache append, in one pass over qkv.
//
// Replaces three launches (head_rmsnorm, value_residual_packed, kv_cache_update) that each stream the
// [tpf, (Hq + 2 Hk) * 64] tensor through HBM.  Every rounding point of the unfused chain is kept
// (normalised Q / K and mixed V are rounded to bf16 before anything else uses them, sums of squares
// are added in the same order), so the outputs are bit-identical to running the three kernels.
// One CTA handles 64 tokens of one KV head: its K head, its V head and the gqa Q heads that share it.
#include "common.cuh"
#include "rope.cuh"

namespace qb {

constexpr int kPostTile = 64;
constexpr int kPostThreads = 256;
constexpr int kPostVPitch = 72;  // smem row pitch of the V tile in 16-bit words

struct QkvPostArgs {
  const uint16_t* qkv_in;
  const uint16_t* qkv_first;  // may be null: no value residual
  const float* lamb;
  uint16_t* qkv_out;
  const int32_t* frame_t;
  const int32_t* frozen;
  void* K_cache;
  void* Vt_cache;
  int32_t* segments;
  int32_t* n_segments;
  const float* rope_xy;
  const float* k_scale;  // optional per-head cache scales (see qb_kv_params)
  const float* v_scale;
  int qkv_dim, n_q_heads, n_kv_heads, gqa;
  int tpf, nb, pd, max_segments;
  float eps;
};

__device__ __forceinline__ void unpack16(const uint4& a, const uint4& b, float (&f)[16]) {
  const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    f[2 * j] = bf16lo(w[j]);
    f[2 * j + 1] = bf16hi(w[j]);
  }
}

// RMS norm of one 64-wide head held by 4 consecutive lanes (16 elements each).  The squares are
// added in the order of the stand-alone kernel: 8 + 8 sequentially, then pairs of lanes.
__device__ __forceinline__ void head_norm16(float (&f)[16], float eps, uint4& o0, uint4& o1) {
  float sa = 0.f, sb = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) sa += f[j] * f[j];
#pragma unroll
  for (int j = 8; j < 16; ++j) sb += f[j] * f[j];
  float ss = sa + sb;
  ss += __shfl_xor_sync(0xffffffffu, ss, 1);
  ss += __shfl_xor_sync(0xffffffffu, ss, 2);
  const float inv = 1.0f / sqrtf(ss * (1.0f / 64.0f) + eps);
  uint32_t w[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) w[j] = pack_bf16x2(__fmul_rn(f[2 * j], inv), __fmul_rn(f[2 * j + 1], inv));
  o0 = make_uint4(w[0], w[1], w[2], w[3]);
  o1 = make_uint4(w[4], w[5], w[6], w[7]);
}

template <bool kFp8>
__global__ void __launch_bounds__(kPostThreads) qkv_post_kernel(const QkvPostArgs a) {
  grid_dep_wait();    // inputs come from the kernels before this one
  grid_dep_launch();  // the next kernel may begin its set-up
  constexpr int kEs = kFp8 ? 1 : 2;
  __shared__ float tm[16];
  __shared__ __align__(16) uint16_t vt[kPostTile * kPostVPitch];

  const int head = blockIdx.y;
  const int t0 = blockIdx.x * kPostTile;
  const int ft = *after_wait(a.frame_t);  // written on the device (incremented after every frame): an ordinary load
  const int frozen = *after_wait(a.frozen);
  const int L = a.nb * a.tpf;
  const int cap = L + a.tpf;
  const int bucket = (ft + a.pd - 1) / a.pd;
  const int slot = bucket % a.nb;
  const bool is_write = (ft % a.pd) == 0;
  const bool ring = is_write && frozen == 0;
  const int k_off = a.n_q_heads * 64, v_off = (a.n_q_heads + a.n_kv_heads) * 64;

  if (threadIdx.x < 8) temporal_cos_sin(ft, threadIdx.x, tm);
  const float inv_k = a.k_scale != nullptr ? __fdiv_rn(1.0f, __ldg(a.k_scale + head)) : 1.0f;  // * 1 changes no bit
  const float inv_v = a.v_scale != nullptr ? __fdiv_rn(1.0f, __ldg(a.v_scale + head)) : 1.0f;
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 32) {  // segment table: one thread of the grid
    int s[6] = {0, 0, 0, 0, 0, 0};
    int n;
    if (is_write && bucket >= a.nb) {
      s[1] = slot * a.tpf;
      s[2] = (slot + 1) * a.tpf;
      s[3] = (a.nb - slot - 1) * a.tpf;
      s[4] = L;
      s[5] = a.tpf;
      n = 3;
    } else {
      s[1] = min(bucket, a.nb) * a.tpf;
      s[2] = L;
      s[3] = a.tpf;
      n = 2;
    }
    for (int i = 0; i < 2 * a.max_segments; ++i) a.segments[i] = i < 6 ? s[i] : 0;
    a.n_segments[0] = n;
  }

  // Every global load of this thread is issued before the first result is needed: the kernel is a chain
  // of short phases, and one memory latency per phase would dominate its run time.
  const int tt = threadIdx.x >> 2, q = threadIdx.x & 3;
  const int t = t0 + tt;
  const size_t row = static_cast<size_t>(t) * a.qkv_dim;
  constexpr int kMaxGqa = 4;
  uint4 qa[kMaxGqa], qb4[kMaxGqa];
#pragma unroll
  for (int h = 0; h < kMaxGqa; ++h) {
    if (h < a.gqa) {
      const size_t off = row + (head * a.gqa + h) * 64 + q * 16;
      qa[h] = *reinterpret_cast<const uint4*>(a.qkv_in + off);
      qb4[h] = *reinterpret_cast<const uint4*>(a.qkv_in + off + 8);
    }
  }
  const size_t koff = row + k_off + head * 64 + q * 16;
  const uint4 ka = *reinterpret_cast<const uint4*>(a.qkv_in + koff);
  const uint4 kb = *reinterpret_cast<const uint4*>(a.qkv_in + koff + 8);
  float xy[16];
  {
    const float4* rp = reinterpret_cast<const float4*>(a.rope_xy + static_cast<size_t>(t) * 16);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float4 v = __ldg(rp + i);
      xy[4 * i] = v.x; xy[4 * i + 1] = v.y; xy[4 * i + 2] = v.z; xy[4 * i + 3] = v.w;
    }
  }

  // ---- V: value residual, round, keep a copy for the transpose, write the packed output
  const float lam = a.qkv_first != nullptr ? *a.lamb : 0.f;
  for (int v = threadIdx.x; v < kPostTile * 8; v += kPostThreads) {
    const int tt = v >> 3, c = v & 7;
    const size_t off = static_cast<size_t>(t0 + tt) * a.qkv_dim + v_off + head * 64 + c * 8;
    uint4 x = *reinterpret_cast<const uint4*>(a.qkv_in + off);
    if (a.qkv_first != nullptr) {
      const uint4 y = *reinterpret_cast<const uint4*>(a.qkv_first + off);
      const uint32_t xw[4] = {x.x, x.y, x.z, x.w}, yw[4] = {y.x, y.y, y.z, y.w};
      uint32_t w[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const float c0 = bf16lo(xw[j]), c1 = bf16hi(xw[j]);
        w[j] = pack_bf16x2(__fadd_rn(c0, __fmul_rn(lam, __fsub_rn(bf16lo(yw[j]), c0))),
                           __fadd_rn(c1, __fmul_rn(lam, __fsub_rn(bf16hi(yw[j]), c1))));
      }
      x = make_uint4(w[0], w[1], w[2], w[3]);
    }
    *reinterpret_cast<uint4*>(&vt[tt * kPostVPitch + c * 8]) = x;
    *reinterpret_cast<uint4*>(a.qkv_out + off) = x;
  }
  __syncthreads();

  // ---- Q heads that share this KV head, then K: 4 lanes per token, 16 elements per lane
#pragma unroll
  for (int h = 0; h < kMaxGqa; ++h) {
    if (h < a.gqa) {
      const size_t off = row + (head * a.gqa + h) * 64 + q * 16;
      float f[16];
      unpack16(qa[h], qb4[h], f);
      uint4 o0, o1;
      head_norm16(f, a.eps, o0, o1);
      *reinterpret_cast<uint4*>(a.qkv_out + off) = o0;
      *reinterpret_cast<uint4*>(a.qkv_out + off + 8) = o1;
    }
  }
  for (int h = kMaxGqa; h < a.gqa; ++h) {  // more Q heads per KV head than were fetched ahead
    const size_t off = row + (head * a.gqa + h) * 64 + q * 16;
    float f[16];
    unpack16(*reinterpret_cast<const uint4*>(a.qkv_in + off), *reinterpret_cast<const uint4*>(a.qkv_in + off + 8), f);
    uint4 o0, o1;
    head_norm16(f, a.eps, o0, o1);
    *reinterpret_cast<uint4*>(a.qkv_out + off) = o0;
    *reinterpret_cast<uint4*>(a.qkv_out + off + 8) = o1;
  }
  {
    const size_t off = koff;
    float f[16];
    unpack16(ka, kb, f);
    uint4 o0, o1;
    head_norm16(f, a.eps, o0, o1);
    *reinterpret_cast<uint4*>(a.qkv_out + off) = o0;
    *reinterpret_cast<uint4*>(a.qkv_out + off + 8) = o1;
    unpack16(o0, o1, f);  // rotate what the stand-alone append would read back: the bf16-rounded values
    float y0[8], y1[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float c, s;
      pair_cos_sin(q * 8 + j, xy, tm, c, s);
      y0[j] = __fmul_rn(__fsub_rn(__fmul_rn(f[2 * j], c), __fmul_rn(f[2 * j + 1], s)), inv_k);
      y1[j] = __fmul_rn(__fadd_rn(__fmul_rn(f[2 * j + 1], c), __fmul_rn(f[2 * j], s)), inv_k);
    }
    uint8_t* kc = static_cast<uint8_t*>(a.K_cache);
    const size_t row_bytes = 64 * kEs;
    const size_t tail = (static_cast<size_t>(head) * cap + L + t) * row_bytes;
    const size_t rr = (static_cast<size_t>(head) * cap + static_cast<size_t>(slot) * a.tpf + t) * row_bytes;
    if (kFp8) {
      // 8 bytes per lane; neighbouring lanes pair up so that every store is 16 bytes:
      // the even lane stores y0 of both, the odd lane y1 of both
      const uint2 m0 = make_uint2(pack_e4m3x4(y0[0], y0[1], y0[2], y0[3]), pack_e4m3x4(y0[4], y0[5], y0[6], y0[7]));
      const uint2 m1 = make_uint2(pack_e4m3x4(y1[0], y1[1], y1[2], y1[3]), pack_e4m3x4(y1[4], y1[5], y1[6], y1[7]));
      const bool odd = q & 1;
      const uint2 give = odd ? m0 : m1;
      uint2 got;
      got.x = __shfl_xor_sync(0xffffffffu, give.x, 1);
      got.y = __shfl_xor_sync(0xffffffffu, give.y, 1);
      const uint4 o = odd ? make_uint4(got.x, got.y, m1.x, m1.y) : make_uint4(m0.x, m0.y, got.x, got.y);
      const size_t col = (odd ? 32 : 0) + (q >> 1) * 16;
      *reinterpret_cast<uint4*>(kc + tail + col) = o;
      if (ring) *reinterpret_cast<uint4*>(kc + rr + col) = o;
    } else {
      const uint4 o0b = make_uint4(pack_bf16x2(y0[0], y0[1]), pack_bf16x2(y0[2], y0[3]), pack_bf16x2(y0[4], y0[5]), pack_bf16x2(y0[6], y0[7]));
      const uint4 o1b = make_uint4(pack_bf16x2(y1[0], y1[1]), pack_bf16x2(y1[2], y1[3]), pack_bf16x2(y1[4], y1[5]), pack_bf16x2(y1[6], y1[7]));
      *reinterpret_cast<uint4*>(kc + tail + q * 16) = o0b;
      *reinterpret_cast<uint4*>(kc + tail + 64 + q * 16) = o1b;
      if (ring) {
        *reinterpret_cast<uint4*>(kc + rr + q * 16) = o0b;
        *reinterpret_cast<uint4*>(kc + rr + 64 + q * 16) = o1b;
      }
    }
  }

  // ---- V: transposed 16-byte stores, one channel x (8 | 16) tokens each
  constexpr int kTokPerVec = 16 / kEs;
  constexpr int kVecPerCh = kPostTile / kTokPerVec;
  uint8_t* vc = static_cast<uint8_t*>(a.Vt_cache);
  for (int v = threadIdx.x; v < 64 * kVecPerCh; v += kPostThreads) {
    const int d = v / kVecPerCh, j = v % kVecPerCh;
    const int t1 = j * kTokPerVec;
    uint32_t w[4];
    if (kFp8) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = pack_e4m3x4(__fmul_rn(bf16_bits_to_f32(vt[(t1 + 4 * i) * kPostVPitch + d]), inv_v), __fmul_rn(bf16_bits_to_f32(vt[(t1 + 4 * i + 1) * kPostVPitch + d]), inv_v),
                           __fmul_rn(bf16_bits_to_f32(vt[(t1 + 4 * i + 2) * kPostVPitch + d]), inv_v), __fmul_rn(bf16_bits_to_f32(vt[(t1 + 4 * i + 3) * kPostVPitch + d]), inv_v));
    } else {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint16_t lo = vt[(t1 + 2 * i) * kPostVPitch + d], hi = vt[(t1 + 2 * i + 1) * kPostVPitch + d];
        w[i] = a.v_scale != nullptr ? pack_bf16x2(__fmul_rn(bf16_bits_to_f32(lo), inv_v), __fmul_rn(bf16_bits_to_f32(hi), inv_v))
                                    : static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
    }
    const uint4 o = make_uint4(w[0], w[1], w[2], w[3]);
    const size_t ch = (static_cast<size_t>(head) * 64 + d) * cap;
    *reinterpret_cast<uint4*>(vc + (ch + L + t0 + t1) * kEs) = o;
    if (ring) *reinterpret_cast<uint4*>(vc + (ch + static_cast<size_t>(slot) * a.tpf + t0 + t1) * kEs) = o;
  }
}

}  // namespace qb

using namespace qb;

extern "C" int32_t qb_qkv_post(const void* qkv_in, const void* qkv_first, const float* lamb, void* qkv_out, const int32_t* frame_t,
                               const int32_t* frozen, void* K_cache, void* Vt_cache, int32_t* segments, int32_t* n_segments,
                               const float* rope_xy, const qb_kv_params* p, float eps, void* stream) {
  QB_REQUIRE(p != nullptr, QB_ERR_INVALID_ARG, "qkv_post: params are NULL");
  QB_REQUIRE(qkv_in && qkv_out && frame_t && frozen && K_cache && Vt_cache && segments && n_segments && rope_xy, QB_ERR_INVALID_ARG,
             "qkv_post: NULL pointer");
  QB_REQUIRE((qkv_first == nullptr) == (lamb == nullptr), QB_ERR_INVALID_ARG, "qkv_post: qkv_first and lamb come together");
  QB_REQUIRE(p->quilt_factor == 1, QB_ERR_UNSUPPORTED, "qkv_post: quilt_factor %d is not supported (only 1)", p->quilt_factor);
  QB_REQUIRE(p->packed_qkv == 1, QB_ERR_UNSUPPORTED, "qkv_post: only the packed-QKV layout is supported");
  QB_REQUIRE(p->n_kv_heads > 0 && p->n_q_heads > 0 && p->n_q_heads % p->n_kv_heads == 0, QB_ERR_INVALID_ARG,
             "qkv_post: n_q_heads %d must be a positive multiple of n_kv_heads %d", p->n_q_heads, p->n_kv_heads);
  QB_REQUIRE(p->H_spatial > 0 && p->W_spatial > 0 && p->num_buckets > 0 && p->pinned_dilation > 0, QB_ERR_INVALID_ARG,
             "qkv_post: sizes must be positive");
  QB_REQUIRE(p->kv_dtype == QB_BF16 || p->kv_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "qkv_post: kv_dtype %d", p->kv_dtype);
  QB_REQUIRE(p->max_segments >= 3, QB_ERR_INVALID_ARG, "qkv_post: max_segments %d < 3", p->max_segments);
  const int tpf = p->H_spatial * p->W_spatial;
  QB_REQUIRE(tpf % kPostTile == 0, QB_ERR_UNSUPPORTED, "qkv_post: H*W = %d must be a multiple of %d", tpf, kPostTile);
  QB_REQUIRE(aligned16(qkv_in) && aligned16(qkv_first) && aligned16(qkv_out) && aligned16(K_cache) && aligned16(Vt_cache) &&
                 aligned16(rope_xy),
             QB_ERR_ALIGN, "qkv_post: pointers must be 16-byte aligned");
  QkvPostArgs a{};
  a.qkv_in = static_cast<const uint16_t*>(qkv_in);
  a.qkv_first = static_cast<const uint16_t*>(qkv_first);
  a.lamb = lamb;
  a.qkv_out = static_cast<uint16_t*>(qkv_out);
  a.frame_t = frame_t; a.frozen = frozen;
  a.K_cache = K_cache; a.Vt_cache = Vt_cache;
  a.segments = segments; a.n_segments = n_segments;
  a.rope_xy = rope_xy;
  a.k_scale = p->k_scale; a.v_scale = p->v_scale;
  a.qkv_dim = (p->n_q_heads + 2 * p->n_kv_heads) * 64;
  a.n_q_heads = p->n_q_heads; a.n_kv_heads = p->n_kv_heads; a.gqa = p->n_q_heads / p->n_kv_heads;
  a.tpf = tpf; a.nb = p->num_buckets; a.pd = p->pinned_dilation; a.max_segments = p->max_segments;
  a.eps = eps;
  dim3 grid(tpf / kPostTile, p->n_kv_heads);
  if (p->kv_dtype == QB_E4M3)
    return launch_dep("qkv_post", qkv_post_kernel<true>, grid, dim3(kPostThreads), 0, static_cast<cudaStream_t>(stream), a);
  return launch_dep("qkv_post", qkv_post_kernel<false>, grid, dim3(kPostThreads), 0, static_cast<cudaStream_t>(stream), a);
}
