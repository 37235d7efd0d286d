// KV-cache append: RoPE(K) -> narrow -> K rows; V -> narrow -> transposed columns; segment table.
//
// One CTA handles 64 tokens of one KV head.  K rows of a tile are one contiguous block in the
// cache, written with 16-byte stores straight from registers; V is transposed through shared
// memory so that each 16-byte store covers 8 (bf16) or 16 (e4m3) consecutive tokens of one
// channel.  Everything is written twice when the frame lands in the ring (tail slot + ring slot).
// Pure HBM traffic: 2 * tpf * Hk * 64 * 2 bytes read, 1x or 2x that (halved for e4m3) written.
#include "common.cuh"
#include "rope.cuh"

namespace qb {

constexpr int kKvTile = 64;      // tokens per CTA
constexpr int kKvThreads = 256;
constexpr int kVPitch = 72;      // smem row pitch of the V tile in 16-bit words

struct KvArgs {
  // K and V of token t, head h start at k_src / v_src + t * row_stride + h * head_stride (16-bit words): the packed
  // projection has row_stride = qkv_dim, head_stride = 64; separate [Hk * tpf, 64] tensors have 64 and tpf * 64
  const uint16_t* k_src;
  const uint16_t* v_src;
  size_t row_stride, head_stride;
  const int32_t* frame_t;
  const int32_t* frozen;
  void* K_cache;
  void* Vt_cache;
  int32_t* segments;
  int32_t* n_segments;
  const float* rope_xy;
  const float* k_scale;  // optional per-head scales: the cache holds value * (1 / scale[head])
  const float* v_scale;
  // Quilt: the cache keeps every quilt-th token of a frame, cached token i being token qoff + i * quilt; tpf below is
  // the cached count, so slots, capacity and the segment table are those of a frame of tpf tokens
  // (src/quark/kernels/kv_cache_update/reference.py:201-207, spec.py:66-76).  quilt = 1, qoff = 0: every token.
  int quilt, qoff;
  int tpf, nb, pd, max_segments;
};

template <bool kFp8>
__global__ void __launch_bounds__(kKvThreads) kv_append_kernel(const KvArgs a) {
  constexpr int kPairs = kFp8 ? 16 : 8;        // rotation pairs per thread
  constexpr int kThreadsPerTok = 32 / kPairs;  // 2 or 4
  constexpr int kEs = kFp8 ? 1 : 2;
  __shared__ float tm[16];
  __shared__ __align__(16) uint16_t vt[kKvTile * kVPitch];

  const int head = blockIdx.y;
  const int t0 = blockIdx.x * kKvTile;
  const int ft = *a.frame_t;
  const int frozen = *a.frozen;
  const int L = a.nb * a.tpf;
  const int cap = L + a.tpf;
  const int bucket = (ft + a.pd - 1) / a.pd;
  const int slot = bucket % a.nb;
  const bool is_write = (ft % a.pd) == 0;
  const bool ring = is_write && frozen == 0;

  if (threadIdx.x < 8) temporal_cos_sin(ft, threadIdx.x, tm);
  // multiplying by exactly 1 changes no bit, so the scale-free call stays what it was
  const float inv_k = a.k_scale != nullptr ? __fdiv_rn(1.0f, __ldg(a.k_scale + head)) : 1.0f;
  const float inv_v = a.v_scale != nullptr ? __fdiv_rn(1.0f, __ldg(a.v_scale + head)) : 1.0f;

  // segment table: one thread of the whole grid
  if (blockIdx.x == 0 && blockIdx.y == 0 && threadIdx.x == 32) {
    int s[6] = {0, 0, 0, 0, 0, 0};
    int n;
    if (is_write && bucket >= a.nb) {
      s[0] = 0;                    s[1] = slot * a.tpf;
      s[2] = (slot + 1) * a.tpf;   s[3] = (a.nb - slot - 1) * a.tpf;
      s[4] = L;                    s[5] = a.tpf;
      n = 3;
    } else {
      s[0] = 0;                    s[1] = min(bucket, a.nb) * a.tpf;
      s[2] = L;                    s[3] = a.tpf;
      n = 2;
    }
    for (int i = 0; i < 2 * a.max_segments; ++i) a.segments[i] = i < 6 ? s[i] : 0;
    a.n_segments[0] = n;
  }

  // stage V (raw bf16) for the transpose
  for (int v = threadIdx.x; v < kKvTile * 8; v += kKvThreads) {
    const int tt = v >> 3, c = v & 7;
    if (t0 + tt >= a.tpf) continue;  // a cached frame shorter than the tile (a multiple of 16 tokens)
    const uint4 x = *reinterpret_cast<const uint4*>(a.v_src + static_cast<size_t>(a.qoff + (t0 + tt) * a.quilt) * a.row_stride + head * a.head_stride + c * 8);
    *reinterpret_cast<uint4*>(&vt[tt * kVPitch + c * 8]) = x;
  }
  __syncthreads();

  // ---- K: rotate, narrow, store rows
  if (threadIdx.x < kKvTile * kThreadsPerTok && t0 + threadIdx.x / kThreadsPerTok < a.tpf) {
    const int tt = threadIdx.x / kThreadsPerTok;
    const int q = threadIdx.x % kThreadsPerTok;
    const int t = t0 + tt;
    const int ts = a.qoff + t * a.quilt;  // the token this cache row holds: its position sets the rotation
    const uint16_t* src = a.k_src + static_cast<size_t>(ts) * a.row_stride + head * a.head_stride + q * kPairs * 2;
    float xy[16];
    {
      const float4* r = reinterpret_cast<const float4*>(a.rope_xy + static_cast<size_t>(ts) * 16);
      const float4 r0 = __ldg(r), r1 = __ldg(r + 1), r2 = __ldg(r + 2), r3 = __ldg(r + 3);
      xy[0] = r0.x; xy[1] = r0.y; xy[2] = r0.z; xy[3] = r0.w; xy[4] = r1.x; xy[5] = r1.y; xy[6] = r1.z; xy[7] = r1.w;
      xy[8] = r2.x; xy[9] = r2.y; xy[10] = r2.z; xy[11] = r2.w; xy[12] = r3.x; xy[13] = r3.y; xy[14] = r3.z; xy[15] = r3.w;
    }
    float y0[kPairs], y1[kPairs];
#pragma unroll
    for (int v = 0; v < kPairs / 4; ++v) {
      const uint4 x = *reinterpret_cast<const uint4*>(src + v * 8);
      const uint32_t w[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int pl = v * 4 + j;            // pair index inside this thread
        const int p = q * kPairs + pl;       // pair index inside the head
        float c, s;
        pair_cos_sin(p, xy, tm, c, s);
        const float x0 = bf16lo(w[j]), x1 = bf16hi(w[j]);
        y0[pl] = __fmul_rn(__fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s)), inv_k);
        y1[pl] = __fmul_rn(__fadd_rn(__fmul_rn(x1, c), __fmul_rn(x0, s)), inv_k);
      }
    }
    uint4 o0, o1;
    if (kFp8) {
      o0 = make_uint4(pack_e4m3x4(y0[0], y0[1], y0[2], y0[3]), pack_e4m3x4(y0[4], y0[5], y0[6], y0[7]),
                      pack_e4m3x4(y0[8 % kPairs], y0[9 % kPairs], y0[10 % kPairs], y0[11 % kPairs]),
                      pack_e4m3x4(y0[12 % kPairs], y0[13 % kPairs], y0[14 % kPairs], y0[15 % kPairs]));
      o1 = make_uint4(pack_e4m3x4(y1[0], y1[1], y1[2], y1[3]), pack_e4m3x4(y1[4], y1[5], y1[6], y1[7]),
                      pack_e4m3x4(y1[8 % kPairs], y1[9 % kPairs], y1[10 % kPairs], y1[11 % kPairs]),
                      pack_e4m3x4(y1[12 % kPairs], y1[13 % kPairs], y1[14 % kPairs], y1[15 % kPairs]));
    } else {
      o0 = make_uint4(pack_bf16x2(y0[0], y0[1]), pack_bf16x2(y0[2], y0[3]), pack_bf16x2(y0[4], y0[5]), pack_bf16x2(y0[6], y0[7]));
      o1 = make_uint4(pack_bf16x2(y1[0], y1[1]), pack_bf16x2(y1[2], y1[3]), pack_bf16x2(y1[4], y1[5]), pack_bf16x2(y1[6], y1[7]));
    }
    uint8_t* kc = static_cast<uint8_t*>(a.K_cache);
    const size_t col0 = static_cast<size_t>(q) * 16;  // byte offset of this thread's y0 vector in a row
    const size_t row_bytes = 64 * kEs;
    const size_t tail = (static_cast<size_t>(head) * cap + L + t) * row_bytes;
    *reinterpret_cast<uint4*>(kc + tail + col0) = o0;
    *reinterpret_cast<uint4*>(kc + tail + 32 * kEs + col0) = o1;
    if (ring) {
      const size_t rr = (static_cast<size_t>(head) * cap + static_cast<size_t>(slot) * a.tpf + t) * row_bytes;
      *reinterpret_cast<uint4*>(kc + rr + col0) = o0;
      *reinterpret_cast<uint4*>(kc + rr + 32 * kEs + col0) = o1;
    }
  }

  // ---- V: transposed 16-byte stores, one channel x (8 | 16) tokens each
  constexpr int kTokPerVec = 16 / kEs;
  constexpr int kVecPerCh = kKvTile / kTokPerVec;
  uint8_t* vc = static_cast<uint8_t*>(a.Vt_cache);
  for (int v = threadIdx.x; v < 64 * kVecPerCh; v += kKvThreads) {
    const int d = v / kVecPerCh, j = v % kVecPerCh;
    const int tt = j * kTokPerVec;
    if (t0 + tt >= a.tpf) continue;
    uint4 o;
    if (kFp8) {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i)
        w[i] = pack_e4m3x4(__fmul_rn(bf16_bits_to_f32(vt[(tt + 4 * i) * kVPitch + d]), inv_v), __fmul_rn(bf16_bits_to_f32(vt[(tt + 4 * i + 1) * kVPitch + d]), inv_v),
                           __fmul_rn(bf16_bits_to_f32(vt[(tt + 4 * i + 2) * kVPitch + d]), inv_v), __fmul_rn(bf16_bits_to_f32(vt[(tt + 4 * i + 3) * kVPitch + d]), inv_v));
      o = make_uint4(w[0], w[1], w[2], w[3]);
    } else {
      uint32_t w[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        const uint16_t lo = vt[(tt + 2 * i) * kVPitch + d], hi = vt[(tt + 2 * i + 1) * kVPitch + d];
        w[i] = a.v_scale != nullptr ? pack_bf16x2(__fmul_rn(bf16_bits_to_f32(lo), inv_v), __fmul_rn(bf16_bits_to_f32(hi), inv_v))
                                    : static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
      }
      o = make_uint4(w[0], w[1], w[2], w[3]);
    }
    const size_t ch = (static_cast<size_t>(head) * 64 + d) * cap;
    *reinterpret_cast<uint4*>(vc + (ch + L + t0 + tt) * kEs) = o;
    if (ring) *reinterpret_cast<uint4*>(vc + (ch + static_cast<size_t>(slot) * a.tpf + t0 + tt) * kEs) = o;
  }
}

// rope_xy[t][0..7] = cos, [8..15] = sin of the 4 x-angles and 4 y-angles of token t.
// Angles are evaluated the way numpy evaluates the table: positions from an f64 linspace
// narrowed to f32, multiplied in f64 by (1 + i * step) * pi, narrowed to f32.
__global__ void rope_table_kernel(float* out, int H, int W) {
  const int idx = blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= H * W * 8) return;
  const int t = idx >> 3, i = idx & 7;
  const int fi = i & 3;
  const bool is_y = i >= 4;
  const int n = is_y ? H : W;
  const int pos_i = is_y ? t / W : t % W;
  const double start = __dadd_rn(-1.0, __ddiv_rn(1.0, static_cast<double>(n)));
  const double stop = __dsub_rn(1.0, __ddiv_rn(1.0, static_cast<double>(n)));
  double pos = start;
  if (n > 1) {
    const double step = __ddiv_rn(__dsub_rn(stop, start), static_cast<double>(n - 1));
    pos = pos_i == n - 1 ? stop : __dadd_rn(__dmul_rn(static_cast<double>(pos_i), step), start);
  }
  const float pos_f = static_cast<float>(pos);
  const double max_freq = __dmul_rn(static_cast<double>(min(H, W)), 0.8);
  const double fstop = __ddiv_rn(max_freq, 2.0);
  const double fstep = __ddiv_rn(__dsub_rn(fstop, 1.0), 3.0);
  const double lin = fi == 3 ? fstop : __dadd_rn(__dmul_rn(static_cast<double>(fi), fstep), 1.0);
  const double freq = __dmul_rn(lin, 3.141592653589793);
  const float ang = static_cast<float>(__dmul_rn(static_cast<double>(pos_f), freq));
  float s, c;
  sincosf(ang, &s, &c);
  out[t * 16 + i] = c;
  out[t * 16 + 8 + i] = s;
}

// ---------------------------------------------------------------- shadow cache in the attention's compute dtype
// When the attention computes in another dtype than the cache stores (kv_cache = fp8 with attn_compute = bf16, or the
// reverse), the reference casts K and V as it loads them (src/quark/kernels/owl_attn/kernel.py:342-348).  Tensor-core
// operands go from shared memory to the MMA without passing through registers here, so the cast happens once per
// appended row instead: a second pair of caches in the compute dtype is kept beside the first, and after every append
// this kernel converts the rows that append wrote (the tail slot always, the ring slot on write frames), reading the
// stored values, so the shadow holds exactly cast(cache) - what a cast on load would produce.  Traffic: the appended
// rows only, not the whole cache.
struct KvCastArgs {
  const void* K_cache;
  const void* Vt_cache;
  void* K_shadow;
  void* Vt_shadow;
  const int32_t* frame_t;
  const int32_t* frozen;
  int tpf, nb, pd;
};

template <bool kSrcFp8>
__device__ __forceinline__ void cast16(const void* src, void* dst, size_t idx) {
  if (kSrcFp8) {  // 16 e4m3 -> 16 bf16, exact
    const uint4 v = *reinterpret_cast<const uint4*>(static_cast<const uint8_t*>(src) + idx);
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      o[2 * j] = e4m3x2_to_bf16x2(static_cast<uint16_t>(w[j] & 0xFFFF));
      o[2 * j + 1] = e4m3x2_to_bf16x2(static_cast<uint16_t>(w[j] >> 16));
    }
    uint16_t* d = static_cast<uint16_t*>(dst) + idx;
    *reinterpret_cast<uint4*>(d) = make_uint4(o[0], o[1], o[2], o[3]);
    *reinterpret_cast<uint4*>(d + 8) = make_uint4(o[4], o[5], o[6], o[7]);
  } else {  // 16 bf16 -> 16 e4m3, nearest even, saturating (qb_quantize_e4m3)
    const uint16_t* sp = static_cast<const uint16_t*>(src) + idx;
    const uint4 a = *reinterpret_cast<const uint4*>(sp), b = *reinterpret_cast<const uint4*>(sp + 8);
    const uint32_t w[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    uint32_t o[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) o[j] = pack_e4m3x4(bf16lo(w[2 * j]), bf16hi(w[2 * j]), bf16lo(w[2 * j + 1]), bf16hi(w[2 * j + 1]));
    *reinterpret_cast<uint4*>(static_cast<uint8_t*>(dst) + idx) = make_uint4(o[0], o[1], o[2], o[3]);
  }
}

template <bool kSrcFp8>
__global__ void __launch_bounds__(kKvThreads) kv_cast_appended_kernel(const KvCastArgs a) {
  grid_dep_wait();    // the rows were written by the append just before
  grid_dep_launch();
  const int head = blockIdx.y;
  const int t0 = blockIdx.x * kKvTile;
  const int ft = *after_wait(a.frame_t);
  const int frozen = *after_wait(a.frozen);
  const int L = a.nb * a.tpf;
  const int cap = L + a.tpf;
  const bool ring = (ft % a.pd) == 0 && frozen == 0;
  if (blockIdx.z == 1 && !ring) return;
  const int base = blockIdx.z == 0 ? L : (((ft + a.pd - 1) / a.pd) % a.nb) * a.tpf;
  const int ntok = min(kKvTile, a.tpf - t0);  // a multiple of 16
  // K: ntok rows of 64 values, contiguous
  const size_t krow0 = (static_cast<size_t>(head) * cap + base + t0) * 64;
  for (int i = threadIdx.x; i < ntok * 4; i += kKvThreads) cast16<kSrcFp8>(a.K_cache, a.K_shadow, krow0 + static_cast<size_t>(i) * 16);
  // V^T: 64 channel rows, ntok consecutive tokens of each
  const int per_row = ntok / 16;
  for (int i = threadIdx.x; i < 64 * per_row; i += kKvThreads) {
    const int d = i / per_row, j = i % per_row;
    cast16<kSrcFp8>(a.Vt_cache, a.Vt_shadow, (static_cast<size_t>(head) * 64 + d) * cap + base + t0 + 16 * j);
  }
}

}  // namespace qb

using namespace qb;

extern "C" int32_t qb_rope_table_build(float* rope_xy, int32_t H_spatial, int32_t W_spatial, void* stream) {
  QB_REQUIRE(rope_xy != nullptr, QB_ERR_INVALID_ARG, "rope_table_build: NULL pointer");
  QB_REQUIRE(H_spatial > 0 && W_spatial > 0, QB_ERR_INVALID_ARG, "rope_table_build: H_spatial and W_spatial must be > 0 (got %d, %d)",
             H_spatial, W_spatial);
  const int n = H_spatial * W_spatial * 8;
  rope_table_kernel<<<(n + 255) / 256, 256, 0, static_cast<cudaStream_t>(stream)>>>(rope_xy, H_spatial, W_spatial);
  return check_launch("rope_table_build");
}

static int32_t kv_append(const void* k_src, const void* v_src, size_t row_stride, size_t head_stride, const int32_t* frame_t,
                         const int32_t* frozen, void* K_cache, void* Vt_cache, int32_t* segments, int32_t* n_segments, const float* rope_xy,
                         const qb_kv_params* p, void* stream) {
  QB_REQUIRE(k_src && v_src && frame_t && frozen && K_cache && Vt_cache && segments && n_segments && rope_xy, QB_ERR_INVALID_ARG,
             "kv_cache_update: NULL pointer");
  QB_REQUIRE(p->quilt_factor >= 1 && p->quilt_offset >= 0 && p->quilt_offset < p->quilt_factor, QB_ERR_INVALID_ARG,
             "kv_cache_update: quilt_factor %d, quilt_offset %d", p->quilt_factor, p->quilt_offset);
  QB_REQUIRE(p->n_kv_heads > 0 && p->n_q_heads >= 0 && p->H_spatial > 0 && p->W_spatial > 0 && p->num_buckets > 0 &&
                 p->pinned_dilation > 0,
             QB_ERR_INVALID_ARG, "kv_cache_update: sizes must be positive");
  QB_REQUIRE(p->kv_dtype == QB_BF16 || p->kv_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "kv_cache_update: kv_dtype %d", p->kv_dtype);
  QB_REQUIRE(p->max_segments >= 3, QB_ERR_INVALID_ARG, "kv_cache_update: max_segments %d < 3", p->max_segments);
  QB_REQUIRE((p->H_spatial * p->W_spatial) % p->quilt_factor == 0, QB_ERR_INVALID_ARG, "kv_cache_update: H*W = %d is not a multiple of quilt_factor %d",
             p->H_spatial * p->W_spatial, p->quilt_factor);
  const int tpf = p->H_spatial * p->W_spatial / p->quilt_factor;  // tokens of a frame that the cache keeps
  QB_REQUIRE(tpf % 16 == 0, QB_ERR_UNSUPPORTED, "kv_cache_update: H*W / quilt_factor = %d must be a multiple of 16 (one 16-byte vector of V^T)", tpf);
  QB_REQUIRE(aligned16(k_src) && aligned16(v_src) && aligned16(K_cache) && aligned16(Vt_cache) && aligned16(rope_xy), QB_ERR_ALIGN,
             "kv_cache_update: pointers must be 16-byte aligned");
  KvArgs a{};
  a.k_src = static_cast<const uint16_t*>(k_src);
  a.v_src = static_cast<const uint16_t*>(v_src);
  a.row_stride = row_stride; a.head_stride = head_stride;
  a.frame_t = frame_t; a.frozen = frozen;
  a.K_cache = K_cache; a.Vt_cache = Vt_cache;
  a.segments = segments; a.n_segments = n_segments;
  a.rope_xy = rope_xy;
  a.k_scale = p->k_scale; a.v_scale = p->v_scale;
  a.quilt = p->quilt_factor; a.qoff = p->quilt_offset;
  a.tpf = tpf; a.nb = p->num_buckets; a.pd = p->pinned_dilation; a.max_segments = p->max_segments;
  dim3 grid((tpf + kKvTile - 1) / kKvTile, p->n_kv_heads);
  if (p->kv_dtype == QB_E4M3)
    kv_append_kernel<true><<<grid, kKvThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  else
    kv_append_kernel<false><<<grid, kKvThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
  return check_launch("kv_cache_update");
}

extern "C" int32_t qb_kv_cache_update(const void* qkv, const int32_t* frame_t, const int32_t* frozen, void* K_cache, void* Vt_cache,
                                      int32_t* segments, int32_t* n_segments, const float* rope_xy, const qb_kv_params* p,
                                      void* stream) {
  QB_REQUIRE(p != nullptr, QB_ERR_INVALID_ARG, "kv_cache_update: params are NULL");
  QB_REQUIRE(qkv != nullptr, QB_ERR_INVALID_ARG, "kv_cache_update: NULL pointer");
  QB_REQUIRE(p->packed_qkv == 1, QB_ERR_INVALID_ARG, "kv_cache_update: separate K and V go through qb_kv_cache_update_kv");
  const uint16_t* base = static_cast<const uint16_t*>(qkv);
  return kv_append(base + p->n_q_heads * 64, base + (p->n_q_heads + p->n_kv_heads) * 64,
                   static_cast<size_t>(p->n_q_heads + 2 * p->n_kv_heads) * 64, 64, frame_t, frozen, K_cache, Vt_cache, segments, n_segments,
                   rope_xy, p, stream);
}

extern "C" int32_t qb_kv_cache_update_kv(const void* K, const void* V, const int32_t* frame_t, const int32_t* frozen, void* K_cache,
                                         void* Vt_cache, int32_t* segments, int32_t* n_segments, const float* rope_xy,
                                         const qb_kv_params* p, void* stream) {
  QB_REQUIRE(p != nullptr, QB_ERR_INVALID_ARG, "kv_cache_update: params are NULL");
  QB_REQUIRE(p->packed_qkv == 0, QB_ERR_INVALID_ARG, "kv_cache_update: the packed projection goes through qb_kv_cache_update");
  const size_t tpf = static_cast<size_t>(p->H_spatial) * p->W_spatial;  // K and V hold every token, quilt or not
  return kv_append(K, V, 64, tpf * 64, frame_t, frozen, K_cache, Vt_cache, segments, n_segments, rope_xy, p, stream);
}

extern "C" int32_t qb_kv_cast_appended(const void* K_cache, const void* Vt_cache, void* K_shadow, void* Vt_shadow, const int32_t* frame_t,
                                       const int32_t* frozen, const qb_kv_params* p, void* stream) {
  QB_REQUIRE(p != nullptr && K_cache && Vt_cache && K_shadow && Vt_shadow && frame_t && frozen, QB_ERR_INVALID_ARG, "kv_cast_appended: NULL pointer");
  QB_REQUIRE(p->n_kv_heads > 0 && p->H_spatial > 0 && p->W_spatial > 0 && p->num_buckets > 0 && p->pinned_dilation > 0 && p->quilt_factor >= 1,
             QB_ERR_INVALID_ARG, "kv_cast_appended: sizes must be positive");
  QB_REQUIRE(p->kv_dtype == QB_BF16 || p->kv_dtype == QB_E4M3, QB_ERR_INVALID_ARG, "kv_cast_appended: kv_dtype %d", p->kv_dtype);
  QB_REQUIRE((p->H_spatial * p->W_spatial) % p->quilt_factor == 0, QB_ERR_INVALID_ARG, "kv_cast_appended: H*W is not a multiple of quilt_factor");
  const int tpf = p->H_spatial * p->W_spatial / p->quilt_factor;
  QB_REQUIRE(tpf % 16 == 0, QB_ERR_UNSUPPORTED, "kv_cast_appended: H*W / quilt_factor = %d must be a multiple of 16", tpf);
  QB_REQUIRE(aligned16(K_cache) && aligned16(Vt_cache) && aligned16(K_shadow) && aligned16(Vt_shadow), QB_ERR_ALIGN,
             "kv_cast_appended: pointers must be 16-byte aligned");
  KvCastArgs a{};
  a.K_cache = K_cache; a.Vt_cache = Vt_cache; a.K_shadow = K_shadow; a.Vt_shadow = Vt_shadow;
  a.frame_t = frame_t; a.frozen = frozen;
  a.tpf = tpf; a.nb = p->num_buckets; a.pd = p->pinned_dilation;
  const dim3 grid((tpf + kKvTile - 1) / kKvTile, p->n_kv_heads, 2);
  if (p->kv_dtype == QB_E4M3)
    return launch_dep("kv_cast_appended", kv_cast_appended_kernel<true>, grid, dim3(kKvThreads), 0, static_cast<cudaStream_t>(stream), a);
  return launch_dep("kv_cast_appended", kv_cast_appended_kernel<false>, grid, dim3(kKvThreads), 0, static_cast<cudaStream_t>(stream), a);
}
