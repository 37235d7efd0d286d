/*
 * quark_b200 - C ABI of the sm_100a kernel library for the Waypoint-1.5 DiT per-NFE hot path.
 *
 * One shared library (libquark_b200.so) replaces everything below the reference's
 * `quark.functional` (qf.*) layer for this path.  The reference reaches its kernels through
 * Python: qf.* -> Launcher -> PTX text -> cuModuleLoadData / cuLaunchKernel via ctypes
 * (src/quark/drivers/cuda.py:159-239, src/quark/runtime/cuda.py:81-110) or cublasLtMatmul via
 * ctypes (src/quark/runtime/cublas.py:265-459).  A maintainer binds these entry points with
 * ctypes in the same way.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless its name ends in `_host`;
 *   - `stream` is a cudaStream_t / CUstream passed as void* (NULL = default stream);
 *   - tensors are row-major and contiguous; bf16 and e4m3 are raw 16- and 8-bit words;
 *   - every function returns QB_OK (0) or a negative qb_status, never aborts the process,
 *     never synchronises the device and never allocates device memory except where the
 *     comment says so (the qb_malloc family and qb_device_status);
 *   - after an error qb_last_error_string() holds a message for the calling thread;
 *   - compute calls are stream-capturable: scalars that change per step (frame_t, frozen,
 *     segments) live in device memory, so a captured CUDA graph can be replayed.
 *
 * Paths relative to the reference project are cited as "ref:".
 */
#ifndef QUARK_B200_H
#define QUARK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
  QB_OK = 0,
  QB_ERR_INVALID_ARG = -1, /* bad shape / NULL pointer / inconsistent sizes */
  QB_ERR_UNSUPPORTED = -2, /* legal in the reference, not implemented here (e.g. b_shuffled weights) */
  QB_ERR_ALIGN = -3,       /* pointer or row pitch not 16-byte aligned */
  QB_ERR_LAUNCH = -4,      /* CUDA reported an error at launch */
  QB_ERR_DEVICE = -5,      /* no CUDA device, or not compute capability 10.0 */
  QB_ERR_WORKSPACE = -6,   /* workspace missing or too small */
  QB_ERR_CUDA = -7         /* a CUDA runtime call failed (message has the detail) */
} qb_status;

/* dtype codes; names follow ref: src/quark/runtime/tensor.py:57-69 */
typedef enum { QB_BF16 = 0, QB_E4M3 = 1, QB_F32 = 2, QB_S32 = 3 } qb_dtype;

/* ------------------------------------------------------------------ library / device */
int32_t qb_version(void);
const char* qb_last_error_string(void);
/* Number of CUDA devices, 0 when there is none (never fails). */
int32_t qb_device_count(void);
/* QB_OK iff `device` exists and is compute capability 10.0. */
int32_t qb_device_check(int32_t device);
int32_t qb_set_device(int32_t device);
/* Reads and clears the device status word that kernels set when a bounded wait ran out
 * (bit 0 GEMM, bit 1 attention, bit 3 the cross-GPU reduction) or a segment table was malformed (bit 2).
 * Synchronises. */
int32_t qb_device_status(uint32_t* status_host);
/* Number of kernels this library has launched since it was loaded (launches recorded into a CUDA
 * graph during capture count once, replays do not count). */
uint64_t qb_kernel_launch_count(void);
/* The hot-path kernels are launched so that each may begin its set-up (barriers, TMEM, weight prefetch)
 * while the kernel before it in the stream is still running (programmatic dependent launch); each waits
 * for that kernel to complete before it reads its results or writes global memory, so results do not
 * change.  enabled = 0 turns this off (as does QB_DEPENDENT_LAUNCH=0 in the environment when the library
 * is loaded).  Returns the previous setting.  No counterpart in the reference. */
int32_t qb_set_dependent_launch(int32_t enabled);

/* ------------------------------------------------------------------ memory / streams / graphs
 * Replaces the ctypes libcuda subset the reference's tensor class uses
 * (ref: src/quark/runtime/cuda.py:118-800: mem_alloc, memcpy_htod/dtoh/dtod, memset,
 * stream/event helpers, and src/quark/graph.py:105-173 for capture). */
int32_t qb_malloc(void** ptr_host, size_t bytes);
int32_t qb_free(void* ptr);
int32_t qb_host_alloc(void** ptr_host, size_t bytes); /* pinned host memory */
int32_t qb_host_free(void* ptr_hostmem);
/* kind: 0 host->device, 1 device->host, 2 device->device; asynchronous on `stream` */
int32_t qb_memcpy_async(void* dst, const void* src, size_t bytes, int32_t kind, void* stream);
int32_t qb_memset_async(void* dst, int32_t byte_value, size_t bytes, void* stream);
int32_t qb_memset32_async(void* dst, uint32_t value, size_t count, void* stream);
int32_t qb_stream_create(void** stream_host);
int32_t qb_stream_destroy(void* stream);
int32_t qb_stream_sync(void* stream);
int32_t qb_device_sync(void);
int32_t qb_event_create(void** event_host);
int32_t qb_event_destroy(void* event);
int32_t qb_event_record(void* event, void* stream);
int32_t qb_event_sync(void* event);
int32_t qb_event_elapsed_ms(void* start, void* stop, float* ms_host);
int32_t qb_graph_begin(void* stream);
int32_t qb_graph_end(void* stream, void** graph_exec_host);
int32_t qb_graph_launch(void* graph_exec, void* stream);
int32_t qb_graph_destroy(void* graph_exec);

/* ------------------------------------------------------------------ GEMM
 * C[M,N] = epilogue(A[M,K] . B[N,K]^T), f32 accumulation, epilogue order
 *   acc * (a_scale * w_scale[n]) -> + bias[n] -> SiLU -> * gate[m / (M/G), n] + residual[m, n] -> cast
 * Replaces qf.gemm (ref: src/quark/functional/gemm.py:597-635), i.e. GemmKernel
 * (ref: src/quark/kernels/gemm/kernel.py:831-895, epilogue order src/quark/lang/epilogue.py:387-420)
 * and the cublasLtMatmul path (ref: src/quark/runtime/cublas.py:265-459).
 *
 * compute_dtype QB_BF16 needs A and B in bf16; QB_E4M3 needs B in e4m3 and A in e4m3 or bf16.
 * A bf16 A is first narrowed to e4m3 (round-to-nearest-even, saturating, unscaled) into the
 * workspace, which is what the reference's cuBLAS route does with a separate launch
 * (ref: src/quark/kernels/gemm/cublas_dispatch.py:164-168).
 * bias / gate / residual / a_scale / w_scale may be NULL (scales default to 1: the reference
 * has no scales).  gate and residual come together.  C may be bf16, f32 or e4m3.
 * Needs K % 16 == 0, N % 8 == 0 and 16-byte aligned pointers. */
typedef struct {
  int32_t M, N, K;
  int32_t a_dtype, b_dtype, c_dtype; /* qb_dtype */
  int32_t compute_dtype;             /* QB_BF16 or QB_E4M3 */
  int32_t activation;                /* 0 none, 1 SiLU */
  int32_t gate_groups;               /* G: gate is [G, N], each row covers M/G rows */
  int32_t split_k;                   /* 0 = choose; >= 1 forces the number of K slices */
  int32_t tile_n;                    /* 0 = choose; 64, 128 or 256 */
  int32_t reserved;                  /* flags.  bit 0, slice mode: 0 = sum K slices inside a thread-block cluster when there
                                        are 2, 4 or 8 of them (no workspace traffic); 1 = always through the workspace.
                                        bit 1: B is constant (weights; no kernel in flight writes it), so its first tiles
                                        may be fetched before the kernels ahead of this one in the stream have finished */
  const float* a_scale; /* [1]  optional */
  const float* w_scale; /* [N]  optional */
} qb_gemm_params;

/* Bytes of workspace qb_gemm needs for `p` (tile counters, the e4m3 copy of a bf16 A, K-slice
 * partial sums); 0 when the call touches no scratch memory.  The counters occupy the first 64 KiB
 * of the workspace whatever the shape, so calls of different shapes may share one workspace; that
 * area must be zero before the first use, and qb_gemm leaves it zero.  Calls that share a workspace
 * must not overlap on the GPU. */
size_t qb_gemm_workspace_bytes(const qb_gemm_params* p);
int32_t qb_gemm(const void* A, const void* B, void* C, const void* bias, const void* gate, const void* residual,
                const qb_gemm_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* qb_gemm without a workspace argument, for callers that must not allocate device memory.
 * No counterpart in the reference.
 * Some hosts cannot call cudaMalloc where they call the GEMM: a frame loop with a hard latency
 * budget (cudaMalloc may synchronise the whole device), a plugin that was handed a fixed memory
 * budget by the application that embeds it, or code that runs while another allocator (a game
 * engine's, a framework's caching allocator) owns all of the device memory.  This entry point gives
 * them the same GEMM on scratch memory that is part of the library image: a file-scope device array
 * of qb_gemm_static_scratch_capacity() = 8 MiB bytes, present on every GPU that loads the library
 * until the process exits.  It performs no cudaMalloc / cudaFree and calls no allocating routine.
 * Limits: a GEMM whose scratch need (qb_gemm_workspace_bytes) exceeds the capacity is rejected with
 * QB_ERR_WORKSPACE and a message that states both numbers.  All calls share the one array, which
 * keeps the previous call's contents (the part that must start at zero is cleared on the stream by
 * every call): two calls that overlap on the GPU (different streams, no ordering) race on it.
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress); make
 * that first call before any stream capture begins.  The address is that of the calling thread's
 * current device (cudaGetDevice), which must be the device `stream` belongs to; the lookup is safe
 * against two host threads making their first calls at once, and cudaDeviceReset invalidates it for
 * that device.  A call that is rejected enqueues nothing.  Results are bit-identical to qb_gemm. */
size_t qb_gemm_static_scratch_capacity(void);
int32_t qb_gemm_static_scratch(const void* A, const void* B, void* C, const void* bias, const void* gate, const void* residual,
                               const qb_gemm_params* p, void* stream);

/* X -> e4m3, round-to-nearest-even, saturate to +-448, NaN -> 0x7F, no scale.
 * Replaces qf.quantize_e4m3 (ref: src/quark/functional/quantize_e4m3.py:25-69,
 * src/quark/kernels/quantize_e4m3/kernel.py:107-176). src_dtype: QB_BF16 or QB_F32. */
int32_t qb_quantize_e4m3(const void* X, void* out, size_t n, int32_t src_dtype, void* stream);
/* Per-row scaled narrowing of a bf16 matrix X [rows, cols] (a weight [out, in]): scale[r] = max |X[r, :]| / 448
 * (1 for an all-zero row), out[r, c] = e4m3(X[r, c] * (1 / scale[r])), every step rounded to nearest in f32.
 * scale_out receives the f32 [rows] dequantisation scales that qb_gemm takes as w_scale.  An extension: the
 * reference narrows its weights without a scale (ref: src/quark/nn/layers.py:291-304).  cols % 8 == 0. */
int32_t qb_quantize_e4m3_rows(const void* X, void* out, float* scale_out, int32_t rows, int32_t cols, void* stream);
/* out[0..n) (bf16) = X[0..n) (e4m3), exact (every e4m3 value is a bf16 value; NaN stays NaN).  The widening half
 * of the reference's cast-on-load for a cache whose dtype differs from the attention's compute dtype
 * (ref: src/quark/kernels/owl_attn/kernel.py:342-348), here as a pass of its own. */
int32_t qb_dequantize_e4m3(const void* X, void* out, size_t n, void* stream);

/* ------------------------------------------------------------------ KV-cache append
 * Reads the K and V columns of packed qkv [tpf, (Hq + 2 Hk) * 64] bf16, applies ortho-RoPE to K
 * in f32, narrows to kv_dtype, writes K rows and transposed V columns to the tail slot
 * (rows [L, L + tpf)) always and to ring slot ((ft + pd - 1) / pd) % nb iff ft % pd == 0 and
 * frozen == 0, and rewrites the 3-entry segment table.
 * Replaces qf.kv_cache_update (ref: src/quark/functional/kv_cache_update.py:187-265,
 * src/quark/kernels/kv_cache_update/kernel.py:395-766; cache layout
 * src/quark/kernels/kv_cache_update/spec.py:11-14).
 *   K_cache  [Hk * capacity, 64]    Vt_cache [Hk * 64, capacity]    capacity = (nb + 1) * tpf
 *   segments s32[6], n_segments s32[1], frame_t s32[1], frozen s32[1]: device scalars.
 * rope_xy: f32 [tpf, 16] = per token 8 cosines then 8 sines of the 4 x- and 4 y-angles
 * (build with qb_rope_table_build, or on the host as the reference's numpy table does). */
typedef struct {
  int32_t n_q_heads, n_kv_heads;
  int32_t H_spatial, W_spatial;
  int32_t num_buckets, pinned_dilation;
  int32_t kv_dtype;     /* QB_BF16 or QB_E4M3 */
  int32_t max_segments; /* 3 */
  int32_t quilt_factor; /* the cache keeps every quilt_factor-th token of a frame (1: all); capacity, slots and
                         * segments are then those of H*W / quilt_factor tokens per frame */
  int32_t packed_qkv;   /* 1: qb_kv_cache_update (packed projection); 0: qb_kv_cache_update_kv (separate K, V) */
  int32_t quilt_offset; /* which residue: cached token i is token quilt_offset + i * quilt_factor */
  /* Optional per-KV-head quantisation scales, f32 [n_kv_heads] each (NULL = 1, the reference's scale-free caches;
   * an extension, see qb_attn_params): the cache holds narrow(RoPE(K) * (1 / k_scale[h])) and narrow(V * (1 / v_scale[h])),
   * the reciprocal and the product both rounded to nearest in f32.  qb_owl_attn given the same scales undoes them. */
  const float* k_scale;
  const float* v_scale;
} qb_kv_params;

int32_t qb_kv_cache_update(const void* qkv, const int32_t* frame_t, const int32_t* frozen, void* K_cache, void* Vt_cache,
                           int32_t* segments, int32_t* n_segments, const float* rope_xy, const qb_kv_params* p, void* stream);
/* The same with K and V as tensors of their own, head-major [Hk * tpf, 64] bf16 each (the reference's
 * packed_qkv=False layout, src/quark/kernels/kv_cache_update/reference.py:183-186); p->packed_qkv must be 0. */
int32_t qb_kv_cache_update_kv(const void* K, const void* V, const int32_t* frame_t, const int32_t* frozen, void* K_cache, void* Vt_cache,
                              int32_t* segments, int32_t* n_segments, const float* rope_xy, const qb_kv_params* p, void* stream);

/* head_rmsnorm + value_residual_packed + kv_cache_update in one pass over the packed QKV projection
 * (ref: the three calls of TransformerBlock.forward, src/quark/models/waypoint_15.py:398-407).
 * qkv_out receives the normalised Q and K heads and the mixed V (what owl_attn reads, and what the
 * first block hands to later blocks as qkv_first); the caches and the segment table are updated as by
 * qb_kv_cache_update.  qkv_first / lamb may both be NULL (first block: no value residual).  Results
 * are bit-identical to the three separate entry points.  n_q_heads must be a multiple of n_kv_heads. */
int32_t qb_qkv_post(const void* qkv_in, const void* qkv_first, const float* lamb, void* qkv_out, const int32_t* frame_t,
                    const int32_t* frozen, void* K_cache, void* Vt_cache, int32_t* segments, int32_t* n_segments,
                    const float* rope_xy, const qb_kv_params* p, float eps, void* stream);

/* The QKV projection with qb_qkv_post as its epilogue: qkv_out = post(A @ B^T), caches and segment table
 * updated, in one launch; the projection's raw output never goes to memory.  Same bytes as qb_gemm
 * followed by qb_qkv_post (ref: qkv_proj then the three calls of TransformerBlock.forward,
 * src/quark/models/waypoint_15.py:396-407).  gp describes the GEMM (M = H*W tokens, N = (n_q_heads +
 * 2 n_kv_heads) * 64, bf16 output, no activation; a_scale / w_scale as in qb_gemm; tile_n and split_k are
 * overridden: 128-column tiles hold two whole heads, one K slice).  qkv_out and K_cache must be 32-byte aligned.  Workspace as
 * for qb_gemm with tile_n = 128, split_k = 1. */
int32_t qb_gemm_qkv_post(const void* A, const void* B, void* qkv_out, const void* qkv_first, const float* lamb,
                         const int32_t* frame_t, const int32_t* frozen, void* K_cache, void* Vt_cache, int32_t* segments,
                         int32_t* n_segments, const float* rope_xy, const qb_gemm_params* gp, const qb_kv_params* kp, float eps,
                         void* workspace, size_t workspace_bytes, void* stream);

/* Fills rope_xy [H*W, 16] on the device: token t -> (h, w) = (t / W, t % W).  The angles follow
 * ref: src/quark/kernels/kv_cache_update/reference.py:61-106 (f64 position x frequency, narrowed
 * to f32); cos/sin are the CUDA single-precision functions. */
int32_t qb_rope_table_build(float* rope_xy, int32_t H_spatial, int32_t W_spatial, void* stream);

/* Keeps a second pair of caches (K_shadow, Vt_shadow: the shapes of K_cache, Vt_cache, in the OTHER of the two dtypes)
 * equal to cast(cache) by converting the rows the append just before wrote: the tail slot always, the ring slot when
 * frame_t is a write frame and *frozen == 0 (the same arithmetic as the append).  p describes the cache as for the
 * append (p->kv_dtype = the dtype of K_cache / Vt_cache).  e4m3 -> bf16 is exact, bf16 -> e4m3 rounds to nearest even
 * and saturates (qb_quantize_e4m3).  This is the reference's cast on load for a cache dtype that differs from the
 * attention's compute dtype (ref: src/quark/kernels/owl_attn/kernel.py:342-348), done once per appended row instead of
 * once per attended row per call; qb_owl_attn then runs on the shadow pair with kv_dtype = compute_dtype.  Call it after
 * every append; a cache written by other means (restored, reset) is brought over whole with qb_quantize_e4m3 /
 * qb_dequantize_e4m3. */
int32_t qb_kv_cast_appended(const void* K_cache, const void* Vt_cache, void* K_shadow, void* Vt_shadow, const int32_t* frame_t,
                            const int32_t* frozen, const qb_kv_params* p, void* stream);

/* ------------------------------------------------------------------ owl_attn
 * Segment-sparse GQA flash attention with inline ortho-RoPE on Q, head_dim 64.
 * Replaces qf.owl_attn (ref: src/quark/functional/owl_attn.py:322-394,
 * src/quark/kernels/owl_attn/kernel.py:324-790).  qkv packed [tpf, (Hq + 2 Hk) * 64] bf16 (only
 * the Q columns are read), caches as above, out [tpf, Hq * 64] bf16.  Attends to the union of
 * the first n_segments (start, length) entries; starts must be multiples of 16.  out_q (optional,
 * may be NULL) receives the same result narrowed to e4m3 for a following fp8 GEMM.
 * compute_dtype QB_BF16 (bf16 caches) or QB_E4M3 (e4m3 caches; Q after RoPE and P are narrowed
 * to e4m3).  k_scale / v_scale: optional f32 [Hk] per-head dequantisation scales (NULL = 1). */
typedef struct {
  int32_t n_kv_heads, gqa_ratio;
  int32_t H_spatial, W_spatial;
  int32_t num_buckets, pinned_dilation;
  int32_t kv_dtype;      /* QB_BF16 or QB_E4M3 */
  int32_t compute_dtype; /* QB_BF16 or QB_E4M3 */
  int32_t max_segments;  /* 3 */
  int32_t packed_qkv;    /* 1: qkv is the packed projection, out is [tpf, Hq * 64]; 0: qkv is Q alone, head-major
                          * [Hq * tpf, 64], and so is out (src/quark/kernels/owl_attn/reference.py:62-69, :106-110) */
  int32_t quilt_factor;  /* the caches keep H*W / quilt_factor tokens per frame (1: all): capacity = (nb + 1) * that */
  int32_t kv_splits;     /* 0 = choose; > 1 splits the keys over CTAs (needs workspace) */
  const float* k_scale;
  const float* v_scale;
} qb_attn_params;

/* e4m3 probabilities: by default every second exponential of a score row is built on the FMA pipe as
 * 2^floor(x) * (1 + frac(x) - 0.052) (relative error -5.2 % .. +2.3 %, below the 6.25 % an e4m3 code spans) so that
 * the special-function unit is not the kernel's bottleneck; on = 1 computes all of them with ex2.approx, as the
 * reference kernel does (ref: src/quark/kernels/owl_attn/kernel.py:587-614), at about 12 % more time per call.
 * Process-wide; returns the previous setting.  QB_ATTN_EXACT_EXP=1 in the environment sets it at load time.
 * bf16 attention always uses ex2.approx. */
int32_t qb_set_attn_exact_exp(int32_t on);

/* Bytes of workspace qb_owl_attn needs for `p`: 0 unless the keys of one (query tile, head) are shared by
 * several CTAs, which is chosen when query tiles x heads would leave most SMs idle (360p; a tensor-parallel
 * rank with few heads) or forced with kv_splits.  The workspace starts with one ticket per (query tile,
 * head) in a fixed 16 KiB area (so calls of different geometries may share a workspace), which must be zero
 * before the first use (the kernel leaves it zero), followed by the CTAs' partial results; it must not be the workspace of qb_gemm.  Shares are summed in a fixed order. */
size_t qb_owl_attn_workspace_bytes(const qb_attn_params* p);
int32_t qb_owl_attn(const void* qkv, const void* K_cache, const void* Vt_cache, const int32_t* segments,
                    const int32_t* n_segments, const int32_t* frame_t, void* out, void* out_q, const float* rope_xy,
                    const qb_attn_params* p, void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------ norm / elementwise ops
 * bf16 in, f32 math, bf16 out unless noted.  `out_q` (optional) receives the same result
 * narrowed to e4m3 so the next fp8 GEMM needs no separate cast. */

/* y = x * rsqrt(mean(x^2) + eps) * (1 + scale[g]) + bias[g], then SiLU if activation == 1.
 * X [rows, D], scale / bias [G, D]; out may be NULL when out_q is given (only the e4m3 result is wanted).
 * ref: src/quark/functional/ada_rmsnorm.py:61,
 * src/quark/kernels/ada_rmsnorm/reference.py:10-29. */
int32_t qb_ada_rmsnorm(const void* X, const void* scale, const void* bias, void* out, void* out_q, int32_t rows, int32_t D,
                       int32_t groups, float eps, int32_t activation, void* stream);
/* RMS norm of each 64-wide Q and K head of packed qkv [rows, (Hq + 2 Hk) * Dh]; V copied.
 * ref: src/quark/kernels/head_rmsnorm/reference.py:10-26. */
int32_t qb_head_rmsnorm(const void* X, void* out, int32_t rows, int32_t n_q_heads, int32_t n_kv_heads, int32_t Dh, float eps,
                        void* stream);
/* out = cur with V columns v + lamb * (v_first - v); lamb f32[1] on the device.
 * ref: src/quark/kernels/value_residual_packed/reference.py:8-20. */
int32_t qb_value_residual_packed(const void* cur, const void* first, const float* lamb, void* out, int32_t rows, int32_t D_full,
                                 int32_t v_col_offset, int32_t v_width, void* stream);
/* out = x + gate[g] * y.  ref: src/quark/kernels/ada_gate_residual/reference.py:10-22. */
int32_t qb_ada_gate_residual(const void* X, const void* Y, const void* gate, void* out, int32_t rows, int32_t D, int32_t groups,
                             void* stream);
/* out = x * sigmoid(x).  ref: src/quark/kernels/silu/reference.py:10-18. */
int32_t qb_silu(const void* X, void* out, void* out_q, size_t n, void* stream);
/* out = x * rsqrt(mean(x^2 over the last dimension) + eps), bf16 [rows, D], no gain.
 * ref: src/quark/kernels/rmsnorm/reference.py:10-22 (qf.rmsnorm, src/quark/functional/rmsnorm.py:29-45). */
int32_t qb_rmsnorm(const void* X, void* out, int32_t rows, int32_t D, float eps, void* stream);
/* out = x + y, bf16, n elements.  ref: src/quark/kernels/elementwise/reference.py:10-19 (op "add"; nn.Add). */
int32_t qb_add(const void* X, const void* Y, void* out, size_t n, void* stream);
/* out = x + dsig[0] * v; dsig f32[1] on the device.  ref: src/quark/functional/euler_step.py:36-41. */
int32_t qb_euler_step(const void* X, const void* V, const float* dsig, void* out, size_t n, void* stream);
/* out[0..n) = standard normals (bf16 or f32) from Philox4x32-10 + Box-Muller; stateless: the draw is a function
 * of (counter[0] * counter_stride, seed0, seed1) alone, so the call can sit in a captured graph and a caller that
 * advances counter[0] by one per draw with counter_stride >= ceil(n / 4) never reuses a Philox counter.
 * counter is a u32 on the device.  ref: src/quark/functional/randn.py:33-82, src/quark/kernels/randn/kernel.py:200-254
 * (same counters, key, uniform mapping and output layout as its default tile; counter_stride = 1 is its meaning of
 * counter_offset). */
int32_t qb_randn(const uint32_t* counter, void* out, size_t n, int32_t out_dtype, uint32_t counter_stride, uint32_t seed0, uint32_t seed1,
                 void* stream);
/* Mixture-of-experts routing ("correct" mode: every token goes to its own top_k experts, no capacity bound):
 * weights[e][m] (f32, [E, M]) = softmax over token m's top_k logits at its top_k experts, 0 elsewhere; ties go to
 * the lower expert index.  logits bf16 [M, E], E <= 32.  ref: src/quark/kernels/moe_router_correct/reference.py:38-49.
 * For the dense schedule (every expert over every token); the slot-sorted schedule below is the default. */
int32_t qb_moe_route(const void* logits, float* weights, int32_t M, int32_t E, int32_t top_k, void* stream);
/* The same routing as slot tables for the slot-sorted schedule (ref: the tables of
 * src/quark/kernels/moe_router_correct/reference.py:51-120, src/quark/nn/moe.py:252-363, whose row tile is 32; here
 * 128, the GEMM kernel's).  n = qb_moe_slots(M, E, top_k) rows, a multiple of 128 that holds every expert's run padded
 * to whole tiles.  slot_token [n]: the token in each slot, -1 for padding; slot_weight [n]: its routing weight;
 * tile_expert [n / 128]: the expert of each 128-row tile, -1 past the last used tile; token_slot [M, top_k]: the slot of
 * token m's k-th choice, k in order of decreasing logit; counts [E] (may be NULL): tokens per expert.  Within an expert
 * the slots follow (token, k) order: the tables are a function of the logits alone. */
size_t qb_moe_slots(int32_t M, int32_t E, int32_t top_k);
int32_t qb_moe_route_slots(const void* logits, int32_t* slot_token, float* slot_weight, int32_t* tile_expert, int32_t* token_slot,
                           int32_t* counts, int32_t M, int32_t E, int32_t top_k, void* stream);
/* out[s, :] = X[slot_token[s], :] for rows of row_bytes bytes (a multiple of 16), zeros where slot_token[s] < 0: the
 * activations in slot order, the A operand of the grouped in-projection (the reference's moe_inproj gathers while it
 * loads, src/quark/functional/moe_inproj.py). */
int32_t qb_moe_gather(const void* X, const int32_t* slot_token, void* out, int32_t n_slots, int32_t row_bytes, void* stream);
/* Grouped GEMM: C[128 i .. 128 i + 127, :] = epilogue(A[same rows] . B[e N .. e N + N - 1, :]^T) with e = tile_expert[i];
 * tiles with e < 0 are skipped (their rows of C are left as they are).  A [p->M, K] with p->M a multiple of 128,
 * B [n_experts * p->N, K], C [p->M, p->N]; plain or SiLU epilogue, no bias / gate / scales.  Replaces qf.moe_inproj and
 * qf.moe_outproj (ref: src/quark/nn/moe.py:307-338). */
size_t qb_gemm_grouped_workspace_bytes(const qb_gemm_params* p);
int32_t qb_gemm_grouped(const void* A, const void* B, void* C, const int32_t* tile_expert, int32_t n_experts, const qb_gemm_params* p,
                        void* workspace, size_t workspace_bytes, void* stream);
/* out[m, :] = bf16(sum over k of slot_weight[s] * partials[s, :], s = token_slot[m, k]), the sum in f32 in order of
 * increasing slot (= expert index; the order of qb_moe_combine, so both schedules give the same bits), one narrowing.  Replaces qf.moe_reduce (ref: src/quark/kernels/moe_reduce/reference.py:16-33). */
int32_t qb_moe_reduce(const float* partials, const float* slot_weight, const int32_t* token_slot, void* out, int32_t M, int32_t D, int32_t top_k,
                      void* stream);
/* out[m, :] (bf16 [M, D]) = sum over experts with weights[e][m] != 0 of weights[e][m] * partials[e][m][:] (f32
 * [E, M, D]), summed in f32, narrowed once.  ref: src/quark/kernels/moe_reduce/reference.py:16-33. */
int32_t qb_moe_combine(const float* partials, const float* weights, void* out, int32_t M, int32_t D, int32_t E, void* stream);
/* counter[0] += 1.  ref: src/quark/kernels/increment/kernel.py:1-7. */
int32_t qb_increment(int32_t* counter, void* stream);
/* latent [1, C*H*W] -> tokens [(H/ph)*(W/pw), d_model] = patches . W[d_model, C*ph*pw]^T.
 * ref: src/quark/kernels/patchify/reference.py:8-23. */
int32_t qb_patchify(const void* X, const void* W, void* out, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw,
                    int32_t d_model, void* stream);
/* tokens [(H/ph)*(W/pw), d_model] -> latent [1, C*H*W] = scatter(tokens . W[C*ph*pw, d_model]^T + bias).
 * ref: src/quark/kernels/unpatchify/reference.py:8-24. */
int32_t qb_unpatchify(const void* X, const void* W, const void* bias, void* out, int32_t C, int32_t H, int32_t Wd, int32_t ph,
                      int32_t pw, int32_t d_model, void* stream);

/* The data movement of patchify / unpatchify alone (bf16): latent [C, H, W] <-> tokens
 * [(H/ph)*(W/pw), C*ph*pw] with feature index c*ph*pw + r*pw + q, so that the contraction can run on
 * qb_gemm: patchify = qb_patch_gather + qb_gemm, unpatchify = qb_gemm (with bias) + qb_patch_scatter.
 * Same results as qb_patchify / qb_unpatchify up to the f32 summation order
 * (ref: src/quark/kernels/patchify/reference.py:8-23, src/quark/kernels/unpatchify/reference.py:8-24). */
int32_t qb_patch_gather(const void* latent, void* tokens_out, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw, void* stream);
int32_t qb_patch_scatter(const void* tokens_in, void* latent_out, int32_t C, int32_t H, int32_t Wd, int32_t ph, int32_t pw, void* stream);

/* ------------------------------------------------------------------ one session over several GPUs
 * The reference is single-GPU (ref: src/quark/models/waypoint_15.py:318, :333: B = 1, one device); nothing below has a
 * counterpart there.  When a block is sharded by KV-head group, out-proj and fc2 are row-parallel and their partial
 * outputs [rows, D] bf16 must be summed over the ranks before gate and residual are applied.  qb_tp_reduce does that
 * sum, `x + gate * sum`, and optionally the AdaRMSNorm that follows, as one kernel per rank over peer-mapped memory
 * (plain loads and stores over NVLink; no TMA, no multicast), in place of an NCCL all-reduce and two more launches:
 *   x_new[m, :] = residual[m, :] + gate[m / (rows / G), :] * bf16(sum over ranks r, in rank order, of y_r[m, :])
 *   h[m, :]     = ada_rmsnorm(x_new[m, :]; norm_scale, norm_bias, eps, norm_activation)        (when norm_scale != NULL)
 * with the rounding points of qb_ada_gate_residual and qb_ada_rmsnorm, so every rank ends up with the same bytes.
 *
 * Each rank owns an arena of qb_tp_arena_bytes(rows, D) bytes from qb_malloc, zeroed once, laid out as
 * [4 KiB of flags | y slot 0 | y slot 1 | x slot 0 | x slot 1 | h (bf16) | hq (e4m3)] (byte offsets of the six buffers from
 * qb_tp_arena_offsets).  The rank's row-parallel GEMM writes its partial into its own y slot p->x_slot; the kernel reads
 * every rank's y and leaves x_new (x slot p->x_slot), h and hq (if emit_h / emit_hq) complete in every rank's arena.
 * Schedules (p->schedule: 0 = the library's choice, which is one-shot; 1 = one-shot, 2 = two-shot, 3 = pushed, see
 * qb_gemm_tp; all ranks must agree): one-shot, the fastest measured at 2, 4 and 8 ranks,
 * has every rank read all rows of every peer's y and compute the whole result for itself (one exchange of
 * flags, nothing written to a peer); two-shot has rank r reduce rows [r * rows / world, (r + 1) * rows / world) only and
 * store them into EVERY rank's arena (traffic stays near twice the partial, a second exchange of flags).
 * arena[r] is rank r's arena as mapped in the calling process: arena[rank] the rank's own pointer, the others from
 * qb_ipc_open of a handle that rank r made with qb_ipc_export.  Consecutive calls must alternate x_slot (the block does:
 * 0 after attention, 1 after the MLP): the residual of one call is the x_new of the call before, and a y slot is
 * rewritten two calls later.  All ranks must make the same sequence of calls.  A rank waits (bounded: wait_limit_us,
 * 0 = about one second) for its peers' kernels of the same call to start and, two-shot, to deliver their rows; when
 * the limit runs out the kernel raises bit 3 of the device status word and returns with the outputs unspecified.
 * Stream-capturable. */
typedef struct {
  int32_t world, rank;
  int32_t rows, D;                   /* the partial is [rows, D] bf16; rows % world == 0, D % 8 == 0, D <= 8192 */
  int32_t gate_groups, norm_groups;  /* gate [gate_groups, D], norm_scale / norm_bias [norm_groups, D] */
  int32_t norm_activation;           /* 0 none, 1 SiLU (the output norm) */
  int32_t x_slot;                    /* 0 or 1: which y buffer holds the partials and which x buffer receives x_new */
  int32_t emit_h, emit_hq;           /* write the norm's result as bf16 / as e4m3 */
  int32_t wait_limit_us;             /* 0 = default */
  float eps;
  int32_t schedule;                  /* 0 = choose (one-shot), 1 = one-shot, 2 = two-shot, 3 = two-shot over partials that qb_gemm_tp
                                        has already stored into the owners' staging areas */
  int32_t reserved;
  void* arena[8];
} qb_tp_params;

/* The row-parallel GEMM of a rank with its output sent straight to where it is summed: row m of the bf16 partial
 * [p->M, p->N] = A . B^T (no epilogue, one K slice) is stored into y slot 0 of the arena of rank m / (M / world), at
 * block tp->rank of that area ([source rank][M / world rows][N]), with plain stores over NVLink.  Follow it with
 * qb_tp_reduce with schedule = 3 on every rank, which sums the blocks of its own area.  tp: world, rank, rows = M,
 * D = N and the arenas are read; the other fields are ignored.  Workspace as for qb_gemm.  No counterpart in the
 * reference. */
int32_t qb_gemm_tp(const void* A, const void* B, const qb_gemm_params* p, const qb_tp_params* tp, void* workspace, size_t workspace_bytes,
                   void* stream);
size_t qb_tp_arena_bytes(int32_t rows, int32_t D);
/* offsets6_host[0..5] = byte offsets of y slot 0, y slot 1, x slot 0, x slot 1, h, hq inside an arena. */
int32_t qb_tp_arena_offsets(int32_t rows, int32_t D, size_t* offsets6_host);
int32_t qb_tp_reduce(const void* residual, const void* gate, const void* norm_scale, const void* norm_bias, const qb_tp_params* p,
                     void* stream);
/* The same protocol with all `world` ranks run as ONE cooperative launch on the calling GPU, over arenas that all live on
 * it (residuals[r] is rank r's residual): for tests on a single GPU, where kernels that wait on one another must not be
 * separate launches.  p->rank is ignored. */
int32_t qb_tp_reduce_emulated(const void* const* residuals, const void* gate, const void* norm_scale, const void* norm_bias,
                              const qb_tp_params* p, void* stream);
/* CUDA IPC for the arenas: a 64-byte handle of a qb_malloc allocation, and its mapping in another process of the same
 * node (the exporting GPU must be visible to the importing process and peer access possible). */
int32_t qb_ipc_export(void* device_ptr, void* handle64_host);
int32_t qb_ipc_open(const void* handle64_host, void** ptr_host);
int32_t qb_ipc_close(void* ptr);

#ifdef __cplusplus
}
#endif
#endif /* QUARK_B200_H */
