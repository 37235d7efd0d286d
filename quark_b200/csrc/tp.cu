// Sum of the row-parallel partial outputs over the GPUs of one node, fused with what follows it in the block:
//   x_new = residual + gate * bf16(sum_r y_r)          (the all-reduce + ada_gate_residual of the unfused wiring)
//   h     = ada_rmsnorm(x_new) (bf16 and / or e4m3)    (the next AdaRMSNorm, optional)
// as ONE kernel per rank over peer-mapped buffers, in place of ncclAllReduce + two more launches.
//
// Every rank owns an "arena" of the same layout in its own device memory, mapped into every peer (CUDA IPC):
//   flags | y slot 0 | y slot 1 (this rank's partial, written by its GEMM) | x slot 0 | x slot 1 | h (bf16) | hq (e4m3)
// Partials are summed in rank order with plain peer loads, so every rank computes the same bits.  No TMA, no multicast,
// no multimem: ordinary ld / st over NVLink, so the kernel runs unchanged on any number of GPUs.  Two schedules:
//   one-shot (few ranks)  every rank reads ALL rows of every peer's y and computes the whole result for itself; one
//                         exchange of flags, (world - 1) x the partial read over NVLink, nothing written to a peer;
//   two-shot (many ranks) rank r sums rows [r * rows / world, (r + 1) * rows / world) only and stores them into EVERY
//                         rank's arena; the traffic per rank stays near 2 x the partial, at the price of a second
//                         exchange of flags (a rank's kernel ends only when every peer's rows have arrived).
//   pushed                two-shot, but the partials are already where they are summed: the row-parallel GEMM (qb_gemm_tp)
//                         stored each row of its partial into the staging area of the rank that owns the row (y slot 0 of
//                         that rank's arena, one block of rows per source rank), so the kernel reads local memory only and
//                         no load crosses NVLink; the flag exchange at its start tells it that the peers' GEMMs have ended.
//
// Synchronisation is by epoch counters in the arenas, pushed into the memory of the rank that polls them:
//   y_ready[r]   = e   written into every peer by rank r when its kernel e starts (its GEMM before it has finished)
//   x_arrived[r] = e   (two-shot) written into every peer by rank r's last CTA after all of its stores
// Every wait is bounded: when it runs out the kernel raises QB_DEV_WAIT_TIMEOUT_TP in the device status word, skips
// the data phase and returns; nothing spins for ever.
// Buffer reuse: consecutive calls alternate between the two y slots and the two x slots.  A rank rewrites a y slot two
// calls later, after its own kernel of the call in between has ended; that kernel waited for every peer's y_ready of
// that call, which a peer sends only after its kernel of the call before (the reader of the slot) has ended.  In the
// two-shot schedule a peer writes x slot (e + 1) only after this rank announced epoch e + 1, i.e. after its own
// kernel e, the last reader of the other slot as a residual, has ended.
//
// Kernels that wait on one another must not be separate launches on one GPU, so the single-GPU test entry
// (qb_tp_reduce_emulated) runs all ranks as the y-dimension of ONE cooperative launch over arenas that all live on
// that GPU.
#include <cstring>

#include "common.cuh"
#include "sm100.cuh"

namespace qb {

constexpr unsigned QB_DEV_WAIT_TIMEOUT_TP = 1u << 3;
constexpr int kTpMaxWorld = 8;
constexpr int kTpThreads = 256;
constexpr size_t kTpFlagBytes = 4096;
// flag words (u32 index into the flag area); every flag has a 128-byte line of its own
constexpr int kFlagYReady = 0;       // + 32 * rank
constexpr int kFlagXArrived = 256;   // + 32 * rank
constexpr int kFlagDone = 512;
constexpr int kFlagEpoch = 544;

struct TpArgs {
  uint8_t* arena[kTpMaxWorld];
  const uint16_t* residual[kTpMaxWorld];  // the emulated launch has one per rank; a real launch uses [rank]
  const uint16_t* gate;                   // [gate groups, D]
  const uint16_t* nscale;                 // [norm groups, D] or null: no norm
  const uint16_t* nbias;
  int world, rank, emulate, one_shot, pushed;
  int rows, D, gate_rows_per_group, norm_rows_per_group;
  int xslot, activation, emit_h, emit_hq;
  float eps;
  long long wait_cycles;
  unsigned int* status;
};

__device__ __forceinline__ void st_release_sys(unsigned int* p, unsigned int v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned int ld_acquire_sys(const unsigned int* p) {
  unsigned int v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_volatile_v4(const void* p) {
  uint4 v;
  asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}

// Waits until flags[first + 32 * p] has reached epoch e for every rank p; false when the limit ran out.
// (Polling with relaxed loads and one system-scope fence after the last flag was measured: the fence, which every CTA
// then executes, costs far more than acquire loads do - 13.7 against 8.7 us for a launch without peers.)
__device__ __forceinline__ bool tp_wait_all(const unsigned int* flags, int first, int world, unsigned int e, long long limit) {
  const long long t0 = clock64();
  for (int p = 0; p < world; ++p) {
    while (static_cast<int>(ld_acquire_sys(flags + first + 32 * p) - e) < 0) {
      if (clock64() - t0 > limit) return false;
      __nanosleep(40);
    }
  }
  return true;
}

__device__ __forceinline__ void tp_unpack8(const uint4& u, float (&f)[8]) {
  f[0] = bf16lo(u.x); f[1] = bf16hi(u.x); f[2] = bf16lo(u.y); f[3] = bf16hi(u.y);
  f[4] = bf16lo(u.z); f[5] = bf16hi(u.z); f[6] = bf16lo(u.w); f[7] = bf16hi(u.w);
}
__device__ __forceinline__ uint4 tp_pack8(const float (&f)[8]) {
  return make_uint4(pack_bf16x2(f[0], f[1]), pack_bf16x2(f[2], f[3]), pack_bf16x2(f[4], f[5]), pack_bf16x2(f[6], f[7]));
}

// kMaxVec: 16-byte vectors of a row per thread (D <= 8 * kTpThreads * kMaxVec); an instantiation per width keeps the
// registers of the common D = 2048 low enough for every row's CTA to be resident at once.
// kW: the most ranks the instantiation sums (2, 4 or 8): the partials of a vector are all requested before the first is
// used, one register quadruple each.
template <int kMaxVec, int kW>
__global__ void __launch_bounds__(kTpThreads, (kMaxVec == 1 && kW <= 4) ? 4 : 2) tp_reduce_kernel(const TpArgs a) {
  grid_dep_wait();    // this rank's partial comes from the GEMM before this kernel
  grid_dep_launch();
  __shared__ float red[kTpThreads / 32];
  __shared__ unsigned int s_epoch;
  __shared__ int s_ok;

  const int rank = a.emulate ? static_cast<int>(blockIdx.y) : a.rank;
  uint8_t* mine = a.arena[rank];
  unsigned int* flags = reinterpret_cast<unsigned int*>(mine);
  const size_t plane = static_cast<size_t>(a.rows) * a.D * 2;  // one bf16 [rows, D] buffer
  const size_t off_y = kTpFlagBytes + plane * a.xslot, off_x = kTpFlagBytes + plane * (2 + a.xslot), off_h = kTpFlagBytes + plane * 4,
               off_hq = kTpFlagBytes + plane * 5;

  // What does not depend on the peers is requested before the flags are looked at, so that it arrives while thread 0
  // exchanges them: this rank's own partial (its GEMM has finished: the grid dependency above), the residual and the
  // gate of the CTA's first row.
  const int rpr_ = a.one_shot ? a.rows : a.rows / a.world;
  const int row0 = a.one_shot ? static_cast<int>(blockIdx.x) : rank * rpr_ + static_cast<int>(blockIdx.x);
  uint4 pre_y[kMaxVec], pre_r[kMaxVec], pre_g[kMaxVec];
#pragma unroll
  for (int i = 0; i < kMaxVec; ++i) {
    const int c = (i * kTpThreads + threadIdx.x) * 8;
    pre_y[i] = pre_r[i] = pre_g[i] = make_uint4(0u, 0u, 0u, 0u);
    if (c < a.D && static_cast<int>(blockIdx.x) < rpr_) {
      const size_t roff = static_cast<size_t>(row0) * a.D;
      if (!a.pushed) pre_y[i] = ld_volatile_v4(mine + off_y + (roff + c) * 2);
      pre_r[i] = *reinterpret_cast<const uint4*>(a.residual[rank] + roff + c);
      pre_g[i] = *reinterpret_cast<const uint4*>(a.gate + static_cast<size_t>(row0 / a.gate_rows_per_group) * a.D + c);
    }
  }

  if (threadIdx.x == 0) {
    const unsigned int e = flags[kFlagEpoch] + 1u;  // written by this rank's previous launch, which has ended
    s_epoch = e;
    if (blockIdx.x == 0) {
      for (int p = 0; p < a.world; ++p) st_release_sys(reinterpret_cast<unsigned int*>(a.arena[p]) + kFlagYReady + 32 * rank, e);
    }
    // Once a wait has run out on this GPU (the bit stays up until the host reads the status word) the session is
    // broken: later calls do not wait their full limit again, they pass straight through.
    const bool broken = (*reinterpret_cast<volatile unsigned int*>(a.status) & QB_DEV_WAIT_TIMEOUT_TP) != 0;
    const bool ok = !broken && tp_wait_all(flags, kFlagYReady, a.world, e, a.wait_cycles);
    if (!ok) atomicOr(a.status, QB_DEV_WAIT_TIMEOUT_TP);
    s_ok = ok ? 1 : 0;
  }
  __syncthreads();
  const unsigned int e = s_epoch;

  if (s_ok) {
    // one-shot: every row, results kept on this rank; two-shot: this rank's share of the rows, results sent to every rank
    const int rpr = a.one_shot ? a.rows : a.rows / a.world;
    const int first_dst = a.one_shot ? rank : 0, end_dst = a.one_shot ? rank + 1 : a.world;
    for (int lr = blockIdx.x; lr < rpr; lr += gridDim.x) {
      const int row = a.one_shot ? lr : rank * rpr + lr;
      const size_t roff = static_cast<size_t>(row) * a.D;
      const size_t goff = static_cast<size_t>(row / a.gate_rows_per_group) * a.D;
      uint4 xv[kMaxVec];
      float ss = 0.f;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int c = (i * kTpThreads + threadIdx.x) * 8;
        if (c < a.D) {
          // every peer's vector is requested before the first is used: one NVLink round trip, not `world` of them
          const bool first = lr == static_cast<int>(blockIdx.x);  // this row's own inputs are in registers already
          uint4 yv[kW];
#pragma unroll
          for (int p = 0; p < kW; ++p)
            if (p < a.world) {
              if (a.pushed) yv[p] = ld_volatile_v4(mine + kTpFlagBytes + ((static_cast<size_t>(p) * rpr + lr) * a.D + c) * 2);  // local staging
              else if (first && p == rank) yv[p] = pre_y[i];
              else yv[p] = ld_volatile_v4(a.arena[p] + off_y + (roff + c) * 2);
            }
          float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
          for (int p = 0; p < kW; ++p) {  // rank order: every rank that summed these rows would get the same bits
            if (p < a.world) {
              float y[8];
              tp_unpack8(yv[p], y);
#pragma unroll
              for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(acc[j], y[j]);
            }
          }
          float r[8], g[8];
          tp_unpack8(first ? pre_r[i] : *reinterpret_cast<const uint4*>(a.residual[rank] + roff + c), r);
          tp_unpack8(first ? pre_g[i] : *reinterpret_cast<const uint4*>(a.gate + goff + c), g);
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const float s = __bfloat162float(__float2bfloat16_rn(acc[j]));  // the summed partial as a bf16 tensor
            r[j] = __fadd_rn(r[j], __fmul_rn(g[j], s));                     // x + gate * y, as ada_gate_residual
          }
          xv[i] = tp_pack8(r);
          float f[8];
          tp_unpack8(xv[i], f);  // the norm reads the bf16-rounded x_new, as a kernel of its own would
#pragma unroll
          for (int j = 0; j < 8; ++j) ss += f[j] * f[j];
        }
      }
      float inv = 0.f;
      if (a.nscale != nullptr) {  // block-wide sum of squares, in the order of ada_rmsnorm_kernel
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        __syncthreads();  // red[] of the previous row has been read by everybody
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kTpThreads / 32; ++w) tot += red[w];
        inv = 1.0f / sqrtf(tot / static_cast<float>(a.D) + a.eps);
      }
      const size_t noff = a.nscale != nullptr ? static_cast<size_t>(row / a.norm_rows_per_group) * a.D : 0;
#pragma unroll
      for (int i = 0; i < kMaxVec; ++i) {
        const int c = (i * kTpThreads + threadIdx.x) * 8;
        if (c < a.D) {
          uint4 hv = make_uint4(0u, 0u, 0u, 0u);
          uint2 hq = make_uint2(0u, 0u);
          if (a.nscale != nullptr) {
            float f[8], s[8], b[8];
            tp_unpack8(xv[i], f);
            tp_unpack8(*reinterpret_cast<const uint4*>(a.nscale + noff + c), s);
            tp_unpack8(*reinterpret_cast<const uint4*>(a.nbias + noff + c), b);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
              float y = __fmul_rn(f[j], inv);
              y = __fadd_rn(__fmul_rn(y, __fadd_rn(1.0f, s[j])), b[j]);
              f[j] = a.activation == 1 ? silu_f(y) : y;
            }
            hv = tp_pack8(f);
            float q[8];
            tp_unpack8(hv, q);  // the e4m3 copy is narrowed from the bf16-rounded value
            hq = make_uint2(pack_e4m3x4(q[0], q[1], q[2], q[3]), pack_e4m3x4(q[4], q[5], q[6], q[7]));
          }
          for (int p = first_dst; p < end_dst; ++p) {
            uint8_t* dst = a.arena[p];
            *reinterpret_cast<uint4*>(dst + off_x + (roff + c) * 2) = xv[i];
            if (a.nscale != nullptr && a.emit_h) *reinterpret_cast<uint4*>(dst + off_h + (roff + c) * 2) = hv;
            if (a.nscale != nullptr && a.emit_hq) *reinterpret_cast<uint2*>(dst + off_hq + (roff + c)) = hq;
          }
        }
      }
    }
  }

  // The CTA that draws the last ticket closes the epoch.  Two-shot: its stores to the peers must be visible system-wide
  // before the peers are told, so one thread per CTA fences after the CTA's barrier (the barrier orders the other
  // threads' stores before that thread, and its fence is cumulative), draws the ticket, and the last one signals and
  // then waits for every peer's rows.
  __syncthreads();
  if (threadIdx.x == 0) {
    if (!a.one_shot) __threadfence_system();
    const unsigned int ticket = atomicAdd(flags + kFlagDone, 1u);
    if (ticket == gridDim.x - 1) {
      flags[kFlagDone] = 0;  // ready for the next launch
      if (!a.one_shot) {
        __threadfence_system();
        for (int p = 0; p < a.world; ++p) st_release_sys(reinterpret_cast<unsigned int*>(a.arena[p]) + kFlagXArrived + 32 * rank, e);
        const bool broken = (*reinterpret_cast<volatile unsigned int*>(a.status) & QB_DEV_WAIT_TIMEOUT_TP) != 0;
        if (!broken && !tp_wait_all(flags, kFlagXArrived, a.world, e, a.wait_cycles)) atomicOr(a.status, QB_DEV_WAIT_TIMEOUT_TP);
      }
      flags[kFlagEpoch] = e;
    }
  }
}

}  // namespace qb

using namespace qb;

typedef void (*TpKernel)(const TpArgs);
template <int kW>
static TpKernel tp_kernel_for_width(int D) {
  if (D <= 8 * kTpThreads) return tp_reduce_kernel<1, kW>;
  if (D <= 16 * kTpThreads) return tp_reduce_kernel<2, kW>;
  return tp_reduce_kernel<4, kW>;
}
static TpKernel tp_kernel_for(int world, int D) {
  if (world <= 2) return tp_kernel_for_width<2>(D);
  if (world <= 4) return tp_kernel_for_width<4>(D);
  return tp_kernel_for_width<8>(D);
}

extern "C" size_t qb_tp_arena_bytes(int32_t rows, int32_t D) {
  if (rows <= 0 || D <= 0) return 0;
  return kTpFlagBytes + static_cast<size_t>(rows) * D * 11;  // y0, y1, x0, x1, h in bf16, hq in e4m3
}

extern "C" int32_t qb_tp_arena_offsets(int32_t rows, int32_t D, size_t* offsets6_host) {
  QB_REQUIRE(rows > 0 && D > 0 && offsets6_host != nullptr, QB_ERR_INVALID_ARG, "tp_arena_offsets: bad arguments");
  const size_t plane = static_cast<size_t>(rows) * D * 2;
  for (int i = 0; i < 6; ++i) offsets6_host[i] = kTpFlagBytes + plane * i;
  return QB_OK;
}

extern "C" int32_t qb_ipc_export(void* device_ptr, void* handle64_host) {
  QB_REQUIRE(device_ptr != nullptr && handle64_host != nullptr, QB_ERR_INVALID_ARG, "ipc_export: NULL pointer");
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "a CUDA IPC memory handle is 64 bytes");
  cudaIpcMemHandle_t h;
  QB_CUDA_OK(cudaIpcGetMemHandle(&h, device_ptr));
  memcpy(handle64_host, &h, 64);
  return QB_OK;
}

extern "C" int32_t qb_ipc_open(const void* handle64_host, void** ptr_host) {
  QB_REQUIRE(handle64_host != nullptr && ptr_host != nullptr, QB_ERR_INVALID_ARG, "ipc_open: NULL pointer");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64_host, 64);
  QB_CUDA_OK(cudaIpcOpenMemHandle(ptr_host, h, cudaIpcMemLazyEnablePeerAccess));
  return QB_OK;
}

extern "C" int32_t qb_ipc_close(void* ptr) {
  QB_REQUIRE(ptr != nullptr, QB_ERR_INVALID_ARG, "ipc_close: NULL pointer");
  QB_CUDA_OK(cudaIpcCloseMemHandle(ptr));
  return QB_OK;
}

static int32_t tp_fill(TpArgs& a, const qb_tp_params* p, const void* gate, const void* norm_scale, const void* norm_bias) {
  QB_REQUIRE(p != nullptr && gate != nullptr, QB_ERR_INVALID_ARG, "tp_reduce: NULL pointer");
  QB_REQUIRE(p->world >= 1 && p->world <= kTpMaxWorld && p->rank >= 0 && p->rank < p->world, QB_ERR_INVALID_ARG, "tp_reduce: rank %d of %d",
             p->rank, p->world);
  QB_REQUIRE(p->rows > 0 && p->rows % p->world == 0, QB_ERR_INVALID_ARG, "tp_reduce: %d rows do not split over %d ranks", p->rows, p->world);
  QB_REQUIRE(p->D > 0 && p->D % 8 == 0 && p->D <= 8 * kTpThreads * 4, QB_ERR_UNSUPPORTED, "tp_reduce: D = %d must be a multiple of 8, at most %d",
             p->D, 8 * kTpThreads * 4);
  QB_REQUIRE(p->gate_groups >= 1 && p->rows % p->gate_groups == 0, QB_ERR_INVALID_ARG, "tp_reduce: gate_groups %d", p->gate_groups);
  QB_REQUIRE((norm_scale == nullptr) == (norm_bias == nullptr), QB_ERR_INVALID_ARG, "tp_reduce: norm scale and bias come together");
  QB_REQUIRE(norm_scale == nullptr || (p->norm_groups >= 1 && p->rows % p->norm_groups == 0), QB_ERR_INVALID_ARG, "tp_reduce: norm_groups %d",
             p->norm_groups);
  QB_REQUIRE(p->x_slot == 0 || p->x_slot == 1, QB_ERR_INVALID_ARG, "tp_reduce: x_slot %d", p->x_slot);
  QB_REQUIRE(p->norm_activation == 0 || p->norm_activation == 1, QB_ERR_INVALID_ARG, "tp_reduce: norm_activation %d", p->norm_activation);
  QB_REQUIRE(aligned16(gate) && aligned16(norm_scale) && aligned16(norm_bias), QB_ERR_ALIGN, "tp_reduce: pointers must be 16-byte aligned");
  for (int r = 0; r < p->world; ++r) {
    QB_REQUIRE(p->arena[r] != nullptr && aligned16(p->arena[r]), QB_ERR_INVALID_ARG, "tp_reduce: arena %d is NULL or misaligned", r);
    a.arena[r] = static_cast<uint8_t*>(p->arena[r]);
  }
  a.gate = static_cast<const uint16_t*>(gate);
  a.nscale = static_cast<const uint16_t*>(norm_scale);
  a.nbias = static_cast<const uint16_t*>(norm_bias);
  a.world = p->world; a.rank = p->rank;
  a.rows = p->rows; a.D = p->D;
  a.gate_rows_per_group = p->rows / p->gate_groups;
  a.norm_rows_per_group = norm_scale ? p->rows / p->norm_groups : p->rows;
  QB_REQUIRE(p->schedule >= 0 && p->schedule <= 3, QB_ERR_INVALID_ARG, "tp_reduce: schedule %d", p->schedule);
  a.one_shot = p->schedule <= 1;  // also the choice when none is made: measured ahead of the two-shot forms at 2, 4 and 8 ranks
  a.pushed = p->schedule == 3;
  a.xslot = p->x_slot; a.activation = p->norm_activation;
  a.emit_h = p->emit_h != 0; a.emit_hq = p->emit_hq != 0;
  a.eps = p->eps;
  // about 1 s at B200 clocks unless the caller asks for less (tests of the timeout path do)
  a.wait_cycles = p->wait_limit_us > 0 ? static_cast<long long>(p->wait_limit_us) * 2000ll : kWaitCycleLimit;
  a.status = status_word();
  QB_REQUIRE(a.status != nullptr, QB_ERR_CUDA, "tp_reduce: device status word unavailable");
  return QB_OK;
}

extern "C" int32_t qb_tp_reduce(const void* residual, const void* gate, const void* norm_scale, const void* norm_bias, const qb_tp_params* p,
                                void* stream) {
  TpArgs a{};
  int32_t rc = tp_fill(a, p, gate, norm_scale, norm_bias);
  if (rc != QB_OK) return rc;
  QB_REQUIRE(residual != nullptr && aligned16(residual), QB_ERR_INVALID_ARG, "tp_reduce: residual is NULL or misaligned");
  a.residual[a.rank] = static_cast<const uint16_t*>(residual);
  a.emulate = 0;
  int sms = 148, dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
  const int rpr = a.one_shot ? p->rows : p->rows / p->world;
  const int grid = rpr < 4 * sms ? rpr : 4 * sms;
  return launch_dep("tp_reduce", tp_kernel_for(p->world, p->D), dim3(grid), dim3(kTpThreads), 0, static_cast<cudaStream_t>(stream), a);
}

extern "C" int32_t qb_tp_reduce_emulated(const void* const* residuals, const void* gate, const void* norm_scale, const void* norm_bias,
                                         const qb_tp_params* p, void* stream) {
  TpArgs a{};
  int32_t rc = tp_fill(a, p, gate, norm_scale, norm_bias);
  if (rc != QB_OK) return rc;
  QB_REQUIRE(residuals != nullptr, QB_ERR_INVALID_ARG, "tp_reduce_emulated: NULL pointer");
  for (int r = 0; r < p->world; ++r) {
    QB_REQUIRE(residuals[r] != nullptr && aligned16(residuals[r]), QB_ERR_INVALID_ARG, "tp_reduce_emulated: residual %d is NULL or misaligned", r);
    a.residual[r] = static_cast<const uint16_t*>(residuals[r]);
  }
  a.emulate = 1;
  const int rpr = a.one_shot ? p->rows : p->rows / p->world;
  int dev = 0, sms = 0, per_sm = 0;
  QB_CUDA_OK(cudaGetDevice(&dev));
  QB_CUDA_OK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  TpKernel kernel = tp_kernel_for(p->world, p->D);
  QB_CUDA_OK(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kTpThreads, 0));
  int gx = rpr;
  while (gx > 1 && static_cast<long>(gx) * p->world > static_cast<long>(sms) * per_sm) gx = (gx + 1) / 2;  // all CTAs must be resident at once
  QB_REQUIRE(static_cast<long>(gx) * p->world <= static_cast<long>(sms) * per_sm, QB_ERR_UNSUPPORTED, "tp_reduce_emulated: %d ranks do not fit on the GPU at once",
             p->world);
  void* kargs[] = {&a};
  ++g_launch_count;
  cudaError_t e = cudaLaunchCooperativeKernel(reinterpret_cast<void*>(kernel), dim3(gx, p->world), dim3(kTpThreads), kargs, 0,
                                              static_cast<cudaStream_t>(stream));
  if (e != cudaSuccess) return fail(QB_ERR_LAUNCH, "tp_reduce_emulated: %s", cudaGetErrorString(e));
  return QB_OK;
}
