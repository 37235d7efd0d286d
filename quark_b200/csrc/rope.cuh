// Ortho-RoPE pieces shared by the KV-cache append and the attention kernel.
//
// head_dim 64 -> 32 rotation pairs per token.  Pair p rotates input elements (x[2p], x[2p+1]);
// the outputs are de-interleaved: y[p] = x[2p] cos - x[2p+1] sin, y[p + 32] = x[2p+1] cos + x[2p] sin.
//   p in [0, 8)   angle = x-position  * pixel frequency (p >> 1)          table columns 0..3
//   p in [8, 16)  angle = y-position  * pixel frequency ((p - 8) >> 1)    table columns 4..7
//   p in [16, 32) angle = frame index * temporal frequency ((p - 16) >> 1)
// The spatial cos / sin come from a per-geometry table rope_xy[token][16] (8 cosines, then 8
// sines); the 8 temporal angles depend on the frame counter, a device scalar, and are evaluated
// in the kernel.
#pragma once

#include <cstdint>

namespace qb {

// 1 / 10000^(i / 8), i = 0..7, evaluated in single precision the way numpy evaluates
// `1.0 / (theta ** (arange(0, 16, 2, dtype=float32) / 16))`; stored as bit patterns.
static __device__ __constant__ uint32_t kTemporalFreqBits[8] = {1065353216u, 1050798235u, 1036831949u, 1023510243u,
                                                               1008981770u, 995049016u,  981668463u,  967166816u};

// cos / sin of the 8 temporal angles of frame `ft` into out[0..7] (cos) and out[8..15] (sin).
__device__ __forceinline__ void temporal_cos_sin(int ft, int i, float* out) {
  const float ang = __fmul_rn(static_cast<float>(ft), __uint_as_float(kTemporalFreqBits[i]));
  float s, c;
  sincosf(ang, &s, &c);
  out[i] = c;
  out[8 + i] = s;
}

// (cos, sin) of rotation pair p for a token whose 16 spatial values are in `xy` and the frame's
// 16 temporal values in `tm`.
__device__ __forceinline__ void pair_cos_sin(int p, const float* xy, const float* tm, float& c, float& s) {
  if (p < 16) {
    const int i = p >> 1;
    c = xy[i];
    s = xy[8 + i];
  } else {
    const int i = (p - 16) >> 1;
    c = tm[i];
    s = tm[8 + i];
  }
}

}  // namespace qb
