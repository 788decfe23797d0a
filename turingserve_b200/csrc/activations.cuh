// One-input activations of the feed-forwards, in 32-bit.
#pragma once

#include "common.cuh"

enum TsActivation : int { TS_ACT_NONE = 0, TS_ACT_GELU_TANH = 1, TS_ACT_RELU2 = 2, TS_ACT_SILU = 3, TS_ACT_GELU = 4 };
constexpr int TS_ACT_LAST = 4;

__device__ __forceinline__ float ts_activate(float z, int kind) {
  if (kind == TS_ACT_GELU_TANH) return 0.5f * z * (1.f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
  if (kind == TS_ACT_RELU2) {
    const float r = fmaxf(z, 0.f);
    return r * r;
  }
  if (kind == TS_ACT_SILU) return z / (1.f + expf(-z));
  if (kind == TS_ACT_GELU) return 0.5f * z * (1.f + erff(0.7071067811865476f * z));
  return z;
}

// The same on its way to a rounding to T: for bfloat16 the tanh form of GELU is z * sigmoid(2 u), u = 0.79788456 (z +
// 0.044715 z^3), with the hardware's approximate exponential and reciprocal (about 2^-21 relative, against a bfloat16 step of
// 2^-9), and SiLU likewise; the 32-bit type keeps the exact functions.
template <typename T> __device__ __forceinline__ float ts_activate_for(float z, int kind) { return ts_activate(z, kind); }
template <> __device__ __forceinline__ float ts_activate_for<bf16>(float z, int kind) {
  if (kind == TS_ACT_GELU_TANH) return __fdividef(z, 1.f + __expf(-1.5957691216057308f * (z + 0.044715f * z * z * z)));
  if (kind == TS_ACT_SILU) return __fdividef(z, 1.f + __expf(-z));
  return ts_activate(z, kind);
}
