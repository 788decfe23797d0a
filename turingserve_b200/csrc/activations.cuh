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
