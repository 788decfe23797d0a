// A residual stream kept as S parallel copies (hyper-connections), all in 32-bit whatever the engine's type.
// A sublayer reads ONE vector u = sum_s in[s] x_s, and its output y comes back into all copies at once:
//     x_t <- sum_s mix[s, t] x_s + out[t] y          (mix indexed [from, to]).
// As with the single-copy stream the write-back is put off into the kernel that prepares the NEXT sublayer's
// input, so one kernel per sublayer does
//     (1) the pending write-back of the previous sublayer's y (mix, out; or, first != 0, the start of all copies
//         from the embedding rows times a constant),
//     (2) u = sum_s in[s] x_s   (in == null: the plain sum, which is what the model's last norm reads),
//     (3) the RMS norm of u, T(u * rsqrt(mean(u^2) + eps) * w), w in 32-bit (a weight stored around zero has had
//         its 1 added when it was loaded).
// streams: [T, S, hidden] 32-bit, updated in place.  y: [T, hidden] in the engine's type, or a product left
// unreduced by its kernel (part [splits, T, hidden] 32-bit partial sums + bias, summed in split order and rounded
// as the product's own epilogue would have).  S == 1 with mix = out = in = 1 is the ordinary pre-norm residual.
// One block a token; a thread keeps its columns' S values in registers between (1) and (2), u goes through
// shared memory between (2) and (3).
#include "common.cuh"

namespace {

constexpr int HS_MAX = 8;                  // copies of the stream a model may have

struct HsWeights {
  float mix[HS_MAX * HS_MAX];              // [from][to]
  float out[HS_MAX];
  float in[HS_MAX];
};

template <typename T, int S>
__global__ void __launch_bounds__(256)
hyper_norm_kernel(T* __restrict__ out, float* __restrict__ streams, const T* __restrict__ y,
                  const float* __restrict__ part, int splits, size_t split_stride, const T* __restrict__ bias,
                  const float* __restrict__ mix_w, const float* __restrict__ out_w, const float* __restrict__ in_w,
                  const float* __restrict__ w, float eps, int hidden, int first, float alpha) {
  pdl_launch_dependents();
  extern __shared__ float u_s[];           // [hidden]
  __shared__ float scratch[32];
  __shared__ HsWeights hw;
  // (the link weights are model tensors: nothing in the step writes them, so they are read before the wait)
  if (threadIdx.x < S * S) hw.mix[threadIdx.x] = mix_w != nullptr ? mix_w[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    hw.out[threadIdx.x] = out_w != nullptr ? out_w[threadIdx.x] : 1.f;
    hw.in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
  }
  pdl_wait();
  __syncthreads();
  const size_t row = blockIdx.x;
  float* xs = streams + row * S * hidden;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float yv = 0.f;
    const bool has_y = y != nullptr || part != nullptr;
    if (part != nullptr) {
      for (int sp = 0; sp < splits; ++sp) yv += __ldcg(part + (size_t)sp * split_stride + row * hidden + i);
      yv = round_to<T>(yv + (bias != nullptr ? to_f(bias[i]) : 0.f));
    } else if (y != nullptr) {
      yv = to_f(y[row * hidden + i]);
    }
    float nx[S];
    if (first) {
#pragma unroll
      for (int t = 0; t < S; ++t) nx[t] = alpha * yv;
    } else {
      float x[S];
#pragma unroll
      for (int s = 0; s < S; ++s) x[s] = xs[(size_t)s * hidden + i];
      if (has_y) {
#pragma unroll
        for (int t = 0; t < S; ++t) {
          float a = 0.f;
#pragma unroll
          for (int s = 0; s < S; ++s) a = fmaf(hw.mix[s * S + t], x[s], a);
          nx[t] = fmaf(hw.out[t], yv, a);
        }
      } else {
#pragma unroll
        for (int t = 0; t < S; ++t) nx[t] = x[t];
      }
    }
    float u = 0.f;
#pragma unroll
    for (int t = 0; t < S; ++t) {
      if (first || has_y) xs[(size_t)t * hidden + i] = nx[t];
      u = fmaf(hw.in[t], nx[t], u);
    }
    u_s[i] = u;
    ss = fmaf(u, u, ss);
  }
  if (out == nullptr) return;
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)           // (a thread reads back what it wrote itself)
    out[row * hidden + i] = from_f<T>(u_s[i] * rstd * w[i]);
}


// The same for rows a multiple of 4 long and at most 4 * CH * blockDim: every load of a thread (its 16 bytes of every
// copy, of y or of its partial sums) is issued before the first is used, the new copies and u stay in registers, the
// stream moves as float4: one round trip to memory.
template <typename T, int S, int CH>
__global__ void __launch_bounds__(256)
hyper_norm_vec_kernel(T* __restrict__ out, float* __restrict__ streams, const T* __restrict__ y,
                      const float* __restrict__ part, int splits, size_t split_stride, const T* __restrict__ bias,
                      const float* __restrict__ mix_w, const float* __restrict__ out_w, const float* __restrict__ in_w,
                      const float* __restrict__ w, float eps, int hidden, int first, float alpha) {
  pdl_launch_dependents();
  __shared__ float scratch[32];
  __shared__ HsWeights hw;
  if (threadIdx.x < S * S) hw.mix[threadIdx.x] = mix_w != nullptr ? mix_w[threadIdx.x] : (threadIdx.x / S == threadIdx.x % S ? 1.f : 0.f);
  if (threadIdx.x < S) {
    hw.out[threadIdx.x] = out_w != nullptr ? out_w[threadIdx.x] : 1.f;
    hw.in[threadIdx.x] = in_w != nullptr ? in_w[threadIdx.x] : 1.f;
  }
  pdl_wait();
  __syncthreads();
  const size_t row = blockIdx.x;
  float* xs = streams + row * S * hidden;
  const bool has_y = y != nullptr || part != nullptr;
  float u[CH][4];
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
      float yv[4] = {0.f, 0.f, 0.f, 0.f};
      if (part != nullptr) {
        float4 p4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < splits; ++sp) {
          const float4 q4 = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * split_stride + row * hidden + i));
          p4.x += q4.x; p4.y += q4.y; p4.z += q4.z; p4.w += q4.w;
        }
        const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) yv[k] = round_to<T>(pv[k] + (bias != nullptr ? to_f(bias[i + k]) : 0.f));
      } else if (y != nullptr) {
#pragma unroll
        for (int k = 0; k < 4; ++k) yv[k] = to_f(y[row * hidden + i + k]);
      }
      float x[S][4], nx[S][4];
      if (!first) {
#pragma unroll
        for (int s = 0; s < S; ++s) {
          const float4 v = *reinterpret_cast<const float4*>(xs + (size_t)s * hidden + i);
          x[s][0] = v.x; x[s][1] = v.y; x[s][2] = v.z; x[s][3] = v.w;
        }
      }
#pragma unroll
      for (int t = 0; t < S; ++t) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          if (first) nx[t][k] = alpha * yv[k];
          else if (has_y) {
            float a = 0.f;
#pragma unroll
            for (int s = 0; s < S; ++s) a = fmaf(hw.mix[s * S + t], x[s][k], a);
            nx[t][k] = fmaf(hw.out[t], yv[k], a);
          } else nx[t][k] = x[t][k];
        }
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) u[c][k] = 0.f;
#pragma unroll
      for (int t = 0; t < S; ++t) {
        if (first || has_y) *reinterpret_cast<float4*>(xs + (size_t)t * hidden + i) = make_float4(nx[t][0], nx[t][1], nx[t][2], nx[t][3]);
#pragma unroll
        for (int k = 0; k < 4; ++k) u[c][k] = fmaf(hw.in[t], nx[t][k], u[c][k]);
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) ss = fmaf(u[c][k], u[c][k], ss);
    }
  }
  if (out == nullptr) return;
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
#pragma unroll
      for (int k = 0; k < 4; ++k) out[row * hidden + i + k] = from_f<T>(u[c][k] * rstd * w[i + k]);
    }
  }
}

template <typename T>
int launch_hyper(int S, dim3 grid, dim3 block, size_t smem, cudaStream_t s, T* out, float* streams, const T* y,
                 const float* part, int splits, size_t split_stride, const T* bias, const float* mix_w,
                 const float* out_w, const float* in_w, const float* w, float eps, int hidden, int first, float alpha) {
  // rows a multiple of 4 long on 16-byte boundaries, up to 4 copies: the kernel that keeps the row in registers
  const bool vec = S <= 4 && hidden % 4 == 0 && hidden <= 4 * 4 * 256 && !((uintptr_t)streams & 15) && !((uintptr_t)part & 15);
  const int ch = hidden <= 1024 ? 1 : (hidden <= 2048 ? 2 : 4);
  const dim3 vblock((((hidden / 4 + ch - 1) / ch) + 31) / 32 * 32);
#define TS_HV(N, CH)                                                                                                  \
  ts_launch(hyper_norm_vec_kernel<T, N, CH>, grid, vblock, 0, s, out, streams, y, part, splits, split_stride, bias, mix_w, \
            out_w, in_w, w, eps, hidden, first, alpha)
#define TS_HS(N)                                                                                                      \
  case N:                                                                                                             \
    if (vec && N <= 4) {                                                                                              \
      constexpr int M = N <= 4 ? N : 1;                                                                               \
      if (ch == 1) TS_HV(M, 1);                                                                                       \
      else if (ch == 2) TS_HV(M, 2);                                                                                  \
      else TS_HV(M, 4);                                                                                               \
      break;                                                                                                          \
    }                                                                                                                 \
    if (smem > 48 * 1024) cudaFuncSetAttribute(hyper_norm_kernel<T, N>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    ts_launch(hyper_norm_kernel<T, N>, grid, block, smem, s, out, streams, y, part, splits, split_stride, bias, mix_w, \
              out_w, in_w, w, eps, hidden, first, alpha);                                                             \
    break
  switch (S) {
    TS_HS(1); TS_HS(2); TS_HS(3); TS_HS(4); TS_HS(5); TS_HS(6); TS_HS(7); TS_HS(8);
    default: return -1;
  }
#undef TS_HS
#undef TS_HV
  return 0;
}

}  // namespace

TS_API int ts_hyper_norm_max_streams() { return HS_MAX; }

// out [T, hidden] (may be null: only the write-back); streams [T, S, hidden] 32-bit; y [T, hidden] or null; part /
// splits / bias: y as a product left unreduced; mix [S, S], outw [S], inw [S] 32-bit on the device (null: identity /
// ones); w [hidden] 32-bit; first != 0: every copy starts as alpha * y.
TS_API int ts_hyper_norm(void* out, float* streams, const void* y, const float* part, int splits, const void* bias,
                         const float* mix, const float* outw, const float* inw, const float* w, float eps, int T, int S,
                         int hidden, int first, float alpha, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (S < 1 || S > HS_MAX) TS_REFUSE(TS_ERR_LIMIT, "ts_hyper_norm: %d copies of the stream (limit %d)", S, HS_MAX);
  if (hidden <= 0 || hidden > 48 * 1024) TS_REFUSE(TS_ERR_LIMIT, "ts_hyper_norm: rows of %d", hidden);
  if (first && y == nullptr && part == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_hyper_norm: a stream starts from a tensor");
  if (out != nullptr && w == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_hyper_norm: a norm without a weight");
  cudaStream_t s = (cudaStream_t)stream;
  const int th = hidden >= 1024 ? 256 : 128;
  const size_t smem = sizeof(float) * hidden;
  int rc;
  if (dtype == TS_F32)
    rc = launch_hyper<float>(S, dim3(T), dim3(th), smem, s, (float*)out, streams, (const float*)y, part, splits,
                             (size_t)T * hidden, (const float*)bias, mix, outw, inw, w, eps, hidden, first, alpha);
  else if (dtype == TS_BF16)
    rc = launch_hyper<bf16>(S, dim3(T), dim3(th), smem, s, (bf16*)out, streams, (const bf16*)y, part, splits,
                            (size_t)T * hidden, (const bf16*)bias, mix, outw, inw, w, eps, hidden, first, alpha);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_hyper_norm: dtype %d", dtype);
  if (rc != 0) TS_REFUSE(TS_ERR_LIMIT, "ts_hyper_norm: %d copies", S);
  TS_LAUNCH_CHECK();
}
