// Row-wise kernels of models whose residual stream is kept in 32-bit whatever the engine's type:
//   * the stream's own norm (RMS, or a layer norm with mean, weight and bias), which first takes the pending
//     branch outputs (times a constant) and a vector common to all rows into the stream,
//   * an RMS norm over a 32-bit row with a sigmoid gate from a second tensor (the output stage of a
//     linear-attention mixer),
//   * one-input activations (tanh-form GELU, squared ReLU, SiLU).
// All arithmetic is 32-bit with one rounding to the output type.
#include "activations.cuh"
#include "common.cuh"

namespace {

// stream[row] (+)= alpha * add1[row] + alpha * add2[row] + vec;  out[row] = T(stream * rsqrt(mean(stream^2) + eps) * w),
// or with a norm bias nb the layer norm T((stream - mean) * rsqrt(mean((stream - mean)^2) + eps) * w + nb).
// first != 0: the stream row is not read (this call starts it).  add1 / add2 / vec (32-bit, one row) may be null.
template <typename T, typename WT>
__global__ void rmsnorm_wide_kernel(T* __restrict__ out, float* __restrict__ stream, const T* __restrict__ add1,
                                    const T* __restrict__ add2, const WT* __restrict__ w, float eps, int hidden,
                                    int first, float alpha, const float* __restrict__ vec, const WT* __restrict__ nb) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float ss = 0.f, s1 = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
    float v = first ? 0.f : stream[base + i];
    if (add1 != nullptr) v += alpha * to_f(add1[base + i]);
    if (add2 != nullptr) v += alpha * to_f(add2[base + i]);
    if (vec != nullptr) v += vec[i];
    stream[base + i] = v;
    ss += v * v;
    s1 += v;
  }
  if (out == nullptr) return;
  if (nb != nullptr) {
    const float mean = block_sum(s1, scratch) / (float)hidden;
    float dev = 0.f;
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      const float d = stream[base + i] - mean;
      dev += d * d;
    }
    dev = block_sum(dev, scratch);
    const float rstd = 1.f / sqrtf(dev / (float)hidden + eps);
    for (int i = threadIdx.x; i < hidden; i += blockDim.x)
      out[base + i] = from_f<T>((stream[base + i] - mean) * rstd * to_f(w[i]) + to_f(nb[i]));
    return;
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    out[base + i] = from_f<T>(stream[base + i] * rstd * to_f(w[i]));
}

// The same, for rows whose length is a multiple of 4 and at most 4 * 4 * blockDim: every thread keeps its values in
// registers between the sum and the result, the stream moves as float4 (one round trip to memory instead of two).
template <typename T, typename WT, int CH>
__global__ void __launch_bounds__(256)
rmsnorm_wide_vec_kernel(T* __restrict__ out, float* __restrict__ stream, const T* __restrict__ add1,
                        const T* __restrict__ add2, const WT* __restrict__ w, float eps, int hidden, int first,
                        const float* __restrict__ part, int splits, size_t split_stride, const T* __restrict__ bias,
                        float alpha, const float* __restrict__ vec, const WT* __restrict__ nb) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const size_t base = (size_t)blockIdx.x * hidden;
  float v[CH][4];
  float ss = 0.f, s1 = 0.f;
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
      float4 s4 = first ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(stream + base + i);
      v[c][0] = s4.x; v[c][1] = s4.y; v[c][2] = s4.z; v[c][3] = s4.w;
      if (part != nullptr) {
        // a product left unreduced by its kernel: the partial sums in split order, the bias, and the rounding the
        // product's own epilogue would have done
        float4 p4 = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int sp = 0; sp < splits; ++sp) {
          const float4 q4 = __ldcg(reinterpret_cast<const float4*>(part + (size_t)sp * split_stride + base + i));
          p4.x += q4.x; p4.y += q4.y; p4.z += q4.z; p4.w += q4.w;
        }
        const float pv[4] = {p4.x, p4.y, p4.z, p4.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) v[c][k] += alpha * round_to<T>(pv[k] + (bias != nullptr ? to_f(bias[i + k]) : 0.f));
      }
#pragma unroll
      for (int k = 0; k < 4; ++k) {
        if (add1 != nullptr) v[c][k] += alpha * to_f(add1[base + i + k]);
        if (add2 != nullptr) v[c][k] += alpha * to_f(add2[base + i + k]);
        if (vec != nullptr) v[c][k] += vec[i + k];
        ss += v[c][k] * v[c][k];
        s1 += v[c][k];
      }
      *reinterpret_cast<float4*>(stream + base + i) = make_float4(v[c][0], v[c][1], v[c][2], v[c][3]);
    }
  }
  if (out == nullptr) return;
  if (nb != nullptr) {
    // layer norm: the deviations from the mean are taken from the registers, so the variance is a sum of squares of
    // small numbers and not a difference of large ones
    const float mean = block_sum(s1, scratch) / (float)hidden;
    float dev = 0.f;
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int i = (c * blockDim.x + threadIdx.x) * 4;
      if (i < hidden) {
#pragma unroll
        for (int k = 0; k < 4; ++k) {
          v[c][k] -= mean;
          dev += v[c][k] * v[c][k];
        }
      }
    }
    dev = block_sum(dev, scratch);
    const float rstd = 1.f / sqrtf(dev / (float)hidden + eps);
#pragma unroll
    for (int c = 0; c < CH; ++c) {
      const int i = (c * blockDim.x + threadIdx.x) * 4;
      if (i < hidden) {
#pragma unroll
        for (int k = 0; k < 4; ++k) out[base + i + k] = from_f<T>(v[c][k] * rstd * to_f(w[i + k]) + to_f(nb[i + k]));
      }
    }
    return;
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)hidden + eps);
#pragma unroll
  for (int c = 0; c < CH; ++c) {
    const int i = (c * blockDim.x + threadIdx.x) * 4;
    if (i < hidden) {
#pragma unroll
      for (int k = 0; k < 4; ++k) out[base + i + k] = from_f<T>(v[c][k] * rstd * to_f(w[i + k]));
    }
  }
}

// out[row] = T(x * rsqrt(mean(x^2) + eps) * w * sigmoid(gate[row]));  x is 32-bit, the gate has its own row stride
template <typename T, typename WT>
__global__ void gated_rmsnorm_kernel(T* __restrict__ out, const float* __restrict__ x, const T* __restrict__ gate,
                                     int gate_stride, const WT* __restrict__ w, float eps, int n) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const float* xr = x + (size_t)blockIdx.x * n;
  const T* gr = gate + (size_t)blockIdx.x * gate_stride;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += xr[i] * xr[i];
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float g = 1.f / (1.f + expf(-to_f(gr[i])));
    out[(size_t)blockIdx.x * n + i] = from_f<T>(xr[i] * rstd * to_f(w[i]) * g);
  }
}

template <typename T>
__global__ void activation_kernel(T* __restrict__ out, const T* __restrict__ x, size_t n, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    out[i] = from_f<T>(ts_activate(to_f(x[i]), kind));
}

// out = act(T(sum over splits of part + bias)): the activation fed by a product left unreduced
template <typename T>
__global__ void activation_parts_kernel(T* __restrict__ out, const float* __restrict__ part, int splits, size_t split_stride,
                                        const T* __restrict__ bias, size_t n, int cols, int kind) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
    float v = 0.f;
    for (int sp = 0; sp < splits; ++sp) v += __ldcg(part + (size_t)sp * split_stride + i);
    if (bias != nullptr) v += to_f(bias[i % cols]);
    out[i] = from_f<T>(ts_activate(round_to<T>(v), kind));
  }
}


// gate functions of the kernels below
enum TsGate : int { TS_GATE_SIGMOID = 0, TS_GATE_SILU = 1 };
__device__ __forceinline__ float ts_gate(float g, int kind) {
  const float sg = 1.f / (1.f + expf(-g));
  return kind == TS_GATE_SILU ? g * sg : sg;
}
// On its way to a rounding to bfloat16 the hardware's approximate exponential and reciprocal serve (about 2^-21 relative,
// against a bfloat16 step of 2^-9; see silu_for); the 32-bit type keeps the exact ones.
template <typename T> __device__ __forceinline__ float ts_gate_for(float g, int kind) { return ts_gate(g, kind); }
template <> __device__ __forceinline__ float ts_gate_for<bf16>(float g, int kind) {
  const float sg = __fdividef(1.f, 1.f + __expf(-g));
  return kind == TS_GATE_SILU ? g * sg : sg;
}

// An RMS norm over a 32-bit row in `groups` equal parts, each by its own root mean square, with a gate from a second
// tensor that multiplies either what is normed (gate_first) or the normed result:
//   gate_first:  v = x * gate(z);  out = T(v * rsqrt(mean_part(v^2) + eps) * w * scale)
//   else:        out = T(x * rsqrt(mean_part(x^2) + eps) * w * gate(z) * scale)
// grid (T, groups); out and the gate have row strides of their own (a column slice of a wider tensor).
template <typename T>
__global__ void gated_group_rmsnorm_kernel(T* __restrict__ out, int out_stride, const float* __restrict__ x,
                                           const T* __restrict__ gate, int gate_stride, const float* __restrict__ w,
                                           float eps, int n, int groups, int gate_kind, int gate_first, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int m = n / groups, c0 = blockIdx.y * m;
  const float* xr = x + (size_t)blockIdx.x * n + c0;
  const T* gr = gate + (size_t)blockIdx.x * gate_stride + c0;
  T* orow = out + (size_t)blockIdx.x * out_stride + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    float v = xr[i];
    if (gate_first) v *= ts_gate_for<T>(to_f(gr[i]), gate_kind);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)m + eps);
  for (int i = threadIdx.x; i < m; i += blockDim.x) {
    const float g = ts_gate_for<T>(to_f(gr[i]), gate_kind);
    const float v = gate_first ? xr[i] * g * rstd * w[c0 + i] : xr[i] * rstd * w[c0 + i] * g;
    orow[i] = from_f<T>(v * scale);
  }
}

// out[t, i] = T(a[t, i] * gate(z[t, i]) * scale): the gate on a mixer's heads before its output projection
template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ out, int out_stride, const T* __restrict__ a, int a_stride,
                                const T* __restrict__ gate, int gate_stride, int n, size_t total, int gate_kind, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / n;
    const int i = (int)(idx - t * n);
    out[t * out_stride + i] = from_f<T>(to_f(a[t * a_stride + i]) * ts_gate_for<T>(to_f(gate[t * gate_stride + i]), gate_kind) * scale);
  }
}

int threads_for(int n) { return n >= 2048 ? 512 : (n >= 512 ? 256 : 128); }

}  // namespace

// The rows a multiple of 4 long and at most 4,096 (ts_rmsnorm_wide_takes_parts) may also take a product left
// unreduced: part [splits, T, hidden] 32-bit partial sums (+ bias), added to the stream after the rounding the
// product's epilogue would have done.
TS_API int ts_rmsnorm_wide_takes_parts(int hidden) { return hidden % 4 == 0 && hidden <= 4 * 4 * 256; }

//
// alpha multiplies what is added (add1, add2, the product); vec (32-bit [hidden], may be null) is added to every row;
// nbias (the type of w, may be null): with it the norm is a layer norm (mean taken off, variance about the mean,
// times w plus nbias) instead of the RMS norm.
TS_API int ts_rmsnorm_wide(void* out, float* stream, const void* add1, const void* add2, const void* w, float eps,
                           int T, int hidden, int first, int dtype, int w_dtype, const float* part, int splits,
                           const void* bias, float alpha, const float* vec, const void* nbias, void* stream_) {
  if (T <= 0) return 0;
  if (first && add1 == nullptr && part == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_rmsnorm_wide: a stream starts from a tensor");
  if (part != nullptr && (!ts_rmsnorm_wide_takes_parts(hidden) || ((uintptr_t)stream & 15) || ((uintptr_t)part & 15)))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_rmsnorm_wide: partial sums with rows of %d", hidden);
  cudaStream_t s = (cudaStream_t)stream_;
  const int th = threads_for(hidden);
  if (hidden % 4 == 0 && hidden <= 4 * 4 * 256 && !((uintptr_t)stream & 15)) {
    const int ch = hidden <= 1024 ? 1 : (hidden <= 2048 ? 2 : 4);
    const int tv = ((hidden / 4 + ch - 1) / ch + 31) / 32 * 32;
#define TS_WV(TT, WT, CH)                                                                                           \
  ts_launch(rmsnorm_wide_vec_kernel<TT, WT, CH>, dim3(T), dim3(tv), 0, s, (TT*)out, stream, (const TT*)add1, (const TT*)add2, \
            (const WT*)w, eps, hidden, first, part, splits, (size_t)T * hidden, (const TT*)bias, alpha, vec, (const WT*)nbias)
#define TS_WVC(TT, WT)      \
  do {                      \
    if (ch == 1) TS_WV(TT, WT, 1); \
    else if (ch == 2) TS_WV(TT, WT, 2); \
    else TS_WV(TT, WT, 4);  \
  } while (0)
    if (dtype == TS_F32 && w_dtype == TS_F32) TS_WVC(float, float);
    else if (dtype == TS_BF16 && w_dtype == TS_BF16) TS_WVC(bf16, bf16);
    else if (dtype == TS_BF16 && w_dtype == TS_F32) TS_WVC(bf16, float);
    else TS_REFUSE(TS_ERR_DTYPE, "ts_rmsnorm_wide: dtype %d with scale dtype %d", dtype, w_dtype);
#undef TS_WVC
#undef TS_WV
    TS_LAUNCH_CHECK();
  }
#define TS_WN(TT, WT)                                                                                         \
  ts_launch(rmsnorm_wide_kernel<TT, WT>, dim3(T), dim3(th), 0, s, (TT*)out, stream, (const TT*)add1, (const TT*)add2, \
            (const WT*)w, eps, hidden, first, alpha, vec, (const WT*)nbias)
  if (dtype == TS_F32 && w_dtype == TS_F32) TS_WN(float, float);
  else if (dtype == TS_BF16 && w_dtype == TS_BF16) TS_WN(bf16, bf16);
  else if (dtype == TS_BF16 && w_dtype == TS_F32) TS_WN(bf16, float);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_rmsnorm_wide: dtype %d with scale dtype %d", dtype, w_dtype);
#undef TS_WN
  TS_LAUNCH_CHECK();
}

TS_API int ts_gated_rmsnorm(void* out, const float* x, const void* gate, int gate_stride, const void* w, float eps,
                            int T, int n, int dtype, int w_dtype, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  const int th = threads_for(n);
#define TS_GN(TT, WT)                                                                                          \
  ts_launch(gated_rmsnorm_kernel<TT, WT>, dim3(T), dim3(th), 0, s, (TT*)out, x, (const TT*)gate, gate_stride, \
            (const WT*)w, eps, n)
  if (dtype == TS_F32 && w_dtype == TS_F32) TS_GN(float, float);
  else if (dtype == TS_BF16 && w_dtype == TS_BF16) TS_GN(bf16, bf16);
  else if (dtype == TS_BF16 && w_dtype == TS_F32) TS_GN(bf16, float);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_gated_rmsnorm: dtype %d with scale dtype %d", dtype, w_dtype);
#undef TS_GN
  TS_LAUNCH_CHECK();
}

// part: [splits, rows, cols] 32-bit partial sums of a product; out [rows, cols].
TS_API int ts_activation_parts(void* out, const float* part, int splits, const void* bias, int rows, int cols, int kind,
                               int dtype, void* stream) {
  const size_t n = (size_t)rows * cols;
  if (n == 0) return 0;
  if (kind < 1 || kind > TS_ACT_LAST) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_activation_parts: kind %d", kind);
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = (int)((n + 255) / 256 < 148 * 8 ? (n + 255) / 256 : 148 * 8);
  if (dtype == TS_F32)
    ts_launch(activation_parts_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)out, part, splits, n, (const float*)bias,
              n, cols, kind);
  else if (dtype == TS_BF16)
    ts_launch(activation_parts_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (bf16*)out, part, splits, n, (const bf16*)bias, n,
              cols, kind);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_activation_parts: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// kind: 1 tanh-form GELU, 2 squared ReLU, 3 SiLU, 4 GELU with the error function.  out may be x.
TS_API int ts_activation(void* out, const void* x, long long n, int kind, int dtype, void* stream) {
  if (n <= 0) return 0;
  if (kind < 1 || kind > TS_ACT_LAST) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_activation: kind %d", kind);
  cudaStream_t s = (cudaStream_t)stream;
  const int blocks = (int)((n + 1023) / 1024 < 148 * 8 ? (n + 1023) / 1024 : 148 * 8);
  if (dtype == TS_F32)
    ts_launch(activation_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)out, (const float*)x, (size_t)n, kind);
  else if (dtype == TS_BF16)
    ts_launch(activation_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (bf16*)out, (const bf16*)x, (size_t)n, kind);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_activation: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// the same, 8 bfloat16 columns (16 bytes of each operand) a thread: rows and strides in multiples of 8 on 16-byte boundaries
__global__ void gate_mul_vec_kernel(bf16* __restrict__ out, int out_stride, const bf16* __restrict__ a, int a_stride,
                                    const bf16* __restrict__ gate, int gate_stride, int n8, size_t total8, int gate_kind, float scale) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total8; idx += (size_t)gridDim.x * blockDim.x) {
    const size_t t = idx / n8;
    const int i = (int)(idx - t * n8) * 8;
    const uint4 av = *reinterpret_cast<const uint4*>(a + t * a_stride + i);
    const uint4 gv = *reinterpret_cast<const uint4*>(gate + t * gate_stride + i);
    const __nv_bfloat162* ah = reinterpret_cast<const __nv_bfloat162*>(&av);
    const __nv_bfloat162* gh = reinterpret_cast<const __nv_bfloat162*>(&gv);
    uint4 ov;
    __nv_bfloat162* oh = reinterpret_cast<__nv_bfloat162*>(&ov);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 af = __bfloat1622float2(ah[j]), gf = __bfloat1622float2(gh[j]);
      oh[j] = __floats2bfloat162_rn(af.x * ts_gate_for<bf16>(gf.x, gate_kind) * scale, af.y * ts_gate_for<bf16>(gf.y, gate_kind) * scale);
    }
    *reinterpret_cast<uint4*>(out + t * out_stride + i) = ov;
  }
}

// x [T, n] 32-bit; gate [T, gate_stride] and out [T, out_stride] in `dtype`; w [n] 32-bit.  gate_kind: 0 sigmoid, 1 SiLU.
TS_API int ts_gated_group_rmsnorm(void* out, int out_stride, const float* x, const void* gate, int gate_stride,
                                  const float* w, float eps, int T, int n, int groups, int gate_kind, int gate_first,
                                  float scale, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (groups < 1 || n % groups) TS_REFUSE(TS_ERR_SHAPE, "ts_gated_group_rmsnorm: %d columns in %d parts", n, groups);
  if (groups > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_gated_group_rmsnorm: %d parts", groups);
  cudaStream_t s = (cudaStream_t)stream;
  const int th = threads_for(n / groups);
  if (dtype == TS_F32)
    ts_launch(gated_group_rmsnorm_kernel<float>, dim3(T, groups), dim3(th), 0, s, (float*)out, out_stride, x, (const float*)gate,
              gate_stride, w, eps, n, groups, gate_kind, gate_first, scale);
  else if (dtype == TS_BF16)
    ts_launch(gated_group_rmsnorm_kernel<bf16>, dim3(T, groups), dim3(th), 0, s, (bf16*)out, out_stride, x, (const bf16*)gate,
              gate_stride, w, eps, n, groups, gate_kind, gate_first, scale);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_gated_group_rmsnorm: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// out [T, out_stride], a [T, a_stride], gate [T, gate_stride], n columns each.  out may be a.
TS_API int ts_gate_mul(void* out, int out_stride, const void* a, int a_stride, const void* gate, int gate_stride, int T,
                       int n, int gate_kind, float scale, int dtype, void* stream) {
  const size_t total = (size_t)T * n;
  if (total == 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_BF16 && n % 8 == 0 && out_stride % 8 == 0 && a_stride % 8 == 0 && gate_stride % 8 == 0 &&
      !(((uintptr_t)out | (uintptr_t)a | (uintptr_t)gate) & 15)) {
    const size_t total8 = total / 8;
    const int vb = (int)((total8 + 255) / 256 < 148 * 16 ? (total8 + 255) / 256 : 148 * 16);
    ts_launch(gate_mul_vec_kernel, dim3(vb), dim3(256), 0, s, (bf16*)out, out_stride, (const bf16*)a, a_stride, (const bf16*)gate,
              gate_stride, n / 8, total8, gate_kind, scale);
    TS_LAUNCH_CHECK();
  }
  const int blocks = (int)((total + 255) / 256 < 148 * 8 ? (total + 255) / 256 : 148 * 8);
  if (dtype == TS_F32)
    ts_launch(gate_mul_kernel<float>, dim3(blocks), dim3(256), 0, s, (float*)out, out_stride, (const float*)a, a_stride,
              (const float*)gate, gate_stride, n, total, gate_kind, scale);
  else if (dtype == TS_BF16)
    ts_launch(gate_mul_kernel<bf16>, dim3(blocks), dim3(256), 0, s, (bf16*)out, out_stride, (const bf16*)a, a_stride,
              (const bf16*)gate, gate_stride, n, total, gate_kind, scale);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_gate_mul: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}
