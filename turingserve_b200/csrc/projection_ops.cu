// What sits between a projection and the attention that consumes it, for mixers that norm, rotate or re-project
// their queries and keys; 32-bit arithmetic and one rounding everywhere:
//   ts_rms_rows          out = x[:, col0 : col0 + n] / rms * w               (a column slice of wider rows)
//   ts_qk_rownorm_write  q and k normed over their WHOLE rows (all heads at once), q times a temperature that grows
//                        with the position; normed keys into the key cache, the keys as projected into the value cache
//   ts_latent_kv_write   one cached row a token: [rms(latent) * w | rotated key part]
//   ts_rotate_pairs      rotation of neighbouring pairs (2i, 2i+1), angle = position * freq[i] in 32-bit, cosine and
//                        sine times a magnitude; strided source and destination
//   ts_rope_headnorm_write  rotation of the pairs (i, i + R/2) of every q and k head, angle = position * freq[i] in 32-bit,
//                        then each head over its root mean square (no weight); q in place, k and v rows into a cache
//                        whose key and value rows have widths of their own
//   ts_batched_linear    out[t, h, :] = w[h] x[t, h, :], a product per head over strided rows (FFMA, fixed k order; up to
//                        16 rows: a warp an output column, streaming its weight row)
#include "common.cuh"

namespace {

template <typename T>
__global__ void rms_rows_kernel(T* __restrict__ out, const T* __restrict__ x, int x_stride, int col0, int n,
                                const float* __restrict__ w, float eps) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const T* xr = x + (size_t)blockIdx.x * x_stride + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = to_f(xr[i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x) out[(size_t)blockIdx.x * n + i] = from_f<T>(to_f(xr[i]) * rstd * w[i]);
}

template <typename T>
__global__ void qk_rownorm_write_kernel(T* __restrict__ proj, int stride, const float* __restrict__ q_w,
                                        const float* __restrict__ k_w, float eps, const int* __restrict__ positions,
                                        float coef, int every, T* __restrict__ k_cache, T* __restrict__ v_cache,
                                        const int* __restrict__ slots, int H, int G, int D, int page) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  T* row = proj + (size_t)t * stride;
  const int hd = H * D, gd = G * D;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < hd; i += blockDim.x) {
    const float v = to_f(row[i]);
    sq = fmaf(v, v, sq);
  }
  for (int i = threadIdx.x; i < gd; i += blockDim.x) {
    const float v = to_f(row[hd + i]);
    sk = fmaf(v, v, sk);
  }
  sq = block_sum(sq, scratch);
  sk = block_sum(sk, scratch);
  const int p = positions[t];
  // (p + 1) / every as an integer division: the floor of the quotient of two positive integers
  const float heat = coef != 0.f ? 1.f + coef * logf((float)((p + 1) / every) + 1.f) : 1.f;
  const float rq = heat / sqrtf(sq / (float)hd + eps), rk = 1.f / sqrtf(sk / (float)gd + eps);
  const int slot = slots != nullptr ? slots[t] : -1;
  if (slot >= 0) {
    const size_t pg = slot / page, off = slot % page;
    for (int i = threadIdx.x; i < gd; i += blockDim.x) {
      const int g = i / D, d = i % D;
      const size_t at = ((pg * G + g) * page + off) * D + d;
      const T raw = row[hd + i];
      k_cache[at] = from_f<T>(to_f(raw) * rk * k_w[i]);
      v_cache[at] = raw;
    }
  }
  for (int i = threadIdx.x; i < hd; i += blockDim.x) row[i] = from_f<T>(to_f(row[i]) * rq * q_w[i]);
}

__device__ __forceinline__ void pair_angle(int pos, float f, float magnitude, float& c, float& s) {
  const float a = (float)pos * f;
  sincosf(a, &s, &c);
  c *= magnitude;
  s *= magnitude;
}

template <typename T>
__global__ void latent_kv_write_kernel(const T* __restrict__ proj, int stride, int col0, const float* __restrict__ w,
                                       float eps, const int* __restrict__ positions, const float* __restrict__ freq,
                                       float magnitude, int rot_dims, T* __restrict__ k_cache,
                                       const int* __restrict__ slots, int rank, int R, int page) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ float scratch[32];
  const int t = blockIdx.x;
  const int slot = slots[t];
  if (slot < 0) return;
  const T* row = proj + (size_t)t * stride + col0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < rank; i += blockDim.x) {
    const float v = to_f(row[i]);
    ss = fmaf(v, v, ss);
  }
  ss = block_sum(ss, scratch);
  const float rstd = 1.f / sqrtf(ss / (float)rank + eps);
  T* dst = k_cache + ((size_t)(slot / page) * page + slot % page) * (rank + R);        // one kv head
  for (int i = threadIdx.x; i < rank; i += blockDim.x) dst[i] = from_f<T>(to_f(row[i]) * rstd * w[i]);
  const int pos = positions[t];
  for (int i = threadIdx.x; i < R / 2 + (R & 1); i += blockDim.x) {
    const int d = 2 * i;
    if (d < rot_dims) {                                  // (rot_dims is even and at most R)
      float c, s;
      pair_angle(pos, freq[i], magnitude, c, s);
      const float u = to_f(row[rank + d]), v = to_f(row[rank + d + 1]);
      dst[rank + d] = from_f<T>(u * c - v * s);
      dst[rank + d + 1] = from_f<T>(v * c + u * s);
    } else {
      dst[rank + d] = row[rank + d];
      if (d + 1 < R) dst[rank + d + 1] = row[rank + d + 1];
    }
  }
}

template <typename T>
__global__ void rotate_pairs_kernel(T* __restrict__ dst, int dst_ts, int dst_hs, const T* __restrict__ src, int src_ts,
                                    int src_hs, const int* __restrict__ positions, const float* __restrict__ freq,
                                    float magnitude, int rot_dims, int H, int R) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int pos = positions[t];
  const int half = R / 2 + (R & 1);
  for (int idx = threadIdx.x; idx < H * half; idx += blockDim.x) {
    const int h = idx / half, i = idx % half, d = 2 * i;
    const T* a = src + (size_t)t * src_ts + (size_t)h * src_hs;
    T* o = dst + (size_t)t * dst_ts + (size_t)h * dst_hs;
    if (d < rot_dims) {                                  // (rot_dims is even and at most R)
      float c, s;
      pair_angle(pos, freq[i], magnitude, c, s);
      const float u = to_f(a[d]), v = to_f(a[d + 1]);
      o[d] = from_f<T>(u * c - v * s);
      o[d + 1] = from_f<T>(v * c + u * s);
    } else {
      o[d] = a[d];
      if (d + 1 < R) o[d + 1] = a[d + 1];
    }
  }
}

constexpr int BL_M = 64, BL_N = 64, BL_K = 16, BL_PAD = 4;

template <typename T>
__global__ void __launch_bounds__(256)
batched_linear_kernel(T* __restrict__ out, int out_ts, int out_hs, const T* __restrict__ x, int x_ts, int x_hs,
                      const T* __restrict__ w, int M, int N, int K) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ __align__(16) float As[BL_K][BL_M + BL_PAD];
  __shared__ __align__(16) float Ws[BL_K][BL_N + BL_PAD];
  const int tid = threadIdx.x;
  const int h = blockIdx.z;
  const int m0 = blockIdx.y * BL_M, n0 = blockIdx.x * BL_N;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};
  const int am = m0 + lr;
  const T* a_row = am < M ? x + (size_t)am * x_ts + (size_t)h * x_hs : nullptr;
  const int wn = n0 + lr;
  const T* w_row = wn < N ? w + ((size_t)h * N + wn) * K : nullptr;
  for (int k0 = 0; k0 < K; k0 += BL_K) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_row != nullptr && k < K) ? to_f(a_row[k]) : 0.f;
      Ws[lk + i][lr] = (w_row != nullptr && k < K) ? to_f(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < BL_K; ++k) {
      const float4 a = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float4 b = *reinterpret_cast<const float4*>(&Ws[k][tx * 4]);
      const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + ty * 4 + i;
    if (m >= M) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n < N) out[(size_t)m * out_ts + (size_t)h * out_hs + n] = from_f<T>(acc[i][j]);
    }
  }
}

// Few rows: the weights are what is read.  A warp owns one output column of one head; its lanes stream that weight
// row 16 bytes at a time and keep a partial sum for each of up to BLR_ROWS token rows (whose pieces come out of L1/L2,
// shared by all warps); a lane's share of k and the order of the sums are the same whatever the number of rows.
constexpr int BLR_ROWS = 8, BLR_WARPS = 8;

template <typename T>
__global__ void __launch_bounds__(BLR_WARPS * 32)
batched_linear_rows_kernel(T* __restrict__ out, int out_ts, int out_hs, const T* __restrict__ x, int x_ts, int x_hs,
                           const T* __restrict__ w, int M, int N, int K) {
  pdl_launch_dependents();
  constexpr int PER = 16 / (int)sizeof(T);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.y, n = blockIdx.x * BLR_WARPS + warp;
  if (n >= N) return;
  const T* w_row = w + ((size_t)h * N + n) * K;
  // (the weights are nobody's output: their first pieces are on their way before the wait for the predecessor)
  uint4 first = make_uint4(0u, 0u, 0u, 0u);
  if (lane * PER < K) first = *reinterpret_cast<const uint4*>(w_row + lane * PER);
  pdl_wait();
  for (int m0 = 0; m0 < M; m0 += BLR_ROWS) {
    float acc[BLR_ROWS];
#pragma unroll
    for (int r = 0; r < BLR_ROWS; ++r) acc[r] = 0.f;
    for (int k = lane * PER; k < K; k += 32 * PER) {
      const uint4 wv = k == lane * PER ? first : *reinterpret_cast<const uint4*>(w_row + k);
      const T* we = reinterpret_cast<const T*>(&wv);
#pragma unroll
      for (int r = 0; r < BLR_ROWS; ++r) {
        if (m0 + r < M) {
          const uint4 xv = *reinterpret_cast<const uint4*>(x + (size_t)(m0 + r) * x_ts + (size_t)h * x_hs + k);
          const T* xe = reinterpret_cast<const T*>(&xv);
#pragma unroll
          for (int u = 0; u < PER; ++u) acc[r] = fmaf(to_f(xe[u]), to_f(we[u]), acc[r]);
        }
      }
    }
#pragma unroll
    for (int r = 0; r < BLR_ROWS; ++r) {
      const float v = warp_sum(acc[r]);
      if (lane == 0 && m0 + r < M) out[(size_t)(m0 + r) * out_ts + (size_t)h * out_hs + n] = from_f<T>(v);
    }
  }
}

// One warp a (token, head), RHN_WARPS heads a block.  The head's D values pass through shared memory: rotated in
// 32-bit (dimension i < R/2 with dimension i + R/2, the rest as they are), then, with norm != 0, divided by
// sqrt(mean of their squares + eps), rounded once; q heads go back where they came from, k heads into the key
// cache.  The block with blockIdx.y == 0 also copies the token's value rows.  A slot of -1 caches nothing.
constexpr int RHN_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(RHN_WARPS * 32)
rope_headnorm_write_kernel(T* __restrict__ proj, int stride, int k_off, int v_off, const int* __restrict__ positions,
                           const float* __restrict__ freq, int rot_dims, int norm, float eps, T* __restrict__ k_cache,
                           T* __restrict__ v_cache, const int* __restrict__ slots, int H, int G, int D, int V, int page) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float rhn_s[];
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y * RHN_WARPS + warp;
  const int slot = slots != nullptr ? slots[t] : -1;
  T* row = proj + (size_t)t * stride;
  if (head < H + G) {
    float* x = rhn_s + warp * D;
    T* src = head < H ? row + (size_t)head * D : row + k_off + (size_t)(head - H) * D;
    const float pos = (float)positions[t];
    const int half = rot_dims / 2;
    float ss = 0.f;
    for (int i = lane; i < half; i += 32) {
      float sn, cs;
      sincosf(pos * freq[i], &sn, &cs);
      const float u = to_f(src[i]), v = to_f(src[i + half]);
      const float a = u * cs - v * sn, b = v * cs + u * sn;
      x[i] = a;
      x[i + half] = b;
      ss += a * a + b * b;
    }
    for (int i = rot_dims + lane; i < D; i += 32) {
      const float v = to_f(src[i]);
      x[i] = v;
      ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    __syncwarp();
    const float r = norm ? 1.f / sqrtf(ss / (float)D + eps) : 1.f;
    T* dst = src;
    if (head >= H) {
      dst = nullptr;
      if (slot >= 0) {
        const size_t pg = slot / page, off = slot % page;
        dst = k_cache + ((pg * G + (head - H)) * page + off) * D;
      }
    }
    if (dst != nullptr)
      for (int i = lane; i < D; i += 32) dst[i] = from_f<T>(x[i] * r);
  }
  if (blockIdx.y == 0 && slot >= 0 && v_cache != nullptr) {
    const size_t pg = slot / page, off = slot % page;
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) {
      const int g = i / V, d = i % V;
      v_cache[((pg * G + g) * page + off) * V + d] = row[v_off + i];
    }
  }
}

// The same for bfloat16 heads of up to 256 columns (a multiple of 8) on 16-byte boundaries whose rotated halves are
// multiples of 8 too: a lane holds 8 neighbouring columns in registers (one 16-byte load, one 16-byte store), its
// partner columns i +- R/2 come from the lane R/16 further by shuffles, and the block works the cosines and sines of
// the token out once, into shared memory, for all its heads.  L lanes a head: 16 for heads of up to 128 columns (a
// warp takes two heads), else 32.  The rotation's arithmetic is that of the kernel above, operation for operation.
__device__ __forceinline__ void bf16x8_to_f(const uint4& v, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 t = __bfloat1622float2(h[j]);
    f[2 * j] = t.x;
    f[2 * j + 1] = t.y;
  }
}

template <int L>
__global__ void __launch_bounds__(RHN_WARPS * 32)
rope_headnorm_write_vec_kernel(bf16* __restrict__ proj, int stride, int k_off, int v_off, const int* __restrict__ positions,
                               const float* __restrict__ freq, int rot_dims, int norm, float eps, bf16* __restrict__ k_cache,
                               bf16* __restrict__ v_cache, const int* __restrict__ slots, int H, int G, int D, int V, int page,
                               const float* __restrict__ part, int splits) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float rhn_s[];                     // cosines [R/2], sines [R/2]
  constexpr int PER = 32 / L;                                        // heads a warp
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int sub = lane % L, which = lane / L;
  const int head = (blockIdx.y * RHN_WARPS + warp) * PER + which;
  const int c = sub * 8;                                             // this lane's first column of the head
  const bool holds = head < H + G && c < D;
  const int slot = slots != nullptr ? slots[t] : -1;
  bf16* row = proj + (size_t)t * stride;
  const int half = rot_dims / 2, hl = half / 8;
  float* cs = rhn_s;
  float* sn = rhn_s + half;
  const float pos = (float)positions[t];
  for (int i = threadIdx.x; i < half; i += blockDim.x) sincosf(pos * freq[i], sn + i, cs + i);
  // `part` set: the projection arrives unreduced, [splits, T, stride] partial sums; a column's value is their sum in
  // ascending order rounded to bfloat16, as the product's own last pass would have left it in `proj`
  const size_t split_stride = (size_t)gridDim.x * stride;
  const float* prow = part != nullptr ? part + (size_t)t * stride : nullptr;
  const int col0 = !holds ? 0 : (head < H ? head * D : k_off + (head - H) * D);
  bf16* src = row + col0 + (holds ? c : 0);
  float f[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  if (holds) {
    if (prow == nullptr) {
      bf16x8_to_f(*reinterpret_cast<const uint4*>(src), f);
    } else {
      for (int sp = 0; sp < splits; ++sp) {
        const float4* p4 = reinterpret_cast<const float4*>(prow + sp * split_stride + col0 + c);
        const float4 a = p4[0], b = p4[1];
        f[0] += a.x; f[1] += a.y; f[2] += a.z; f[3] += a.w;
        f[4] += b.x; f[5] += b.y; f[6] += b.z; f[7] += b.w;
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) f[j] = round_to<bf16>(f[j]);
    }
  }
  __syncthreads();
  // the lane that holds the other column of this lane's pairs (itself: columns that are not rotated)
  const int partner = which * L + (sub < hl ? sub + hl : (sub < 2 * hl ? sub - hl : sub));
  float g[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) g[j] = __shfl_sync(0xffffffffu, f[j], partner);
  if (sub < 2 * hl) {
    const bool low = sub < hl;                                       // holds u of (u, v); else v
    const int i0 = (low ? sub : sub - hl) * 8;
    const float4 c0 = *reinterpret_cast<const float4*>(cs + i0), c1 = *reinterpret_cast<const float4*>(cs + i0 + 4);
    const float4 s0 = *reinterpret_cast<const float4*>(sn + i0), s1 = *reinterpret_cast<const float4*>(sn + i0 + 4);
    const float cv[8] = {c0.x, c0.y, c0.z, c0.w, c1.x, c1.y, c1.z, c1.w};
    const float sv[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
#pragma unroll
    for (int j = 0; j < 8; ++j) f[j] = low ? f[j] * cv[j] - g[j] * sv[j] : f[j] * cv[j] + g[j] * sv[j];
  }
  float ss = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) ss = fmaf(f[j], f[j], ss);
#pragma unroll
  for (int o = L / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);        // (stays within the head's lanes)
  const float r = norm ? 1.f / sqrtf(ss / (float)D + eps) : 1.f;
  bf16* dst = src;
  if (head >= H) {
    dst = nullptr;
    if (slot >= 0 && holds) {
      const size_t pg = slot / page, off = slot % page;
      dst = k_cache + ((pg * G + (head - H)) * page + off) * D + c;
    }
  }
  if (holds && dst != nullptr) {
    uint4 o;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __halves2bfloat162(from_f<bf16>(f[2 * j] * r), from_f<bf16>(f[2 * j + 1] * r));
    *reinterpret_cast<uint4*>(dst) = o;
  }
  if (blockIdx.y == 0 && slot >= 0 && v_cache != nullptr) {
    const size_t pg = slot / page, off = slot % page;
    if (prow != nullptr) {
      for (int i = threadIdx.x; i < G * V; i += blockDim.x) {
        float f = 0.f;
        for (int sp = 0; sp < splits; ++sp) f += prow[sp * split_stride + v_off + i];
        const int g = i / V, d = i % V;
        v_cache[((pg * G + g) * page + off) * V + d] = from_f<bf16>(f);
      }
    } else if (V % 8 == 0 && v_off % 8 == 0 && !((uintptr_t)v_cache & 15)) {
      for (int i = threadIdx.x * 8; i < G * V; i += blockDim.x * 8) {
        const int g = i / V, d = i % V;
        *reinterpret_cast<uint4*>(v_cache + ((pg * G + g) * page + off) * V + d) = *reinterpret_cast<const uint4*>(row + v_off + i);
      }
    } else {
      for (int i = threadIdx.x; i < G * V; i += blockDim.x) {
        const int g = i / V, d = i % V;
        v_cache[((pg * G + g) * page + off) * V + d] = row[v_off + i];
      }
    }
  }
}

int threads_for_row(int n) { return n >= 2048 ? 512 : (n >= 512 ? 256 : 128); }

}  // namespace

#define TS_BY_TYPE(name, CALL)                                   \
  do {                                                           \
    if (dtype == TS_F32) { using TT = float; CALL; }             \
    else if (dtype == TS_BF16) { using TT = bf16; CALL; }        \
    else TS_REFUSE(TS_ERR_DTYPE, name ": dtype %d", dtype);      \
  } while (0)

TS_API int ts_rms_rows(void* out, const void* x, int x_stride, int col0, int n, const float* w, float eps, int T, int dtype,
                       void* stream) {
  if (T <= 0 || n <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  TS_BY_TYPE("ts_rms_rows", ts_launch(rms_rows_kernel<TT>, dim3(T), dim3(threads_for_row(n)), 0, s, (TT*)out, (const TT*)x,
                                      x_stride, col0, n, w, eps));
  TS_LAUNCH_CHECK();
}

// proj [T, stride]: q in columns [0, H D), k in [H D, (H + G) D).  slots null: nothing is cached.
TS_API int ts_qk_rownorm_write(void* proj, int stride, const float* q_w, const float* k_w, float eps, const int* positions,
                               float coef, int every, void* k_cache, void* v_cache, const int* slots, int T, int H, int G,
                               int D, int page, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (every < 1) TS_REFUSE(TS_ERR_SHAPE, "ts_qk_rownorm_write: every = %d", every);
  cudaStream_t s = (cudaStream_t)stream;
  TS_BY_TYPE("ts_qk_rownorm_write",
             ts_launch(qk_rownorm_write_kernel<TT>, dim3(T), dim3(threads_for_row(H * D)), 0, s, (TT*)proj, stride, q_w, k_w,
                       eps, positions, coef, every, (TT*)k_cache, (TT*)v_cache, slots, H, G, D, page));
  TS_LAUNCH_CHECK();
}

// proj [T, stride]: the latent in columns [col0, col0 + rank), the key part to rotate in the R columns behind it.
// k_cache [pages, 1, page, rank + R].
TS_API int ts_latent_kv_write(const void* proj, int stride, int col0, const float* w, float eps, const int* positions,
                              const float* freq, float magnitude, int rot_dims, void* k_cache, const int* slots, int T,
                              int rank, int R, int page, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (rot_dims % 2 || rot_dims > R) TS_REFUSE(TS_ERR_SHAPE, "ts_latent_kv_write: %d rotated dimensions of %d", rot_dims, R);
  cudaStream_t s = (cudaStream_t)stream;
  TS_BY_TYPE("ts_latent_kv_write",
             ts_launch(latent_kv_write_kernel<TT>, dim3(T), dim3(threads_for_row(rank)), 0, s, (const TT*)proj, stride, col0, w,
                       eps, positions, freq, magnitude, rot_dims, (TT*)k_cache, slots, rank, R, page));
  TS_LAUNCH_CHECK();
}

// dst[t, h, :R] = rotate(src[t, h, :R]); strides in elements.
TS_API int ts_rotate_pairs(void* dst, int dst_ts, int dst_hs, const void* src, int src_ts, int src_hs, const int* positions,
                           const float* freq, float magnitude, int rot_dims, int T, int H, int R, int dtype, void* stream) {
  if (T <= 0 || H <= 0 || R <= 0) return 0;
  if (rot_dims % 2 || rot_dims > R) TS_REFUSE(TS_ERR_SHAPE, "ts_rotate_pairs: %d rotated dimensions of %d", rot_dims, R);
  cudaStream_t s = (cudaStream_t)stream;
  TS_BY_TYPE("ts_rotate_pairs",
             ts_launch(rotate_pairs_kernel<TT>, dim3(T), dim3(threads_for_row(H * R / 2)), 0, s, (TT*)dst, dst_ts, dst_hs,
                       (const TT*)src, src_ts, src_hs, positions, freq, magnitude, rot_dims, H, R));
  TS_LAUNCH_CHECK();
}

// proj [T, stride]: q heads in columns [0, H D), k heads in [k_off, k_off + G D), value rows in [v_off, v_off + G V).
// freq: 32-bit [rot_dims / 2].  k_cache [pages, G, page, D], v_cache [pages, G, page, V]; slots null: nothing is cached.
// `part` (float32 [splits, T, stride], 16-byte aligned) set: the projection is still the partial sums of a product
// cut along K; the kernel sums them on the way, and of `proj` only the q columns are written.  bfloat16 rows of heads
// that are multiples of 8 wide, at most 256, with a multiple of 16 rotated dimensions only (TS_ERR_ALIGN otherwise: the
// caller finishes the product first).
TS_API int ts_rope_headnorm_write_supports_parts(int stride, int k_off, int D, int dtype) {
  return dtype == TS_BF16 && D % 8 == 0 && D <= 256 && stride % 8 == 0 && k_off % 8 == 0;
}

TS_API int ts_rope_headnorm_write(void* proj, int stride, int k_off, int v_off, const int* positions, const float* freq,
                                  int rot_dims, int norm, float eps, void* k_cache, void* v_cache, const int* slots, int T,
                                  int H, int G, int D, int V, int page, int dtype, const float* part, int splits,
                                  void* stream) {
  if (T <= 0) return 0;
  if (part != nullptr && (!ts_rope_headnorm_write_supports_parts(stride, k_off, D, dtype) || ((uintptr_t)part & 15) ||
                          ((uintptr_t)proj & 15) || ((uintptr_t)k_cache & 15) || splits < 1))
    TS_REFUSE(TS_ERR_ALIGN, "ts_rope_headnorm_write: unreduced input needs bfloat16 heads of multiples of 8 on 16-byte boundaries");
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > D) TS_REFUSE(TS_ERR_SHAPE, "ts_rope_headnorm_write: %d rotated dimensions of %d", rot_dims, D);
  if (rot_dims > 0 && freq == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_rope_headnorm_write: a rotation without frequencies");
  if (D <= 0 || D > 4096) TS_REFUSE(TS_ERR_LIMIT, "ts_rope_headnorm_write: heads of %d (limit 4096)", D);
  const int groups = ceil_div(H + G, RHN_WARPS);
  if (groups > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_rope_headnorm_write: %d heads", H + G);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = sizeof(float) * RHN_WARPS * D;
  if (smem > 48 * 1024) {
    cudaError_t e1 = cudaFuncSetAttribute(rope_headnorm_write_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    cudaError_t e2 = cudaFuncSetAttribute(rope_headnorm_write_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e1 != cudaSuccess || e2 != cudaSuccess) TS_REFUSE((int)(e1 != cudaSuccess ? e1 : e2), "ts_rope_headnorm_write: shared memory %zu", smem);
  }
  if (ts_rope_headnorm_write_supports_parts(stride, k_off, D, dtype) && rot_dims % 16 == 0 && !((uintptr_t)proj & 15) &&
      !((uintptr_t)k_cache & 15)) {
    const int per = D <= 128 ? 2 : 1;                                  // heads a warp
    const int vgroups = ceil_div(H + G, RHN_WARPS * per);
    const size_t vsmem = sizeof(float) * (rot_dims + 8);
    auto kernel = per == 2 ? rope_headnorm_write_vec_kernel<16> : rope_headnorm_write_vec_kernel<32>;
    ts_launch(kernel, dim3(T, vgroups), dim3(RHN_WARPS * 32), vsmem, s, (bf16*)proj, stride, k_off, v_off,
              positions, freq, rot_dims, norm, eps, (bf16*)k_cache, (bf16*)v_cache, slots, H, G, D, V, page, part, splits);
    TS_LAUNCH_CHECK();
  }
  if (part != nullptr) TS_REFUSE(TS_ERR_ALIGN, "ts_rope_headnorm_write: unreduced input with %d rotated dimensions", rot_dims);
  TS_BY_TYPE("ts_rope_headnorm_write",
             ts_launch(rope_headnorm_write_kernel<TT>, dim3(T, groups), dim3(RHN_WARPS * 32), smem, s, (TT*)proj, stride, k_off,
                       v_off, positions, freq, rot_dims, norm, eps, (TT*)k_cache, (TT*)v_cache, slots, H, G, D, V, page));
  TS_LAUNCH_CHECK();
}

// Rotation of NEIGHBOURING pairs (2i, 2i + 1), i < rot_dims / 2, of every q and k head by position * freq[i] (32-bit
// product, sincosf), fused with the cache write: q heads in place, k heads into the key cache, the token's value rows
// copied into the value cache.  One warp a (token, head); a lane takes whole pairs, so nothing crosses lanes.  The block
// with blockIdx.y == 0 also copies the value rows.  A slot of -1 (or slots == null) caches nothing.
template <typename T>
__global__ void __launch_bounds__(RHN_WARPS * 32)
rope_pairs_write_kernel(T* __restrict__ proj, int stride, int k_off, int v_off, const int* __restrict__ positions,
                        const float* __restrict__ freq, float magnitude, int rot_dims, T* __restrict__ k_cache,
                        T* __restrict__ v_cache, const int* __restrict__ slots, int H, int G, int D, int V, int page) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int head = blockIdx.y * RHN_WARPS + warp;
  const int slot = slots != nullptr ? slots[t] : -1;
  T* row = proj + (size_t)t * stride;
  if (head < H + G) {
    T* src = head < H ? row + (size_t)head * D : row + k_off + (size_t)(head - H) * D;
    T* dst = src;
    if (head >= H) {
      dst = nullptr;
      if (slot >= 0) {
        const size_t pg = slot / page, off = slot % page;
        dst = k_cache + ((pg * G + (head - H)) * page + off) * D;
      }
    }
    if (dst != nullptr) {
      const float pos = (float)positions[t];
      for (int i = lane; i < rot_dims / 2; i += 32) {
        float sn, cs;
        sincosf(pos * freq[i], &sn, &cs);
        sn *= magnitude;
        cs *= magnitude;
        const float u = to_f(src[2 * i]), v = to_f(src[2 * i + 1]);
        dst[2 * i] = from_f<T>(u * cs - v * sn);
        dst[2 * i + 1] = from_f<T>(v * cs + u * sn);
      }
      if (dst != src)
        for (int i = rot_dims + lane; i < D; i += 32) dst[i] = src[i];
    }
  }
  if (blockIdx.y == 0 && slot >= 0 && v_cache != nullptr) {
    const size_t pg = slot / page, off = slot % page;
    for (int i = threadIdx.x; i < G * V; i += blockDim.x) {
      const int g = i / V, d = i % V;
      v_cache[((pg * G + g) * page + off) * V + d] = row[v_off + i];
    }
  }
}

// proj [T, stride]: q heads in the columns [0, H D), k heads from k_off, value rows (G V) from v_off.
TS_API int ts_rope_pairs_write(void* proj, int stride, int k_off, int v_off, const int* positions, const float* freq,
                               float magnitude, int rot_dims, void* k_cache, void* v_cache, const int* slots, int T, int H,
                               int G, int D, int V, int page, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (rot_dims < 0 || rot_dims % 2 || rot_dims > D) TS_REFUSE(TS_ERR_SHAPE, "ts_rope_pairs_write: %d rotated dimensions of %d", rot_dims, D);
  if (rot_dims > 0 && freq == nullptr) TS_REFUSE(TS_ERR_SHAPE, "ts_rope_pairs_write: a rotation without frequencies");
  const int groups = ceil_div(H + G, RHN_WARPS);
  if (groups > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_rope_pairs_write: %d heads", H + G);
  cudaStream_t s = (cudaStream_t)stream;
  TS_BY_TYPE("ts_rope_pairs_write",
             ts_launch(rope_pairs_write_kernel<TT>, dim3(T, groups), dim3(RHN_WARPS * 32), 0, s, (TT*)proj, stride, k_off, v_off,
                       positions, freq, magnitude, rot_dims, (TT*)k_cache, (TT*)v_cache, slots, H, G, D, V, page));
  TS_LAUNCH_CHECK();
}

// out[t, h, :N] = w[h] (N x K) . x[t, h, :K]; w [H, N, K] contiguous; strides in elements.
TS_API int ts_batched_linear(void* out, int out_ts, int out_hs, const void* x, int x_ts, int x_hs, const void* w, int T, int H,
                             int N, int K, int dtype, void* stream) {
  if (T <= 0 || H <= 0 || N <= 0) return 0;
  if (K <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_batched_linear: K = %d", K);
  dim3 grid(ceil_div(N, BL_N), ceil_div(T, BL_M), H);
  if (grid.y > 65535 || H > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_batched_linear: %d rows / %d heads per launch", T, H);
  cudaStream_t s = (cudaStream_t)stream;
  const int per = dtype == TS_F32 ? 4 : 8;
  if (T <= 2 * BLR_ROWS && K % per == 0 && x_ts % per == 0 && x_hs % per == 0 && !((uintptr_t)x & 15) && !((uintptr_t)w & 15)) {
    dim3 rows_grid(ceil_div(N, BLR_WARPS), H);
    TS_BY_TYPE("ts_batched_linear",
               ts_launch(batched_linear_rows_kernel<TT>, dim3(rows_grid), dim3(BLR_WARPS * 32), 0, s, (TT*)out, out_ts, out_hs,
                         (const TT*)x, x_ts, x_hs, (const TT*)w, T, N, K));
    TS_LAUNCH_CHECK();
  }
  TS_BY_TYPE("ts_batched_linear",
             ts_launch(batched_linear_kernel<TT>, dim3(grid), dim3(256), 0, s, (TT*)out, out_ts, out_hs, (const TT*)x, x_ts, x_hs,
                       (const TT*)w, T, N, K));
  TS_LAUNCH_CHECK();
}
