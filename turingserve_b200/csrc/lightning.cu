// Linear attention with a per-head decay ("lightning attention"): for every request and head a matrix
// state S [D, V] in 32-bit that lives in a state slot between steps,
//     S_t = lam_h S_{t-1} + k_t v_t^T,     o_t = S_t^T q_t,
// with q, k, v = act(projection) taken from one fused projection row [q (H D) | k (H D) | v (H V) | ...].
// The activation (SiLU) is applied here, rounded to the storage type as the projection's own epilogue
// would round it; everything from there on (products with the state, decay, the state itself, the
// output) is 32-bit.  Output: 32-bit rows [T, H V] (a norm over all heads follows in another kernel).
//
// ts_lightning runs the tokens of a step in order, exactly as written above, for single tokens and for
// portions alike, so how a prompt is cut never changes a bit.  The columns of S are independent of one
// another: one block owns LT_COLS columns of one (head, request) and keeps them in REGISTERS over all tokens
// of the step: thread (part, col) holds rows part * LT_ROWS .. of column col.  Tokens arrive in groups of
// LT_GROUP rows: the raw projection rows of the NEXT group are on their way (cp.async, 16 bytes a copy) while
// the present group is computed; a group is activated out of the raw buffer into 32-bit shared memory; its
// partial outputs of the row parts are summed through shared memory, in part order.  Per token a thread does
// 3 * LT_ROWS 32-bit operations on registers with broadcast loads from shared memory.
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int LT_GROUP = 16;     // tokens staged at a time
constexpr int LT_COLS = 16;      // state columns per block (half a warp: a warp holds two row parts)
constexpr int LT_ROWS = 8;       // state rows per thread (registers)

template <typename T> __device__ __forceinline__ float act_silu(float z) { return round_to<T>(silu_for<T>(z)); }

// PLAN: an instance of its own for long portions (its per-thread plan of copies and activations costs 60 registers more,
// which would halve the blocks an SM holds in single-token steps)
template <typename T, bool PLAN>
__global__ void __launch_bounds__(512)
lightning_kernel(float* __restrict__ out, const T* __restrict__ proj, int proj_stride, float* __restrict__ state,
                 const float* __restrict__ decay, const int* __restrict__ q_start, const int* __restrict__ slots,
                 int H, int D, int V, int parts, int fast_rows) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int h = blockIdx.y, b = blockIdx.z;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  const int Dp = parts * LT_ROWS;                          // D rounded up: rows beyond D hold zero keys and queries
  const int col = threadIdx.x & (LT_COLS - 1), part = threadIdx.x / LT_COLS;
  const int j = blockIdx.x * LT_COLS + col;
  const bool live = j < V;
  const float lam = decay[h];
  float* S = state + ((size_t)slots[b] * H + h) * D * V;
  float* q_s = smem;                                       // [LT_GROUP][Dp]
  float* k_s = q_s + LT_GROUP * Dp;                        // [LT_GROUP][Dp]
  float* v_s = k_s + LT_GROUP * Dp;                        // [LT_GROUP][LT_COLS]
  float* o_s = v_s + LT_GROUP * LT_COLS;                   // [LT_GROUP][parts][LT_COLS]

  float s[LT_ROWS];
#pragma unroll
  for (int i = 0; i < LT_ROWS; ++i) {
    const int d = part * LT_ROWS + i;
    s[i] = (live && d < D) ? S[(size_t)d * V + j] : 0.f;
  }
  const int q_off = h * D, k_off = H * D + h * D, v_off = 2 * H * D + h * V;
  // raw rows of a group, as stored: [2 buffers][LT_GROUP][D q | D k | LT_COLS v] (fast_rows: D a multiple of 8 and
  // every piece 16-byte aligned, so the copies are asynchronous 16-byte ones; else plain loads at activation)
  T* raw = reinterpret_cast<T*>(o_s + LT_GROUP * parts * LT_COLS);
  const int raw_row = 2 * D + LT_COLS;
  const int cols_here = min(LT_COLS, V - (int)blockIdx.x * LT_COLS);
  constexpr int PER16 = 16 / (int)sizeof(T);
  // Which pieces of a group a thread copies, and which it activates, is the same for every group: with PLAN (long
  // portions) both are worked out once instead of by two divisions a piece and group.  At most LT_MAX_COPIES 16-byte
  // copies a thread (16 rows of 2 D / PER16 + LT_COLS / PER16 pieces over 2 D threads) and LT_MAX_ACT pieces to activate.
  constexpr int LT_MAX_COPIES = 8, LT_MAX_ACT = 4;
  int cp_row[LT_MAX_COPIES], cp_src[LT_MAX_COPIES], cp_dst[LT_MAX_COPIES];
  int ac_row[LT_MAX_ACT], ac_src[LT_MAX_ACT], ac_dst[LT_MAX_ACT];
  const bool planned = PLAN && fast_rows;
  if (planned) {
    const int chunks_qk = D / PER16, chunks_v = LT_COLS / PER16, per_row = 2 * chunks_qk + chunks_v;
#pragma unroll
    for (int k = 0; k < LT_MAX_COPIES; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      cp_row[k] = LT_GROUP;                                // (beyond every group: never copied)
      cp_src[k] = cp_dst[k] = 0;
      if (i < LT_GROUP * per_row) {
        const int r = i / per_row, c = i % per_row;
        if (c < chunks_qk) {
          cp_row[k] = r;
          cp_src[k] = r * proj_stride + q_off + c * PER16;
          cp_dst[k] = r * raw_row + c * PER16;
        } else if (c < 2 * chunks_qk) {
          cp_row[k] = r;
          cp_src[k] = r * proj_stride + k_off + (c - chunks_qk) * PER16;
          cp_dst[k] = r * raw_row + D + (c - chunks_qk) * PER16;
        } else if ((c - 2 * chunks_qk) * PER16 < cols_here) {
          cp_row[k] = r;
          cp_src[k] = r * proj_stride + v_off + blockIdx.x * LT_COLS + (c - 2 * chunks_qk) * PER16;
          cp_dst[k] = r * raw_row + 2 * D + (c - 2 * chunks_qk) * PER16;
        }
      }
    }
#pragma unroll
    for (int k = 0; k < LT_MAX_ACT; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      ac_row[k] = LT_GROUP;
      ac_src[k] = ac_dst[k] = 0;
      if (i < LT_GROUP * 2 * chunks_qk) {
        const int r = i / (2 * chunks_qk), c = i % (2 * chunks_qk);
        const int which = c >= chunks_qk, cc = (which ? c - chunks_qk : c) * PER16;
        ac_row[k] = r;
        ac_src[k] = r * raw_row + which * D + cc;
        ac_dst[k] = which * LT_GROUP * Dp + r * Dp + cc;   // (k_s lies LT_GROUP * Dp behind q_s)
      }
    }
  }
  auto fetch = [&](int g0, int buf) {
    if (!fast_rows) return;
    if (planned) {
      const int gn = min(LT_GROUP, n - g0);
      const T* first = proj + (size_t)(t0 + g0) * proj_stride;
      T* dst0 = raw + (size_t)buf * LT_GROUP * raw_row;
#pragma unroll
      for (int k = 0; k < LT_MAX_COPIES; ++k)
        if (cp_row[k] < gn) cp_async_16(dst0 + cp_dst[k], first + cp_src[k], true);
      return;
    }
    const int gn = min(LT_GROUP, n - g0);
    const int chunks_qk = D / PER16, chunks_v = LT_COLS / PER16, per_row = 2 * chunks_qk + chunks_v;
    for (int i = threadIdx.x; i < gn * per_row; i += blockDim.x) {
      const int r = i / per_row, c = i % per_row;
      const T* row = proj + (size_t)(t0 + g0 + r) * proj_stride;
      T* dst = raw + ((size_t)buf * LT_GROUP + r) * raw_row;
      if (c < chunks_qk) cp_async_16(dst + c * PER16, row + q_off + c * PER16, true);
      else if (c < 2 * chunks_qk) cp_async_16(dst + D + (c - chunks_qk) * PER16, row + k_off + (c - chunks_qk) * PER16, true);
      else {
        const int cc = (c - 2 * chunks_qk) * PER16;
        const bool ok = cc < cols_here;
        cp_async_16(dst + 2 * D + cc, ok ? row + v_off + blockIdx.x * LT_COLS + cc : proj, ok);
      }
    }
  };
  for (int i = threadIdx.x; i < 2 * LT_GROUP * Dp; i += blockDim.x) q_s[i] = 0.f;      // (q_s and k_s: rows beyond D stay zero)
  fetch(0, 0);
  cp_async_commit();
  int buf = 0;
  for (int g0 = 0; g0 < n; g0 += LT_GROUP, buf ^= 1) {
    const int gn = min(LT_GROUP, n - g0);
    if (g0 + LT_GROUP < n) fetch(g0 + LT_GROUP, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                       // this group's raw rows are here; the group before is stored
    if (planned) {
      const T* raw0 = raw + (size_t)buf * LT_GROUP * raw_row;
#pragma unroll
      for (int k = 0; k < LT_MAX_ACT; ++k) {
        if (ac_row[k] < gn) {
          const uint4 rawv = *reinterpret_cast<const uint4*>(raw0 + ac_src[k]);
          const T* e = reinterpret_cast<const T*>(&rawv);
          float* dst = q_s + ac_dst[k];
#pragma unroll
          for (int u = 0; u < PER16; ++u) dst[u] = act_silu<T>(to_f(e[u]));
        }
      }
    } else if (fast_rows) {
      // 16 bytes (PER16 values) of q or k at a time: the index arithmetic once a piece, not once a value
      const int chunks = D / PER16;
      for (int i = threadIdx.x; i < gn * 2 * chunks; i += blockDim.x) {
        const int r = i / (2 * chunks), c = i % (2 * chunks);
        const int which = c >= chunks, cc = (which ? c - chunks : c) * PER16;
        const uint4 rawv = *reinterpret_cast<const uint4*>(raw + ((size_t)buf * LT_GROUP + r) * raw_row + which * D + cc);
        const T* e = reinterpret_cast<const T*>(&rawv);
        float* dst = (which ? k_s : q_s) + r * Dp + cc;
#pragma unroll
        for (int u = 0; u < PER16; ++u) dst[u] = act_silu<T>(to_f(e[u]));
      }
    } else {
      for (int i = threadIdx.x; i < gn * D; i += blockDim.x) {
        const int r = i / D, d = i % D;
        const T* row = proj + (size_t)(t0 + g0 + r) * proj_stride;
        q_s[r * Dp + d] = act_silu<T>(to_f(row[q_off + d]));
        k_s[r * Dp + d] = act_silu<T>(to_f(row[k_off + d]));
      }
    }
    for (int i = threadIdx.x; i < gn * LT_COLS; i += blockDim.x) {
      const int r = i / LT_COLS, c = i % LT_COLS;
      float vv = 0.f;
      if (c < cols_here) {
        vv = fast_rows ? to_f(raw[((size_t)buf * LT_GROUP + r) * raw_row + 2 * D + c])
                       : to_f(proj[(size_t)(t0 + g0 + r) * proj_stride + v_off + blockIdx.x * LT_COLS + c]);
        vv = act_silu<T>(vv);
      }
      v_s[i] = vv;
    }
    __syncthreads();
#pragma unroll 2
    for (int r = 0; r < gn; ++r) {
      const float vj = v_s[r * LT_COLS + col];
      const float4* qr = reinterpret_cast<const float4*>(q_s + r * Dp + part * LT_ROWS);
      const float4* kr = reinterpret_cast<const float4*>(k_s + r * Dp + part * LT_ROWS);
      float o = 0.f, o2 = 0.f;                                 // two chains of four instead of one of eight
#pragma unroll
      for (int i = 0; i < LT_ROWS / 4; ++i) {
        const float4 k4 = kr[i], q4 = qr[i];
        s[4 * i + 0] = fmaf(lam, s[4 * i + 0], k4.x * vj);
        o = fmaf(s[4 * i + 0], q4.x, o);
        s[4 * i + 1] = fmaf(lam, s[4 * i + 1], k4.y * vj);
        o2 = fmaf(s[4 * i + 1], q4.y, o2);
        s[4 * i + 2] = fmaf(lam, s[4 * i + 2], k4.z * vj);
        o = fmaf(s[4 * i + 2], q4.z, o);
        s[4 * i + 3] = fmaf(lam, s[4 * i + 3], k4.w * vj);
        o2 = fmaf(s[4 * i + 3], q4.w, o2);
      }
      o_s[(r * parts + part) * LT_COLS + col] = o + o2;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < gn * LT_COLS; i += blockDim.x) {
      const int r = i / LT_COLS, c = i % LT_COLS;
      const int jj = blockIdx.x * LT_COLS + c;
      if (jj >= V) continue;
      float o = 0.f;
      for (int p = 0; p < parts; ++p) o += o_s[(r * parts + p) * LT_COLS + c];
      out[(size_t)(t0 + g0 + r) * H * V + h * V + jj] = o;
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < LT_ROWS; ++i) {
    const int d = part * LT_ROWS + i;
    if (live && d < D) S[(size_t)d * V + j] = s[i];
  }
}

}  // namespace

// proj: [T, proj_stride] rows holding q at column 0, k at H D, v at 2 H D.  state: [slots, H, D, V] 32-bit.
// decay: [H] 32-bit on the device.  out: [T, H V] 32-bit.
// longest: the most tokens a request brings (0: not known); from LT_LATE_TOKENS on the kernel is launched late (see
// ts_launch_late).
constexpr int LT_LATE_TOKENS = 64;

TS_API int ts_lightning_ex(float* out, const void* proj, int proj_stride, float* state, const float* decay,
                           const int* q_start, const int* slots, int B, int H, int D, int V, int longest, int dtype,
                           void* stream);

TS_API int ts_lightning(float* out, const void* proj, int proj_stride, float* state, const float* decay,
                        const int* q_start, const int* slots, int B, int H, int D, int V, int dtype, void* stream) {
  return ts_lightning_ex(out, proj, proj_stride, state, decay, q_start, slots, B, H, D, V, 0, dtype, stream);
}

TS_API int ts_lightning_ex(float* out, const void* proj, int proj_stride, float* state, const float* decay,
                           const int* q_start, const int* slots, int B, int H, int D, int V, int longest, int dtype,
                           void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || D <= 0 || V <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_lightning: %d heads of %d x %d", H, D, V);
  const int parts = ceil_div(D, LT_ROWS);
  if (parts * LT_COLS > 512) TS_REFUSE(TS_ERR_LIMIT, "ts_lightning: keys of %d (limit %d)", D, 512 / LT_COLS * LT_ROWS);
  if (B > 65535 || H > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_lightning: %d requests / %d heads per launch", B, H);
  cudaStream_t s = (cudaStream_t)stream;
  const int elem = dtype == TS_F32 ? 4 : 2, per16 = 16 / elem;
  // asynchronous 16-byte copies of the raw rows: every piece of a row (q, k, this block's v columns) must start on
  // a 16-byte boundary in global and in shared memory
  const int fast_rows = D % per16 == 0 && V % per16 == 0 && proj_stride % per16 == 0 && !((uintptr_t)proj & 15);
  const size_t smem = sizeof(float) * LT_GROUP * ((size_t)2 * parts * LT_ROWS + LT_COLS + (size_t)parts * LT_COLS) +
                      (size_t)2 * LT_GROUP * (2 * D + LT_COLS) * elem;
  dim3 grid(ceil_div(V, LT_COLS), H, B);
#define TS_LT(TT)                                                                                                   \
  do {                                                                                                              \
    static size_t configured = 0;                                                                                   \
    if (smem > 48 * 1024 && smem > configured) {                                                                    \
      cudaError_t e = cudaFuncSetAttribute(lightning_kernel<TT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                                         \
        e = cudaFuncSetAttribute(lightning_kernel<TT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e != cudaSuccess) TS_REFUSE((int)e, "ts_lightning: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
      configured = smem;                                                                                            \
    }                                                                                                               \
    if (longest >= LT_LATE_TOKENS)                                                                                  \
      ts_launch_late(lightning_kernel<TT, true>, dim3(grid), dim3(parts * LT_COLS), smem, s, out, (const TT*)proj, proj_stride, \
                     state, decay, q_start, slots, H, D, V, parts, fast_rows);                                      \
    else                                                                                                            \
      ts_launch(lightning_kernel<TT, false>, dim3(grid), dim3(parts * LT_COLS), smem, s, out, (const TT*)proj, proj_stride, \
                state, decay, q_start, slots, H, D, V, parts, fast_rows);                                           \
  } while (0)
  if (dtype == TS_F32) TS_LT(float);
  else if (dtype == TS_BF16) TS_LT(bf16);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_lightning: dtype %d", dtype);
#undef TS_LT
  TS_LAUNCH_CHECK();
}
