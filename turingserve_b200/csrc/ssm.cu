// Selective state-space mixer (the "state-space duality" form with a scalar decay per head): for every request and
// head a matrix state S [N, P] in 32-bit that lives in a state slot between steps.  Per token, with the step size
// dt_h > 0, the decay a_h = exp(-exp(A_h) dt_h), an input row B and a read-out row C (N wide, shared by the heads
// of a group) and the head's input x (P wide):
//     S <- a S + dt B x^T,        y = S^T C + D_h x.
// x, B and C are columns of one fused projection after a causal filter of a few taps per channel (with bias) and
// SiLU; the filter's last taps - 1 inputs are kept behind S in the same slot: [H N P | (taps - 1) x Cn],
// Cn = H P + 2 G N.  The projection row is [z (H P) | x (H P) | B (G N) | C (G N) | dt (H)]; z is a gate that a
// later kernel uses.
//
// Two kernels:
//   ts_ssm_prepare   filter + SiLU of every channel, dt = softplus(dt + dt_bias), a; 32-bit rows
//                    [x | B | C | dt (H) | a (H)]; reads the slot's filter inputs for the tokens before the step's
//                    first, writes nothing to the slot
//   ts_ssm_scan      the recurrence, token by token for portions and single tokens alike (cutting a prompt changes no
//                    bit); one block owns SS_COLS columns of one (head, request) state and keeps them in registers
//                    (SS_ROWS rows a thread); the next group's rows arrive by cp.async while the present one is
//                    computed; afterwards one block of the request stores the filter's new last inputs
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int SS_GROUP = 16;     // tokens staged at a time
constexpr int SS_COLS = 16;      // state columns per block
constexpr int SS_ROWS = 8;       // state rows per thread (registers)
constexpr int SS_MAX_TAPS = 8;

__device__ __forceinline__ void ss_cp_async_4(void* smem, const void* gmem) {
  const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ float ss_softplus(float x) { return x > 20.f ? x : log1pf(expf(x)); }

// grid (ceil(T / SS_PREP_TOKENS), ceil((Cn + H) / blockDim)): a thread takes one channel (or one head's dt and a) of
// SS_PREP_TOKENS neighbouring tokens.  The tokens' raw inputs are all loaded before the first is used; the filter's
// window slides through registers, and is refilled (from the rows before, or from the slot's memory where they lie before
// the step's first token) only at the first token of the thread and where another request begins.
constexpr int SS_PREP_TOKENS = 8;

// (SS_PREP_TOKENS_ = 1 for steps of few tokens, where every token is likely a request of its own and the launch has
// few threads as it is; the arithmetic of a token is the same in both instances, bit for bit)
template <typename T, int SS_PREP_TOKENS_>
__global__ void __launch_bounds__(256)
ssm_prepare_kernel(float* __restrict__ ready, const T* __restrict__ proj, int proj_stride, int xbc_off, int dt_off,
                   const float* __restrict__ conv_w, const float* __restrict__ conv_b, const float* __restrict__ a_log,
                   const float* __restrict__ dt_bias, const float* __restrict__ state, size_t state_stride,
                   size_t tail_off, const int* __restrict__ token_request, const int* __restrict__ q_start,
                   const int* __restrict__ slots, int T_, int H, int Cn, int taps) {
  pdl_launch_dependents();
  pdl_wait();
  const int t_base = blockIdx.x * SS_PREP_TOKENS_;
  const int c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= Cn + H) return;
  const int W = Cn + 2 * H;
  const int count = min(SS_PREP_TOKENS_, T_ - t_base);
  if (c >= Cn) {
    const int h = c - Cn;
    const float bias = dt_bias[h], rate = expf(a_log[h]);
    for (int k = 0; k < count; ++k) {
      const int t = t_base + k;
      const float dt = ss_softplus(to_f(proj[(size_t)t * proj_stride + dt_off + h]) + bias);
      ready[(size_t)t * W + Cn + h] = dt;
      ready[(size_t)t * W + Cn + H + h] = expf(-rate * dt);
    }
    return;
  }
  float x[SS_PREP_TOKENS_];
#pragma unroll
  for (int k = 0; k < SS_PREP_TOKENS_; ++k)
    x[k] = k < count ? to_f(proj[(size_t)(t_base + k) * proj_stride + xbc_off + c]) : 0.f;
  float wgt[SS_MAX_TAPS];
#pragma unroll
  for (int u = 0; u < SS_MAX_TAPS; ++u) wgt[u] = u < taps ? conv_w[c * taps + u] : 0.f;
  const float bias = conv_b != nullptr ? conv_b[c] : 0.f;
  const int keep = taps - 1;
  float win[SS_MAX_TAPS - 1];                          // the inputs before the present token, oldest first (keep of them)
#pragma unroll
  for (int k = 0; k < SS_PREP_TOKENS_; ++k) {
    if (k < count) {
      const int t = t_base + k;
      const int b = token_request[t];
      const int t0 = q_start[b], i = t - t0;
      if (k == 0 || i == 0) {
        const float* tail = state + (size_t)slots[b] * state_stride + tail_off;       // [taps - 1][Cn]
#pragma unroll
        for (int u = 0; u < SS_MAX_TAPS - 1; ++u) {
          if (u < keep) {
            const int rel = i - keep + u;              // the input's place, counted from the step's first token
            win[u] = rel >= 0 ? to_f(proj[(size_t)(t0 + rel) * proj_stride + xbc_off + c]) : tail[(size_t)(rel + keep) * Cn + c];
          }
        }
      }
      float acc = bias;
#pragma unroll
      for (int u = 0; u < SS_MAX_TAPS - 1; ++u)
        if (u < keep) acc = fmaf(wgt[u], win[u], acc);
      // (the present token's weight is the last of its taps; the index is not known at compile time)
      float w_now = wgt[0];
#pragma unroll
      for (int u = 1; u < SS_MAX_TAPS; ++u)
        if (u == keep) w_now = wgt[u];
      acc = fmaf(w_now, x[k], acc);
      ready[(size_t)t * W + c] = acc / (1.f + expf(-acc));
#pragma unroll
      for (int u = 0; u < SS_MAX_TAPS - 2; ++u)
        if (u + 1 < keep) win[u] = win[u + 1];
#pragma unroll
      for (int u = 0; u < SS_MAX_TAPS - 1; ++u)
        if (u == keep - 1) win[u] = x[k];
    }
  }
}

// PLAN: an instance of its own for long portions (its per-thread copy plan costs 60 registers more, which would halve the
// blocks an SM holds in single-token steps: 51 -> 59 us at 112 heads)
template <typename T, bool PLAN>
__global__ void __launch_bounds__(512)
ssm_scan_kernel(float* __restrict__ out, const float* __restrict__ ready, const T* __restrict__ proj, int proj_stride,
                int xbc_off, float* __restrict__ state, size_t state_stride, const float* __restrict__ skip,
                const int* __restrict__ q_start, const int* __restrict__ slots, int H, int G, int N, int P, int taps,
                int parts, int vec4) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ __align__(16) float smem[];
  const int h = blockIdx.y, b = blockIdx.z;
  const int t0 = q_start[b], n = q_start[b + 1] - t0;
  if (n <= 0) return;
  const int g = h / (H / G);
  const int inner = H * P, GN = G * N, Cn = inner + 2 * GN, W = Cn + 2 * H;
  const int Np = parts * SS_ROWS;                          // N rounded up: rows beyond N hold zero B and C
  const int col = threadIdx.x & (SS_COLS - 1), part = threadIdx.x / SS_COLS;
  const int j = blockIdx.x * SS_COLS + col;
  const bool live = j < P;
  float* base = state + (size_t)slots[b] * state_stride;
  float* S = base + (size_t)h * N * P;
  const int stage = SS_GROUP * (2 * Np + SS_COLS + 4);     // floats of one staged group: B | C | x | (dt, a) pairs (+ pad)
  float* o_s = smem + 2 * stage;                           // [SS_GROUP][parts][SS_COLS]
  const int cols_here = min(SS_COLS, P - (int)blockIdx.x * SS_COLS);

  float s[SS_ROWS];
#pragma unroll
  for (int i = 0; i < SS_ROWS; ++i) {
    const int d = part * SS_ROWS + i;
    s[i] = (live && d < N) ? S[(size_t)d * P + j] : 0.f;
  }
  for (int i = threadIdx.x; i < 2 * stage; i += blockDim.x) smem[i] = 0.f;     // (what no copy writes stays zero)
  __syncthreads();

  // Which pieces of a group a thread copies is the same for every group: with PLAN (long portions) it is worked out
  // once (the divisions of the index by the pieces a row would otherwise cost more instructions a group than the copies
  // themselves; for a single token the plan itself is what costs: 28.7 -> 36.9 us).  16-byte pieces: at most
  // SS_MAX_COPIES a thread (16 rows of N / 2 + 4 pieces over 16 ceil(N / 8) threads).
  constexpr int SS_MAX_COPIES = 8;
  int cp_row[SS_MAX_COPIES], cp_src[SS_MAX_COPIES], cp_dst[SS_MAX_COPIES];
  if (PLAN && vec4) {
    const int nb = N / 4, nx = cols_here / 4, per_row = 2 * nb + nx;
#pragma unroll
    for (int k = 0; k < SS_MAX_COPIES; ++k) {
      const int i = threadIdx.x + k * blockDim.x;
      cp_row[k] = SS_GROUP;                                // (beyond every group: never copied)
      cp_src[k] = cp_dst[k] = 0;
      if (i < SS_GROUP * per_row) {
        const int r = i / per_row, c = i % per_row;
        cp_row[k] = r;
        if (c < nb) {
          cp_src[k] = r * W + inner + g * N + 4 * c;
          cp_dst[k] = r * Np + 4 * c;
        } else if (c < 2 * nb) {
          cp_src[k] = r * W + inner + GN + g * N + 4 * (c - nb);
          cp_dst[k] = SS_GROUP * Np + r * Np + 4 * (c - nb);
        } else {
          cp_src[k] = r * W + h * P + blockIdx.x * SS_COLS + 4 * (c - 2 * nb);
          cp_dst[k] = 2 * SS_GROUP * Np + r * SS_COLS + 4 * (c - 2 * nb);
        }
      }
    }
  }
  auto fetch = [&](int g0, int buf) {
    const int gn = min(SS_GROUP, n - g0);
    float* Bs = smem + (size_t)buf * stage;
    float* Cs = Bs + SS_GROUP * Np;
    float* xs = Cs + SS_GROUP * Np;
    float* da = xs + SS_GROUP * SS_COLS;
    if (PLAN && vec4) {
      const float* first = ready + (size_t)(t0 + g0) * W;
#pragma unroll
      for (int k = 0; k < SS_MAX_COPIES; ++k)
        if (cp_row[k] < gn) cp_async_16(Bs + cp_dst[k], first + cp_src[k], true);
    } else if (vec4) {
      const int nb = N / 4, nx = cols_here / 4, per_row = 2 * nb + nx;
      for (int i = threadIdx.x; i < gn * per_row; i += blockDim.x) {
        const int r = i / per_row, c = i % per_row;
        const float* row = ready + (size_t)(t0 + g0 + r) * W;
        if (c < nb) cp_async_16(Bs + r * Np + 4 * c, row + inner + g * N + 4 * c, true);
        else if (c < 2 * nb) cp_async_16(Cs + r * Np + 4 * (c - nb), row + inner + GN + g * N + 4 * (c - nb), true);
        else cp_async_16(xs + r * SS_COLS + 4 * (c - 2 * nb), row + h * P + blockIdx.x * SS_COLS + 4 * (c - 2 * nb), true);
      }
    } else {
      const int per_row = 2 * N + cols_here;
      for (int i = threadIdx.x; i < gn * per_row; i += blockDim.x) {
        const int r = i / per_row, c = i % per_row;
        const float* row = ready + (size_t)(t0 + g0 + r) * W;
        if (c < N) ss_cp_async_4(Bs + r * Np + c, row + inner + g * N + c);
        else if (c < 2 * N) ss_cp_async_4(Cs + r * Np + (c - N), row + inner + GN + g * N + (c - N));
        else ss_cp_async_4(xs + r * SS_COLS + (c - 2 * N), row + h * P + blockIdx.x * SS_COLS + (c - 2 * N));
      }
    }
    for (int i = threadIdx.x; i < 2 * gn; i += blockDim.x) {
      const int r = i >> 1, which = i & 1;
      ss_cp_async_4(da + i, ready + (size_t)(t0 + g0 + r) * W + Cn + which * H + h);
    }
  };

  const float dskip = skip != nullptr ? skip[h] : 0.f;
  fetch(0, 0);
  cp_async_commit();
  int buf = 0;
  for (int g0 = 0; g0 < n; g0 += SS_GROUP, buf ^= 1) {
    const int gn = min(SS_GROUP, n - g0);
    if (g0 + SS_GROUP < n) fetch(g0 + SS_GROUP, buf ^ 1);
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                       // this group's rows are here; the group before is stored
    const float* Bs = smem + (size_t)buf * stage;
    const float* Cs = Bs + SS_GROUP * Np;
    const float* xs = Cs + SS_GROUP * Np;
    const float* da = xs + SS_GROUP * SS_COLS;
#pragma unroll 2
    for (int r = 0; r < gn; ++r) {
      const float dt = da[2 * r], a = da[2 * r + 1];
      const float xv = xs[r * SS_COLS + col];
      const float kx = dt * xv;
      const float4* br = reinterpret_cast<const float4*>(Bs + r * Np + part * SS_ROWS);
      const float4* cr = reinterpret_cast<const float4*>(Cs + r * Np + part * SS_ROWS);
      float o = 0.f, o2 = 0.f;                             // two chains of four instead of one of eight
#pragma unroll
      for (int i = 0; i < SS_ROWS / 4; ++i) {
        const float4 b4 = br[i], c4 = cr[i];
        s[4 * i + 0] = fmaf(a, s[4 * i + 0], b4.x * kx);
        o = fmaf(s[4 * i + 0], c4.x, o);
        s[4 * i + 1] = fmaf(a, s[4 * i + 1], b4.y * kx);
        o2 = fmaf(s[4 * i + 1], c4.y, o2);
        s[4 * i + 2] = fmaf(a, s[4 * i + 2], b4.z * kx);
        o = fmaf(s[4 * i + 2], c4.z, o);
        s[4 * i + 3] = fmaf(a, s[4 * i + 3], b4.w * kx);
        o2 = fmaf(s[4 * i + 3], c4.w, o2);
      }
      // (the skip term rides with part 0: the loop below reads nothing of the staged rows, which the next group's
      // copies may already be writing over)
      o_s[(r * parts + part) * SS_COLS + col] = o + o2 + (part == 0 ? dskip * xv : 0.f);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < gn * SS_COLS; i += blockDim.x) {
      const int r = i / SS_COLS, c = i % SS_COLS;
      const int jj = blockIdx.x * SS_COLS + c;
      if (jj >= P) continue;
      float o = 0.f;
      for (int p = 0; p < parts; ++p) o += o_s[(r * parts + p) * SS_COLS + c];
      out[(size_t)(t0 + g0 + r) * inner + h * P + jj] = o;
    }
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < SS_ROWS; ++i) {
    const int d = part * SS_ROWS + i;
    if (live && d < N) S[(size_t)d * P + j] = s[i];
  }
  // the filter's new last inputs: the step's last taps - 1 raw rows, or, of a step shorter than that, the old ones
  // moved up (a thread reads all it needs of a channel before it writes that channel)
  if (blockIdx.x == 0 && h == 0 && taps > 1) {
    float* tail = base + (size_t)H * N * P;
    const int keep = taps - 1;
    for (int c = threadIdx.x; c < Cn; c += blockDim.x) {
      float v[SS_MAX_TAPS];
#pragma unroll
      for (int r = 0; r < SS_MAX_TAPS - 1; ++r) {
        if (r < keep) {
          const int rel = n - keep + r;
          v[r] = rel >= 0 ? to_f(proj[(size_t)(t0 + rel) * proj_stride + xbc_off + c]) : tail[(size_t)(rel + keep) * Cn + c];
        }
      }
#pragma unroll
      for (int r = 0; r < SS_MAX_TAPS - 1; ++r)
        if (r < keep) tail[(size_t)r * Cn + c] = v[r];
    }
  }
}

}  // namespace

// proj [T, proj_stride]: the filtered channels [x | B | C] (Cn = H P + 2 G N) from column xbc_off, dt (H) from column
// dt_off.  conv_w [Cn, taps], conv_b [Cn] (may be null), a_log, dt_bias [H]: 32-bit.  state [slots, state_stride]
// 32-bit, the filter's inputs from tail_off within a slot.  ready [T, Cn + 2 H] 32-bit.
TS_API int ts_ssm_prepare(float* ready, const void* proj, int proj_stride, int xbc_off, int dt_off, const float* conv_w,
                          const float* conv_b, const float* a_log, const float* dt_bias, const float* state,
                          long long state_stride, long long tail_off, const int* token_request, const int* q_start,
                          const int* slots, int T, int H, int Cn, int taps, int dtype, void* stream) {
  if (T <= 0) return 0;
  if (taps < 1 || taps > SS_MAX_TAPS) TS_REFUSE(TS_ERR_LIMIT, "ts_ssm_prepare: a filter of %d taps (1 to %d)", taps, SS_MAX_TAPS);
  cudaStream_t s = (cudaStream_t)stream;
  const bool few = T <= 64;
  dim3 grid(few ? T : ceil_div(T, SS_PREP_TOKENS), ceil_div(Cn + H, 256));
  if (grid.y > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_ssm_prepare: %d channels", Cn);
#define TS_SP1(TT, N)                                                                                                 \
  ts_launch(ssm_prepare_kernel<TT, N>, grid, dim3(256), 0, s, ready, (const TT*)proj, proj_stride, xbc_off, dt_off, conv_w, \
            conv_b, a_log, dt_bias, state, (size_t)state_stride, (size_t)tail_off, token_request, q_start, slots, T, H, Cn, taps)
#define TS_SP(TT)                     \
  do {                                \
    if (few) TS_SP1(TT, 1);           \
    else TS_SP1(TT, SS_PREP_TOKENS);  \
  } while (0)
  if (dtype == TS_F32) TS_SP(float);
  else if (dtype == TS_BF16) TS_SP(bf16);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_ssm_prepare: dtype %d", dtype);
#undef TS_SP
#undef TS_SP1
  TS_LAUNCH_CHECK();
}

// out [T, H P] 32-bit; ready as ts_ssm_prepare left it; skip [H] 32-bit (D, may be null); state [slots, state_stride]:
// [H N P | (taps - 1) x Cn], read and left updated at each request's slot.
// longest: the most tokens a request brings (0: not known); from SS_LATE_TOKENS on the kernel is launched late (see
// ts_launch_late).
constexpr int SS_LATE_TOKENS = 64;

TS_API int ts_ssm_scan(float* out, const float* ready, const void* proj, int proj_stride, int xbc_off, float* state,
                       long long state_stride, const float* skip, const int* q_start, const int* slots, int B, int H,
                       int G, int N, int P, int taps, int longest, int dtype, void* stream) {
  if (B <= 0) return 0;
  if (H <= 0 || G <= 0 || H % G || N <= 0 || P <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_ssm_scan: %d heads in %d groups, state %d x %d", H, G, N, P);
  if (taps < 1 || taps > SS_MAX_TAPS) TS_REFUSE(TS_ERR_LIMIT, "ts_ssm_scan: a filter of %d taps (1 to %d)", taps, SS_MAX_TAPS);
  const int parts = ceil_div(N, SS_ROWS);
  if (parts * SS_COLS > 512) TS_REFUSE(TS_ERR_LIMIT, "ts_ssm_scan: a state of %d rows (limit %d)", N, 512 / SS_COLS * SS_ROWS);
  if (B > 65535 || H > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_ssm_scan: %d requests / %d heads per launch", B, H);
  cudaStream_t s = (cudaStream_t)stream;
  const int W = H * P + 2 * G * N + 2 * H;
  // 16-byte copies: every piece of a row (B, C, this block's x columns) on a 16-byte boundary
  const int vec4 = N % 4 == 0 && P % 4 == 0 && W % 4 == 0 && !((uintptr_t)ready & 15);
  const size_t smem = sizeof(float) * ((size_t)2 * SS_GROUP * (2 * parts * SS_ROWS + SS_COLS + 4) + (size_t)SS_GROUP * parts * SS_COLS);
  dim3 grid(ceil_div(P, SS_COLS), H, B);
#define TS_SC(TT)                                                                                                       \
  do {                                                                                                                  \
    static size_t configured = 0;                                                                                       \
    if (smem > 48 * 1024 && smem > configured) {                                                                        \
      cudaError_t e = cudaFuncSetAttribute(ssm_scan_kernel<TT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      if (e == cudaSuccess)                                                                                             \
        e = cudaFuncSetAttribute(ssm_scan_kernel<TT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);    \
      if (e != cudaSuccess) TS_REFUSE((int)e, "ts_ssm_scan: shared memory %zu: %s", smem, cudaGetErrorString(e));       \
      configured = smem;                                                                                                \
    }                                                                                                                   \
    if (longest >= SS_LATE_TOKENS)                                                                                      \
      ts_launch_late(ssm_scan_kernel<TT, true>, grid, dim3(parts * SS_COLS), smem, s, out, ready, (const TT*)proj, proj_stride, xbc_off, \
                     state, (size_t)state_stride, skip, q_start, slots, H, G, N, P, taps, parts, vec4);                 \
    else                                                                                                                \
      ts_launch(ssm_scan_kernel<TT, false>, grid, dim3(parts * SS_COLS), smem, s, out, ready, (const TT*)proj, proj_stride, xbc_off, \
                state, (size_t)state_stride, skip, q_start, slots, H, G, N, P, taps, parts, vec4);                      \
  } while (0)
  if (dtype == TS_F32) TS_SC(float);
  else if (dtype == TS_BF16) TS_SC(bf16);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_ssm_scan: dtype %d", dtype);
#undef TS_SC
  TS_LAUNCH_CHECK();
}
