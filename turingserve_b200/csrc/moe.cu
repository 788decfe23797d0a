// Routed feed-forward (mixture of experts): router with top-k choice, the grouping of (token, choice)
// pairs by expert, products over the groups, and the sum of a token's choices.  Nothing here reads a
// count back to the host: every launch is sized for the worst case and blocks without work leave, so the
// chain can sit in a captured graph.
//
//   ts_router_topk     z = Wr x in 32-bit (one block a token, fixed summation order), score = sigmoid(z) or
//                      softmax(z); the `top` largest by z (ties: the lower index), or, with a correction vector, by
//                      score + correction; weights = their scores (never the correction), optionally divided by
//                      their sum.
//   ts_moe_align       pairs p = t * top + r sorted by expert: offsets[E + 1], order[P] (sorted place -> pair),
//                      place[P] (pair -> sorted place), and the list of row tiles (expert, first row) the
//                      grouped products walk; experts from `with_tiles` on get a group but no tiles (experts
//                      without weights, whose output is their input).
//   ts_grouped_linear  out[i, :] = act(a_i . W[e(i)]^T) for the sorted places i; a_i is row i of `x`, or, when
//                      `order` is given, row order[i] / top of `x` times row_scale[order[i]] (rounded to the
//                      storage type: the weighted input of an expert).  32-bit accumulation in ascending k
//                      (FFMA; tensor cores for bfloat16 with K a multiple of 8): a row's result does not
//                      depend on its tile-mates.
//   ts_moe_combine     out[t, :] = sum over r (ascending) of (w[t, r] *) y[place[t * top + r], :], in 32-bit; a pair
//                      whose sorted place is *pass_from or later contributes the token's own input row instead.
#include "activations.cuh"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int GL_BM = 64, GL_BN = 64, GL_BK = 16, GL_PAD = 4;

// ---------------------------------------------------------------------------------------------------
// One block of RT_THREADS a token: thread i owns the columns i, i + RT_THREADS, ... of the token's row and keeps one sum
// per expert of a group of eight, so the loads of a step of the loop are all independent (the router's rows come
// from memory once a step: a chain of dependent loads would cost a round trip each); the threads' sums are added
// lane by lane, then warp by warp, in a fixed order.  Warp 0 then picks the experts.
constexpr int RT_THREADS = 256;

template <typename T>
__global__ void __launch_bounds__(RT_THREADS)
router_topk_kernel(int* __restrict__ idx_out, float* __restrict__ w_out, const T* __restrict__ x,
                   const float* __restrict__ wr, int T_, int E, int K, int top, int softmax, int renorm,
                   const float* __restrict__ correction) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  float* z = smem;                       // [E]
  float* part = smem + E;                // [RT_THREADS / 32][8]
  float* pick = part + RT_THREADS / 32 * 8;   // [E] what the choice goes by, when it is not z itself
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* xr = x + (size_t)t * K;
  for (int e0 = 0; e0 < E; e0 += 8) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll 2
    for (int k = threadIdx.x; k < K; k += RT_THREADS) {
      const float xv = to_f(xr[k]);
#pragma unroll
      for (int i = 0; i < 8; ++i)
        if (e0 + i < E) acc[i] = fmaf(xv, __ldg(wr + (size_t)(e0 + i) * K + k), acc[i]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float v = warp_sum(acc[i]);
      if (lane == 0) part[warp * 8 + i] = v;
    }
    __syncthreads();
    if (threadIdx.x < 8 && e0 + threadIdx.x < E) {
      float v = 0.f;
      for (int w = 0; w < RT_THREADS / 32; ++w) v += part[w * 8 + threadIdx.x];
      z[e0 + threadIdx.x] = v;
    }
    __syncthreads();
  }
  if (warp != 0) return;
  __syncwarp();
  float zmax = -INFINITY, denom = 1.f;
  if (softmax) {
    for (int e = lane; e < E; e += 32) zmax = fmaxf(zmax, z[e]);
    zmax = warp_max(zmax);
    float d = 0.f;
    for (int e = lane; e < E; e += 32) d += expf(z[e] - zmax);
    denom = warp_sum(d);
  }
  const float* by = z;
  if (correction != nullptr) {
    for (int e = lane; e < E; e += 32)
      pick[e] = (softmax ? expf(z[e] - zmax) / denom : 1.f / (1.f + expf(-z[e]))) + correction[e];
    by = pick;
    __syncwarp();
  }
  float total = 0.f;
  for (int r = 0; r < top; ++r) {
    float best = -INFINITY;
    int arg = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = by[e];
      if (v > best) {              // ascending e: the first of equal values stays
        best = v;
        arg = e;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, arg, o);
      if (ob > best || (ob == best && oa < arg)) {
        best = ob;
        arg = oa;
      }
    }
    if (arg == 0x7fffffff) arg = 0;              // only when every score left is -inf or NaN
    const float logit = correction != nullptr ? z[arg] : best;
    const float score = softmax ? expf(logit - zmax) / denom : 1.f / (1.f + expf(-logit));
    total += score;
    if (lane == 0) {
      idx_out[(size_t)t * top + r] = arg;
      w_out[(size_t)t * top + r] = score;
      if (correction != nullptr) pick[arg] = -INFINITY;
      else z[arg] = -INFINITY;
    }
    __syncwarp();
  }
  if (renorm && lane == 0)
    for (int r = 0; r < top; ++r) w_out[(size_t)t * top + r] /= (total + 1e-20f);
}

// ---------------------------------------------------------------------------------------------------
// One block.  tiles: [0] = number of row tiles, then (expert, first sorted row) pairs.
__global__ void __launch_bounds__(1024)
moe_align_kernel(const int* __restrict__ idx, int P, int E, int* __restrict__ offsets, int* __restrict__ order,
                 int* __restrict__ place, int* __restrict__ tiles, int tile_rows, int with_tiles) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ int sm_i[];
  int* count = sm_i;          // [E]
  int* cursor = sm_i + E;     // [E]
  for (int e = threadIdx.x; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  for (int p = threadIdx.x; p < P; p += blockDim.x) atomicAdd(&count[min(max(idx[p], 0), E - 1)], 1);
  __syncthreads();
  if (threadIdx.x == 0) {
    int at = 0, n = 0;
    for (int e = 0; e < E; ++e) {
      offsets[e] = at;
      cursor[e] = at;
      for (int r = 0; e < with_tiles && r < count[e]; r += tile_rows) {
        tiles[1 + 2 * n] = e;
        tiles[2 + 2 * n] = at + r;
        ++n;
      }
      at += count[e];
    }
    offsets[E] = at;
    tiles[0] = n;
  }
  __syncthreads();
  // a pair's place inside its expert's group is whatever the cursor gives: a row's result does not depend
  // on where in a tile it sits
  for (int p = threadIdx.x; p < P; p += blockDim.x) {
    const int at = atomicAdd(&cursor[min(max(idx[p], 0), E - 1)], 1);
    order[at] = p;
    place[p] = at;
  }
}

// ---------------------------------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void __launch_bounds__(256)
grouped_linear_kernel(TO* __restrict__ out, const TI* __restrict__ x, const TI* __restrict__ w,
                      const int* __restrict__ order, const float* __restrict__ row_scale,
                      const int* __restrict__ offsets, const int* __restrict__ tiles, int top, int N, int K, int act) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.y >= tiles[0]) return;
  const int e = tiles[1 + 2 * blockIdx.y], m0 = tiles[2 + 2 * blockIdx.y];
  const int m_end = offsets[e + 1];
  __shared__ __align__(16) float As[GL_BK][GL_BM + GL_PAD];
  __shared__ __align__(16) float Ws[GL_BK][GL_BN + GL_PAD];
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * GL_BN;
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int ty = tid >> 4, tx = tid & 15;
  float acc[4][4] = {};

  const int am = m0 + lr;
  const TI* a_row = nullptr;
  float a_scale = 1.f;
  bool scaled = false;
  if (am < m_end) {
    if (order != nullptr) {
      const int p = order[am];
      a_row = x + (size_t)(p / top) * K;
      if (row_scale != nullptr) {
        a_scale = row_scale[p];
        scaled = true;
      }
    } else {
      a_row = x + (size_t)am * K;
    }
  }
  const int wn = n0 + lr;
  const TI* w_row = wn < N ? w + ((size_t)e * N + wn) * K : nullptr;

  for (int k0 = 0; k0 < K; k0 += GL_BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      float a = (a_row != nullptr && k < K) ? to_f(a_row[k]) : 0.f;
      if (scaled) a = round_to<TI>(a * a_scale);
      As[lk + i][lr] = a;
      Ws[lk + i][lr] = (w_row != nullptr && k < K) ? to_f(w_row[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < GL_BK; ++k) {
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
    if (m >= m_end) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      out[(size_t)m * N + n] = from_f<TO>(ts_activate(acc[i][j], act));
    }
  }
}


// The same product on the tensor cores (bfloat16 operands, 32-bit accumulation): tiles of 64 sorted rows x 64
// output columns, k in steps of 64 through a 4-stage cp.async pipeline into XOR-swizzled shared memory; each
// of the 4 warps owns 16 rows.  Where the rows are weighted, the staged tile of inputs is multiplied in shared
// memory (32-bit, rounded to bfloat16) before the products read it.  K must be a multiple of 8.
constexpr int GM_BM = 64, GM_BN = 64, GM_BK = 64, GM_STAGES = 4, GM_WARPS = 4;
static_assert(GM_BM == GL_BM, "both grouped kernels walk the same row tiles");

template <typename TO>
__global__ void __launch_bounds__(GM_WARPS * 32)
grouped_linear_mma_kernel(TO* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ w,
                          const int* __restrict__ order, const float* __restrict__ row_scale,
                          const int* __restrict__ offsets, const int* __restrict__ tiles, int top, int N, int K, int act) {
  pdl_launch_dependents();
  pdl_wait();
  if ((int)blockIdx.y >= tiles[0]) return;
  const int e = tiles[1 + 2 * blockIdx.y], m0 = tiles[2 + 2 * blockIdx.y];
  const int m_end = offsets[e + 1];
  extern __shared__ __align__(128) unsigned char gsm[];
  constexpr int A_STAGE = GM_BM * GM_BK * 2, B_STAGE = GM_BN * GM_BK * 2;
  unsigned char* a_s = gsm;
  unsigned char* b_s = gsm + GM_STAGES * A_STAGE;
  __shared__ const bf16* a_rows[GM_BM];
  __shared__ float a_scales[GM_BM];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n0 = blockIdx.x * GM_BN;
  if (tid < GM_BM) {
    const int am = m0 + tid;
    const bf16* row = nullptr;
    float sc = 1.f;
    if (am < m_end) {
      if (order != nullptr) {
        const int p = order[am];
        row = x + (size_t)(p / top) * K;
        if (row_scale != nullptr) sc = row_scale[p];
      } else {
        row = x + (size_t)am * K;
      }
    }
    a_rows[tid] = row;
    a_scales[tid] = sc;
  }
  __syncthreads();
  const bf16* wb = w + (size_t)e * N * K;
  const int k_tiles = (K + GM_BK - 1) / GM_BK;

  auto load_tile = [&](int kt, int stage) {
    const int k0 = kt * GM_BK;
    for (int idx = tid; idx < GM_BM * 8; idx += GM_WARPS * 32) {
      const int r = idx >> 3, c = idx & 7;
      const bool ok = a_rows[r] != nullptr && k0 + c * 8 < K;
      cp_async_16(a_s + stage * A_STAGE + swz<GM_BK>(r, c), ok ? a_rows[r] + k0 + c * 8 : x, ok);
    }
    for (int idx = tid; idx < GM_BN * 8; idx += GM_WARPS * 32) {
      const int r = idx >> 3, c = idx & 7;
      const bool ok = n0 + r < N && k0 + c * 8 < K;
      cp_async_16(b_s + stage * B_STAGE + swz<GM_BK>(r, c), ok ? wb + (size_t)(n0 + r) * K + k0 + c * 8 : w, ok);
    }
  };

  float acc[GM_BN / 8][4];
#pragma unroll
  for (int i = 0; i < GM_BN / 8; ++i) acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f;
#pragma unroll
  for (int s_ = 0; s_ < GM_STAGES - 1; ++s_) {
    if (s_ < k_tiles) load_tile(s_, s_);
    cp_async_commit();
  }
  for (int kt = 0; kt < k_tiles; ++kt) {
    if (kt + GM_STAGES - 1 < k_tiles) load_tile(kt + GM_STAGES - 1, (kt + GM_STAGES - 1) % GM_STAGES);
    cp_async_commit();
    cp_async_wait<GM_STAGES - 1>();
    __syncthreads();
    unsigned char* as_ = a_s + (kt % GM_STAGES) * A_STAGE;
    const unsigned char* bs_ = b_s + (kt % GM_STAGES) * B_STAGE;
    if (row_scale != nullptr) {
      for (int idx = tid; idx < GM_BM * 8; idx += GM_WARPS * 32) {
        const int r = idx >> 3, c = idx & 7;
        const float sc = a_scales[r];
        __nv_bfloat162* v = reinterpret_cast<__nv_bfloat162*>(as_ + swz<GM_BK>(r, c));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 f = __bfloat1622float2(v[i]);
          v[i] = __floats2bfloat162_rn(f.x * sc, f.y * sc);
        }
      }
      __syncthreads();
    }
#pragma unroll
    for (int ks = 0; ks < GM_BK / 16; ++ks) {
      const int mat = lane >> 3, r = lane & 7;
      unsigned a[4];
      ldmatrix_x4(a[0], a[1], a[2], a[3], as_ + swz<GM_BK>(warp * 16 + (mat & 1) * 8 + r, ks * 2 + (mat >> 1)));
#pragma unroll
      for (int np = 0; np < GM_BN / 16; ++np) {
        unsigned b0, b1, b2, b3;
        ldmatrix_x4(b0, b1, b2, b3, bs_ + swz<GM_BK>(np * 16 + (mat >> 1) * 8 + r, ks * 2 + (mat & 1)));
        mma_bf16(acc[2 * np], a, b0, b1);
        mma_bf16(acc[2 * np + 1], a, b2, b3);
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();
#pragma unroll
  for (int nt = 0; nt < GM_BN / 8; ++nt)
#pragma unroll
    for (int e_ = 0; e_ < 4; ++e_) {
      const int m = m0 + warp * 16 + (lane >> 2) + 8 * (e_ >> 1);
      const int n = n0 + nt * 8 + (lane & 3) * 2 + (e_ & 1);
      if (m < m_end && n < N) out[(size_t)m * N + n] = from_f<TO>(ts_activate(acc[nt][e_], act));
    }
}

// The same product for steps of a few tokens, where an expert has a handful of rows and the time is the experts'
// weights crossing from memory once: no shared memory, no barrier, and the arithmetic on the tensor cores so that the
// instruction stream stays thin (an FFMA version spent 108 instructions a warp per 512 bytes of weights and was
// bound by issue slots at a third of the memory bandwidth).  A warp owns EIGHT output columns of one row tile and up
// to eight input rows at a time: per 32 columns of k, lane (g, t) loads 16 bytes of weight row n0 + g and 16 bytes of
// input row g, both at k + 8 t, and feeds them to two m16n8k16 products.  (The products' k index is a permutation
// of the real one, the same for both operands, so the sum is the same sum.)  GV_UNROLL steps of loads are in flight.
// Rows 8..15 of the product are zero.  A tile with more rows is walked eight at a time.
constexpr int GV_ROWS = 8, GV_WARPS = 8, GV_UNROLL = 8;
constexpr int GV_STREAM_ROWS = 64;      // steps with at most this many (token, choice) pairs take this kernel

template <typename TO>
__global__ void __launch_bounds__(GV_WARPS * 32)
grouped_linear_stream_kernel(TO* __restrict__ out, const bf16* __restrict__ x, const bf16* __restrict__ w,
                             const int* __restrict__ order, const float* __restrict__ row_scale,
                             const int* __restrict__ offsets, const int* __restrict__ tiles, int top, int N, int K, int act) {
  pdl_launch_dependents();
  // (the tile list is written by the kernel before this one: nothing can be fetched ahead of the wait)
  pdl_wait();
  if ((int)blockIdx.y >= tiles[0]) return;
  const int e = tiles[1 + 2 * blockIdx.y], m0 = tiles[2 + 2 * blockIdx.y];
  const int m_end = min(offsets[e + 1], m0 + GL_BM);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int n0 = (blockIdx.x * GV_WARPS + warp) * 8;
  if (n0 >= N) return;
  const bool n_ok = n0 + g < N;
  const bf16* wrow = w + ((size_t)e * N + (n_ok ? n0 + g : n0)) * K + t * 8;
  for (int r0 = m0; r0 < m_end; r0 += GV_ROWS) {
    const int row = r0 + g;
    const bool row_ok = row < m_end;
    const bf16* xrow = x + t * 8;
    float scale = 1.f;
    if (row_ok) {
      if (order != nullptr) {
        const int p = order[row];
        xrow += (size_t)(p / top) * K;
        if (row_scale != nullptr) scale = row_scale[p];
      } else {
        xrow += (size_t)row * K;
      }
    }
    const bool scaled = row_scale != nullptr && order != nullptr;
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    for (int k0 = 0; k0 < K; k0 += 32 * GV_UNROLL) {
      uint4 wv[GV_UNROLL], xv[GV_UNROLL];
#pragma unroll
      for (int u = 0; u < GV_UNROLL; ++u) {
        const int k = k0 + u * 32;
        const bool k_ok = k + t * 8 < K;
        wv[u] = (k_ok && n_ok) ? __ldcs(reinterpret_cast<const uint4*>(wrow + k)) : make_uint4(0u, 0u, 0u, 0u);
        xv[u] = (k_ok && row_ok) ? *reinterpret_cast<const uint4*>(xrow + k) : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < GV_UNROLL; ++u) {
        if (scaled) {
          __nv_bfloat162* x2 = reinterpret_cast<__nv_bfloat162*>(&xv[u]);
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const float2 f = __bfloat1622float2(x2[i]);
            x2[i] = __floats2bfloat162_rn(f.x * scale, f.y * scale);
          }
        }
        const unsigned a1[4] = {xv[u].x, 0u, xv[u].y, 0u};
        const unsigned a2[4] = {xv[u].z, 0u, xv[u].w, 0u};
        mma_bf16(acc, a1, wv[u].x, wv[u].y);
        mma_bf16(acc, a2, wv[u].z, wv[u].w);
      }
    }
    if (row_ok) {
#pragma unroll
      for (int i = 0; i < 2; ++i) {
        const int n = n0 + 2 * t + i;
        if (n < N) out[(size_t)row * N + n] = from_f<TO>(ts_activate(acc[i], act));
      }
    }
  }
}

// xs[i, :] = x[order[i] / top, :] (* row_scale[order[i]], rounded to the storage type): the experts' input rows in
// sorted order, for the path that hands each expert's rows to a many-row product of its own.
template <typename T>
__global__ void moe_gather_kernel(T* __restrict__ xs, const T* __restrict__ x, const int* __restrict__ order,
                                  const float* __restrict__ row_scale, int top, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int p = order[blockIdx.x];
  const T* src = x + (size_t)(p / top) * K;
  T* dst = xs + (size_t)blockIdx.x * K;
  if (row_scale != nullptr) {
    const float sc = row_scale[p];
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = from_f<T>(to_f(src[k]) * sc);
  } else {
    for (int k = threadIdx.x; k < K; k += blockDim.x) dst[k] = src[k];
  }
}

template <typename T>
__global__ void moe_combine_kernel(T* __restrict__ out, const float* __restrict__ y, const int* __restrict__ place,
                                   const float* __restrict__ pair_w, int top, int N, const T* __restrict__ x,
                                   const int* __restrict__ pass_from, const T* __restrict__ add) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int first_pass = pass_from != nullptr ? *pass_from : 0x7fffffff;
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    float acc = 0.f;
    for (int r = 0; r < top; ++r) {
      const size_t p = (size_t)t * top + r;
      const int at = place[p];
      const float v = at >= first_pass ? to_f(x[(size_t)t * N + n]) : y[(size_t)at * N + n];
      acc += pair_w != nullptr ? pair_w[p] * v : v;
    }
    if (add != nullptr) acc += to_f(add[(size_t)t * N + n]);       // (an expert that every token uses)
    out[(size_t)t * N + n] = from_f<T>(acc);
  }
}

}  // namespace

TS_API int ts_moe_tile_rows() { return GL_BM; }

// x: [T, K] in `dtype`; wr: [E, K] 32-bit.  idx_out / w_out: [T, top].
// correction: 32-bit [E] or null.
TS_API int ts_router_topk(int* idx_out, float* w_out, const void* x, const float* wr, int T, int E, int K, int top,
                          int softmax, int renorm, int dtype, const float* correction, void* stream) {
  if (T <= 0) return 0;
  if (E <= 0 || top <= 0 || top > E) TS_REFUSE(TS_ERR_SHAPE, "ts_router_topk: top %d of %d experts", top, E);
  if (E > 2048) TS_REFUSE(TS_ERR_LIMIT, "ts_router_topk: %d experts (limit 2048)", E);
  cudaStream_t s = (cudaStream_t)stream;
  const size_t smem = sizeof(float) * (2 * E + RT_THREADS / 32 * 8);
  if (dtype == TS_F32)
    ts_launch(router_topk_kernel<float>, dim3(T), dim3(RT_THREADS), smem, s, idx_out, w_out, (const float*)x, wr, T,
              E, K, top, softmax, renorm, correction);
  else if (dtype == TS_BF16)
    ts_launch(router_topk_kernel<bf16>, dim3(T), dim3(RT_THREADS), smem, s, idx_out, w_out, (const bf16*)x, wr, T,
              E, K, top, softmax, renorm, correction);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_router_topk: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// tiles needs 1 + 2 * (ceil(P / tile_rows) + E) ints.
// with_tiles: the experts [0, with_tiles) get row tiles (E: all of them).
TS_API int ts_moe_align(const int* idx, int P, int E, int* offsets, int* order, int* place, int* tiles, int with_tiles,
                        void* stream) {
  if (P <= 0) return 0;
  if (E > 4096) TS_REFUSE(TS_ERR_LIMIT, "ts_moe_align: %d experts (limit 4096)", E);
  ts_launch(moe_align_kernel, dim3(1), dim3(1024), sizeof(int) * 2 * E, (cudaStream_t)stream, idx, P, E, offsets, order,
            place, tiles, GL_BM, with_tiles);
  TS_LAUNCH_CHECK();
}


TS_API int ts_moe_gather(void* xs, const void* x, const int* order, const float* row_scale, int P, int top, int K, int dtype,
                         void* stream) {
  if (P <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    ts_launch(moe_gather_kernel<float>, dim3(P), dim3(256), 0, s, (float*)xs, (const float*)x, order, row_scale, top, K);
  else if (dtype == TS_BF16)
    ts_launch(moe_gather_kernel<bf16>, dim3(P), dim3(256), 0, s, (bf16*)xs, (const bf16*)x, order, row_scale, top, K);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_moe_gather: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}

// w: [E, N, K].  out: [P, N].  act: 0 none, 1 tanh-form GELU, 2 squared ReLU, 3 SiLU.
TS_API int ts_grouped_linear(void* out, const void* x, const void* w, const int* order, const float* row_scale,
                             const int* offsets, const int* tiles, int P, int E, int top, int N, int K, int act,
                             int dtype, int out_dtype, void* stream) {
  if (P <= 0 || N <= 0) return 0;
  if (K <= 0) TS_REFUSE(TS_ERR_SHAPE, "ts_grouped_linear: K = %d", K);
  cudaStream_t s = (cudaStream_t)stream;
  dim3 grid(ceil_div(N, GL_BN), ceil_div(P, GL_BM) + E);
  if (grid.y > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_grouped_linear: %d rows too many for one launch", P);
  if (dtype == TS_BF16 && K % 8 == 0 && !(((uintptr_t)x | (uintptr_t)w) & 15) && P <= GV_STREAM_ROWS) {
    dim3 sgrid(ceil_div(N, GV_WARPS * 8), ceil_div(P, GL_BM) + E);
    if (out_dtype == TS_BF16)
      ts_launch(grouped_linear_stream_kernel<bf16>, dim3(sgrid), dim3(GV_WARPS * 32), 0, s, (bf16*)out, (const bf16*)x,
                (const bf16*)w, order, row_scale, offsets, tiles, top, N, K, act);
    else if (out_dtype == TS_F32)
      ts_launch(grouped_linear_stream_kernel<float>, dim3(sgrid), dim3(GV_WARPS * 32), 0, s, (float*)out, (const bf16*)x,
                (const bf16*)w, order, row_scale, offsets, tiles, top, N, K, act);
    else
      TS_REFUSE(TS_ERR_DTYPE, "ts_grouped_linear: dtype %d -> %d", dtype, out_dtype);
    TS_LAUNCH_CHECK();
  }
  if (dtype == TS_BF16 && K % 8 == 0 && !(((uintptr_t)x | (uintptr_t)w) & 15)) {
    const size_t smem = (size_t)GM_STAGES * (GM_BM + GM_BN) * GM_BK * 2;
    static bool configured = false;
    if (!configured) {
      cudaError_t e1 = cudaFuncSetAttribute(grouped_linear_mma_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      cudaError_t e2 = cudaFuncSetAttribute(grouped_linear_mma_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e1 != cudaSuccess || e2 != cudaSuccess) TS_REFUSE((int)(e1 != cudaSuccess ? e1 : e2), "ts_grouped_linear: shared memory %zu", smem);
      configured = true;
    }
    if (out_dtype == TS_BF16)
      ts_launch(grouped_linear_mma_kernel<bf16>, dim3(grid), dim3(GM_WARPS * 32), smem, s, (bf16*)out, (const bf16*)x,
                (const bf16*)w, order, row_scale, offsets, tiles, top, N, K, act);
    else if (out_dtype == TS_F32)
      ts_launch(grouped_linear_mma_kernel<float>, dim3(grid), dim3(GM_WARPS * 32), smem, s, (float*)out, (const bf16*)x,
                (const bf16*)w, order, row_scale, offsets, tiles, top, N, K, act);
    else
      TS_REFUSE(TS_ERR_DTYPE, "ts_grouped_linear: dtype %d -> %d", dtype, out_dtype);
    TS_LAUNCH_CHECK();
  }
#define TS_GLK(TI, TO)                                                                                           \
  ts_launch(grouped_linear_kernel<TI, TO>, dim3(grid), dim3(256), 0, s, (TO*)out, (const TI*)x, (const TI*)w, order, \
            row_scale, offsets, tiles, top, N, K, act)
  if (dtype == TS_F32 && out_dtype == TS_F32) TS_GLK(float, float);
  else if (dtype == TS_BF16 && out_dtype == TS_BF16) TS_GLK(bf16, bf16);
  else if (dtype == TS_BF16 && out_dtype == TS_F32) TS_GLK(bf16, float);
  else TS_REFUSE(TS_ERR_DTYPE, "ts_grouped_linear: dtype %d -> %d", dtype, out_dtype);
#undef TS_GLK
  TS_LAUNCH_CHECK();
}

// x (out's type, [T, N]) and pass_from (one int on the device): pairs sorted to place *pass_from or later add the
// token's own row of x instead of a row of y; both null: none do.  add (out's type, [T, N], may be null): added to
// every token's sum.
TS_API int ts_moe_combine(void* out, const float* y, const int* place, const float* pair_w, int T, int top, int N, int dtype,
                          const void* x, const int* pass_from, const void* add, void* stream) {
  if (T <= 0) return 0;
  cudaStream_t s = (cudaStream_t)stream;
  if (dtype == TS_F32)
    ts_launch(moe_combine_kernel<float>, dim3(T), dim3(256), 0, s, (float*)out, y, place, pair_w, top, N, (const float*)x, pass_from, (const float*)add);
  else if (dtype == TS_BF16)
    ts_launch(moe_combine_kernel<bf16>, dim3(T), dim3(256), 0, s, (bf16*)out, y, place, pair_w, top, N, (const bf16*)x, pass_from, (const bf16*)add);
  else
    TS_REFUSE(TS_ERR_DTYPE, "ts_moe_combine: dtype %d", dtype);
  TS_LAUNCH_CHECK();
}
