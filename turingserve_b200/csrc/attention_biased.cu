// Paged grouped-query attention with a score that is more than a scaled dot product, any sizes, 32-bit
// arithmetic whatever the storage type:
//     s = q.k * scale;   s <- cap * tanh(s / cap)  (cap > 0);   s <- s - slope_h * (i - j)  (slopes given)
// for the query at position i and the key at position j <= i, with a window w only j > i - w, and with blocks of c
// positions (counted from the sequence's position 0) only j >= floor(i / c) * c; softmax over the visible keys, whose
// denominator also holds exp(sink_h) when sinks are given (a learned number per head that has no key and no value:
// the weights of a row then sum to less than one); a request without context gives zeros.  Key rows (Dk wide) and value rows
// (Dv wide) have widths of their own; with no value tensor the values ARE the first Dv columns of the key rows
// (a cache that keeps one latent row a token serves all heads as keys and as values).  Queries and outputs
// are addressed by a token stride and a head stride, so they may be column slices of wider rows.
//
// Work split as in the plain any-size kernel: one block per (tile of AB_ROWS query rows, kv head, request, key
// split), a row being one (token, head-in-group) pair so that the heads of a group share each key tile; keys 32 at
// a time, lane j scores key j from shared memory, online softmax per row, then each lane accumulates its Dv / 32
// output columns.  Requests that bring ONE token may have their keys cut over `splits` blocks; each leaves
// (m, l, unnormalised sum) in scratch and the block that comes last for its (request, kv head, row tile)
// (a ticket counter; nobody waits) merges them in split order.
#include "common.cuh"

namespace {

constexpr int AB_ROWS = 16;     // query rows per block
constexpr int AB_KT = 32;       // keys per tile (one per lane)
constexpr int AB_WARPS = 4;
constexpr int AB_RPW = AB_ROWS / AB_WARPS;
constexpr int AB_MAX_DPL = 16;  // Dv <= 512

// 1 / (l + exp(sink - m)) for sums l taken against the maximum m: what the unnormalised output is multiplied by.
// Against the larger of m and the sink, so that neither exponential can overflow.  No visible key: 0.
__device__ __forceinline__ float sink_inverse(float m, float l, const float* sink) {
  if (!(l > 0.f)) return 0.f;
  if (sink == nullptr) return 1.f / l;
  const float s = *sink;
  const float top = fmaxf(m, s);
  const float down = expf(m - top);
  return down / (l * down + expf(s - top));
}

template <typename T, int DPL>
__global__ void __launch_bounds__(AB_WARPS * 32)
attention_biased_kernel(T* __restrict__ out, int out_ts, int out_hs, const T* __restrict__ q, int q_ts, int q_hs,
                        const T* __restrict__ k_cache, const T* __restrict__ v_cache,
                        const int* __restrict__ block_tables, const int* __restrict__ q_start,
                        const int* __restrict__ seq_lens, int table_width, int H, int KVH, int Dk, int Dv, int page,
                        float scale, float softcap, const float* __restrict__ slopes, int window, int splits,
                        float* __restrict__ scratch, int* __restrict__ counters, int chunk,
                        const float* __restrict__ sinks) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = H / KVH;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int seq_len = seq_lens[b];
  const int n_rows = q_len * G;
  const int tiles = (n_rows + AB_ROWS - 1) / AB_ROWS;
  // blockIdx.x = row tile * splits + split; only single-token requests are split
  const int my_splits = (q_len == 1) ? splits : 1;
  const int tile = blockIdx.x / splits, split = blockIdx.x % splits;
  if (tile >= tiles || split >= my_splits) return;
  const int row0 = tile * AB_ROWS;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int prefix = seq_len - q_len;
  const bool v_in_k = v_cache == nullptr;

  float* q_s = smem;                           // [AB_ROWS][Dk]
  float* k_s = q_s + AB_ROWS * Dk;             // [AB_KT][Dk + 1]
  float* v_s = k_s + AB_KT * (Dk + 1);         // [AB_KT][Dv] (absent when the values are in the key rows)
  __shared__ size_t key_off[AB_KT];
  __shared__ int last_flag;

  for (int idx = threadIdx.x; idx < AB_ROWS * Dk; idx += blockDim.x) {
    const int r = idx / Dk, d = idx % Dk;
    const int row = row0 + r;
    float v = 0.f;
    if (row < n_rows) {
      const int t = row / G, g = row % G;
      v = to_f(q[(size_t)(qs + t) * q_ts + (size_t)(kvh * G + g) * q_hs + d]);
    }
    q_s[idx] = v;
  }

  const int last_row = min(row0 + AB_ROWS, n_rows) - 1;
  const int t_lo = row0 / G, t_hi = last_row / G;
  int j_hi = prefix + t_hi;                                           // last key any row of the tile sees
  int j_lo = window > 0 ? max(0, prefix + t_lo - window + 1) : 0;
  if (chunk > 0) j_lo = max(j_lo, (prefix + t_lo) / chunk * chunk);      // (a block's start never moves back with the position)
  if (my_splits > 1) {
    // this block's share of the key tiles
    const int n_tiles = (j_hi - j_lo) / AB_KT + 1;
    const int per = (n_tiles + my_splits - 1) / my_splits;
    const int first = j_lo + split * per * AB_KT;
    j_hi = min(j_hi, first + per * AB_KT - 1);
    j_lo = first;
  }

  float m[AB_RPW], l[AB_RPW], acc[AB_RPW][DPL], slope[AB_RPW];
  int p_row[AB_RPW], lo_row[AB_RPW];
#pragma unroll
  for (int r = 0; r < AB_RPW; ++r) {
    m[r] = -INFINITY;
    l[r] = 0.f;
#pragma unroll
    for (int i = 0; i < DPL; ++i) acc[r][i] = 0.f;
    const int row = row0 + warp * AB_RPW + r;
    const int t = row / G;
    p_row[r] = (row < n_rows) ? prefix + t : -1;
    lo_row[r] = (window > 0) ? max(0, p_row[r] - window + 1) : 0;
    if (chunk > 0 && p_row[r] >= 0) lo_row[r] = max(lo_row[r], p_row[r] / chunk * chunk);
    slope[r] = (slopes != nullptr && row < n_rows) ? slopes[kvh * G + row % G] : 0.f;
  }

  if (seq_len > 0 && j_hi >= j_lo) {
    for (int j0 = j_lo; j0 <= j_hi; j0 += AB_KT) {
      __syncthreads();
      if (threadIdx.x < AB_KT) {
        const int j = j0 + threadIdx.x;
        size_t off = 0;
        if (j <= j_hi) {
          const int pg = block_tables[(size_t)b * table_width + j / page];
          off = ((size_t)pg * KVH + kvh) * page + (size_t)(j % page);
        }
        key_off[threadIdx.x] = off;
      }
      __syncthreads();
      for (int idx = threadIdx.x; idx < AB_KT * Dk; idx += blockDim.x) {
        const int kk = idx / Dk, d = idx % Dk;
        k_s[kk * (Dk + 1) + d] = (j0 + kk <= j_hi) ? to_f(k_cache[key_off[kk] * Dk + d]) : 0.f;
      }
      if (!v_in_k) {
        for (int idx = threadIdx.x; idx < AB_KT * Dv; idx += blockDim.x) {
          const int kk = idx / Dv, d = idx % Dv;
          v_s[kk * Dv + d] = (j0 + kk <= j_hi) ? to_f(v_cache[key_off[kk] * Dv + d]) : 0.f;
        }
      }
      __syncthreads();
      const int j = j0 + lane;
      const float* vbase = v_in_k ? k_s : v_s;
      const int vstride = v_in_k ? Dk + 1 : Dv;
#pragma unroll
      for (int r = 0; r < AB_RPW; ++r) {
        if (p_row[r] < j0) continue;                 // whole tile is in this row's future (warp-uniform)
        const float* qr = q_s + (warp * AB_RPW + r) * Dk;
        const float* kr = k_s + lane * (Dk + 1);
        float s0 = 0.f, s1 = 0.f;
        int d = 0;
        for (; d + 1 < Dk; d += 2) {
          s0 = fmaf(qr[d], kr[d], s0);
          s1 = fmaf(qr[d + 1], kr[d + 1], s1);
        }
        if (d < Dk) s0 = fmaf(qr[d], kr[d], s0);
        float s = (s0 + s1) * scale;
        if (softcap > 0.f) s = softcap * tanhf(s / softcap);
        s -= slope[r] * (float)(p_row[r] - j);
        const bool ok = (j <= p_row[r]) && (j >= lo_row[r]) && (j <= j_hi);
        s = ok ? s : -INFINITY;
        const float m_new = fmaxf(m[r], warp_max(s));
        if (m_new == -INFINITY) continue;            // nothing visible yet (warp-uniform)
        const float p = ok ? expf(s - m_new) : 0.f;
        const float corr = (m[r] == -INFINITY) ? 0.f : expf(m[r] - m_new);
        l[r] = l[r] * corr + warp_sum(p);
        m[r] = m_new;
#pragma unroll
        for (int i = 0; i < DPL; ++i) acc[r][i] *= corr;
        for (int kk = 0; kk < AB_KT; ++kk) {
          const float pk = __shfl_sync(0xffffffffu, p, kk);
          const float* vr = vbase + kk * vstride;
#pragma unroll
          for (int i = 0; i < DPL; ++i) {
            const int dd = lane + 32 * i;
            if (dd < Dv) acc[r][i] = fmaf(pk, vr[dd], acc[r][i]);
          }
        }
      }
    }
  }

  if (my_splits == 1) {
#pragma unroll
    for (int r = 0; r < AB_RPW; ++r) {
      const int row = row0 + warp * AB_RPW + r;
      if (row >= n_rows) continue;
      const int t = row / G, g = row % G;
      const float inv = sink_inverse(m[r], l[r], sinks != nullptr ? sinks + kvh * G + g : nullptr);
      T* o = out + (size_t)(qs + t) * out_ts + (size_t)(kvh * G + g) * out_hs;
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int dd = lane + 32 * i;
        if (dd < Dv) o[dd] = from_f<T>(acc[r][i] * inv);
      }
    }
    return;
  }

  // partial results: [request][kv head][tile][split][AB_ROWS][Dv + 2]
  const size_t rec = (size_t)Dv + 2;
  const size_t group = ((size_t)(b * KVH + kvh) * gridDim.x / splits + tile) * splits;
  float* mine = scratch + (group + split) * AB_ROWS * rec;
#pragma unroll
  for (int r = 0; r < AB_RPW; ++r) {
    float* dst = mine + (size_t)(warp * AB_RPW + r) * rec;
    if (lane == 0) {
      dst[0] = m[r];
      dst[1] = l[r];
    }
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int dd = lane + 32 * i;
      if (dd < Dv) dst[2 + dd] = acc[r][i];
    }
  }
  __threadfence();
  __syncthreads();
  int* counter = counters + (size_t)(b * KVH + kvh) * (gridDim.x / splits) + tile;
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(counter, 1);
    last_flag = ticket == my_splits - 1;
    if (last_flag) *counter = 0;                                     // ready for the next launch
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
#pragma unroll
  for (int r = 0; r < AB_RPW; ++r) {
    const int row = row0 + warp * AB_RPW + r;
    if (row >= n_rows) continue;
    const float* src = scratch + group * AB_ROWS * rec + (size_t)(warp * AB_RPW + r) * rec;
    float mm = -INFINITY;
    for (int sp = 0; sp < my_splits; ++sp) mm = fmaxf(mm, __ldcg(src + (size_t)sp * AB_ROWS * rec));
    float ll = 0.f, o[DPL];
#pragma unroll
    for (int i = 0; i < DPL; ++i) o[i] = 0.f;
    for (int sp = 0; sp < my_splits; ++sp) {
      const float* part = src + (size_t)sp * AB_ROWS * rec;
      const float pm = __ldcg(part);
      if (pm == -INFINITY) continue;
      const float w = expf(pm - mm);
      ll = fmaf(__ldcg(part + 1), w, ll);
#pragma unroll
      for (int i = 0; i < DPL; ++i) {
        const int dd = lane + 32 * i;
        if (dd < Dv) o[i] = fmaf(__ldcg(part + 2 + dd), w, o[i]);
      }
    }
    const int t = row / G, g = row % G;
    const float inv = sink_inverse(mm, ll, sinks != nullptr ? sinks + kvh * G + g : nullptr);
    T* dst = out + (size_t)(qs + t) * out_ts + (size_t)(kvh * G + g) * out_hs;
#pragma unroll
    for (int i = 0; i < DPL; ++i) {
      const int dd = lane + 32 * i;
      if (dd < Dv) dst[dd] = from_f<T>(o[i] * inv);
    }
  }
}

template <typename T, int DPL>
int launch(void* out, int out_ts, int out_hs, const void* q, int q_ts, int q_hs, const void* k_cache, const void* v_cache,
           const int* block_tables, const int* q_start, const int* seq_lens, int B, int table_width, int max_q_len, int H,
           int KVH, int Dk, int Dv, int page, float scale, float softcap, const float* slopes, int window, int splits,
           float* scratch, int* counters, int chunk, const float* sinks, cudaStream_t s) {
  const int G = H / KVH;
  const size_t smem = sizeof(float) * ((size_t)AB_ROWS * Dk + (size_t)AB_KT * (Dk + 1) + (v_cache ? (size_t)AB_KT * Dv : 0));
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_biased_kernel<T, DPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_biased: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = smem;
  }
  dim3 grid(ceil_div(max_q_len * G, AB_ROWS) * splits, KVH, B);
  ts_launch(attention_biased_kernel<T, DPL>, dim3(grid), dim3(AB_WARPS * 32), smem, s, (T*)out, out_ts, out_hs, (const T*)q,
            q_ts, q_hs, (const T*)k_cache, (const T*)v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, Dk, Dv,
            page, scale, softcap, slopes, window, splits, scratch, counters, chunk, sinks);
  TS_LAUNCH_CHECK();
}

}  // namespace

// Floats of scratch a launch with `splits` > 1 needs (0 for one split).
TS_API long long ts_attention_biased_scratch_floats(int B, int KVH, int H, int max_q_len, int Dv, int splits) {
  if (splits <= 1) return 0;
  const long long tiles = ceil_div(max_q_len * (H / KVH), AB_ROWS);
  return (long long)B * KVH * tiles * splits * AB_ROWS * (Dv + 2);
}

// k_cache [pages, KVH, page, Dk]; v_cache [pages, KVH, page, Dv] or null (values = first Dv columns of the key
// rows).  softcap <= 0: no cap; slopes null: no distance bias; window <= 0: none; chunk <= 0: no blocks; sinks
// (32-bit [H]) null: none.  splits > 1 needs scratch
// (ts_attention_biased_scratch_floats) and zeroed counters, one per (request, kv head, row tile).
TS_API int ts_attention_biased(void* out, int out_ts, int out_hs, const void* q, int q_ts, int q_hs, const void* k_cache,
                               const void* v_cache, const int* block_tables, const int* q_start, const int* seq_lens, int B,
                               int table_width, int max_q_len, int H, int KVH, int Dk, int Dv, int page, float scale,
                               float softcap, const float* slopes, int window, int splits, float* scratch, int* counters,
                               int dtype, int chunk, const float* sinks, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  if (KVH <= 0 || H % KVH) TS_REFUSE(TS_ERR_SHAPE, "ts_attention_biased: %d heads over %d kv heads", H, KVH);
  if (Dk <= 0 || Dv <= 0 || Dv > 32 * AB_MAX_DPL || (v_cache == nullptr && Dv > Dk))
    TS_REFUSE(TS_ERR_LIMIT, "ts_attention_biased: keys of %d, values of %d (limit %d)", Dk, Dv, 32 * AB_MAX_DPL);
  if (Dk > 1024) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_biased: keys of %d (limit 1024)", Dk);
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_biased: %d requests / %d kv heads per launch", B, KVH);
  if (splits < 1) splits = 1;
  if (splits > 1 && (scratch == nullptr || counters == nullptr)) TS_REFUSE(TS_ERR_SHAPE, "ts_attention_biased: splits without scratch");
  cudaStream_t s = (cudaStream_t)stream;
  const int dpl = ceil_div(Dv, 32);
#define TS_AB(TT, N)                                                                                                   \
  return launch<TT, N>(out, out_ts, out_hs, q, q_ts, q_hs, k_cache, v_cache, block_tables, q_start, seq_lens, B, table_width, \
                       max_q_len, H, KVH, Dk, Dv, page, scale, softcap, slopes, window, splits, scratch, counters, chunk, sinks, s)
#define TS_AB_T(TT)                     \
  do {                                  \
    if (dpl <= 2) TS_AB(TT, 2);         \
    if (dpl <= 4) TS_AB(TT, 4);         \
    if (dpl <= 8) TS_AB(TT, 8);         \
    TS_AB(TT, 16);                      \
  } while (0)
  if (dtype == TS_F32) TS_AB_T(float);
  if (dtype == TS_BF16) TS_AB_T(bf16);
#undef TS_AB_T
#undef TS_AB
  TS_REFUSE(TS_ERR_DTYPE, "ts_attention_biased: dtype %d", dtype);
}
