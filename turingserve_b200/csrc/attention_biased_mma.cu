// The attention of attention_biased.cu (capped scores, distance bias per head, window, blocks of positions, a sink in
// the softmax's denominator, values of their own width or inside the key rows) on the tensor cores, bfloat16 storage, for key rows that are a multiple of 64 wide.
//
// Work split as in the prompt-portion kernel: one block per (tile of 64 query ROWS, kv head, request), a row being
// one (token, head-in-group) pair, four warps of 16 rows (m16n8k16), keys 64 at a time through a cp.async pipeline
// into XOR-swizzled shared memory.  What differs:
//   * the query tile lives in shared memory too (ldmatrix per k-step), so key rows of 576 columns do not cost 144
//     registers a thread;
//   * scores leave the accumulator in 32-bit, are scaled, capped (tanh from the exponential: absolute error of a
//     few 1e-7 of the cap) and biased there; the softmax weights stay 32-bit in the sums and enter the second
//     product as TWO bfloat16 terms (p = hi + lo, two products), so they carry 16 bits of mantissa, not 8;
//   * wide value rows are cut into chunks of DV columns, one block each (a block's accumulator is 16 x DV per warp):
//     a latent row of 512 value columns is two blocks that each redo the scores (128 accumulator registers a thread:
//     the shared memory of a 576-wide tile allows one block an SM anyway);
//   * requests that bring ONE token may have their keys cut over `splits` blocks; each leaves (m, l, unnormalised
//     sum) in scratch and the block that comes last (a ticket counter; nobody waits) merges them in split order; a
//     second and a third instance of the kernel take such requests when their rows fill one or two warps (below).
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int BM_WARPS = 4;
constexpr int BM_ROWS = BM_WARPS * 16;
constexpr int BM_TILE = 64;
constexpr int BM_PAGES_S = 512;
constexpr int BM_MAX_SPLITS = 16;   // blocks a single-token request's keys are cut over
constexpr int BM_MAX_RECORDS = 64;  // partial results the last block merges (four a block where the warps share a tile's keys)
constexpr float BM_LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float capped(float s, float cap, float inv_cap) {
  const float t = __expf(2.f * s * inv_cap);
  return cap * (1.f - __fdividef(2.f, t + 1.f));
}

// SPREAD (1 or 2; 0: off): for requests that bring ONE token whose rows (the heads of one kv head) fill SPREAD warps'
// 16 rows at most.  The 4 / SPREAD warps of a row group all take its rows and 64 / (4 / SPREAD) keys of every tile
// each (instead of idling) and leave as many partial results a block, which the merge folds like those of blocks.
template <int DK, int DV, bool V_IN_K, int STAGES, int SPREAD>
__global__ void __launch_bounds__(BM_WARPS * 32)
attention_biased_mma_kernel(bf16* __restrict__ out, int out_ts, int out_hs, const bf16* __restrict__ q, int q_ts, int q_hs,
                            const bf16* __restrict__ k_cache, const bf16* __restrict__ v_cache,
                            const int* __restrict__ block_tables, const int* __restrict__ q_start,
                            const int* __restrict__ seq_lens, int table_width, int H, int KVH, int page, float scale,
                            float softcap, const float* __restrict__ slopes, int window, int v_chunks, int splits,
                            float* __restrict__ scratch, int* __restrict__ counters, int block_of,
                            const float* __restrict__ sinks) {
  pdl_launch_dependents();
  pdl_wait();
  constexpr int CHK = DK / 8, KS = DK / 16, NT = DV / 8, CHV = DV / 8;
  constexpr int WPG = SPREAD ? BM_WARPS / SPREAD : 1;                // warps that share a row group's keys
  constexpr int NTW = BM_TILE / 8 / WPG;                             // groups of 8 keys of a tile this warp takes
  extern __shared__ __align__(128) unsigned char smem[];
  const int b = blockIdx.z, kvh = blockIdx.y;
  const int G = H / KVH;
  const int qs = q_start[b];
  const int q_len = q_start[b + 1] - qs;
  const int seq_len = seq_lens[b];
  const int n_rows = q_len * G;
  const int n_row_tiles = (n_rows + BM_ROWS - 1) / BM_ROWS;
  const int my_splits = (q_len == 1) ? splits : 1;
  const int split = blockIdx.x % splits, chunk = (blockIdx.x / splits) % v_chunks, tile = blockIdx.x / (splits * v_chunks);
  if (tile >= n_row_tiles || split >= my_splits) return;
  const int row0 = (n_row_tiles - 1 - tile) * BM_ROWS;               // longest tiles first
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int prefix = seq_len - q_len;
  if (SPREAD && (q_len != 1 || n_rows > 16 * SPREAD)) return;        // (the launcher sends only such requests)
  const int wrow = SPREAD ? (warp / WPG) * 16 : warp * 16;           // first row of this warp within the tile
  const int nt0 = SPREAD ? (warp % WPG) * NTW : 0;                   // its first group of 8 keys within a tile

  unsigned char* q_s = smem;                                         // [64][DK]
  unsigned char* k_s = q_s + BM_ROWS * DK * 2;                       // [STAGES][64][DK]
  unsigned char* v_s = k_s + STAGES * BM_TILE * DK * 2;              // [STAGES][64][DV] (absent when the values are in the key rows)
  __shared__ int pages_s[BM_PAGES_S];
  __shared__ int last_flag;

  // this thread's two rows
  int pos[2], lo[2];                                                 // the row's position and the first key it sees
  float slope[2], sink2[2];                                          // (the sink in the exp2 domain; -inf: none)
  bf16* optr[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row0 + wrow + (lane >> 2) + 8 * r;
    if (row < n_rows) {
      const int t = row / G, g = row % G;
      pos[r] = prefix + t;
      lo[r] = window > 0 ? max(0, pos[r] - window + 1) : 0;
      if (block_of > 0) lo[r] = max(lo[r], pos[r] / block_of * block_of);
      slope[r] = slopes != nullptr ? slopes[kvh * G + g] : 0.f;
      sink2[r] = sinks != nullptr ? sinks[kvh * G + g] * BM_LOG2E : -INFINITY;
      optr[r] = out + (size_t)(qs + t) * out_ts + (size_t)(kvh * G + g) * out_hs + chunk * DV;
    } else {
      pos[r] = -1;                                                   // sees nothing, writes nothing
      lo[r] = 0;
      slope[r] = 0.f;
      sink2[r] = -INFINITY;
      optr[r] = nullptr;
    }
  }
  // the query tile
  // (only the rows that exist: what the others' places in shared memory hold reaches nothing, since every row of a
  // product depends on its own query row alone and a row without a position is masked whatever its scores are)
  for (int idx = threadIdx.x; idx < min(BM_ROWS, n_rows - row0) * CHK; idx += BM_WARPS * 32) {
    const int r = idx / CHK, c = idx % CHK;
    const int row = row0 + r;
    cp_async_16(q_s + swz<DK>(r, c), q + (size_t)(qs + row / G) * q_ts + (size_t)(kvh * G + row % G) * q_hs + c * 8, true);
  }
  cp_async_commit();

  // keys any row of the block can see, and this block's share of them
  const int last_row = min(row0 + BM_ROWS, n_rows) - 1;
  int j_hi = prefix + last_row / G;
  int j_lo = window > 0 ? max(0, prefix + row0 / G - window + 1) : 0;
  if (block_of > 0) j_lo = max(j_lo, (prefix + row0 / G) / block_of * block_of);
  if (my_splits > 1) {
    const int all = (j_hi - j_lo) / BM_TILE + 1;
    const int per = (all + my_splits - 1) / my_splits;
    const int first = j_lo + split * per * BM_TILE;
    j_hi = min(j_hi, first + per * BM_TILE - 1);
    j_lo = first;
  }
  const int n_tiles = (seq_len > 0 && j_hi >= j_lo) ? (j_hi - j_lo) / BM_TILE + 1 : 0;
  const int w_first = row0 + wrow, w_last = min(w_first + 15, n_rows - 1);
  const int w_pos_lo = prefix + w_first / G, w_pos_hi = (w_first < n_rows) ? prefix + w_last / G : -1;

  const int page_shift = (page & (page - 1)) == 0 ? 31 - __clz(page) : -1;
  const int page_first = j_lo / page;
  const int n_pages = n_tiles > 0 ? j_hi / page - page_first + 1 : 0;
  const bool pages_staged = n_pages <= BM_PAGES_S;
  if (pages_staged) {
    for (int i = threadIdx.x; i < n_pages; i += BM_WARPS * 32)
      pages_s[i] = block_tables[(size_t)b * table_width + page_first + i];
    __syncthreads();
  }
  const int v_width = DV * v_chunks;                                 // a value row's width in its own tensor

  // A tile's keys are dealt out to groups of LPK lanes, which bring a key row's 16-byte pieces: the row's place in the
  // cache is worked out once a key, not once a piece (index arithmetic per piece cost more issue slots than the products).
  constexpr int LPK = CHK >= 32 ? 32 : (CHK >= 16 ? 16 : 8);         // lanes a key
  constexpr int KPI = BM_WARPS * (32 / LPK);                         // keys the block brings in one round
  auto load_tile = [&](int t, int stage) {
    const int j0 = j_lo + t * BM_TILE;
    unsigned char* ks_ = k_s + (size_t)stage * BM_TILE * DK * 2;
    unsigned char* vs_ = v_s + (size_t)stage * BM_TILE * DV * 2;
    const int c0 = lane % LPK;
#pragma unroll 2
    for (int key = warp * (32 / LPK) + lane / LPK; key < BM_TILE; key += KPI) {
      const int j = j0 + key;
      const bool ok = j <= j_hi;
      size_t tok = 0;
      if (ok) {
        const int lp = page_shift >= 0 ? (j >> page_shift) : (j / page);
        const int pg = pages_staged ? pages_s[lp - page_first] : block_tables[(size_t)b * table_width + lp];
        tok = ((size_t)pg * KVH + kvh) * page + (size_t)(j - lp * page);
      }
      const bf16* krow = k_cache + tok * DK;
#pragma unroll
      for (int c = c0; c < CHK; c += LPK) cp_async_16(ks_ + swz<DK>(key, c), krow + c * 8, ok);
      if (!V_IN_K) {
        const bf16* vrow = v_cache + tok * v_width + chunk * DV;
#pragma unroll
        for (int c = c0; c < CHV; c += LPK) cp_async_16(vs_ + swz<DV>(key, c), vrow + c * 8, ok);
      }
    }
  };

  float o[NT][4];
#pragma unroll
  for (int i = 0; i < NT; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  const float inv_cap = softcap > 0.f ? 1.f / softcap : 0.f;

#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (s < n_tiles) load_tile(s, s);
    cp_async_commit();
  }
  for (int t = 0; t < n_tiles; ++t) {
    if (t + STAGES - 1 < n_tiles) load_tile(t + STAGES - 1, (t + STAGES - 1) % STAGES);
    cp_async_commit();
    cp_async_wait<STAGES - 1>();
    __syncthreads();
    const unsigned char* ks_ = k_s + (size_t)(t % STAGES) * BM_TILE * DK * 2;
    const unsigned char* vs_ = V_IN_K ? ks_ : v_s + (size_t)(t % STAGES) * BM_TILE * DV * 2;
    const int j0 = j_lo + t * BM_TILE;
    const bool in_future = j0 > w_pos_hi;                                          // warp-uniform
    const bool in_past = (window > 0 && (j0 + BM_TILE - 1) < (w_pos_lo - window + 1)) ||
                         (block_of > 0 && w_pos_lo >= 0 && (j0 + BM_TILE - 1) < w_pos_lo / block_of * block_of);
    if (!in_future && !in_past) {
      float s_acc[NTW][4];
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt) s_acc[nt][0] = s_acc[nt][1] = s_acc[nt][2] = s_acc[nt][3] = 0.f;
#pragma unroll 4
      for (int ks = 0; ks < KS; ++ks) {
        const int mat = lane >> 3, r = lane & 7;
        unsigned qf[4];
        ldmatrix_x4(qf[0], qf[1], qf[2], qf[3], q_s + swz<DK>(wrow + (mat & 1) * 8 + r, ks * 2 + (mat >> 1)));
#pragma unroll
        for (int np = 0; np < NTW / 2; ++np) {
          const int key = (nt0 / 2 + np) * 16 + (mat >> 1) * 8 + r;
          const int c = ks * 2 + (mat & 1);
          unsigned b0, b1, b2, b3;
          ldmatrix_x4(b0, b1, b2, b3, ks_ + swz<DK>(key, c));
          mma_bf16(s_acc[2 * np], qf, b0, b1);
          mma_bf16(s_acc[2 * np + 1], qf, b2, b3);
        }
      }
      // scale, cap, bias, mask; online softmax in the exp2 domain
      float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int j = j0 + (nt0 + nt) * 8 + (lane & 3) * 2 + (e & 1);
          const int p = pos[e >> 1];
          float v = s_acc[nt][e] * scale;
          if (softcap > 0.f) v = capped(v, softcap, inv_cap);
          v = (v - slope[e >> 1] * (float)(p - j)) * BM_LOG2E;
          const bool ok = (j <= p) && (j >= lo[e >> 1]) && (j <= j_hi);
          v = ok ? v : -INFINITY;
          s_acc[nt][e] = v;
          mx[e >> 1] = fmaxf(mx[e >> 1], v);
        }
      float corr[2], m_use[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 1));
        mx[r] = fmaxf(mx[r], __shfl_xor_sync(0xffffffffu, mx[r], 2));
        const float m_new = fmaxf(m_run[r], mx[r]);
        m_use[r] = (m_new == -INFINITY) ? 0.f : m_new;             // a row that has seen nothing yet
        corr[r] = exp2f(m_run[r] - m_use[r]);
        m_run[r] = m_new;
      }
      float rs[2] = {0.f, 0.f};
#pragma unroll
      for (int nt = 0; nt < NTW; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float p = exp2f(s_acc[nt][e] - m_use[e >> 1]);
          s_acc[nt][e] = p;
          rs[e >> 1] += p;
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 1);
        rs[r] += __shfl_xor_sync(0xffffffffu, rs[r], 2);
        l_run[r] = l_run[r] * corr[r] + rs[r];
      }
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        o[i][0] *= corr[0];
        o[i][1] *= corr[0];
        o[i][2] *= corr[1];
        o[i][3] *= corr[1];
      }
      // O += P . V, 16 keys at a time; P as two bfloat16 terms
#pragma unroll
      for (int kk = 0; kk < NTW / 2; ++kk) {
        unsigned hi[4], lo[4];
#pragma unroll
        for (int x = 0; x < 4; ++x) {
          const float a0 = s_acc[2 * kk + (x >> 1)][(x & 1) * 2], a1 = s_acc[2 * kk + (x >> 1)][(x & 1) * 2 + 1];
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(a0, a1);
          hi[x] = *reinterpret_cast<const unsigned*>(&h2);
          lo[x] = pack_bf16(a0 - __low2float(h2), a1 - __high2float(h2));
        }
#pragma unroll
        for (int i = 0; i < NT; i += 2) {
          const int mat = lane >> 3, r = lane & 7;
          const int key = (nt0 / 2 + kk) * 16 + (mat & 1) * 8 + r;
          const int c = i + (mat >> 1);
          unsigned b0, b1, b2, b3;
          if (V_IN_K) ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + swz<DK>(key, chunk * CHV + c));
          else ldmatrix_x4_trans(b0, b1, b2, b3, vs_ + swz<DV>(key, c));
          mma_bf16(o[i], hi, b0, b1);
          mma_bf16(o[i + 1], hi, b2, b3);
          mma_bf16(o[i], lo, b0, b1);
          mma_bf16(o[i + 1], lo, b2, b3);
        }
      }
    }
    __syncthreads();
  }
  cp_async_wait<0>();

  if (!SPREAD && my_splits == 1) {
#pragma unroll
    for (int r = 0; r < 2; ++r) {
      if (optr[r] == nullptr) continue;
      float inv = 0.f;
      if (l_run[r] > 0.f) {
        // the sink joins the denominator; both against the larger of the running maximum and the sink
        const float top = fmaxf(m_run[r], sink2[r]);
        const float down = exp2f(m_run[r] - top);
        inv = down / (l_run[r] * down + exp2f(sink2[r] - top));
      }
#pragma unroll
      for (int i = 0; i < NT; ++i) {
        const int d = i * 8 + (lane & 3) * 2;
        *reinterpret_cast<__nv_bfloat162*>(optr[r] + d) = __floats2bfloat162_rn(o[i][2 * r] * inv, o[i][2 * r + 1] * inv);
      }
    }
    return;
  }

  // partial results of a single-token request: [request][kv head][chunk][split][row][DV + 4] (one row tile: G <= 64)
  constexpr int REC = DV + 4;                                        // m, l, two floats of padding, the sums (16-byte rows)
  const size_t group = ((size_t)(b * KVH + kvh) * v_chunks + chunk) * splits;
  float* mine = scratch + (group + split) * BM_ROWS * REC;
  // (a block's 64 records: its rows, or, where warps shared the keys, 16 rows of each of the four warps)
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = wrow + (lane >> 2) + 8 * r;
    if (row >= n_rows) continue;
    float* dst = mine + (size_t)(SPREAD ? warp * 16 + row % 16 : row) * REC;
    if ((lane & 3) == 0) {
      dst[0] = m_run[r];
      dst[1] = l_run[r];
    }
#pragma unroll
    for (int i = 0; i < NT; ++i) {
      const int d = i * 8 + (lane & 3) * 2;
      *reinterpret_cast<float2*>(dst + 4 + d) = make_float2(o[i][2 * r], o[i][2 * r + 1]);
    }
  }
  __threadfence();
  __syncthreads();
  int* counter = counters + (size_t)(b * KVH + kvh) * v_chunks + chunk;
  if (threadIdx.x == 0) {
    const int ticket = atomicAdd(counter, 1);
    last_flag = ticket == my_splits - 1;
    if (last_flag) *counter = 0;                                     // ready for the next launch
  }
  __syncthreads();
  if (!last_flag) return;
  __threadfence();
  // The merge, by the block that came last.  Every load of another block's numbers is independent of the others and
  // issued before any is used: a chain of dependent L2 round trips, one a split, would cost more than the attention.
  const float* all = scratch + group * BM_ROWS * REC;
  const int n_rec = my_splits * WPG;
  // record k of row `row`: block k / WPG, and within it, where warps shared the keys, warp k % WPG of the row's group
  auto rec_of = [&](int k, int row) {
    const int in_block = SPREAD ? ((row / 16) * WPG + k % WPG) * 16 + row % 16 : row;
    return all + ((size_t)(k / WPG) * BM_ROWS + in_block) * REC;
  };
  float* m_m = reinterpret_cast<float*>(smem);                       // [64][64] maxima, then weights (the tiles are done with)
  float* l_m = m_m + BM_ROWS * BM_MAX_RECORDS;                       // [64][64] sums
  for (int idx = threadIdx.x; idx < n_rows * n_rec; idx += BM_WARPS * 32) {
    const int row = idx / n_rec, k = idx % n_rec;
    const float2 ml = __ldcg(reinterpret_cast<const float2*>(rec_of(k, row)));
    m_m[row * BM_MAX_RECORDS + k] = ml.x;
    l_m[row * BM_MAX_RECORDS + k] = ml.y;
  }
  __syncthreads();
  for (int row = threadIdx.x; row < n_rows; row += BM_WARPS * 32) {
    float mm = -INFINITY;
    for (int k = 0; k < n_rec; ++k) mm = fmaxf(mm, m_m[row * BM_MAX_RECORDS + k]);
    float ll = 0.f;
    for (int k = 0; k < n_rec; ++k) {
      const float pm = m_m[row * BM_MAX_RECORDS + k];
      const float w = pm == -INFINITY ? 0.f : exp2f(pm - mm);
      m_m[row * BM_MAX_RECORDS + k] = w;
      ll = fmaf(l_m[row * BM_MAX_RECORDS + k], w, ll);
    }
    float inv = 0.f;
    if (ll > 0.f) {
      const float sk = sinks != nullptr ? sinks[kvh * G + row] * BM_LOG2E : -INFINITY;
      const float top = fmaxf(mm, sk);
      const float down = exp2f(mm - top);
      inv = down / (ll * down + exp2f(sk - top));
    }
    for (int k = 0; k < n_rec; ++k) m_m[row * BM_MAX_RECORDS + k] *= inv;
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < n_rows * (DV / 4); idx += BM_WARPS * 32) {
    const int row = idx / (DV / 4), d = (idx % (DV / 4)) * 4;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    for (int k0 = 0; k0 < n_rec; k0 += 16) {                         // sixteen loads in flight, then their sum, in record order
      float4 v[16];
#pragma unroll
      for (int u = 0; u < 16; ++u)
        v[u] = k0 + u < n_rec ? __ldcg(reinterpret_cast<const float4*>(rec_of(k0 + u, row) + 4 + d)) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int u = 0; u < 16; ++u) {
        const float w = k0 + u < n_rec ? m_m[row * BM_MAX_RECORDS + k0 + u] : 0.f;
        a0 = fmaf(v[u].x, w, a0);
        a1 = fmaf(v[u].y, w, a1);
        a2 = fmaf(v[u].z, w, a2);
        a3 = fmaf(v[u].w, w, a3);
      }
    }
    bf16* dst = out + (size_t)qs * out_ts + (size_t)(kvh * G + row) * out_hs + chunk * DV + d;
    *reinterpret_cast<__nv_bfloat162*>(dst) = __floats2bfloat162_rn(a0, a1);
    *reinterpret_cast<__nv_bfloat162*>(dst + 2) = __floats2bfloat162_rn(a2, a3);
  }
}

template <int DK, int DV, bool V_IN_K, int STAGES, int SPREAD>
int launch(bf16* out, int out_ts, int out_hs, const bf16* q, int q_ts, int q_hs, const bf16* k_cache, const bf16* v_cache,
           const int* block_tables, const int* q_start, const int* seq_lens, int B, int table_width, int max_q_len, int H,
           int KVH, int page, float scale, float softcap, const float* slopes, int window, int v_chunks, int splits,
           float* scratch, int* counters, int block_of, const float* sinks, cudaStream_t s) {
  const size_t smem = (size_t)BM_ROWS * DK * 2 + (size_t)STAGES * BM_TILE * DK * 2 + (V_IN_K ? 0 : (size_t)STAGES * BM_TILE * DV * 2);
  static bool configured = false;
  if (!configured) {
    cudaError_t e = cudaFuncSetAttribute(attention_biased_mma_kernel<DK, DV, V_IN_K, STAGES, SPREAD>,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) TS_REFUSE((int)e, "ts_attention_biased_mma: shared memory %zu: %s", smem, cudaGetErrorString(e));
    configured = true;
  }
  const int G = H / KVH;
  dim3 grid(ceil_div(max_q_len * G, BM_ROWS) * v_chunks * splits, KVH, B);
  ts_launch(attention_biased_mma_kernel<DK, DV, V_IN_K, STAGES, SPREAD>, dim3(grid), dim3(BM_WARPS * 32), smem, s, out, out_ts, out_hs, q,
            q_ts, q_hs, k_cache, v_cache, block_tables, q_start, seq_lens, table_width, H, KVH, page, scale, softcap, slopes,
            window, v_chunks, splits, scratch, counters, block_of, sinks);
  TS_LAUNCH_CHECK();
}

// which instance takes (key width, value width, values inside the key rows): 0 none
int instance_of(int Dk, int Dv, int v_in_k) {
  if (!v_in_k && Dk == 64 && Dv == 64) return 1;
  if (!v_in_k && Dk == 128 && Dv == 128) return 2;
  if (v_in_k && Dk == 576 && Dv == 512) return 3;
  if (v_in_k && Dk == 320 && Dv == 256) return 4;
  return 0;
}

}  // namespace

TS_API int ts_attention_biased_mma_supported(int H, int KVH, int Dk, int Dv, int v_in_k, int dtype) {
  return dtype == TS_BF16 && KVH > 0 && H % KVH == 0 && instance_of(Dk, Dv, v_in_k) != 0;
}

// Columns of the value rows one block takes (the value rows are cut into Dv / this chunks).
TS_API int ts_attention_biased_mma_chunk(int Dk, int Dv, int v_in_k) {
  const int i = instance_of(Dk, Dv, v_in_k);
  return i == 0 ? 0 : (i <= 2 ? Dv : 256);
}

TS_API long long ts_attention_biased_mma_scratch_floats(int B, int KVH, int Dk, int Dv, int v_in_k, int splits) {
  const int chunk = ts_attention_biased_mma_chunk(Dk, Dv, v_in_k);
  if (chunk == 0) return 0;
  return (long long)B * KVH * (Dv / chunk) * (splits < 1 ? 1 : splits) * BM_ROWS * (chunk + 4);
}

// As ts_attention_biased; bfloat16 only; q rows 16-byte aligned (strides multiples of 8).  splits > 1 (at most 16,
// and only where a kv head serves at most 64 heads) needs scratch and zeroed counters, one per (request, kv head, chunk).
// spread: every request of the launch brings one token of at most 32 rows; an instance whose warps share each tile's
// keys runs (scratch and counters are needed at every split count).
TS_API int ts_attention_biased_mma(void* out, int out_ts, int out_hs, const void* q, int q_ts, int q_hs, const void* k_cache,
                                   const void* v_cache, const int* block_tables, const int* q_start, const int* seq_lens,
                                   int B, int table_width, int max_q_len, int H, int KVH, int Dk, int Dv, int page,
                                   float scale, float softcap, const float* slopes, int window, int splits, float* scratch,
                                   int* counters, int spread, int block_of, const float* sinks, void* stream) {
  if (B <= 0 || max_q_len <= 0) return 0;
  const int v_in_k = v_cache == nullptr;
  const int inst = (KVH > 0 && H % KVH == 0) ? instance_of(Dk, Dv, v_in_k) : 0;
  if (inst == 0) TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_biased_mma: H=%d KVH=%d keys %d values %d", H, KVH, Dk, Dv);
  if ((q_ts % 8) || (q_hs % 8) || ((uintptr_t)q & 15) || (out_ts % 2) || (out_hs % 2) || ((uintptr_t)out & 3))
    TS_REFUSE(TS_ERR_UNSUPPORTED, "ts_attention_biased_mma: query rows must start on 16-byte boundaries");
  if (B > 65535 || KVH > 65535) TS_REFUSE(TS_ERR_LIMIT, "ts_attention_biased_mma: %d requests / %d kv heads", B, KVH);
  if (splits < 1) splits = 1;
  if (splits > 1 && (splits > BM_MAX_SPLITS || H / KVH > BM_ROWS || scratch == nullptr || counters == nullptr))
    TS_REFUSE(TS_ERR_LIMIT, "ts_attention_biased_mma: %d splits", splits);
  if (spread && (max_q_len != 1 || H / KVH > 32 || scratch == nullptr || counters == nullptr))
    TS_REFUSE(TS_ERR_SHAPE, "ts_attention_biased_mma: the warps share the keys of single tokens with at most 32 rows, through scratch");
  const int groups = H / KVH > 16 ? 2 : 1;                            // row groups of 16 among a request's rows
  cudaStream_t s = (cudaStream_t)stream;
#define TS_BM(DKK, DVV, VK, ST, CHUNKS)                                                                                       \
  do {                                                                                                                        \
    if (spread && groups == 1)                                                                                                \
      return launch<DKK, DVV, VK, ST, 1>((bf16*)out, out_ts, out_hs, (const bf16*)q, q_ts, q_hs, (const bf16*)k_cache,        \
                                         (const bf16*)v_cache, block_tables, q_start, seq_lens, B, table_width, max_q_len,    \
                                         H, KVH, page, scale, softcap, slopes, window, CHUNKS, splits, scratch, counters, block_of, sinks, s); \
    if (spread)                                                                                                               \
      return launch<DKK, DVV, VK, ST, 2>((bf16*)out, out_ts, out_hs, (const bf16*)q, q_ts, q_hs, (const bf16*)k_cache,        \
                                         (const bf16*)v_cache, block_tables, q_start, seq_lens, B, table_width, max_q_len,    \
                                         H, KVH, page, scale, softcap, slopes, window, CHUNKS, splits, scratch, counters, block_of, sinks, s); \
    return launch<DKK, DVV, VK, ST, 0>((bf16*)out, out_ts, out_hs, (const bf16*)q, q_ts, q_hs, (const bf16*)k_cache,      \
                                           (const bf16*)v_cache, block_tables, q_start, seq_lens, B, table_width, max_q_len,  \
                                           H, KVH, page, scale, softcap, slopes, window, CHUNKS, splits, scratch, counters, block_of, sinks, s); \
  } while (0)
  if (inst == 1) TS_BM(64, 64, false, 3, 1);
  if (inst == 2) TS_BM(128, 128, false, 2, 1);                        // (two stages: 80 KB a block, so two blocks share an SM)
  if (inst == 3) TS_BM(576, 256, true, 2, 2);
  TS_BM(320, 256, true, 3, 1);
#undef TS_BM
}
