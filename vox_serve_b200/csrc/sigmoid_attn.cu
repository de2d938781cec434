// Attention whose weights are not normalised over the keys, over a sliding window plus pooled blocks:
//
//   s_ij  = (q_i . k_j) * scale;   s <- cap * tanh(s / cap) (cap > 0)
//   o_i   = out_scale * sum_j sigmoid(s_ij + bias[head]) * v_j
//
// where j runs over the tokens of the window (0 <= i - j < window; window <= 0: all earlier tokens) and, with pool = P > 0,
// over one pooled key / value per block of P positions that ended before the window began (block b = positions bP .. bP + P - 1
// is seen by i when bP + P - 1 <= i - window): the mean of the block's cached keys / values.  A pooled entry is scored, capped,
// biased and weighted exactly as a token is.  Grouped heads: query head h reads key/value head h / (H / G).  Queries, the page cache and the output take the
// compute type; pooled blocks are kept in fp32 in a cache of their own; scores, weights and sums are fp32.
//
// Because nothing is normalised, partial sums over disjoint key ranges simply add up: a row's keys can be dealt to several
// CTAs whose fp32 partial planes are summed afterwards (single-token rows of small batches).
//
//   vb_qk_norm_append    tail of a fused (q | k | v) projection: RMS norm of q and of k over their WHOLE width (all heads at
//                        once, one weight per coordinate), q out, k and v appended to the pages
//   vb_pool_blocks       the blocks completed by the step's rows: mean of their P cached keys / values -> pooled cache
//                        [pages][ceil(page / P)][G][dim]: block b of a request lives in the page of its first position
//   vb_sigmoid_attn      the attention: tiles of a prompt portion's rows (16 rows x the heads of a key/value head per CTA share
//                        every staged key / value chunk) or single rows (optionally split over keys)
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 1
#include "common.cuh"

namespace vb {

template <typename T> __device__ __forceinline__ float sa_to_f(T v);
template <> __device__ __forceinline__ float sa_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float sa_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T sa_from_f(float v);
template <> __device__ __forceinline__ float sa_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 sa_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// ---- projection tail ----------------------------------------------------------------------------------------------------
template <typename CT>
__global__ void __launch_bounds__(256) qk_norm_append_kernel(const float* __restrict__ proj, int ldp, int q_off, int k_off,
                                                             int v_off, const float* __restrict__ wq, const float* __restrict__ wk,
                                                             float eps, CT* __restrict__ q_out, CT* __restrict__ k_cache,
                                                             CT* __restrict__ v_cache, const int32_t* __restrict__ row_req,
                                                             const int32_t* __restrict__ pos, const int32_t* __restrict__ page_indptr,
                                                             const int32_t* __restrict__ page_indices, int page_size, int nq,
                                                             int nk, int nv) {
  __shared__ float red[2][8];
  pdl_sync();
  const size_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = proj + t * ldp;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < nq; i += 256) sq = fmaf(row[q_off + i], row[q_off + i], sq);
  for (int i = threadIdx.x; i < nk; i += 256) sk = fmaf(row[k_off + i], row[k_off + i], sk);
  sq = warp_sum(sq);
  sk = warp_sum(sk);
  if (lane == 0) { red[0][warp] = sq; red[1][warp] = sk; }
  __syncthreads();
  sq = sk = 0.f;
#pragma unroll
  for (int i = 0; i < 8; ++i) { sq += red[0][i]; sk += red[1][i]; }
  const float rq = wq ? 1.f / sqrtf(sq / nq + eps) : 1.f, rk = wk ? 1.f / sqrtf(sk / nk + eps) : 1.f;
  const int b = row_req[t], ps = pos[t];
  const size_t tok = static_cast<size_t>(page_indices[page_indptr[b] + ps / page_size]) * page_size + ps % page_size;
  for (int i = threadIdx.x; i < nq; i += 256) q_out[t * nq + i] = sa_from_f<CT>(row[q_off + i] * rq * (wq ? wq[i] : 1.f));
  for (int i = threadIdx.x; i < nk; i += 256) k_cache[tok * nk + i] = sa_from_f<CT>(row[k_off + i] * rk * (wk ? wk[i] : 1.f));
  for (int i = threadIdx.x; i < nv; i += 256) v_cache[tok * nv + i] = sa_from_f<CT>(row[v_off + i]);
}

// ---- pooled blocks --------------------------------------------------------------------------------------------------------
// grid (blocks a request can complete in the step, B): CTA (k, b) forms the k-th block that the rows of request b complete
template <typename CT>
__global__ void __launch_bounds__(256) pool_blocks_kernel(float* __restrict__ kp, float* __restrict__ vp,
                                                          const CT* __restrict__ k_cache, const CT* __restrict__ v_cache,
                                                          const int32_t* __restrict__ qo, const int32_t* __restrict__ pos,
                                                          const int32_t* __restrict__ page_indptr,
                                                          const int32_t* __restrict__ page_indices, int page_size, int P,
                                                          int pool_slots, int nk, int nv) {
  pdl_sync();
  const int b = blockIdx.y;
  const int r0 = qo[b], n = qo[b + 1] - r0;
  if (n <= 0) return;
  const int p0 = pos[r0], p1 = p0 + n;                 // the step's rows hold positions p0 .. p1 - 1
  const int blk = p0 / P + blockIdx.x;                 // the first block that ends at or after p0, and on
  if (blk * P + P > p1) return;
  const int32_t* pages = page_indices + page_indptr[b];
  const int first = blk * P;
  const size_t dst = static_cast<size_t>(pages[first / page_size]) * pool_slots + (first % page_size) / P;
  const float inv = 1.f / static_cast<float>(P);
  // (grid.z deals the block's values to CTAs: a thread forms one mean, in position order)
  for (int e = blockIdx.z * 256 + threadIdx.x; e < nk + nv; e += gridDim.z * 256) {
    float s = 0.f;
#pragma unroll 4
    for (int i = 0; i < P; ++i) {
      const int ps = first + i;
      const size_t tok = static_cast<size_t>(pages[ps / page_size]) * page_size + ps % page_size;
      s += e < nk ? sa_to_f(k_cache[tok * nk + e]) : sa_to_f(v_cache[tok * nv + e - nk]);
    }
    if (e < nk) kp[dst * nk + e] = s * inv;
    else vp[dst * nv + e - nk] = s * inv;
  }
}

// ---- attention --------------------------------------------------------------------------------------------------------------
struct SigmoidAttnParams {
  const void* q;          // [T][H * dim]
  const void* k_cache;    // [pages][page][G][dim]
  const void* v_cache;    // [pages][page][G][vdim]
  const float* kp;        // [pages][pool_slots][G][dim]  (pool > 0)
  const float* vp;
  const float* head_bias; // [H] or nullptr
  void* out;              // [T][ld_out] compute type
  int ld_out;
  float* part;            // split rows: [splits][rows][H * vdim] fp32 partial planes
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  const int32_t* qo_indptr;
  const int32_t* tile_req;
  const int32_t* tile_row0;
  const int32_t* row_list;
  int n_items, H, G, dim, vdim, page_size, window, pool, pool_slots;
  float scale, cap, out_scale;
  int tile_rows, heads_per_cta, splits;
};

constexpr int SA_ROWS = 16;       // rows of a tile per CTA
constexpr int SA_KEYS = 32;       // keys per staged chunk (a lane per key in the score phase)
constexpr int SA_THREADS = 256;

// keys of position ps: pooled blocks [0, nb) and tokens [lo, ps]
__device__ __forceinline__ void sa_range(const SigmoidAttnParams& p, int ps, int& nb, int& lo) {
  if (p.window <= 0) { nb = 0; lo = 0; return; }
  lo = max(0, ps - p.window + 1);
  nb = (p.pool > 0 && ps - p.window + 1 > 0) ? (ps - p.window + 1) / p.pool : 0;
}

template <typename CT>
__global__ void __launch_bounds__(SA_THREADS) sigmoid_attn_kernel(SigmoidAttnParams p) {
  // (everything in dynamic shared memory: with static arrays beside it the kernel could not be given the device's maximum)
  extern __shared__ __align__(16) float sa_sm[];
  long long* key_off = reinterpret_cast<long long*>(sa_sm);       // [SA_KEYS] element offset of the chunk's keys in their cache
  int* key_id = reinterpret_cast<int*>(key_off + SA_KEYS);        // [SA_KEYS] block index (pooled) or position (token); -1: none
  float* sa_data = reinterpret_cast<float*>(key_id + SA_KEYS);
  pdl_sync();
  const int R = p.H / p.G;
  const int hc_n = (R + p.heads_per_cta - 1) / p.heads_per_cta;
  const int g = blockIdx.y / hc_n, hc = blockIdx.y - g * hc_n;
  const int h0 = g * R + hc * p.heads_per_cta, nh = min(p.heads_per_cta, R - hc * p.heads_per_cta);
  int b, row0, nrows, item_row = blockIdx.x;
  if (p.tile_req) {
    const int sub_n = p.tile_rows / SA_ROWS, tile = blockIdx.x / sub_n, sub = blockIdx.x - tile * sub_n;
    b = p.tile_req[tile];
    const int t0 = p.tile_row0[tile], end = min(p.qo_indptr[b + 1], t0 + p.tile_rows);
    row0 = t0 + sub * SA_ROWS;
    nrows = min(SA_ROWS, end - row0);
  } else {
    row0 = p.row_list ? p.row_list[blockIdx.x] : blockIdx.x;
    b = p.row_req[row0];
    nrows = 1;
  }
  if (nrows <= 0) return;
  const int pairs = nrows * nh, D = p.dim, V = p.vdim, ldk = D + 1;
  float* qs = sa_data;                                 // [pairs][D]
  float* acc = qs + SA_ROWS * p.heads_per_cta * D;     // [pairs][V]
  float* ks = acc + SA_ROWS * p.heads_per_cta * V;     // [SA_KEYS][D + 1]
  float* vs = ks + SA_KEYS * ldk;                      // [SA_KEYS][V]
  const CT* q = static_cast<const CT*>(p.q);
  for (int i = threadIdx.x; i < pairs * D; i += SA_THREADS) {
    const int pr = i / D, d = i - pr * D, r = pr / nh, hh = pr - r * nh;
    qs[i] = sa_to_f(q[(static_cast<size_t>(row0 + r) * p.H + h0 + hh) * D + d]);
  }
  for (int i = threadIdx.x; i < pairs * V; i += SA_THREADS) acc[i] = 0.f;
  const int p_first = p.pos[row0], p_last = p_first + nrows - 1;
  int nb_max, lo_last, nb_first, lo_first;
  sa_range(p, p_last, nb_max, lo_last);
  sa_range(p, p_first, nb_first, lo_first);
  // key items of the tile: pooled blocks [0, nb_max) then tokens [lo_first, p_last]
  const int n_items = nb_max + (p_last - lo_first + 1);
  int it0 = 0, it1 = n_items;
  if (p.splits > 1) {                                   // this CTA's share of the key chunks
    const int chunks = (n_items + SA_KEYS - 1) / SA_KEYS, per = (chunks + p.splits - 1) / p.splits;
    it0 = min(n_items, static_cast<int>(blockIdx.z) * per * SA_KEYS);
    it1 = min(n_items, it0 + per * SA_KEYS);
  }
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  for (int c0 = it0; c0 < it1; c0 += SA_KEYS) {
    __syncthreads();                                    // the previous chunk is consumed (and qs / acc are initialised)
    if (threadIdx.x < SA_KEYS) {
      const int it = c0 + threadIdx.x;
      int id = -1;
      long long off = 0;
      if (it < it1) {
        if (it < nb_max) {
          id = it;
          const int first = it * p.pool;
          off = static_cast<long long>(pages[first / p.page_size]) * p.pool_slots + (first % p.page_size) / p.pool;
        } else {
          id = lo_first + it - nb_max;
          off = static_cast<long long>(pages[id / p.page_size]) * p.page_size + id % p.page_size;
        }
      }
      key_id[threadIdx.x] = id;
      key_off[threadIdx.x] = off;
    }
    __syncthreads();
    for (int i = threadIdx.x; i < SA_KEYS * D; i += SA_THREADS) {
      const int kk = i / D, d = i - kk * D;
      float v = 0.f;
      if (key_id[kk] >= 0) {
        const size_t e = (static_cast<size_t>(key_off[kk]) * p.G + g) * D + d;
        v = c0 + kk < nb_max ? p.kp[e] : sa_to_f(kc[e]);
      }
      ks[kk * ldk + d] = v;
    }
    for (int i = threadIdx.x; i < SA_KEYS * V; i += SA_THREADS) {
      const int kk = i / V, d = i - kk * V;
      float v = 0.f;
      if (key_id[kk] >= 0) {
        const size_t e = (static_cast<size_t>(key_off[kk]) * p.G + g) * V + d;
        v = c0 + kk < nb_max ? p.vp[e] : sa_to_f(vc[e]);
      }
      vs[kk * V + d] = v;
    }
    __syncthreads();
    const int id = key_id[lane];
    const bool pooled = c0 + lane < nb_max;
    for (int pr = warp; pr < pairs; pr += SA_THREADS / 32) {
      const int r = pr / nh, hh = pr - r * nh, ps = p_first + r;
      int nb, lo;
      sa_range(p, ps, nb, lo);
      const bool seen = id >= 0 && (pooled ? id < nb : (id >= lo && id <= ps));
      float w = 0.f;
      if (__any_sync(0xffffffffu, seen)) {
        const float* qr = qs + pr * D;
        const float* kr = ks + lane * ldk;
        float s = 0.f;
        for (int d = 0; d < D; ++d) s = fmaf(qr[d], kr[d], s);
        s *= p.scale;
        if (p.cap > 0.f) s = p.cap * tanhf(s / p.cap);
        if (p.head_bias) s += p.head_bias[h0 + hh];
        w = seen ? 1.f / (1.f + expf(-s)) : 0.f;
      } else {
        continue;
      }
      float* a = acc + pr * V;
      for (int v0 = 0; v0 < V; v0 += 32) {
        const int vi = v0 + lane;
        float o = 0.f;
#pragma unroll 8
        for (int kk = 0; kk < SA_KEYS; ++kk) {
          const float wk = __shfl_sync(0xffffffffu, w, kk);
          if (vi < V) o = fmaf(wk, vs[kk * V + vi], o);
        }
        if (vi < V) a[vi] += o;
      }
    }
  }
  __syncthreads();
  if (p.splits > 1) {
    float* part = p.part + (static_cast<size_t>(blockIdx.z) * p.n_items + item_row) * p.H * V;
    for (int i = threadIdx.x; i < pairs * V; i += SA_THREADS) {
      const int pr = i / V, d = i - pr * V, hh = pr % nh;
      part[(h0 + hh) * V + d] = acc[i];
    }
    return;
  }
  CT* out = static_cast<CT*>(p.out);
  for (int i = threadIdx.x; i < pairs * V; i += SA_THREADS) {
    const int pr = i / V, d = i - pr * V, r = pr / nh, hh = pr - r * nh;
    out[static_cast<size_t>(row0 + r) * p.ld_out + (h0 + hh) * V + d] = sa_from_f<CT>(p.out_scale * acc[i]);
  }
}

// ---- the same on tensor-core tiles (bf16, head sizes in multiples of 16, values up to 128 per head) ---------------------------
// CTA = 4 warps = 64 query rows: 64 / nh rows of a prompt portion's tile times nh = 1 / 2 / 4 heads of one key/value head (warp w
// holds 16 token rows of one head), or -- single-token rows -- one token's heads (one row per warp in use).  Chunks of 64 keys
// (pooled blocks, rounded to bf16 here, then tokens) are staged once for all of them; S = Q K^T by mma.sync m16n8k16 with fp32
// accumulators, the weights sigmoid(cap(S) + bias) are formed on the accumulator fragments, masked, rounded to bf16 and fed
// back as the A operand of O += P V (values read through transposing ldmatrix).
constexpr int SM_KEYS = 64;

// sigmoid(cap(s) + bias) from exponentials of the fast unit (relative error ~1e-6: below the bf16 rounding the weight gets as an
// mma operand): cap tanh(s / cap) = cap - 2 cap / (exp(2 s / cap) + 1), sigmoid(x) = 1 / (1 + exp(-x)); both saturate cleanly
__device__ __forceinline__ float sa_fast_weight(float s, float cap, float inv_cap2, float bias) {
  if (cap > 0.f) s = cap - __fdividef(2.f * cap, __expf(s * inv_cap2) + 1.f);
  return __fdividef(1.f, 1.f + __expf(-(s + bias)));
}

template <int NV>
__global__ void __launch_bounds__(128) sigmoid_attn_mma_kernel(SigmoidAttnParams p) {
  extern __shared__ __align__(16) unsigned char sm_raw[];
  using bf16 = __nv_bfloat16;
  const int D = p.dim, V = p.vdim, QLD = D + 8, VLD = V + 8, D8 = D / 8, V8 = V / 8;
  bf16* Qs = reinterpret_cast<bf16*>(sm_raw);                     // [64][QLD]
  bf16* Ks = Qs + 64 * QLD;                                       // [SM_KEYS][QLD]
  bf16* Vs = Ks + SM_KEYS * QLD;                                  // [SM_KEYS][VLD]
  long long* key_off = reinterpret_cast<long long*>(Vs + SM_KEYS * VLD);
  int* key_id = reinterpret_cast<int*>(key_off + SM_KEYS);
  int* see = key_id + SM_KEYS;                                    // [SM_KEYS][2]: the first and last position that sees the key
  pdl_sync();
  const int R = p.H / p.G, nh = p.heads_per_cta, wph = 4 / nh;    // warps per head
  const int hc_n = (R + nh - 1) / nh;
  const int g = blockIdx.y / hc_n, hc = blockIdx.y - g * hc_n;
  const int h0 = g * R + hc * nh, nh_eff = min(nh, R - hc * nh), TR = 16 * wph;
  int b, row0, nrows;
  const int item_row = blockIdx.x;
  if (p.tile_req) {
    const int sub_n = p.tile_rows / TR, tile = blockIdx.x / sub_n, sub = blockIdx.x - tile * sub_n;
    b = p.tile_req[tile];
    const int t0 = p.tile_row0[tile], end = min(p.qo_indptr[b + 1], t0 + p.tile_rows);
    row0 = t0 + sub * TR;
    nrows = min(TR, end - row0);
  } else {
    row0 = p.row_list ? p.row_list[blockIdx.x] : blockIdx.x;
    b = p.row_req[row0];
    nrows = 1;
  }
  if (nrows <= 0) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int my_h = warp / wph, my_rb = (warp - my_h * wph) * 16;   // this warp's head and first token row
  const bool active = my_h < nh_eff && my_rb < nrows;
  const bf16* q = static_cast<const bf16*>(p.q);
  for (int i = tid; i < 64 * D8; i += 128) {
    const int pr = i / D8, c = (i - pr * D8) * 8, w_ = pr >> 4, hh = w_ / wph, r = (w_ - hh * wph) * 16 + (pr & 15);
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (hh < nh_eff && r < nrows) v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(row0 + r) * p.H + h0 + hh) * D + c);
    *reinterpret_cast<uint4*>(Qs + pr * QLD + c) = v;
  }
  float O[2 * NV][4];
#pragma unroll
  for (int n = 0; n < 2 * NV; ++n) O[n][0] = O[n][1] = O[n][2] = O[n][3] = 0.f;
  const int p_first = p.pos[row0], p_last = p_first + nrows - 1;
  int nb_max, lo_last, nb_first, lo_first;
  sa_range(p, p_last, nb_max, lo_last);
  sa_range(p, p_first, nb_first, lo_first);
  const int n_items = nb_max + (p_last - lo_first + 1);
  int it0 = 0, it1 = n_items;
  if (p.splits > 1) {
    const int chunks = (n_items + SM_KEYS - 1) / SM_KEYS, per = (chunks + p.splits - 1) / p.splits;
    it0 = min(n_items, static_cast<int>(blockIdx.z) * per * SM_KEYS);
    it1 = min(n_items, it0 + per * SM_KEYS);
  }
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const bf16* kc = static_cast<const bf16*>(p.k_cache);
  const bf16* vc = static_cast<const bf16*>(p.v_cache);
  const float bias = (p.head_bias && my_h < nh_eff) ? p.head_bias[h0 + my_h] : 0.f;
  const int ra = my_rb + (lane >> 2), psa = p_first + ra, psb = psa + 8;
  const int ps_a = ra < nrows ? psa : -1, ps_b = ra + 8 < nrows ? psb : -1;      // (-1: no such row; it sees nothing)
  const float inv_cap2 = p.cap > 0.f ? 2.f / p.cap : 0.f;
  for (int c0 = it0; c0 < it1; c0 += SM_KEYS) {
    __syncthreads();
    if (tid < SM_KEYS) {
      const int it = c0 + tid;
      int id = -1;
      long long off = 0;
      if (it < it1) {
        if (it < nb_max) {
          id = it;
          const int first = it * p.pool;
          off = static_cast<long long>(pages[first / p.page_size]) * p.pool_slots + (first % p.page_size) / p.pool;
        } else {
          id = lo_first + it - nb_max;
          off = static_cast<long long>(pages[id / p.page_size]) * p.page_size + id % p.page_size;
        }
      }
      key_id[tid] = id;
      key_off[tid] = off;
      // a token j is seen from j to j + window - 1, a pooled block from the first position whose window lies wholly behind it
      int from = 0x7fffffff, to = -1;
      if (id >= 0) {
        const bool pooled = it < nb_max;
        from = pooled ? id * p.pool + p.pool - 1 + p.window : id;
        to = (pooled || p.window <= 0) ? 0x7fffffff : id + p.window - 1;
      }
      see[2 * tid] = from;
      see[2 * tid + 1] = to;
    }
    __syncthreads();
    // 16-byte pieces of the chunk's key and value rows, eight per thread at a time: all loads of a batch are issued before the
    // first store (a load behind a shared-memory store would wait for it)
    const int n_pieces = SM_KEYS * (D8 + V8);
    for (int i0 = tid; i0 < n_pieces; i0 += 128 * 8) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 128;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (i < n_pieces) {
          const int kk = i / (D8 + V8), j = i - kk * (D8 + V8);
          const bool is_k = j < D8;
          const int c = (is_k ? j : j - D8) * 8, n = is_k ? D : V;
          if (key_id[kk] >= 0) {
            const size_t e = (static_cast<size_t>(key_off[kk]) * p.G + g) * n + c;
            if (c0 + kk < nb_max) {
              const float* src = (is_k ? p.kp : p.vp) + e;
              const float4 a = __ldg(reinterpret_cast<const float4*>(src)), bq = __ldg(reinterpret_cast<const float4*>(src + 4));
              v[u] = make_uint4(pack_bf16(a.x, a.y), pack_bf16(a.z, a.w), pack_bf16(bq.x, bq.y), pack_bf16(bq.z, bq.w));
            } else {
              v[u] = __ldg(reinterpret_cast<const uint4*>((is_k ? kc : vc) + e));
            }
          }
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = i0 + u * 128;
        if (i < n_pieces) {
          const int kk = i / (D8 + V8), j = i - kk * (D8 + V8);
          const bool is_k = j < D8;
          *reinterpret_cast<uint4*>((is_k ? Ks + kk * QLD : Vs + kk * VLD) + (is_k ? j : j - D8) * 8) = v[u];
        }
      }
    }
    __syncthreads();
    if (!active) continue;
    float S[SM_KEYS / 8][4];
#pragma unroll
    for (int n = 0; n < SM_KEYS / 8; ++n) S[n][0] = S[n][1] = S[n][2] = S[n][3] = 0.f;
    for (int kb = 0; kb < D / 16; ++kb) {
      uint32_t af[4];
      ldmatrix_x4(af, smem_u32(Qs + (warp * 16 + (lane & 15)) * QLD + kb * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int np = 0; np < SM_KEYS / 16; ++np) {
        uint32_t bf[4];
        ldmatrix_x4(bf, smem_u32(Ks + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * QLD + kb * 16 + ((lane >> 3) & 1) * 8));
        mma_bf16_16816(S[2 * np], af, bf[0], bf[1]);
        mma_bf16_16816(S[2 * np + 1], af, bf[2], bf[3]);
      }
    }
    bool any = false;
#pragma unroll
    for (int nt = 0; nt < SM_KEYS / 8; ++nt) {
      const int4 ft = *reinterpret_cast<const int4*>(see + 2 * (nt * 8 + (lane & 3) * 2));      // (from, to) of the lane's two keys
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int ps = e >= 2 ? ps_b : ps_a, from = (e & 1) ? ft.z : ft.x, to = (e & 1) ? ft.w : ft.y;
        float w = 0.f;
        if (ps >= from && ps <= to) {
          w = sa_fast_weight(S[nt][e] * p.scale, p.cap, inv_cap2, bias);
          any = true;
        }
        S[nt][e] = w;
      }
    }
    if (!__any_sync(0xffffffffu, any)) continue;
#pragma unroll
    for (int kb = 0; kb < SM_KEYS / 16; ++kb) {
      uint32_t a[4] = {pack_bf16(S[2 * kb][0], S[2 * kb][1]), pack_bf16(S[2 * kb][2], S[2 * kb][3]),
                       pack_bf16(S[2 * kb + 1][0], S[2 * kb + 1][1]), pack_bf16(S[2 * kb + 1][2], S[2 * kb + 1][3])};
#pragma unroll
      for (int np = 0; np < NV; ++np) {
        if (np * 16 < V) {
          uint32_t bf[4];
          ldmatrix_x4_trans(bf, smem_u32(Vs + (kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * VLD + np * 16 + (lane >> 4) * 8));
          mma_bf16_16816(O[2 * np], a, bf[0], bf[1]);
          mma_bf16_16816(O[2 * np + 1], a, bf[2], bf[3]);
        }
      }
    }
  }
  if (!active) return;
  const int h = h0 + my_h;
#pragma unroll
  for (int nt = 0; nt < 2 * NV; ++nt) {
    const int v = nt * 8 + (lane & 3) * 2;
    if (v >= V) continue;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      const int r = ra + 8 * half;
      if (r >= nrows) continue;
      const float o0 = O[nt][2 * half], o1 = O[nt][2 * half + 1];
      if (p.splits > 1) {
        float* part = p.part + (static_cast<size_t>(blockIdx.z) * p.n_items + item_row) * p.H * V + h * V + v;
        part[0] = o0;
        part[1] = o1;
      } else {
        bf16* out = static_cast<bf16*>(p.out) + static_cast<size_t>(row0 + r) * p.ld_out + h * V + v;
        *reinterpret_cast<uint32_t*>(out) = pack_bf16(p.out_scale * o0, p.out_scale * o1);
      }
    }
  }
}

// out[row] = out_scale * sum of the splits' partial planes, in split order
template <typename CT>
__global__ void sigmoid_attn_sum_kernel(CT* __restrict__ out, int ld_out, const float* __restrict__ part,
                                        const int32_t* __restrict__ row_list, int rows, int n, int splits, float out_scale) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= static_cast<long long>(rows) * n) return;
  const int r = static_cast<int>(i / n), c = static_cast<int>(i - static_cast<long long>(r) * n);
  float s = 0.f;
  for (int k = 0; k < splits; ++k) s += part[(static_cast<size_t>(k) * rows + r) * n + c];
  const int t = row_list ? row_list[r] : r;
  out[static_cast<size_t>(t) * ld_out + c] = sa_from_f<CT>(out_scale * s);
}

}  // namespace vb

using namespace vb;
using bf16 = __nv_bfloat16;

extern "C" {

int vb_qk_norm_append(const float* d_proj, int ldp, int q_off, int k_off, int v_off, const float* d_q_norm,
                      const float* d_k_norm, float eps, void* d_q_out, void* d_k_cache, void* d_v_cache,
                      const int32_t* d_row_req, const int32_t* d_pos, const int32_t* d_page_indptr,
                      const int32_t* d_page_indices, int page_size, int T, int nq, int nk, int nv, int dtype, void* stream) {
  VB_CHECK_ARG(d_proj && d_q_out && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_qk_norm_append: null pointer");
  VB_CHECK_ARG(nq > 0 && nk > 0 && nv > 0 && page_size > 0, "vb_qk_norm_append: bad sizes");
  if (T <= 0) return 0;
  if (dtype == 1)
    VB_LAUNCH_PDL(qk_norm_append_kernel<float>, T, 256, 0, stream, d_proj, ldp, q_off, k_off, v_off, d_q_norm, d_k_norm, eps,
                  static_cast<float*>(d_q_out), static_cast<float*>(d_k_cache), static_cast<float*>(d_v_cache), d_row_req, d_pos,
                  d_page_indptr, d_page_indices, page_size, nq, nk, nv);
  else
    VB_LAUNCH_PDL(qk_norm_append_kernel<bf16>, T, 256, 0, stream, d_proj, ldp, q_off, k_off, v_off, d_q_norm, d_k_norm, eps,
                  static_cast<bf16*>(d_q_out), static_cast<bf16*>(d_k_cache), static_cast<bf16*>(d_v_cache), d_row_req, d_pos,
                  d_page_indptr, d_page_indices, page_size, nq, nk, nv);
  return 0;
}

int vb_pool_blocks(float* d_kp, float* d_vp, const void* d_k_cache, const void* d_v_cache, const int32_t* d_qo_indptr,
                   const int32_t* d_pos, const int32_t* d_page_indptr, const int32_t* d_page_indices, int page_size, int pool,
                   int T, int B, int nk, int nv, int dtype, void* stream) {
  VB_CHECK_ARG(d_kp && d_vp && d_k_cache && d_v_cache && d_qo_indptr && d_pos && d_page_indptr && d_page_indices,
               "vb_pool_blocks: null pointer");
  VB_CHECK_ARG(pool > 0 && page_size > 0 && nk > 0 && nv > 0, "vb_pool_blocks: bad sizes");
  if (T <= 0 || B <= 0) return 0;
  const int slots = (page_size + pool - 1) / pool;
  dim3 grid(T / pool + 1, B, (nk + nv + 255) / 256 < 16 ? (nk + nv + 255) / 256 : 16);
  if (dtype == 1)
    VB_LAUNCH_PDL(pool_blocks_kernel<float>, grid, 256, 0, stream, d_kp, d_vp, static_cast<const float*>(d_k_cache),
                  static_cast<const float*>(d_v_cache), d_qo_indptr, d_pos, d_page_indptr, d_page_indices, page_size, pool, slots, nk, nv);
  else
    VB_LAUNCH_PDL(pool_blocks_kernel<bf16>, grid, 256, 0, stream, d_kp, d_vp, static_cast<const bf16*>(d_k_cache),
                  static_cast<const bf16*>(d_v_cache), d_qo_indptr, d_pos, d_page_indptr, d_page_indices, page_size, pool, slots, nk, nv);
  return 0;
}

int vb_sigmoid_attn(void* d_out, int ld_out, const void* d_q, const void* d_k_cache, const void* d_v_cache, const float* d_kp,
                    const float* d_vp, const float* d_head_bias, const int32_t* d_row_req, const int32_t* d_pos,
                    const int32_t* d_page_indptr, const int32_t* d_page_indices, const int32_t* d_qo_indptr,
                    const int32_t* d_tile_req, const int32_t* d_tile_row0, int n_tiles, int tile_rows,
                    const int32_t* d_row_list, int n_rows, int H, int G, int dim, int vdim, int page_size, int window, int pool,
                    float scale, float cap, float out_scale, float* d_part, long long part_floats, int max_keys, int dtype,
                    void* stream) {
  VB_CHECK_ARG(d_out && d_q && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_sigmoid_attn: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && dim <= 256 && vdim <= 256,
               "vb_sigmoid_attn: H %d, G %d, dim %d, vdim %d (heads a multiple of key/value heads, sizes up to 256)", H, G, dim, vdim);
  VB_CHECK_ARG(pool <= 0 || (d_kp && d_vp && window > 0), "vb_sigmoid_attn: pooled blocks need their cache and a window");
  const bool tiled = d_tile_req != nullptr;
  VB_CHECK_ARG(!tiled || (d_tile_row0 && d_qo_indptr && tile_rows > 0 && tile_rows % SA_ROWS == 0),
               "vb_sigmoid_attn: tiles of a multiple of %d rows", SA_ROWS);
  const int R = H / G;
  // tensor-core tiles: bf16, head sizes in multiples of 16 (keys up to 256, values up to 128 dims), 4-byte aligned output rows
  const bool mma = dtype == 0 && dim % 16 == 0 && vdim % 16 == 0 && vdim <= 128 && ld_out % 2 == 0 && (!tiled || tile_rows == 64) &&
                   reinterpret_cast<uintptr_t>(d_out) % 4 == 0 && reinterpret_cast<uintptr_t>(d_q) % 16 == 0 &&
                   reinterpret_cast<uintptr_t>(d_k_cache) % 16 == 0 && reinterpret_cast<uintptr_t>(d_v_cache) % 16 == 0 &&
                   (pool <= 0 || (reinterpret_cast<uintptr_t>(d_kp) % 16 == 0 && reinterpret_cast<uintptr_t>(d_vp) % 16 == 0));
  const int hpc = mma ? (R >= 4 ? 4 : (R >= 2 ? 2 : 1)) : (R < 4 ? R : 4);
  const int rows_per_cta = mma ? 64 / hpc : SA_ROWS, chunk_keys = mma ? SM_KEYS : SA_KEYS;
  const int items = tiled ? n_tiles * (tile_rows / rows_per_cta) : n_rows;
  if (items <= 0) return 0;
  SigmoidAttnParams p{d_q, d_k_cache, d_v_cache, d_kp, d_vp, d_head_bias, d_out, ld_out, d_part, d_row_req, d_pos, d_page_indptr,
                      d_page_indices, d_qo_indptr, d_tile_req, d_tile_row0, d_row_list, items, H, G, dim, vdim, page_size, window,
                      pool, pool > 0 ? (page_size + pool - 1) / pool : 0, scale, cap, out_scale, tile_rows, hpc, 1};
  const size_t smem = mma ? static_cast<size_t>(64 + SM_KEYS) * (dim + 8) * 2 + static_cast<size_t>(SM_KEYS) * (vdim + 8) * 2 +
                                SM_KEYS * (sizeof(long long) + 3 * sizeof(int))
                          : (static_cast<size_t>(SA_ROWS) * hpc * (dim + vdim) + static_cast<size_t>(SA_KEYS) * (dim + 1 + vdim)) * sizeof(float) +
                                SA_KEYS * (sizeof(long long) + sizeof(int));
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_sigmoid_attn: head sizes need %zu bytes of shared memory", smem);
  const int gy = G * ((R + hpc - 1) / hpc);
  // single rows of a small step: a row's key chunks dealt to several CTAs (partial planes, summed in order afterwards)
  int splits = 1;
  if (!tiled && d_part && max_keys > 0) {
    const int chunks = (max_keys + chunk_keys - 1) / chunk_keys;
    int want = (mma ? 592 : 296) / (items * gy > 0 ? items * gy : 1);
    if (want > 16) want = 16;
    if (want > chunks / 2) want = chunks / 2;
    while (want > 1 && static_cast<long long>(want) * items * H * vdim > part_floats) --want;
    if (want > 1) splits = want;
  }
  p.splits = splits;
  dim3 grid(items, gy, splits);
  if (mma) {
    if (vdim <= 32) {
      if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(sigmoid_attn_mma_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(sigmoid_attn_mma_kernel<2>, grid, 128, smem, stream, p);
    } else if (vdim <= 64) {
      if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(sigmoid_attn_mma_kernel<4>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(sigmoid_attn_mma_kernel<4>, grid, 128, smem, stream, p);
    } else {
      if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(sigmoid_attn_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(sigmoid_attn_mma_kernel<8>, grid, 128, smem, stream, p);
    }
  } else if (dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(sigmoid_attn_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(sigmoid_attn_kernel<float>, grid, SA_THREADS, smem, stream, p);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(sigmoid_attn_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(sigmoid_attn_kernel<bf16>, grid, SA_THREADS, smem, stream, p);
  }
  if (splits > 1) {
    const int n = H * vdim;
    const long long total = static_cast<long long>(items) * n;
    const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
    if (dtype == 1) VB_LAUNCH_PDL(sigmoid_attn_sum_kernel<float>, blocks, 256, 0, stream, static_cast<float*>(d_out), ld_out, d_part, d_row_list, items, n, splits, out_scale);
    else VB_LAUNCH_PDL(sigmoid_attn_sum_kernel<bf16>, blocks, 256, 0, stream, static_cast<bf16*>(d_out), ld_out, d_part, d_row_list, items, n, splits, out_scale);
  }
  return 0;
}

}  // extern "C"
