// Softmax attention with a sliding window over a paged cache whose key and value heads may have different sizes,
// grouped query heads, rotary positions on a leading slice of every head in (even, odd) pairs, cross-layer value mixing
// and a sigmoid output gate.  Operands bf16 or fp32; scores, softmax and the output accumulation in fp32.
//
//   vb_rotary_table      cos / sin of position * frequency, evaluated in double and rounded once (the table is shared by
//                        every layer of a step that has the same rotary constants)
//   vb_qkv_rotary_append the tail of a fused q|k|v|gate projection: rotate q and k, mix v with the first mixing layer's
//                        values of the same token, write q, append k and the mixed v to the layer's pages
//   vb_window_attn       decode rows (and steps that mix them with prompt portions): a CTA per (token row, key/value
//                        head) whose K / V tiles serve all query heads of the group; for head groups or value sizes
//                        beyond its registers, one warp per (token row, query head).  Online softmax, gate, store.
//   vb_window_attn_tiled prompt portions: one CTA per (64 query rows of one request, query head), K/V tiles staged in
//                        shared memory and reused by all rows of the tile: mma.sync tensor-core tiles for bf16 heads whose
//                        sizes are multiples of 16 (keys up to 192 dims, values up to 128), fp32 FMAs otherwise (and always
//                        in fp32 mode).
//   vb_qkv_norm_rotary_append, vb_latent_rope_append, vb_head_pair_combine: projection tails with per-head RMS norms, rotation
//                        in (2i, 2i + 1) or (i, i + half) pairs, a shared rotated key part behind a latent, and the
//                        combination of two score maps per head.
// Besides the sliding window the kernels take a chunk mask (a position sees the keys of its own block of positions), per-token
// strides of the two caches (a value that is a leading slice of the key row), key heads that share a value head, and an fp32
// output beside bf16 operands.
// Cache layout per layer: K [pages][page_size][kv_heads][dim], V [pages][page_size][kv_heads][vdim] unless strides say otherwise.
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 1
#include "common.cuh"

namespace vb {

template <typename T> __device__ __forceinline__ float wa_to_f(T v);
template <> __device__ __forceinline__ float wa_to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float wa_to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T wa_from_f(float v);
template <> __device__ __forceinline__ float wa_from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 wa_from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__global__ void rotary_table_kernel(float* __restrict__ cs, const int32_t* __restrict__ pos, const double* __restrict__ freq,
                                    int T, int half, double mult) {
  pdl_sync();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= T * half) return;
  const int t = i / half, j = i - t * half;
  double s, c;
  sincos(static_cast<double>(pos[t]) * freq[j], &s, &c);
  cs[(static_cast<size_t>(t) * 2) * half + j] = static_cast<float>(c * mult);
  cs[(static_cast<size_t>(t) * 2 + 1) * half + j] = static_cast<float>(s * mult);
}

struct QkvTailParams {
  const float* proj;      // [T][ldp]: q | k | v | (gate) columns
  int ldp, q_off, k_off, v_off;
  const float* cs;        // [T][2][half] or nullptr (no rotation)
  int half;               // rotated dims / 2
  void* q_out;            // [T][H * dim]
  void* k_cache;
  void* v_cache;
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  int page_size, H, G, dim, vdim;
  int vmix;               // 0 none, 1 record v as the first mixing layer's values, 2 mix with them
  float* v_first;         // [T][G * vdim] fp32
  const float* lambda;    // device scalar
};

template <typename CT>
__global__ void qkv_rotary_append_kernel(QkvTailParams p) {
  pdl_sync();
  const int t = blockIdx.x;
  const float* row = p.proj + static_cast<size_t>(t) * p.ldp;
  const int b = p.row_req[t], ps = p.pos[t];
  const int page = p.page_indices[p.page_indptr[b] + ps / p.page_size];
  const size_t tok = static_cast<size_t>(page) * p.page_size + ps % p.page_size;
  const float* cs = p.cs ? p.cs + static_cast<size_t>(t) * 2 * p.half : nullptr;
  CT* q_out = static_cast<CT*>(p.q_out) + static_cast<size_t>(t) * p.H * p.dim;
  CT* k_out = static_cast<CT*>(p.k_cache) + tok * p.G * p.dim;
  CT* v_out = static_cast<CT*>(p.v_cache) + tok * p.G * p.vdim;
  // q and k: pairs (2i, 2i + 1) of the first 2 * half dims of every head are rotated, the rest pass
  const int pairs_per_head = (p.dim + 1) / 2;
  const int nq = p.H * pairs_per_head, nk = p.G * pairs_per_head;
  for (int i = threadIdx.x; i < nq + nk; i += blockDim.x) {
    const bool is_q = i < nq;
    const int j = is_q ? i : i - nq;
    const int h = j / pairs_per_head, pr = j - h * pairs_per_head;
    const float* src = row + (is_q ? p.q_off : p.k_off) + h * p.dim + 2 * pr;
    CT* dst = (is_q ? q_out : k_out) + h * p.dim + 2 * pr;
    const bool has2 = 2 * pr + 1 < p.dim;
    float u = src[0], v = has2 ? src[1] : 0.f;
    if (cs && pr < p.half) {
      const float c = cs[pr], s = cs[p.half + pr];
      const float nu = u * c - v * s, nv = v * c + u * s;
      u = nu;
      v = nv;
    }
    dst[0] = wa_from_f<CT>(u);
    if (has2) dst[1] = wa_from_f<CT>(v);
  }
  const int nv = p.G * p.vdim;
  float lam = 0.f;
  if (p.vmix == 2) lam = *p.lambda;
  for (int i = threadIdx.x; i < nv; i += blockDim.x) {
    float v = row[p.v_off + i];
    if (p.vmix == 1) p.v_first[static_cast<size_t>(t) * nv + i] = v;
    else if (p.vmix == 2) v = (1.f - lam) * v + lam * p.v_first[static_cast<size_t>(t) * nv + i];
    v_out[i] = wa_from_f<CT>(v);
  }
}

// The tail of a fused (query latent | key/value latent | ...) projection of latent attention: both latents are RMS-normed
// with their own weights in fp32; the query latent is written out for its up-projection, the key/value latent is appended
// to the layer's pages as ONE head of kv_rank dims per token (the only thing such a layer caches: keys and values are
// per-head expansions of it).  A layer that reads another layer's latents has no c part (c_cache == nullptr).
struct LatentTailParams {
  const float* proj;      // [T][ldp]
  int ldp, q_off, c_off, q_rank, kv_rank;
  const float* wq;        // [q_rank]
  const float* wc;        // [kv_rank]
  void* cq_out;           // [T][q_rank]
  void* c_cache;          // [pages][page_size][kv_rank]
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  int page_size;
  float eps;
};

template <typename CT>
__global__ void __launch_bounds__(128) latent_norm_append_kernel(LatentTailParams p) {
  __shared__ float red[2][4];
  pdl_sync();
  const size_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* q = p.proj + t * p.ldp + p.q_off;
  const float* c = p.proj + t * p.ldp + p.c_off;
  float sq = 0.f, sc = 0.f;
  for (int i = threadIdx.x; i < p.q_rank; i += 128) sq = fmaf(q[i], q[i], sq);
  if (p.c_cache)
    for (int i = threadIdx.x; i < p.kv_rank; i += 128) sc = fmaf(c[i], c[i], sc);
  sq = warp_sum(sq);
  sc = warp_sum(sc);
  if (lane == 0) { red[0][warp] = sq; red[1][warp] = sc; }
  __syncthreads();
  sq = red[0][0] + red[0][1] + red[0][2] + red[0][3];
  sc = red[1][0] + red[1][1] + red[1][2] + red[1][3];
  const float rq = 1.f / sqrtf(sq / p.q_rank + p.eps);
  CT* qo = static_cast<CT*>(p.cq_out) + t * p.q_rank;
  for (int i = threadIdx.x; i < p.q_rank; i += 128) qo[i] = wa_from_f<CT>(q[i] * rq * p.wq[i]);
  if (p.c_cache == nullptr) return;
  const float rc = 1.f / sqrtf(sc / p.kv_rank + p.eps);
  const int b = p.row_req[t], ps = p.pos[t];
  const size_t tok = static_cast<size_t>(p.page_indices[p.page_indptr[b] + ps / p.page_size]) * p.page_size + ps % p.page_size;
  CT* co = static_cast<CT*>(p.c_cache) + tok * p.kv_rank;
  for (int i = threadIdx.x; i < p.kv_rank; i += 128) co[i] = wa_from_f<CT>(c[i] * rc * p.wc[i]);
}

// The tail of a fused q|k|v|.. projection for heads that are normed before they are rotated: every query and key head
// (for attention with several score maps per head, every map is a head here) is RMS-normed over its dim values with a
// weight shared by all heads (optional), then its first 2 * half dims are rotated -- pairs (2i, 2i + 1) in the
// interleaved layout, pairs (i, i + half) in the half layout -- and written out / appended; values are appended as they are.
// The key cache holds Gk heads per token, the value cache Gv (Gk / Gv key heads read one value head).  One warp per head.
struct QkvNormTailParams {
  const float* proj;      // [T][ldp]
  int ldp, q_off, k_off, v_off;
  const float* cs;        // [T][2][half] or nullptr
  int half, layout;       // layout 0: interleaved pairs, 1: halves
  const float* q_norm;    // [dim] or nullptr
  const float* k_norm;
  float eps;
  void* q_out;            // [T][Hq * dim]
  void* k_cache;          // [pages][page][Gk][dim]
  void* v_cache;          // [pages][page][Gv][vdim]
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  int page_size, Hq, Gk, Gv, dim, vdim;
  int stage_lo, stage_hi; // columns of the row staged in shared memory (stage_hi == 0: read from global memory)
};

// Copies floats [lo, hi) of a projection row into shared memory with every load in flight at once (16-byte loads when the
// row slice is aligned) and returns a pointer that is indexed like the row itself.  The tails below read a row's values
// more than once (norm, rotation partner) and from many threads: one pass over DRAM, the rest from shared memory.
__device__ __forceinline__ const float* stage_row(const float* __restrict__ row, int lo, int hi, float* __restrict__ sm) {
  const int n = hi - lo;
  if (((reinterpret_cast<uintptr_t>(row + lo) & 15) == 0) && (n & 3) == 0) {
    for (int i = threadIdx.x * 4; i < n; i += blockDim.x * 4)
      *reinterpret_cast<float4*>(sm + i) = *reinterpret_cast<const float4*>(row + lo + i);
  } else {
    for (int i = threadIdx.x; i < n; i += blockDim.x) sm[i] = row[lo + i];
  }
  __syncthreads();
  return sm - lo;
}

__device__ __forceinline__ float rotated_value(const float* __restrict__ src, const float* __restrict__ w, float r,
                                               const float* __restrict__ cs, int half, int layout, int d) {
  // value d of a head after norm (scale r, weight w) and rotation
  const float x = src[d] * r * (w ? w[d] : 1.f);
  if (cs == nullptr || d >= 2 * half) return x;
  int i, partner;
  bool first;
  if (layout == 0) { i = d >> 1; first = (d & 1) == 0; partner = d ^ 1; }
  else { first = d < half; i = first ? d : d - half; partner = first ? d + half : d - half; }
  const float y = src[partner] * r * (w ? w[partner] : 1.f);
  const float c = cs[i], sn = cs[half + i];
  return first ? x * c - y * sn : x * c + y * sn;
}

template <typename CT>
__global__ void __launch_bounds__(256) qkv_norm_rotary_append_kernel(QkvNormTailParams p) {
  extern __shared__ __align__(16) float tail_sm[];
  pdl_sync();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* row = p.proj + static_cast<size_t>(t) * p.ldp;
  if (p.stage_hi > 0) row = stage_row(row, p.stage_lo, p.stage_hi, tail_sm);
  const int b = p.row_req[t], ps = p.pos[t];
  const size_t tok = static_cast<size_t>(p.page_indices[p.page_indptr[b] + ps / p.page_size]) * p.page_size + ps % p.page_size;
  const float* cs = p.cs ? p.cs + static_cast<size_t>(t) * 2 * p.half : nullptr;
  CT* q_out = static_cast<CT*>(p.q_out) + static_cast<size_t>(t) * p.Hq * p.dim;
  CT* k_out = static_cast<CT*>(p.k_cache) + tok * p.Gk * p.dim;
  CT* v_out = static_cast<CT*>(p.v_cache) + tok * p.Gv * p.vdim;
  for (int hh = warp; hh < p.Hq + p.Gk; hh += 8) {
    const bool is_q = hh < p.Hq;
    const int h = is_q ? hh : hh - p.Hq;
    const float* src = row + (is_q ? p.q_off : p.k_off) + h * p.dim;
    const float* w = is_q ? p.q_norm : p.k_norm;
    float r = 1.f;
    if (w) {
      float ss = 0.f;
      for (int d = lane; d < p.dim; d += 32) ss = fmaf(src[d], src[d], ss);
      r = 1.f / sqrtf(warp_sum(ss) / p.dim + p.eps);
    }
    CT* dst = (is_q ? q_out : k_out) + h * p.dim;
    for (int d = lane; d < p.dim; d += 32) dst[d] = wa_from_f<CT>(rotated_value(src, w, r, cs, p.half, p.layout, d));
  }
  for (int i = threadIdx.x; i < p.Gv * p.vdim; i += 256) v_out[i] = wa_from_f<CT>(row[p.v_off + i]);
}

// The tail of a fused (queries | key/value latent + shared rotated key part | ...) projection of latent attention whose
// heads have an unrotated part of `dim` and a rotated part of `rot` dims: the latent (kv_rank dims) is RMS-normed with its
// weight, the shared key part is rotated, and both are appended to the layer's pages as ONE row [kv_rank | rot] per token.
// The queries' unrotated parts go to q_out [T][H][dim] (they are carried into latent space by a per-head projection), their
// rotated parts straight to their place behind the latent-space part: q_lat[t][h][kv_rank .. kv_rank + rot).
struct LatentRopeTailParams {
  const float* proj;      // [T][ldp]
  int ldp, q_off, c_off, H, dim, rot, kv_rank;
  const float* wc;        // [kv_rank]
  const float* cs;        // [T][2][half] or nullptr
  int half, layout;
  void* q_out;            // [T][H][dim]
  void* q_lat;            // [T][H][kv_rank + rot]
  void* cache;            // [pages][page][kv_rank + rot]
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  int page_size;
  float eps;
  int stage_lo, stage_hi; // columns of the row staged in shared memory (stage_hi == 0: read from global memory)
};

constexpr int LR_THREADS = 256;

template <typename CT>
__global__ void __launch_bounds__(LR_THREADS) latent_rope_append_kernel(LatentRopeTailParams p) {
  extern __shared__ __align__(16) float tail_sm[];
  __shared__ float red[LR_THREADS / 32];
  pdl_sync();
  const size_t t = blockIdx.x;
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const float* row = p.proj + t * p.ldp;
  if (p.stage_hi > 0) row = stage_row(row, p.stage_lo, p.stage_hi, tail_sm);
  const float* c = row + p.c_off;
  const float* cs = p.cs ? p.cs + t * 2 * p.half : nullptr;
  const int ldc = p.kv_rank + p.rot;
  if (p.cache) {          // (a layer that reads another layer's cached rows has no latent of its own: queries only)
    float sc = 0.f;
    for (int i = threadIdx.x; i < p.kv_rank; i += LR_THREADS) sc = fmaf(c[i], c[i], sc);
    sc = warp_sum(sc);
    if (lane == 0) red[warp] = sc;
    __syncthreads();
    sc = 0.f;
#pragma unroll
    for (int i = 0; i < LR_THREADS / 32; ++i) sc += red[i];
    const float rc = 1.f / sqrtf(sc / p.kv_rank + p.eps);
    const int b = p.row_req[t], ps = p.pos[t];
    const size_t tok = static_cast<size_t>(p.page_indices[p.page_indptr[b] + ps / p.page_size]) * p.page_size + ps % p.page_size;
    CT* co = static_cast<CT*>(p.cache) + tok * ldc;
    for (int i = threadIdx.x; i < p.kv_rank; i += LR_THREADS) co[i] = wa_from_f<CT>(c[i] * rc * p.wc[i]);
    for (int i = threadIdx.x; i < p.rot; i += LR_THREADS)
      co[p.kv_rank + i] = wa_from_f<CT>(rotated_value(c + p.kv_rank, nullptr, 1.f, cs, p.half, p.layout, i));
  }
  const int dq = p.dim + p.rot;
  CT* qo = static_cast<CT*>(p.q_out) + t * p.H * p.dim;
  CT* ql = static_cast<CT*>(p.q_lat) + t * p.H * ldc;
  for (int i = threadIdx.x; i < p.H * dq; i += LR_THREADS) {
    const int h = i / dq, d = i - h * dq;
    const float* src = row + p.q_off + h * dq;
    if (d < p.dim) qo[h * p.dim + d] = wa_from_f<CT>(src[d]);
    else ql[h * ldc + p.kv_rank + d - p.dim] = wa_from_f<CT>(rotated_value(src + p.dim, nullptr, 1.f, cs, p.half, p.layout, d - p.dim));
  }
}

// Attention with two score maps per head over the same values: the maps' outputs a1, a2 (fp32 [T][2H][vdim], laid out per
// key/value group as [map 1 of the group's R heads | map 2 of them]) are combined as o = a1 - lambda * a2, o is divided by
// its root mean square over the head's vdim values, times `post`, times sigmoid(gate).  One warp per (token, head).
template <typename CT>
__global__ void __launch_bounds__(128) head_pair_combine_kernel(CT* __restrict__ out, const float* __restrict__ a,
                                                                const float* __restrict__ gate, int ld_gate, int T, int H,
                                                                int R, int vdim, float lambda, float post, float eps) {
  pdl_sync();
  const int idx = blockIdx.x * 4 + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (idx >= T * H) return;
  const int t = idx / H, h = idx - t * H, g = h / R, j = h - g * R;
  const float* a1 = a + (static_cast<size_t>(t) * 2 * H + g * 2 * R + j) * vdim;
  const float* a2 = a1 + static_cast<size_t>(R) * vdim;
  float ss = 0.f;
  for (int d = lane; d < vdim; d += 32) {
    const float o = a1[d] - lambda * a2[d];
    ss = fmaf(o, o, ss);
  }
  const float r = post / sqrtf(warp_sum(ss) / vdim + eps);
  const float* gt = gate ? gate + static_cast<size_t>(t) * ld_gate + h * vdim : nullptr;
  CT* o_row = out + (static_cast<size_t>(t) * H + h) * vdim;
  for (int d = lane; d < vdim; d += 32) {
    float o = (a1[d] - lambda * a2[d]) * r;
    if (gt) o *= 1.f / (1.f + expf(-gt[d]));
    o_row[d] = wa_from_f<CT>(o);
  }
}

struct WindowAttnParams {
  const void* q;          // [T][H][dim]
  const void* k_cache;
  const void* v_cache;
  void* out;              // [T][H * vdim]
  const float* gate;      // [T][ld_gate] (+ column offset applied by the host) or nullptr
  int ld_gate;
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* page_indptr;
  const int32_t* page_indices;
  const int32_t* qo_indptr;   // tiled kernel: rows of request b are qo[b]..qo[b+1]
  const int32_t* tile_req;    // tiled kernel: request of tile i
  const int32_t* tile_row0;   // tiled kernel: first row of tile i
  int T, H, G, dim, vdim, page_size, window;   // window <= 0: every earlier position is visible
  int chunk;                  // > 0: a position sees only the keys of its own block of `chunk` positions (blocks counted from
                              // position 0 of the sequence)
  int k_ld, v_ld;             // elements per token of the key / value cache (G * dim, (G / v_share) * vdim for caches of their own;
                              // a value that is a leading slice of the key row has v_ld = k_ld)
  int v_share;                // consecutive key heads that read ONE value head (1: every key head has its own)
  int out_f32;                // the output is fp32 whatever the operand type (it feeds a combination of heads done in fp32)
  float scale;
  const int32_t* row_list;    // per-row kernels: the rows to serve (nullptr: rows 0 .. T - 1); T counts the served rows
  int row_heads;              // tensor-core tile kernel on single-token rows: a tile's rows are the query heads of ONE token
                              // that share a key/value head (grid: served rows x key/value heads x splits)
  int splits;                 // grouped kernel: key tiles are dealt round-robin to `splits` CTAs per (row, key/value head)
  float* part;                // [T][H][splits][vdim + 2]: unnormalised output, running max, running sum of every split
};

// first visible key of a query at position pos: the sliding window's start, the start of the position's chunk, or 0
__device__ __forceinline__ int wa_first_key(const WindowAttnParams& p, int pos) {
  int lo = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  if (p.chunk > 0) lo = max(lo, pos - pos % p.chunk);
  return lo;
}
template <typename CT>
__device__ __forceinline__ void wa_store(const WindowAttnParams& p, size_t idx, float v) {
  if (p.out_f32) static_cast<float*>(p.out)[idx] = v;
  else static_cast<CT*>(p.out)[idx] = wa_from_f<CT>(v);
}

template <typename CT>
__device__ __forceinline__ float dot_row(const float* __restrict__ q, const CT* __restrict__ k, int dim);
template <>
__device__ __forceinline__ float dot_row<float>(const float* __restrict__ q, const float* __restrict__ k, int dim) {
  float s = 0.f;
  if ((dim & 3) == 0) {
    for (int d = 0; d < dim; d += 4) {
      const float4 kv = *reinterpret_cast<const float4*>(k + d);
      s = fmaf(q[d], kv.x, s); s = fmaf(q[d + 1], kv.y, s); s = fmaf(q[d + 2], kv.z, s); s = fmaf(q[d + 3], kv.w, s);
    }
  } else {
    for (int d = 0; d < dim; ++d) s = fmaf(q[d], k[d], s);
  }
  return s;
}
template <>
__device__ __forceinline__ float dot_row<__nv_bfloat16>(const float* __restrict__ q, const __nv_bfloat16* __restrict__ k,
                                                        int dim) {
  float s = 0.f;
  if ((dim & 7) == 0) {
    for (int d = 0; d < dim; d += 8) {
      const uint4 kv = *reinterpret_cast<const uint4*>(k + d);
      s = fmaf(q[d], bf16_lo(kv.x), s); s = fmaf(q[d + 1], bf16_hi(kv.x), s);
      s = fmaf(q[d + 2], bf16_lo(kv.y), s); s = fmaf(q[d + 3], bf16_hi(kv.y), s);
      s = fmaf(q[d + 4], bf16_lo(kv.z), s); s = fmaf(q[d + 5], bf16_hi(kv.z), s);
      s = fmaf(q[d + 6], bf16_lo(kv.w), s); s = fmaf(q[d + 7], bf16_hi(kv.w), s);
    }
  } else {
    for (int d = 0; d < dim; ++d) s = fmaf(q[d], __bfloat162float(k[d]), s);
  }
  return s;
}

// rows c0 .. c0 + n_rows - 1 of one key/value head of a request's pages -> dst[row][ldd] as fp32; rows at or past `valid`
// are zero.  16-byte loads when the head size allows (8 bf16 / 4 fp32 per load), element loads otherwise.
template <typename CT>
__device__ __forceinline__ void load_rows_f32(float* __restrict__ dst, int ldd, const CT* __restrict__ cache,
                                              const int32_t* __restrict__ pages, int page_size, int ld, int off, int d_head,
                                              int c0, int n_rows, int valid, int tid, int nthreads) {
  // the head's d_head values of token tok start at cache[tok * ld + off]
  constexpr int VEC = 16 / sizeof(CT);
  if (d_head % VEC == 0 && ld % VEC == 0 && off % VEC == 0) {
    const int nvec = d_head / VEC;
    for (int i = tid; i < n_rows * nvec; i += nthreads) {
      const int kk = i / nvec, d = (i - kk * nvec) * VEC;
      float* o = dst + kk * ldd + d;
      if (kk < valid) {
        const int kj = c0 + kk;
        const size_t tok = static_cast<size_t>(pages[kj / page_size]) * page_size + kj % page_size;
        const uint4 v = *reinterpret_cast<const uint4*>(cache + tok * ld + off + d);
        if constexpr (sizeof(CT) == 2) {
          o[0] = bf16_lo(v.x); o[1] = bf16_hi(v.x); o[2] = bf16_lo(v.y); o[3] = bf16_hi(v.y);
          o[4] = bf16_lo(v.z); o[5] = bf16_hi(v.z); o[6] = bf16_lo(v.w); o[7] = bf16_hi(v.w);
        } else {
          o[0] = __uint_as_float(v.x); o[1] = __uint_as_float(v.y); o[2] = __uint_as_float(v.z); o[3] = __uint_as_float(v.w);
        }
      } else {
#pragma unroll
        for (int e = 0; e < VEC; ++e) o[e] = 0.f;
      }
    }
  } else {
    for (int i = tid; i < n_rows * d_head; i += nthreads) {
      const int kk = i / d_head, d = i - kk * d_head;
      float v = 0.f;
      if (kk < valid) {
        const int kj = c0 + kk;
        const size_t tok = static_cast<size_t>(pages[kj / page_size]) * page_size + kj % page_size;
        v = wa_to_f(cache[tok * ld + off + d]);
      }
      dst[kk * ldd + d] = v;
    }
  }
}

constexpr int WA_WARPS = 4, WA_MAXU = 8;      // value heads up to 32 * WA_MAXU wide

template <typename CT>
__global__ void __launch_bounds__(WA_WARPS * 32) window_attn_kernel(WindowAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int ti = blockIdx.x * WA_WARPS + warp, h = blockIdx.y;
  if (ti >= p.T) return;
  const int t = p.row_list ? p.row_list[ti] : ti;
  float* qs = smf + warp * p.dim;
  const CT* q = static_cast<const CT*>(p.q) + (static_cast<size_t>(t) * p.H + h) * p.dim;
  for (int d = lane; d < p.dim; d += 32) qs[d] = wa_to_f(q[d]) * p.scale;
  __syncwarp();
  const int b = p.row_req[t], ps = p.pos[t], g = h / (p.H / p.G);
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const int lo = wa_first_key(p, ps);
  const int gv = g / p.v_share;
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  float m = -INFINITY, l = 0.f, acc[WA_MAXU];
#pragma unroll
  for (int u = 0; u < WA_MAXU; ++u) acc[u] = 0.f;
  for (int c = lo; c <= ps; c += 32) {
    const int kj = c + lane;
    const bool ok = kj <= ps;
    int tok = 0;
    float s = -INFINITY;
    if (ok) {
      tok = pages[kj / p.page_size] * p.page_size + kj % p.page_size;
      s = dot_row<CT>(qs, kc + static_cast<size_t>(tok) * p.k_ld + g * p.dim, p.dim);
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);          // m = -inf on the first chunk: exp(-inf) = 0
    const float pj = ok ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(pj);
    m = m_new;
#pragma unroll
    for (int u = 0; u < WA_MAXU; ++u) acc[u] *= corr;
    const int n = min(32, ps - c + 1);
    for (int jj = 0; jj < n; ++jj) {
      const float pv = __shfl_sync(0xffffffffu, pj, jj);
      const int tk = __shfl_sync(0xffffffffu, tok, jj);
      const CT* vr = vc + static_cast<size_t>(tk) * p.v_ld + gv * p.vdim;
#pragma unroll
      for (int u = 0; u < WA_MAXU; ++u) {
        const int d = lane + 32 * u;
        if (d < p.vdim) acc[u] = fmaf(pv, wa_to_f(vr[d]), acc[u]);
      }
    }
  }
  const float inv = 1.f / l;
  const size_t out0 = static_cast<size_t>(t) * p.H * p.vdim + h * p.vdim;
  const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * p.vdim : nullptr;
#pragma unroll
  for (int u = 0; u < WA_MAXU; ++u) {
    const int d = lane + 32 * u;
    if (d < p.vdim) {
      float o = acc[u] * inv;
      if (gate) o *= 1.f / (1.f + expf(-gate[d]));
      wa_store<CT>(p, out0 + d, o);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Prompt portions: CTA = (tile of up to 64 consecutive rows of ONE request, query head), 256 threads.  Key / value
// tiles of 32 positions are staged in shared memory as fp32 and shared by all rows; thread (r = tid / 4, c = tid % 4)
// owns row r and, in the score phase, keys c, c + 4, ...; in the output phase the value dims c, c + 4, ....
// The four threads of a row exchange through shuffles (they are neighbours in a warp).
// ------------------------------------------------------------------------------------------------------------------
constexpr int WT_ROWS = 64, WT_KEYS = 32, WT_MAXD = 64;   // per-thread value dims: vdim / 4 <= WT_MAXD

template <typename CT>
__global__ void __launch_bounds__(256) window_attn_tiled_kernel(WindowAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int b = p.tile_req[blockIdx.x], row0 = p.tile_row0[blockIdx.x], h = blockIdx.y;
  const int row_end = min(row0 + WT_ROWS, p.qo_indptr[b + 1]);
  const int nrows = row_end - row0;
  const int dk = p.dim, dv = p.vdim, dkp = dk + 1, dvp = dv + 1;
  float* Qs = smf;                               // [64][dk + 1]
  float* Ks = Qs + WT_ROWS * dkp;                // [32][dk + 1]
  float* Vs = Ks + WT_KEYS * dkp;                // [32][dv + 1]
  float* Ps = Vs + WT_KEYS * dvp;                // [64][33]
  const int tid = threadIdx.x, r = tid >> 2, c = tid & 3;
  const int g = h / (p.H / p.G);
  const CT* q = static_cast<const CT*>(p.q);
  for (int i = tid; i < WT_ROWS * dk; i += 256) {
    const int rr = i / dk, d = i - rr * dk;
    Qs[rr * dkp + d] = rr < nrows ? wa_to_f(q[(static_cast<size_t>(row0 + rr) * p.H + h) * dk + d]) * p.scale : 0.f;
  }
  const int pos0 = p.pos[row0], pos_last = pos0 + nrows - 1;     // rows of a portion are consecutive positions
  const int my_pos = pos0 + r;
  const bool row_ok = r < nrows;
  const int my_lo = wa_first_key(p, my_pos);
  const int lo = wa_first_key(p, pos0);
  const int gv = g / p.v_share;
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  float m = -INFINITY, l = 0.f;
  float acc[WT_MAXD];
#pragma unroll
  for (int u = 0; u < WT_MAXD; ++u) acc[u] = 0.f;
  const int nd = (dv + 3) / 4;
  for (int c0 = lo; c0 <= pos_last; c0 += WT_KEYS) {
    __syncthreads();
    const int valid = min(WT_KEYS, pos_last - c0 + 1);
    load_rows_f32<CT>(Ks, dkp, kc, pages, p.page_size, p.k_ld, g * dk, dk, c0, WT_KEYS, valid, tid, 256);
    load_rows_f32<CT>(Vs, dvp, vc, pages, p.page_size, p.v_ld, gv * dv, dv, c0, WT_KEYS, valid, tid, 256);
    __syncthreads();
    // scores of this thread's 8 keys
    float s[WT_KEYS / 4];
    float mx = -INFINITY;
#pragma unroll
    for (int e = 0; e < WT_KEYS / 4; ++e) {
      const int kk = c + 4 * e, kj = c0 + kk;
      float a = 0.f;
      const float* qr = Qs + r * dkp;
      const float* kr = Ks + kk * dkp;
      for (int d = 0; d < dk; ++d) a = fmaf(qr[d], kr[d], a);
      const bool vis = row_ok && kj <= my_pos && kj >= my_lo;
      s[e] = vis ? a : -INFINITY;
      mx = fmaxf(mx, s[e]);
    }
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
    mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
    const float m_new = fmaxf(m, mx);
    const float corr = m_new == -INFINITY ? 1.f : expf(m - m_new);
    float sum = 0.f;
#pragma unroll
    for (int e = 0; e < WT_KEYS / 4; ++e) {
      const float pj = s[e] == -INFINITY ? 0.f : expf(s[e] - m_new);
      Ps[r * (WT_KEYS + 1) + c + 4 * e] = pj;
      sum += pj;
    }
    sum += __shfl_xor_sync(0xffffffffu, sum, 1);
    sum += __shfl_xor_sync(0xffffffffu, sum, 2);
    l = l * corr + sum;
    m = m_new;
    __syncwarp();
#pragma unroll
    for (int u = 0; u < WT_MAXD; ++u)
      if (u < nd) acc[u] *= corr;
    const float* pr = Ps + r * (WT_KEYS + 1);
    for (int kk = 0; kk < WT_KEYS; ++kk) {
      const float pj = pr[kk];
      const float* vr = Vs + kk * dvp;
#pragma unroll
      for (int u = 0; u < WT_MAXD; ++u) {
        const int d = c + 4 * u;
        if (u < nd && d < dv) acc[u] = fmaf(pj, vr[d], acc[u]);
      }
    }
  }
  if (!row_ok) return;
  const int t = row0 + r;
  const float inv = 1.f / l;
  const size_t out0 = static_cast<size_t>(t) * p.H * dv + h * dv;
  const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * dv : nullptr;
#pragma unroll
  for (int u = 0; u < WT_MAXD; ++u) {
    const int d = c + 4 * u;
    if (u < nd && d < dv) {
      float o = acc[u] * inv;
      if (gate) o *= 1.f / (1.f + expf(-gate[d]));
      wa_store<CT>(p, out0 + d, o);
    }
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Decode rows: CTA = (token row, key/value head), 128 threads.  All R = H / G query heads of the group share every K / V
// tile of 32 positions, staged once in shared memory as fp32 with coalesced loads.  Warp w owns the heads r = w, w + 4, ..:
// lane j scores key j of the tile for them, the softmax statistics of a head stay inside its warp, and in the output phase
// lane d accumulates value dims d, d + 32, .. of the same heads.
// ------------------------------------------------------------------------------------------------------------------
constexpr int WD_KEYS = 32, WD_RU = 4, WD_VU = 8;      // up to 4 * WD_RU query heads per key/value head, vdim <= 32 * WD_VU

template <typename CT>
__global__ void __launch_bounds__(128) window_attn_group_kernel(WindowAttnParams p) {
  extern __shared__ float smf[];
  pdl_sync();
  const int ti = blockIdx.x, g = blockIdx.y, R = p.H / p.G;
  const int t = p.row_list ? p.row_list[ti] : ti;
  const int dk = p.dim, dv = p.vdim, dkp = dk + 1, dvp = dv + 1;
  float* Qs = smf;                      // [R][dk]
  float* Ks = Qs + R * dk;              // [32][dk + 1]
  float* Vs = Ks + WD_KEYS * dkp;       // [32][dv + 1]
  float* Ps = Vs + WD_KEYS * dvp;       // [R][32]
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const CT* q = static_cast<const CT*>(p.q) + (static_cast<size_t>(t) * p.H + g * R) * dk;
  for (int i = tid; i < R * dk; i += 128) Qs[i] = wa_to_f(q[i]) * p.scale;
  const int b = p.row_req[t], ps = p.pos[t];
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const int lo = wa_first_key(p, ps);
  const int gv = g / p.v_share;
  const CT* kc = static_cast<const CT*>(p.k_cache);
  const CT* vc = static_cast<const CT*>(p.v_cache);
  float m[WD_RU], l[WD_RU], acc[WD_RU][WD_VU];
#pragma unroll
  for (int u = 0; u < WD_RU; ++u) {
    m[u] = -INFINITY;
    l[u] = 0.f;
#pragma unroll
    for (int v = 0; v < WD_VU; ++v) acc[u][v] = 0.f;
  }
  const int S = p.splits, sidx = blockIdx.z;
  for (int c0 = lo + sidx * WD_KEYS; c0 <= ps; c0 += S * WD_KEYS) {
    __syncthreads();
    const int nk = min(WD_KEYS, ps - c0 + 1);
    load_rows_f32<CT>(Ks, dkp, kc, pages, p.page_size, p.k_ld, g * dk, dk, c0, WD_KEYS, nk, tid, 128);
    load_rows_f32<CT>(Vs, dvp, vc, pages, p.page_size, p.v_ld, gv * dv, dv, c0, WD_KEYS, nk, tid, 128);
    __syncthreads();
#pragma unroll
    for (int u = 0; u < WD_RU; ++u) {
      const int r = warp + 4 * u;
      if (r >= R) break;
      float s = -INFINITY;
      if (lane < nk) {
        const float* qr = Qs + r * dk;
        const float* kr = Ks + lane * dkp;
        float a = 0.f;
        for (int d = 0; d < dk; ++d) a = fmaf(qr[d], kr[d], a);
        s = a;
      }
      const float m_new = fmaxf(m[u], warp_max(s));
      const float corr = expf(m[u] - m_new);
      const float pj = lane < nk ? expf(s - m_new) : 0.f;
      l[u] = l[u] * corr + warp_sum(pj);
      m[u] = m_new;
      Ps[r * WD_KEYS + lane] = pj;
      __syncwarp();
      const float* pr = Ps + r * WD_KEYS;
#pragma unroll
      for (int v = 0; v < WD_VU; ++v) {
        const int d = lane + 32 * v;
        if (d < dv) {
          float a = acc[u][v] * corr;
          for (int kk = 0; kk < nk; ++kk) a = fmaf(pr[kk], Vs[kk * dvp + d], a);
          acc[u][v] = a;
        }
      }
    }
  }
#pragma unroll
  for (int u = 0; u < WD_RU; ++u) {
    const int r = warp + 4 * u;
    if (r >= R) break;
    const int h = g * R + r;
    if (S > 1) {              // leave this split's share for vb::window_attn_merge_kernel
      float* pt = p.part + ((static_cast<size_t>(ti) * p.H + h) * S + sidx) * (dv + 2);
#pragma unroll
      for (int v = 0; v < WD_VU; ++v) {
        const int d = lane + 32 * v;
        if (d < dv) pt[d] = acc[u][v];
      }
      if (lane == 0) {
        pt[dv] = m[u];
        pt[dv + 1] = l[u];
      }
      continue;
    }
    const float inv = 1.f / l[u];
    const size_t out0 = static_cast<size_t>(t) * p.H * dv + h * dv;
    const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * dv : nullptr;
#pragma unroll
    for (int v = 0; v < WD_VU; ++v) {
      const int d = lane + 32 * v;
      if (d < dv) {
        float o = acc[u][v] * inv;
        if (gate) o *= 1.f / (1.f + expf(-gate[d]));
        wa_store<CT>(p, out0 + d, o);
      }
    }
  }
}

// merges the splits of a (row, head): out = sum_s acc_s e^(m_s - M) / sum_s l_s e^(m_s - M), then the gate
template <typename CT>
__global__ void __launch_bounds__(64) window_attn_merge_kernel(WindowAttnParams p) {
  __shared__ float wgt[32];       // e^(m_s - M) / L of every split (at most 32 splits)
  pdl_sync();
  const int ti = blockIdx.x, h = blockIdx.y, S = p.splits, dv = p.vdim;
  const int t = p.row_list ? p.row_list[ti] : ti;
  const float* pt = p.part + (static_cast<size_t>(ti) * p.H + h) * S * (dv + 2);
  if (threadIdx.x < 32) {
    const int s = threadIdx.x;
    const float m = s < S ? pt[s * (dv + 2) + dv] : -INFINITY, l = s < S ? pt[s * (dv + 2) + dv + 1] : 0.f;
    const float M = warp_max(m);
    const float w = m == -INFINITY ? 0.f : expf(m - M);
    const float L = warp_sum(l * w);
    wgt[s] = w / L;
  }
  __syncthreads();
  const size_t out0 = static_cast<size_t>(t) * p.H * dv + h * dv;
  const float* gate = p.gate ? p.gate + static_cast<size_t>(t) * p.ld_gate + h * dv : nullptr;
  for (int d = threadIdx.x; d < dv; d += blockDim.x) {
    float o = 0.f;
    for (int s = 0; s < S; ++s) o = fmaf(pt[s * (dv + 2) + d], wgt[s], o);
    if (gate) o *= 1.f / (1.f + expf(-gate[d]));
    wa_store<CT>(p, out0 + d, o);
  }
}

// ------------------------------------------------------------------------------------------------------------------
// Prompt portions on the tensor cores (bf16, head sizes multiples of 16 up to 128): CTA = (tile of 64 query rows of one
// request, query head), 4 warps x 16 rows.  Q fragments stay in registers; K / V tiles of 64 positions are staged in shared
// memory as bf16 with 16-byte loads; S = Q K^T and O += P V run as mma.sync m16n8k16 with fp32 accumulators, the softmax
// (scale, window mask, running max and sum) in fp32 on the accumulator fragments, P rounded to bf16 for the second product.
// ------------------------------------------------------------------------------------------------------------------
constexpr int FM = 64, FN = 64, F_KB = 12, F_NT = 16;      // dim <= 16 * F_KB, vdim <= 8 * F_NT
// (KB: the query fragments a thread holds, 16 key dims each; 8 for heads up to 128 dims, 12 up to 192)

template <int KB>
__global__ void __launch_bounds__(128) window_attn_mma_kernel(WindowAttnParams p) {
  extern __shared__ __align__(16) uint8_t smraw[];
  pdl_sync();
  // prompt portions: tile = 64 consecutive rows (positions) of one request and one query head.  Single-token rows
  // (row_heads): tile = the R query heads of ONE token that share key/value head g, all at the token's position; the
  // token's key tiles may be dealt to several CTAs (splits), whose shares vb::window_attn_merge_kernel puts together.
  int b, row0, h, nrows, HH, pstep, pos0, g, S = 1, sidx = 0;
  if (p.row_heads) {
    const int t = p.row_list ? p.row_list[blockIdx.x] : blockIdx.x, R = p.H / p.G;
    b = p.row_req[t]; g = blockIdx.y; row0 = t * p.H + g * R; h = 0; nrows = R; HH = 1; pstep = 0; pos0 = p.pos[t];
    S = p.splits; sidx = blockIdx.z;
  } else {
    // later tiles of a prompt see more keys: they are started first so that the short ones fill the tail
    const int tile = gridDim.x - 1 - blockIdx.x;
    b = p.tile_req[tile]; row0 = p.tile_row0[tile]; h = blockIdx.y;
    nrows = min(row0 + FM, p.qo_indptr[b + 1]) - row0;
    HH = p.H; pstep = 1; pos0 = p.pos[row0]; g = h / (p.H / p.G);
  }
  // keys and values that are one tensor of equal head sizes (latent attention) are staged once and read as both
  // (also values that are a leading slice of the one key head: the shared latent with a rotated key part behind it)
  const bool same_kv = p.k_cache == p.v_cache && p.k_ld == p.v_ld && p.G == 1 && p.v_share == 1 && p.vdim <= p.dim;
  const int dk = p.dim, dv = p.vdim, ldk = dk + 8, ldv = same_kv ? ldk : dv + 8, nkb = dk / 16, nvp = dv / 16;
  // two stages of K [64][dk + 8] | V [64][dv + 8]; the first stage's K region holds the Q tile first
  __nv_bfloat16* Ks = reinterpret_cast<__nv_bfloat16*>(smraw);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const __nv_bfloat16* q = static_cast<const __nv_bfloat16*>(p.q);
  const int qv = dk / 8;
  for (int i = tid; i < FM * qv; i += 128) {
    const int r = i / qv, c = (i - r * qv) * 8;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (r < nrows) v = *reinterpret_cast<const uint4*>(q + (static_cast<size_t>(row0 + r) * HH + h) * dk + c);
    *reinterpret_cast<uint4*>(Ks + r * ldk + c) = v;
  }
  __syncthreads();
  uint32_t qf[KB][4];
#pragma unroll
  for (int kb = 0; kb < KB; ++kb)
    if (kb < nkb) ldmatrix_x4(qf[kb], smem_u32(Ks + (warp * 16 + (lane & 15)) * ldk + kb * 16 + (lane >> 4) * 8));
  const int pos_last = pos0 + (nrows - 1) * pstep;
  const int rA = warp * 16 + (lane >> 2), rB = rA + 8;
  const int posA = pos0 + rA * pstep, posB = pos0 + rB * pstep;
  const bool okA = rA < nrows, okB = rB < nrows;
  const int loA = wa_first_key(p, posA), loB = wa_first_key(p, posB);
  const int lo = wa_first_key(p, pos0);
  const int gv = g / p.v_share;
  const int32_t* pages = p.page_indices + p.page_indptr[b];
  const __nv_bfloat16* kc = static_cast<const __nv_bfloat16*>(p.k_cache);
  const __nv_bfloat16* vc = static_cast<const __nv_bfloat16*>(p.v_cache);
  float o[F_NT][4];
#pragma unroll
  for (int n = 0; n < F_NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.f;
  float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
  const int vv = dv / 8;
  // K / V tiles are double-buffered: the asynchronous copies of tile i + 1 are in flight while tile i is multiplied
  // (cp.async of 16 bytes; rows past the request's last position are filled with zeros by a zero source size)
  const int stage_elems = FN * (ldk + dv + 8);
  // thread t copies 16-byte piece (t % 16) + 16 n of rows (t / 16) + 8 m: the page lookup and the row's cache offset are
  // computed once per row and serve its K and its V pieces
  auto issue_tile = [&](int c0, int stage) {
    __nv_bfloat16* Kd = Ks + stage * stage_elems;
    __nv_bfloat16* Vd = Kd + FN * ldk;
    const int piece = tid & 15;
#pragma unroll 2
    for (int kk = tid >> 4; kk < FN; kk += 8) {
      const int kj = c0 + kk;
      const bool ok = kj <= pos_last;
      const int kq = ok ? kj : pos_last;                 // (a valid address also for the zero-filled rows)
      const int pg = kq / p.page_size;
      const size_t tok = static_cast<size_t>(pages[pg]) * p.page_size + (kq - pg * p.page_size);
      const uint32_t nbytes = ok ? 16u : 0u;
      for (int c = piece; c < qv; c += 16)
        asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(Kd + kk * ldk + c * 8)),
                     "l"(kc + tok * p.k_ld + g * dk + c * 8), "r"(nbytes) : "memory");
      if (!same_kv)
        for (int c = piece; c < vv; c += 16)
          asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_u32(Vd + kk * ldv + c * 8)),
                       "l"(vc + tok * p.v_ld + gv * dv + c * 8), "r"(nbytes) : "memory");
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  __syncthreads();                    // every warp holds its Q fragments: the first stage may be overwritten
  const int c_first = lo + sidx * FN, c_step = FN * S;
  if (c_first <= pos_last) issue_tile(c_first, 0);
  int stage = 0;
  for (int c0 = c_first; c0 <= pos_last; c0 += c_step, stage ^= 1) {
    if (c0 + c_step <= pos_last) {
      issue_tile(c0 + c_step, stage ^ 1);
      asm volatile("cp.async.wait_group 1;" ::: "memory");
    } else {
      asm volatile("cp.async.wait_group 0;" ::: "memory");
    }
    __syncthreads();
    const __nv_bfloat16* Kt = Ks + stage * stage_elems;
    const __nv_bfloat16* Vt = same_kv ? Kt : Kt + FN * ldk;
    // a warp whose 16 rows see nothing of this tile has no work in it
    const int w_first = pos0 + warp * 16 * pstep, w_last = min(pos0 + (warp * 16 + 15) * pstep, pos_last);
    const int w_lo = wa_first_key(p, w_first);
    const bool idle = warp * 16 >= nrows || c0 > w_last || c0 + FN - 1 < w_lo;
    if (!idle) {
    float sc[FN / 8][4];
#pragma unroll
    for (int n = 0; n < FN / 8; ++n) sc[n][0] = sc[n][1] = sc[n][2] = sc[n][3] = 0.f;
#pragma unroll
    for (int kb = 0; kb < KB; ++kb) {
      if (kb < nkb) {
#pragma unroll
        for (int np = 0; np < FN / 16; ++np) {
          uint32_t kf[4];
          ldmatrix_x4(kf, smem_u32(Kt + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * ldk + kb * 16 + ((lane >> 3) & 1) * 8));
          mma_bf16_16816(sc[2 * np], qf[kb], kf[0], kf[1]);
          mma_bf16_16816(sc[2 * np + 1], qf[kb], kf[2], kf[3]);
        }
      }
    }
    float mxA = -INFINITY, mxB = -INFINITY;
#pragma unroll
    for (int n = 0; n < FN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int kj = c0 + n * 8 + (lane & 3) * 2 + (e & 1);
        const bool vis = e < 2 ? (okA && kj <= posA && kj >= loA) : (okB && kj <= posB && kj >= loB);
        const float v = vis ? sc[n][e] * p.scale : -INFINITY;
        sc[n][e] = v;
        if (e < 2) mxA = fmaxf(mxA, v);
        else mxB = fmaxf(mxB, v);
      }
    }
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
    mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
    mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
    const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
    const float cA = nA == -INFINITY ? 1.f : expf(mA - nA), cB = nB == -INFINITY ? 1.f : expf(mB - nB);
    float sA = 0.f, sB = 0.f;
#pragma unroll
    for (int n = 0; n < FN / 8; ++n) {
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const float v = sc[n][e];
        const float pj = v == -INFINITY ? 0.f : expf(v - (e < 2 ? nA : nB));
        sc[n][e] = pj;
        if (e < 2) sA += pj;
        else sB += pj;
      }
    }
    sA += __shfl_xor_sync(0xffffffffu, sA, 1);
    sA += __shfl_xor_sync(0xffffffffu, sA, 2);
    sB += __shfl_xor_sync(0xffffffffu, sB, 1);
    sB += __shfl_xor_sync(0xffffffffu, sB, 2);
    lA = lA * cA + sA;
    lB = lB * cB + sB;
    mA = nA;
    mB = nB;
#pragma unroll
    for (int n = 0; n < F_NT; ++n) {
      o[n][0] *= cA; o[n][1] *= cA; o[n][2] *= cB; o[n][3] *= cB;
    }
#pragma unroll
    for (int kb = 0; kb < FN / 16; ++kb) {
      uint32_t pa[4];
      pa[0] = pack_bf16(sc[2 * kb][0], sc[2 * kb][1]);
      pa[1] = pack_bf16(sc[2 * kb][2], sc[2 * kb][3]);
      pa[2] = pack_bf16(sc[2 * kb + 1][0], sc[2 * kb + 1][1]);
      pa[3] = pack_bf16(sc[2 * kb + 1][2], sc[2 * kb + 1][3]);
#pragma unroll
      for (int np = 0; np < F_NT / 2; ++np) {
        if (np < nvp) {
          uint32_t vf[4];
          ldmatrix_x4_trans(vf, smem_u32(Vt + (kb * 16 + ((lane >> 3) & 1) * 8 + (lane & 7)) * ldv + np * 16 + (lane >> 4) * 8));
          mma_bf16_16816(o[2 * np], pa, vf[0], vf[1]);
          mma_bf16_16816(o[2 * np + 1], pa, vf[2], vf[3]);
        }
      }
    }
    }
    __syncthreads();                  // this stage is free for the copies of the tile after the next
  }
  if (S > 1) {
    // this split's share of every (token, head): unnormalised output, running max, running sum (a split without keys
    // leaves max -inf and sum 0)
#pragma unroll
    for (int half = 0; half < 2; ++half) {
      if (!(half ? okB : okA)) continue;
      const int head = g * nrows + (half ? rB : rA);
      float* pt = p.part + ((static_cast<size_t>(blockIdx.x) * p.H + head) * S + sidx) * (dv + 2);
#pragma unroll
      for (int n = 0; n < F_NT; ++n) {
        const int d = n * 8 + (lane & 3) * 2;
        if (d < dv) { pt[d] = o[n][2 * half]; pt[d + 1] = o[n][2 * half + 1]; }
      }
      if ((lane & 3) == 0) { pt[dv] = half ? mB : mA; pt[dv + 1] = half ? lB : lA; }
    }
    return;
  }
  const float iA = okA ? 1.f / lA : 0.f, iB = okB ? 1.f / lB : 0.f;
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out);
#pragma unroll
  for (int n = 0; n < F_NT; ++n) {
    const int d = n * 8 + (lane & 3) * 2;
    if (d < dv) {
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        if (!(half ? okB : okA)) continue;
        const int t = row0 + (half ? rB : rA);          // (row_heads: token * H + head)
        float x0 = o[n][2 * half] * (half ? iB : iA), x1 = o[n][2 * half + 1] * (half ? iB : iA);
        if (p.gate) {
          const float* gt = p.row_heads ? p.gate + static_cast<size_t>(t / p.H) * p.ld_gate + (t % p.H) * dv + d
                                        : p.gate + static_cast<size_t>(t) * p.ld_gate + h * dv + d;
          x0 *= 1.f / (1.f + expf(-gt[0]));
          x1 *= 1.f / (1.f + expf(-gt[1]));
        }
        const size_t oi = static_cast<size_t>(t) * HH * dv + h * dv + d;
        if (p.out_f32) *reinterpret_cast<float2*>(static_cast<float*>(p.out) + oi) = make_float2(x0, x1);
        else *reinterpret_cast<uint32_t*>(out + oi) = pack_bf16(x0, x1);
      }
    }
  }
}

}  // namespace vb

using namespace vb;
using bf16 = __nv_bfloat16;

extern "C" {

int vb_rotary_table(float* d_cs, const int32_t* d_pos, const double* d_freq, int T, int half, double mult, void* stream) {
  VB_CHECK_ARG(d_cs && d_pos && d_freq && half > 0, "vb_rotary_table: bad arguments");
  if (T <= 0) return 0;
  VB_LAUNCH_PDL(rotary_table_kernel, (T * half + 255) / 256, 256, 0, stream, d_cs, d_pos, d_freq, T, half, mult);
  return 0;
}

int vb_qkv_norm_rotary_append(const float* d_proj, int ldp, int q_off, int k_off, int v_off, const float* d_cs, int half,
                              int layout, const float* d_q_norm, const float* d_k_norm, float eps, void* d_q_out,
                              void* d_k_cache, void* d_v_cache, const int32_t* d_row_req, const int32_t* d_pos,
                              const int32_t* d_page_indptr, const int32_t* d_page_indices, int page_size, int T, int Hq, int Gk,
                              int Gv, int dim, int vdim, int dtype, void* stream) {
  VB_CHECK_ARG(d_proj && d_q_out && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_qkv_norm_rotary_append: null pointer");
  VB_CHECK_ARG(Hq > 0 && Gk > 0 && Gv > 0 && dim > 0 && vdim > 0 && page_size > 0 && half >= 0 && 2 * half <= dim &&
               (layout == 0 || layout == 1), "vb_qkv_norm_rotary_append: bad sizes Hq=%d Gk=%d Gv=%d dim=%d vdim=%d rotated=%d",
               Hq, Gk, Gv, dim, vdim, 2 * half);
  if (T <= 0) return 0;
  QkvNormTailParams p{d_proj, ldp, q_off, k_off, v_off, half > 0 ? d_cs : nullptr, half, layout, d_q_norm, d_k_norm, eps,
                      d_q_out, d_k_cache, d_v_cache, d_row_req, d_pos, d_page_indptr, d_page_indices, page_size, Hq, Gk, Gv,
                      dim, vdim, 0, 0};
  // the q | k | v columns of a row are staged in shared memory when they lie side by side and fit
  const int lo = min(q_off, min(k_off, v_off)), hi = max(q_off + Hq * dim, max(k_off + Gk * dim, v_off + Gv * vdim));
  size_t smem = 0;
  if (hi - lo == (Hq + Gk) * dim + Gv * vdim && static_cast<size_t>(hi - lo) * sizeof(float) <= static_cast<size_t>(VB_MAX_DYN_SMEM)) {
    p.stage_lo = lo; p.stage_hi = hi;
    smem = static_cast<size_t>(hi - lo) * sizeof(float);
  }
  if (dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(qkv_norm_rotary_append_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(qkv_norm_rotary_append_kernel<float>, T, 256, smem, stream, p);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(qkv_norm_rotary_append_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(qkv_norm_rotary_append_kernel<bf16>, T, 256, smem, stream, p);
  }
  return 0;
}

int vb_latent_rope_append(const float* d_proj, int ldp, int q_off, int c_off, int H, int dim, int rot, int kv_rank,
                          const float* d_wc, const float* d_cs, int half, int layout, void* d_q_out, void* d_q_lat,
                          void* d_cache, const int32_t* d_row_req, const int32_t* d_pos, const int32_t* d_page_indptr,
                          const int32_t* d_page_indices, int page_size, int T, float eps, int dtype, void* stream) {
  // d_cache == nullptr: the layer reads rows that another layer cached; only its queries are laid out (c_off, d_wc unused)
  VB_CHECK_ARG(d_proj && d_q_out && d_q_lat && d_row_req && d_pos && d_page_indptr && d_page_indices && (!d_cache || d_wc),
               "vb_latent_rope_append: null pointer");
  const int c_cols = d_cache ? kv_rank + rot : 0;
  if (!d_cache) c_off = q_off;
  VB_CHECK_ARG(H > 0 && dim >= 0 && rot >= 0 && dim + rot > 0 && kv_rank > 0 && page_size > 0 && half >= 0 && 2 * half <= rot &&
               (layout == 0 || layout == 1) && q_off >= 0 && c_off >= 0 && q_off + H * (dim + rot) <= ldp &&
               c_off + c_cols <= ldp, "vb_latent_rope_append: bad sizes H=%d dim=%d rot=%d kv_rank=%d rotated=%d",
               H, dim, rot, kv_rank, 2 * half);
  if (T <= 0) return 0;
  LatentRopeTailParams p{d_proj, ldp, q_off, c_off, H, dim, rot, kv_rank, d_wc, half > 0 ? d_cs : nullptr, half, layout,
                         d_q_out, d_q_lat, d_cache, d_row_req, d_pos, d_page_indptr, d_page_indices, page_size, eps, 0, 0};
  const int lo = min(q_off, c_off), hi = max(q_off + H * (dim + rot), c_off + c_cols);
  size_t smem = 0;
  if (hi - lo == H * (dim + rot) + c_cols && static_cast<size_t>(hi - lo) * sizeof(float) <= static_cast<size_t>(VB_MAX_DYN_SMEM)) {
    p.stage_lo = lo; p.stage_hi = hi;
    smem = static_cast<size_t>(hi - lo) * sizeof(float);
  }
  if (dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(latent_rope_append_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(latent_rope_append_kernel<float>, T, LR_THREADS, smem, stream, p);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(latent_rope_append_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(latent_rope_append_kernel<bf16>, T, LR_THREADS, smem, stream, p);
  }
  return 0;
}

int vb_head_pair_combine(void* d_out, const float* d_a, const float* d_gate, int ld_gate, int T, int H, int R, int vdim,
                         float lambda, float post, float eps, int dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_a && H > 0 && R > 0 && H % R == 0 && vdim > 0, "vb_head_pair_combine: bad arguments");
  if (T <= 0) return 0;
  const int grid = (T * H + 3) / 4;
  if (dtype == 1)
    VB_LAUNCH_PDL(head_pair_combine_kernel<float>, grid, 128, 0, stream, static_cast<float*>(d_out), d_a, d_gate, ld_gate, T, H, R,
                  vdim, lambda, post, eps);
  else
    VB_LAUNCH_PDL(head_pair_combine_kernel<bf16>, grid, 128, 0, stream, static_cast<bf16*>(d_out), d_a, d_gate, ld_gate, T, H, R,
                  vdim, lambda, post, eps);
  return 0;
}

int vb_qkv_rotary_append(const float* d_proj, int ldp, int q_off, int k_off, int v_off, const float* d_cs, int half,
                         void* d_q_out, void* d_k_cache, void* d_v_cache, const int32_t* d_row_req, const int32_t* d_pos,
                         const int32_t* d_page_indptr, const int32_t* d_page_indices, int page_size, int T, int H, int G,
                         int dim, int vdim, int vmix, float* d_v_first, const float* d_lambda, int dtype, void* stream) {
  VB_CHECK_ARG(d_proj && d_q_out && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_qkv_rotary_append: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && page_size > 0 && 2 * half <= dim,
               "vb_qkv_rotary_append: bad sizes H=%d G=%d dim=%d vdim=%d rotated=%d", H, G, dim, vdim, 2 * half);
  VB_CHECK_ARG(vmix == 0 || d_v_first, "vb_qkv_rotary_append: value mixing needs the first layer's values");
  VB_CHECK_ARG(vmix != 2 || d_lambda, "vb_qkv_rotary_append: value mixing needs its coefficient");
  if (T <= 0) return 0;
  QkvTailParams p{d_proj, ldp, q_off, k_off, v_off, half > 0 ? d_cs : nullptr, half, d_q_out, d_k_cache, d_v_cache,
                  d_row_req, d_pos, d_page_indptr, d_page_indices, page_size, H, G, dim, vdim, vmix, d_v_first, d_lambda};
  if (dtype == 1) VB_LAUNCH_PDL(qkv_rotary_append_kernel<float>, T, 256, 0, stream, p);
  else VB_LAUNCH_PDL(qkv_rotary_append_kernel<bf16>, T, 256, 0, stream, p);
  return 0;
}

int vb_latent_norm_append(const float* d_proj, int ldp, int q_off, int c_off, int q_rank, int kv_rank, const float* d_wq,
                          const float* d_wc, void* d_cq_out, void* d_c_cache, const int32_t* d_row_req, const int32_t* d_pos,
                          const int32_t* d_page_indptr, const int32_t* d_page_indices, int page_size, int T, float eps,
                          int dtype, void* stream) {
  VB_CHECK_ARG(d_proj && d_wq && d_cq_out && q_rank > 0 && q_off >= 0 && q_off + q_rank <= ldp,
               "vb_latent_norm_append: bad query latent");
  VB_CHECK_ARG(!d_c_cache || (d_wc && d_row_req && d_pos && d_page_indptr && d_page_indices && kv_rank > 0 && page_size > 0 &&
                              c_off >= 0 && c_off + kv_rank <= ldp), "vb_latent_norm_append: bad key/value latent");
  if (T <= 0) return 0;
  LatentTailParams p{d_proj, ldp, q_off, c_off, q_rank, kv_rank, d_wq, d_wc, d_cq_out, d_c_cache, d_row_req, d_pos,
                     d_page_indptr, d_page_indices, page_size, eps};
  if (dtype == 1) VB_LAUNCH_PDL(latent_norm_append_kernel<float>, T, 128, 0, stream, p);
  else VB_LAUNCH_PDL(latent_norm_append_kernel<bf16>, T, 128, 0, stream, p);
  return 0;
}

int vb_window_attn(void* d_out, const void* d_q, const void* d_k_cache, const void* d_v_cache, const float* d_gate,
                   int ld_gate, const int32_t* d_row_req, const int32_t* d_pos, const int32_t* d_page_indptr,
                   const int32_t* d_page_indices, int T, int H, int G, int dim, int vdim, int page_size, int window,
                   float scale, int dtype, float* d_part, long long part_floats, const int32_t* d_row_list, int head_rows,
                   int chunk, int k_ld, int v_ld, int v_share, int out_f32, void* stream) {
  VB_CHECK_ARG(d_out && d_q && d_k_cache && d_v_cache && d_row_req && d_pos && d_page_indptr && d_page_indices,
               "vb_window_attn: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 32 * WA_MAXU && page_size > 0,
               "vb_window_attn: bad sizes H=%d G=%d dim=%d vdim=%d (vdim <= %d)", H, G, dim, vdim, 32 * WA_MAXU);
  if (T <= 0) return 0;
  if (v_share <= 0) v_share = 1;
  VB_CHECK_ARG(G % v_share == 0, "vb_window_attn: %d key heads do not share value heads %d by %d", G, v_share, v_share);
  if (k_ld <= 0) k_ld = G * dim;
  if (v_ld <= 0) v_ld = (G / v_share) * vdim;
  WindowAttnParams p{d_q, d_k_cache, d_v_cache, d_out, d_gate, ld_gate, d_row_req, d_pos, d_page_indptr, d_page_indices,
                     nullptr, nullptr, nullptr, T, H, G, dim, vdim, page_size, window, chunk, k_ld, v_ld, v_share, out_f32,
                     scale, d_row_list, 0, 1, d_part};
  const int R = H / G;
  const bool mma_ok = dtype == 0 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 16 * F_KB && vdim <= 8 * F_NT &&
                      k_ld % 8 == 0 && v_ld % 8 == 0;
  // head_rows: the query heads that share a key/value head become the rows of a tensor-core tile (bf16, head sizes the
  // tile kernel takes, 2 .. 64 heads per group): the group's K / V tiles are staged once and multiplied on the tensor cores
  if (head_rows && mma_ok && R >= 2 && R <= FM) {
    int splits = 1;
    if (d_part) {
      splits = max(1, min(8, (2 * 148) / max(1, T * G)));
      while (splits > 1 && static_cast<long long>(T) * H * splits * (vdim + 2) > part_floats) --splits;
    }
    p.row_heads = 1;
    p.splits = splits;
    const size_t msmem = 2 * static_cast<size_t>(FN) * (dim + 8 + vdim + 8) * sizeof(__nv_bfloat16);
    if (dim <= 128) {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_mma_kernel<8>, dim3(T, G, splits), 128, msmem, stream, p);
    } else {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<F_KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_mma_kernel<F_KB>, dim3(T, G, splits), 128, msmem, stream, p);
    }
    if (splits > 1) VB_LAUNCH_PDL(window_attn_merge_kernel<bf16>, dim3(T, H), 64, 0, stream, p);
    return 0;
  }
  // a CTA per (row, key/value head) with the K / V tiles shared by the group's query heads, when the group fits its
  // registers and the tiles fit shared memory; one warp per (row, query head) otherwise
  const size_t gsmem = (static_cast<size_t>(R) * dim + static_cast<size_t>(WD_KEYS) * (dim + 1 + vdim + 1) +
                        static_cast<size_t>(R) * WD_KEYS) * sizeof(float);
  if (R <= 4 * WD_RU && vdim <= 32 * WD_VU && gsmem <= 96 * 1024) {
    // few rows leave most SMs idle and every CTA a long serial walk: deal the key tiles of a row to several CTAs
    // (about four CTAs per SM in all) and merge their shares; needs the scratch buffer
    int splits = 1;
    if (d_part) {
      splits = max(1, min(8, (4 * 148) / max(1, T * G)));
      while (splits > 1 && static_cast<long long>(T) * H * splits * (vdim + 2) > part_floats) --splits;
    }
    p.splits = splits;
    dim3 ggrid(T, G, splits);
    if (dtype == 1) {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_group_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_group_kernel<float>, ggrid, 128, gsmem, stream, p);
      if (splits > 1) VB_LAUNCH_PDL(window_attn_merge_kernel<float>, dim3(T, H), 64, 0, stream, p);
    } else {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_group_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_group_kernel<bf16>, ggrid, 128, gsmem, stream, p);
      if (splits > 1) VB_LAUNCH_PDL(window_attn_merge_kernel<bf16>, dim3(T, H), 64, 0, stream, p);
    }
    return 0;
  }
  const size_t smem = static_cast<size_t>(WA_WARPS) * dim * sizeof(float);
  VB_CHECK_ARG(smem <= 48 * 1024, "vb_window_attn: head dim %d too large", dim);
  dim3 grid((T + WA_WARPS - 1) / WA_WARPS, H);
  if (dtype == 1) VB_LAUNCH_PDL(window_attn_kernel<float>, grid, WA_WARPS * 32, smem, stream, p);
  else VB_LAUNCH_PDL(window_attn_kernel<bf16>, grid, WA_WARPS * 32, smem, stream, p);
  return 0;
}

int vb_window_attn_tile_rows(void) { return WT_ROWS; }

int vb_window_attn_tiled(void* d_out, const void* d_q, const void* d_k_cache, const void* d_v_cache, const float* d_gate,
                         int ld_gate, const int32_t* d_pos, const int32_t* d_page_indptr, const int32_t* d_page_indices,
                         const int32_t* d_qo_indptr, const int32_t* d_tile_req, const int32_t* d_tile_row0, int n_tiles,
                         int T, int H, int G, int dim, int vdim, int page_size, int window, float scale, int dtype,
                         int chunk, int k_ld, int v_ld, int v_share, int out_f32, void* stream) {
  VB_CHECK_ARG(d_out && d_q && d_k_cache && d_v_cache && d_pos && d_page_indptr && d_page_indices && d_qo_indptr &&
               d_tile_req && d_tile_row0, "vb_window_attn_tiled: null pointer");
  VB_CHECK_ARG(H > 0 && G > 0 && H % G == 0 && dim > 0 && vdim > 0 && vdim <= 4 * WT_MAXD && page_size > 0,
               "vb_window_attn_tiled: bad sizes H=%d G=%d dim=%d vdim=%d", H, G, dim, vdim);
  if (n_tiles <= 0) return 0;
  if (v_share <= 0) v_share = 1;
  VB_CHECK_ARG(G % v_share == 0, "vb_window_attn_tiled: %d key heads do not share value heads %d by %d", G, v_share, v_share);
  if (k_ld <= 0) k_ld = G * dim;
  if (v_ld <= 0) v_ld = (G / v_share) * vdim;
  WindowAttnParams p{d_q, d_k_cache, d_v_cache, d_out, d_gate, ld_gate, nullptr, d_pos, d_page_indptr, d_page_indices,
                     d_qo_indptr, d_tile_req, d_tile_row0, T, H, G, dim, vdim, page_size, window, chunk, k_ld, v_ld, v_share,
                     out_f32, scale, nullptr, 0, 1, nullptr};
  dim3 grid(n_tiles, H);
  if (dtype == 0 && dim % 16 == 0 && vdim % 16 == 0 && dim <= 16 * F_KB && vdim <= 8 * F_NT && k_ld % 8 == 0 && v_ld % 8 == 0) {
    const size_t msmem = 2 * static_cast<size_t>(FN) * (dim + 8 + vdim + 8) * sizeof(__nv_bfloat16);      // two stages
    if (dim <= 128) {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_mma_kernel<8>, grid, 128, msmem, stream, p);
    } else {
      VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_mma_kernel<F_KB>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
      VB_LAUNCH_PDL(window_attn_mma_kernel<F_KB>, grid, 128, msmem, stream, p);
    }
    return 0;
  }
  const size_t smem = (static_cast<size_t>(WT_ROWS + WT_KEYS) * (dim + 1) + static_cast<size_t>(WT_KEYS) * (vdim + 1) +
                       static_cast<size_t>(WT_ROWS) * (WT_KEYS + 1)) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_window_attn_tiled: heads too large for shared memory");
  if (dtype == 1) {
    VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_tiled_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(window_attn_tiled_kernel<float>, grid, 256, smem, stream, p);
  } else {
    VB_CHECK_CUDA(cudaFuncSetAttribute(window_attn_tiled_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(window_attn_tiled_kernel<bf16>, grid, 256, smem, stream, p);
  }
  return 0;
}

}  // extern "C"
