// Building blocks of the hybrid (attention + linear-attention + mixture-of-experts) decoder stacks whose residual
// stream is kept in fp32: embedding rows into an fp32 stream, LayerNorm with weight and bias (alone, and fused as
// "post-norm -> residual add -> next pre-norm"), and a shape-agnostic linear layer Y = X W^T with fp32 accumulation for
// bf16 or fp32 operands, dense or grouped by expert with gathered input rows.
//
// The linear kernel is the any-shape, any-precision path: every output is ONE sequential fp32 FMA chain over k, so a
// row's result does not depend on which other rows share the launch (batch invariance) and fp32 operands are computed in
// true fp32.  bf16 projections whose shapes fit the tcgen05 kernel (gemm.cu) are routed there by the engine.
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 4
#include "common.cuh"

namespace vb {

template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float block_sum(float v, float* red, int& phase) {
  // red: 64 floats of shared memory used as two alternating halves, so that one barrier per call is enough: a warp can only
  // be one call ahead of the slowest warp, and then it writes the other half.  Every thread gets the total, summed in the
  // same order by every warp.
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
  float* r = red + 32 * (phase & 1);
  ++phase;
  v = warp_sum(v);
  if (lane == 0) r[w] = v;
  __syncthreads();
  float t = lane < nw ? r[lane] : 0.f;
  return warp_sum(t);
}

// out[t] = table[ids[t]] * scale (+ pos_table[pos[t]]: learned absolute positions, added unscaled in fp32); out2: a second
// copy of the rows (stacks that add the embedding again later keep it)
template <typename WT>
__global__ void embed_rows_kernel(float* __restrict__ out, const WT* __restrict__ table, const int32_t* __restrict__ ids,
                                  int W, int vocab, const WT* __restrict__ pos_table, const int32_t* __restrict__ pos,
                                  int n_pos, float scale, float* __restrict__ out2) {
  pdl_sync();
  const int t = blockIdx.x;
  int id = ids[t];
  id = min(max(id, 0), vocab - 1);
  const WT* src = table + static_cast<size_t>(id) * W;
  const WT* ps = nullptr;
  if (pos_table) ps = pos_table + static_cast<size_t>(min(max(pos[t], 0), n_pos - 1)) * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = to_f(src[i]) * scale + (ps ? to_f(ps[i]) : 0.f);
    out[static_cast<size_t>(t) * W + i] = v;
    if (out2) out2[static_cast<size_t>(t) * W + i] = v;
  }
}

// RMS norm of a row with one or two weights: out1[t] = x[r] / sqrt(mean(x[r]^2) + eps) * w1, out2[t] likewise with w2
// (the two sublayers of a parallel block read differently weighted norms of the same row)
template <typename OT>
__global__ void rmsnorm2_kernel(OT* __restrict__ out1, OT* __restrict__ out2, const float* __restrict__ x,
                                const float* __restrict__ w1, const float* __restrict__ w2, int W, float eps,
                                const int32_t* __restrict__ rows) {
  extern __shared__ float sm[];
  float* row = sm;
  float* red = sm + W;
  int phase = 0;
  pdl_sync();
  const size_t t = blockIdx.x;
  const size_t src = rows ? static_cast<size_t>(rows[t]) : t;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = x[src * W + i];
    row[i] = v;
    q = fmaf(v, v, q);
  }
  const float rs = 1.f / sqrtf(block_sum(q, red, phase) / W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = row[i] * rs;
    out1[t * W + i] = from_f<OT>(v * w1[i]);
    if (out2) out2[t * W + i] = from_f<OT>(v * w2[i]);
  }
}

// Stacks that norm what a sublayer returns instead of what it reads; in place on the fp32 stream: x[t] += y[t] / sqrt(mean(y[t]^2) + eps) * w, and (optional)
// out[t] = x[t] in the compute type: what a following sublayer reads when it takes the stream itself, un-normed.
template <typename OT>
__global__ void __launch_bounds__(256) rms_postnorm_residual_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                    const float* __restrict__ w, OT* __restrict__ out, int W,
                                                                    float eps) {
  extern __shared__ float sm[];
  float* row = sm;
  float* red = sm + W;
  int phase = 0;
  pdl_sync();
  const size_t t = blockIdx.x;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = y[t * W + i];
    row[i] = v;
    q = fmaf(v, v, q);
  }
  const float rs = 1.f / sqrtf(block_sum(q, red, phase) / W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = x[t * W + i] + row[i] * rs * w[i];
    x[t * W + i] = v;
    if (out) out[t * W + i] = from_f<OT>(v);
  }
}

__device__ __forceinline__ float act_apply(float v, int act) {
  // 2: relu(v)^2   3: gelu, exact (erf)   4: gelu, tanh form
  if (act == 2) { const float r = fmaxf(v, 0.f); return r * r; }
  if (act == 3) return 0.5f * v * (1.f + erff(v * 0.70710678118654752f));
  if (act == 4) return 0.5f * v * (1.f + tanhf(0.79788456080286536f * (v + 0.044715f * v * v * v)));
  return v;
}

// The tail of a block whose sublayers run in parallel on the same residual row:
//   x[t] += mult * (y1[t] + y2[t])
//   per-token side input (optional): g = gelu_tanh(Wg x[t]) * e[t], y = Wp g, x[t] += mult * y / sqrt(mean(y^2) + eps) * ws
//     with e[t] = side_embed[ids[t]][e_off .. e_off + side_dim)
//   out1[t] = rms_norm(x[t]) * w1, out2[t] = rms_norm(x[t]) * w2 (optional: what the next block's sublayers read)
// Everything in fp32 on the fp32 row; the side matrices are read in their storage type.
struct ResidualSideParams {
  float* x;
  const float* y1;
  const float* y2;
  const void* side_gate;    // [side_dim][W]
  const void* side_proj;    // [W][side_dim]
  const float* side_norm;   // [W]
  const void* side_embed;   // [vocab][ld_e]
  const int32_t* ids;
  void* out1;
  void* out2;
  const float* w1;
  const float* w2;
  int W, side_dim, ld_e, e_off, vocab, T;
  float mult, eps;
};

// eight consecutive elements as fp32 (16-byte loads; the caller guarantees the alignment)
template <typename WT> __device__ __forceinline__ void load8(const WT* __restrict__ p, float (&v)[8]);
template <> __device__ __forceinline__ void load8<float>(const float* __restrict__ p, float (&v)[8]) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}
template <> __device__ __forceinline__ void load8<__nv_bfloat16>(const __nv_bfloat16* __restrict__ p, float (&v)[8]) {
  const uint4 a = *reinterpret_cast<const uint4*>(p);
  v[0] = bf16_lo(a.x); v[1] = bf16_hi(a.x); v[2] = bf16_lo(a.y); v[3] = bf16_hi(a.y);
  v[4] = bf16_lo(a.z); v[5] = bf16_hi(a.z); v[6] = bf16_lo(a.w); v[7] = bf16_hi(a.w);
}

template <typename OT> __device__ __forceinline__ void store4(OT* __restrict__ p, float a, float b, float c, float d);
template <> __device__ __forceinline__ void store4<float>(float* __restrict__ p, float a, float b, float c, float d) {
  *reinterpret_cast<float4*>(p) = make_float4(a, b, c, d);
}
template <> __device__ __forceinline__ void store4<__nv_bfloat16>(__nv_bfloat16* __restrict__ p, float a, float b, float c, float d) {
  *reinterpret_cast<uint2*>(p) = make_uint2(pack_bf16(a, b), pack_bf16(c, d));
}

// The tail of a pre-norm sublayer with a gated residual, in place on the fp32 row:
//   x[t] += sigmoid(r[t] + b) * y[t]      (r: the gate's projection of the sublayer's input, b its bias; r == nullptr: x += y)
//   x[t] += add[t]                        (optional: e.g. the embedding entering a repeated pass over the layers)
//   out[t] = x[t] / sqrt(mean(x[t]^2) + eps) * w      (optional: what the next sublayer reads)
template <typename OT>
__global__ void __launch_bounds__(256) gated_residual_norm_kernel(float* __restrict__ x, const float* __restrict__ y,
                                                                  const float* __restrict__ r, int ld_r,
                                                                  const float* __restrict__ bias, const float* __restrict__ add,
                                                                  OT* __restrict__ out, const float* __restrict__ w, int W,
                                                                  float eps, int vec) {
  extern __shared__ float sm[];
  float* row = sm;
  float* red = sm + W;
  int phase = 0;
  pdl_sync();
  const size_t t = blockIdx.x;
  float q = 0.f;
  if (vec) {
    // rows that move in 16-byte pieces (width, gate stride and every base pointer allow it): all loads of a piece in flight
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      const float4 xv = *reinterpret_cast<const float4*>(x + t * W + i);
      const float4 yv = *reinterpret_cast<const float4*>(y + t * W + i);
      float4 g = make_float4(1.f, 1.f, 1.f, 1.f);
      if (r) {
        const float4 rv = *reinterpret_cast<const float4*>(r + t * ld_r + i);
        const float4 bv = bias ? *reinterpret_cast<const float4*>(bias + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        g.x = 1.f / (1.f + expf(-(rv.x + bv.x))); g.y = 1.f / (1.f + expf(-(rv.y + bv.y)));
        g.z = 1.f / (1.f + expf(-(rv.z + bv.z))); g.w = 1.f / (1.f + expf(-(rv.w + bv.w)));
      }
      float4 v = make_float4(xv.x + g.x * yv.x, xv.y + g.y * yv.y, xv.z + g.z * yv.z, xv.w + g.w * yv.w);
      if (add) {
        const float4 av = *reinterpret_cast<const float4*>(add + t * W + i);
        v.x += av.x; v.y += av.y; v.z += av.z; v.w += av.w;
      }
      *reinterpret_cast<float4*>(x + t * W + i) = v;
      *reinterpret_cast<float4*>(row + i) = v;
      q = fmaf(v.x, v.x, q); q = fmaf(v.y, v.y, q); q = fmaf(v.z, v.z, q); q = fmaf(v.w, v.w, q);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      float g = 1.f;
      if (r) g = 1.f / (1.f + expf(-(r[t * ld_r + i] + (bias ? bias[i] : 0.f))));
      float v = x[t * W + i] + g * y[t * W + i];
      if (add) v += add[t * W + i];
      x[t * W + i] = v;
      row[i] = v;
      q = fmaf(v, v, q);
    }
  }
  if (out == nullptr) return;
  const float rs = 1.f / sqrtf(block_sum(q, red, phase) / W + eps);
  if (vec) {
    for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
      const float4 v = *reinterpret_cast<const float4*>(row + i);
      const float4 wv = *reinterpret_cast<const float4*>(w + i);
      store4<OT>(out + t * W + i, v.x * rs * wv.x, v.y * rs * wv.y, v.z * rs * wv.z, v.w * rs * wv.w);
    }
  } else {
    for (int i = threadIdx.x; i < W; i += blockDim.x) out[t * W + i] = from_f<OT>(row[i] * rs * w[i]);
  }
}

// ROWS rows per CTA: the side matrices are read once per CTA and serve all of its rows (long steps).  A row's result
// depends on nothing but the row; between the one-row form (16 warps) and the four-row form (8 warps) only the order in
// which the norms' sums of squares are added differs.
template <typename WT, typename OT, int ROWS>
__global__ void __launch_bounds__(512) residual_side_kernel(ResidualSideParams p) {
  extern __shared__ float sm[];
  const int W = p.W, SD = p.side_dim;
  float* row = sm;                      // [ROWS][W]
  float* yb = row + ROWS * W;           // [ROWS][W]
  float* g = yb + ROWS * W;             // [ROWS][SD]
  float* red = g + ROWS * SD;           // [64]
  int phase = 0;
  pdl_sync();
  const size_t t0 = static_cast<size_t>(blockIdx.x) * ROWS;
  const int nr = min(ROWS, p.T - static_cast<int>(t0));
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = blockDim.x >> 5;
  const bool w4 = (W & 3) == 0;          // rows move in 16-byte pieces
  if (w4) {
    const int n4 = W >> 2;
    for (int i = threadIdx.x; i < nr * n4; i += blockDim.x) {
      const size_t o = t0 * W + static_cast<size_t>(i) * 4;
      float4 y = *reinterpret_cast<const float4*>(p.y1 + o);
      if (p.y2) {
        const float4 y2 = *reinterpret_cast<const float4*>(p.y2 + o);
        y.x += y2.x; y.y += y2.y; y.z += y2.z; y.w += y2.w;
      }
      const float4 xv = *reinterpret_cast<const float4*>(p.x + o);
      *reinterpret_cast<float4*>(row + static_cast<size_t>(i) * 4) =
          make_float4(fmaf(p.mult, y.x, xv.x), fmaf(p.mult, y.y, xv.y), fmaf(p.mult, y.z, xv.z), fmaf(p.mult, y.w, xv.w));
    }
  } else {
    for (int r = 0; r < nr; ++r)
      for (int i = threadIdx.x; i < W; i += blockDim.x) {
        float y = p.y1[(t0 + r) * W + i];
        if (p.y2) y += p.y2[(t0 + r) * W + i];
        row[r * W + i] = fmaf(p.mult, y, p.x[(t0 + r) * W + i]);
      }
  }
  for (int r = nr; r < ROWS; ++r)
    for (int i = threadIdx.x; i < W; i += blockDim.x) row[r * W + i] = 0.f;
  __syncthreads();
  if (p.side_gate) {
    const WT* Wg = static_cast<const WT*>(p.side_gate);
    const WT* Wp = static_cast<const WT*>(p.side_proj);
    const bool vec = (W & 7) == 0 && (SD & 7) == 0;
    // gate: a warp forms DU dot products at once (DU independent weight streams in flight per lane); every dot product is
    // summed in the same order whatever DU and ROWS are
    constexpr int DU = 4;
    for (int d0 = warp * DU; d0 < SD; d0 += nw * DU) {
      float s[DU][ROWS];
#pragma unroll
      for (int u = 0; u < DU; ++u)
#pragma unroll
        for (int r = 0; r < ROWS; ++r) s[u][r] = 0.f;
      if (vec) {
#pragma unroll 2
        for (int i = lane * 8; i < W; i += 256) {
          float wv[DU][8];
#pragma unroll
          for (int u = 0; u < DU; ++u) {
            if (d0 + u < SD) load8<WT>(Wg + static_cast<size_t>(d0 + u) * W + i, wv[u]);
            else
#pragma unroll
              for (int e = 0; e < 8; ++e) wv[u][e] = 0.f;
          }
#pragma unroll
          for (int r = 0; r < ROWS; ++r) {
            const float4 a = *reinterpret_cast<const float4*>(row + r * W + i), b = *reinterpret_cast<const float4*>(row + r * W + i + 4);
#pragma unroll
            for (int u = 0; u < DU; ++u) {
              float acc = s[u][r];
              acc = fmaf(wv[u][0], a.x, acc); acc = fmaf(wv[u][1], a.y, acc); acc = fmaf(wv[u][2], a.z, acc); acc = fmaf(wv[u][3], a.w, acc);
              acc = fmaf(wv[u][4], b.x, acc); acc = fmaf(wv[u][5], b.y, acc); acc = fmaf(wv[u][6], b.z, acc); acc = fmaf(wv[u][7], b.w, acc);
              s[u][r] = acc;
            }
          }
        }
      } else {
        for (int i = lane; i < W; i += 32)
#pragma unroll
          for (int u = 0; u < DU; ++u) {
            const float wv = d0 + u < SD ? to_f(Wg[static_cast<size_t>(d0 + u) * W + i]) : 0.f;
#pragma unroll
            for (int r = 0; r < ROWS; ++r) s[u][r] = fmaf(wv, row[r * W + i], s[u][r]);
          }
      }
#pragma unroll
      for (int u = 0; u < DU; ++u)
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
          const float tot = warp_sum(s[u][r]);
          if (lane == 0 && r < nr && d0 + u < SD) {
            const int id = min(max(p.ids[t0 + r], 0), p.vocab - 1);
            const WT* e = static_cast<const WT*>(p.side_embed) + static_cast<size_t>(id) * p.ld_e + p.e_off;
            g[r * SD + d0 + u] = act_apply(tot, 4) * to_f(e[d0 + u]);
          }
        }
    }
    for (int i = threadIdx.x; i < (ROWS - nr) * SD; i += blockDim.x) g[nr * SD + i] = 0.f;
    __syncthreads();
    float q[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) q[r] = 0.f;
#pragma unroll 2
    for (int i = threadIdx.x; i < W; i += blockDim.x) {
      const WT* wr = Wp + static_cast<size_t>(i) * SD;
      float s[ROWS];
#pragma unroll
      for (int r = 0; r < ROWS; ++r) s[r] = 0.f;
      if (vec) {
        // 32 weights (four 16-byte loads in flight) at a time
        for (int d = 0; d < SD; d += 32) {
          float wv[4][8];
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            if (d + 8 * c < SD) load8<WT>(wr + d + 8 * c, wv[c]);
            else
#pragma unroll
              for (int e = 0; e < 8; ++e) wv[c][e] = 0.f;
          }
#pragma unroll
          for (int c = 0; c < 4; ++c)
            if (d + 8 * c < SD)
#pragma unroll
              for (int r = 0; r < ROWS; ++r)
#pragma unroll
                for (int e = 0; e < 8; ++e) s[r] = fmaf(wv[c][e], g[r * SD + d + 8 * c + e], s[r]);
        }
      } else {
        for (int d = 0; d < SD; ++d) {
          const float wv = to_f(wr[d]);
#pragma unroll
          for (int r = 0; r < ROWS; ++r) s[r] = fmaf(wv, g[r * SD + d], s[r]);
        }
      }
#pragma unroll
      for (int r = 0; r < ROWS; ++r) {
        yb[r * W + i] = s[r];
        q[r] = fmaf(s[r], s[r], q[r]);
      }
    }
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
      const float rs = 1.f / sqrtf(block_sum(q[r], red, phase) / W + p.eps);
      if (w4) {
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
          const float4 y = *reinterpret_cast<const float4*>(yb + r * W + i), n = *reinterpret_cast<const float4*>(p.side_norm + i);
          float4 v = *reinterpret_cast<float4*>(row + r * W + i);
          v.x = fmaf(p.mult, y.x * rs * n.x, v.x); v.y = fmaf(p.mult, y.y * rs * n.y, v.y);
          v.z = fmaf(p.mult, y.z * rs * n.z, v.z); v.w = fmaf(p.mult, y.w * rs * n.w, v.w);
          *reinterpret_cast<float4*>(row + r * W + i) = v;
        }
      } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x)
          row[r * W + i] = fmaf(p.mult, yb[r * W + i] * rs * p.side_norm[i], row[r * W + i]);
      }
    }
    __syncthreads();
  }
  OT* o1 = static_cast<OT*>(p.out1);
  OT* o2 = static_cast<OT*>(p.out2);
#pragma unroll
  for (int r = 0; r < ROWS; ++r) {
    float q = 0.f;
    if (r < nr) {
      if (w4) {
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
          const float4 v = *reinterpret_cast<const float4*>(row + r * W + i);
          *reinterpret_cast<float4*>(p.x + (t0 + r) * W + i) = v;
          q = fmaf(v.x, v.x, q); q = fmaf(v.y, v.y, q); q = fmaf(v.z, v.z, q); q = fmaf(v.w, v.w, q);
        }
      } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
          const float v = row[r * W + i];
          p.x[(t0 + r) * W + i] = v;
          q = fmaf(v, v, q);
        }
      }
    }
    if (p.out1 == nullptr) continue;
    const float rs = 1.f / sqrtf(block_sum(q, red, phase) / W + p.eps);
    if (r < nr) {
      if (w4) {
        for (int i = threadIdx.x * 4; i < W; i += blockDim.x * 4) {
          float4 v = *reinterpret_cast<const float4*>(row + r * W + i);
          v.x *= rs; v.y *= rs; v.z *= rs; v.w *= rs;
          const float4 a = *reinterpret_cast<const float4*>(p.w1 + i);
          store4<OT>(o1 + (t0 + r) * W + i, v.x * a.x, v.y * a.y, v.z * a.z, v.w * a.w);
          if (o2) {
            const float4 b = *reinterpret_cast<const float4*>(p.w2 + i);
            store4<OT>(o2 + (t0 + r) * W + i, v.x * b.x, v.y * b.y, v.z * b.z, v.w * b.w);
          }
        }
      } else {
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
          const float v = row[r * W + i] * rs;
          o1[(t0 + r) * W + i] = from_f<OT>(v * p.w1[i]);
          if (o2) o2[(t0 + r) * W + i] = from_f<OT>(v * p.w2[i]);
        }
      }
    }
  }
}

// logits <- cap * tanh(logits / cap)
__global__ void softcap_kernel(float* __restrict__ x, long long n, float cap) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) x[i] = cap * tanhf(x[i] / cap);
}

// LayerNorm of a row: (x - mean) / sqrt(mean((x - mean)^2) + eps) * w + b, statistics in two passes over the row
template <typename OT>
__global__ void layernorm_kernel(OT* __restrict__ out, const float* __restrict__ x, const float* __restrict__ w,
                                 const float* __restrict__ b, int W, float eps, const int32_t* __restrict__ rows) {
  extern __shared__ float sm[];
  float* row = sm;
  float* red = sm + W;
  int phase = 0;
  pdl_sync();
  const int t = blockIdx.x;
  const size_t src = rows ? static_cast<size_t>(rows[t]) : static_cast<size_t>(t);
  for (int i = threadIdx.x; i < W; i += blockDim.x) row[i] = x[src * W + i];
  __syncthreads();
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += row[i];
  const float mean = block_sum(s, red, phase) / W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = row[i] - mean;
    q += d * d;
  }
  const float rstd = 1.f / sqrtf(block_sum(q, red, phase) / W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out[static_cast<size_t>(t) * W + i] = from_f<OT>((row[i] - mean) * rstd * w[i] + b[i]);
}

// x[t] += LN(y[t]; w1, b1);  optionally out2[t] = LN(x[t]; w2, b2) (the pre-norm of the sublayer that follows)
template <typename OT>
__global__ void postnorm_residual_kernel(float* __restrict__ x, const float* __restrict__ y, const float* __restrict__ w1,
                                         const float* __restrict__ b1, OT* __restrict__ out2,
                                         const float* __restrict__ w2, const float* __restrict__ b2, int W, float eps,
                                         int planes, long long plane_stride) {
  extern __shared__ float sm[];
  float* row = sm;
  float* red = sm + W;
  int phase = 0;
  pdl_sync();
  const size_t t = blockIdx.x;
  // y may arrive as the fp32 planes of a split-K projection: they are summed here, in plane order
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float v = y[t * W + i];
    for (int s = 1; s < planes; ++s) v += y[s * plane_stride + t * W + i];
    row[i] = v;
  }
  __syncthreads();
  float s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += row[i];
  float mean = block_sum(s, red, phase) / W;
  float q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = row[i] - mean;
    q += d * d;
  }
  float rstd = 1.f / sqrtf(block_sum(q, red, phase) / W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float v = x[t * W + i] + ((row[i] - mean) * rstd * w1[i] + b1[i]);
    x[t * W + i] = v;
    row[i] = v;
  }
  if (out2 == nullptr) return;
  __syncthreads();
  s = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) s += row[i];
  mean = block_sum(s, red, phase) / W;
  q = 0.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    const float d = row[i] - mean;
    q += d * d;
  }
  rstd = 1.f / sqrtf(block_sum(q, red, phase) / W + eps);
  for (int i = threadIdx.x; i < W; i += blockDim.x)
    out2[t * W + i] = from_f<OT>((row[i] - mean) * rstd * w2[i] + b2[i]);
}

// ------------------------------------------------------------------------------------------------------------------
// Y[r][n] = alpha * sum_k X[src(r)][k] * W[g][n][k]
//   dense:   g = 0, r in [0, T), src(r) = r
//   grouped: blockIdx.z = g, r in [row_off[g], row_off[g + 1]), src(r) = gather ? gather[r] : r
//   batched: blockIdx.z = g, every group has the rows [0, T): X, Y advance by x_group_stride, o_group_stride elements per
//            group (heads of one row side by side), gate: Y[r][n] *= sigmoid(gate[r * ld_gate + g])
// epilogue 0: store (OT);  1: W holds N "gate" rows followed by N "up" rows, store silu(gate) * up (OT);
//          2: relu(y)^2;  3: gelu(y), exact;  4: gelu(y), tanh form
// Tile 64 x 64, BK 16, 256 threads, 4 x 4 outputs per thread.
// ------------------------------------------------------------------------------------------------------------------
constexpr int LB_M = 64, LB_N = 64, LB_K = 16;

struct LinearParams {
  void* out;
  const void* x;
  const void* w;
  const int32_t* row_off;
  const int32_t* gather;
  int T, N, K, ldx, ldo, epi;
  long long w_group_stride;     // elements between the weight matrices of consecutive groups
  float alpha;
  long long x_group_stride, o_group_stride;     // batched form (both 0 otherwise)
  const float* gate;
  int ld_gate;
  int gate_values;              // batched form: 0 = one gate per (row, group); N = one per output value (column g * N + n)
  // epilogue 1 with glu_limit > 0: the clamped form g' = min(gate, limit), u' = clamp(up, -limit, limit),
  // out = g' * sigmoid(glu_slope * g') * (u' + 1)
  float glu_limit, glu_slope;
};

template <typename XT, typename WT, typename OT, int EPI>
__global__ void __launch_bounds__(256) linear_kernel(LinearParams p) {
  constexpr int NB = EPI == 1 ? 2 : 1;
  __shared__ float As[LB_K][LB_M + 4];
  __shared__ float Bs[NB][LB_K][LB_N + 4];
  pdl_sync();
  int r_lo = 0, r_hi = p.T;
  if (p.row_off) {
    r_lo = p.row_off[blockIdx.z];
    r_hi = p.row_off[blockIdx.z + 1];
  }
  const int m0 = r_lo + blockIdx.x * LB_M, n0 = blockIdx.y * LB_N;
  if (m0 >= r_hi) return;
  const XT* X = static_cast<const XT*>(p.x) + static_cast<size_t>(blockIdx.z) * p.x_group_stride;
  const WT* Wm = static_cast<const WT*>(p.w) + static_cast<size_t>(blockIdx.z) * p.w_group_stride;
  const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
  // loader: row lr of the tile, 4 consecutive k starting at lk
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  const int ar = m0 + lr;
  const XT* arow = nullptr;
  if (ar < r_hi) arow = X + static_cast<size_t>(p.gather ? p.gather[ar] : ar) * p.ldx;
  const int bn = n0 + lr;
  const WT* brow[NB];
#pragma unroll
  for (int h = 0; h < NB; ++h) brow[h] = bn < p.N ? Wm + (static_cast<size_t>(h) * p.N + bn) * p.K : nullptr;
  float acc[NB][4][4];
#pragma unroll
  for (int h = 0; h < NB; ++h)
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) acc[h][i][j] = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += LB_K) {
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int k = k0 + lk + u;
      As[lk + u][lr] = (arow && k < p.K) ? to_f(arow[k]) : 0.f;
#pragma unroll
      for (int h = 0; h < NB; ++h) Bs[h][lk + u][lr] = (brow[h] && k < p.K) ? to_f(brow[h][k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int k = 0; k < LB_K; ++k) {
      const float4 a4 = *reinterpret_cast<const float4*>(&As[k][ty * 4]);
      const float a[4] = {a4.x, a4.y, a4.z, a4.w};
#pragma unroll
      for (int h = 0; h < NB; ++h) {
        const float4 b4 = *reinterpret_cast<const float4*>(&Bs[h][k][tx * 4]);
        const float b[4] = {b4.x, b4.y, b4.z, b4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i)
#pragma unroll
          for (int j = 0; j < 4; ++j) acc[h][i][j] = fmaf(a[i], b[j], acc[h][i][j]);
      }
    }
    __syncthreads();
  }
  OT* out = static_cast<OT*>(p.out) + static_cast<size_t>(blockIdx.z) * p.o_group_stride;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int r = m0 + ty * 4 + i;
    if (r >= r_hi) continue;
    float gmul = 1.f;
    if (p.gate && !p.gate_values) gmul = 1.f / (1.f + expf(-p.gate[static_cast<size_t>(r) * p.ld_gate + blockIdx.z]));
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= p.N) continue;
      if (p.gate && p.gate_values)
        gmul = 1.f / (1.f + expf(-p.gate[static_cast<size_t>(r) * p.ld_gate + static_cast<size_t>(blockIdx.z) * p.gate_values + n]));
      float v;
      if (EPI == 1) {
        float g = acc[0][i][j], u = acc[NB - 1][i][j];
        if (p.glu_limit > 0.f) {
          g = fminf(g, p.glu_limit);
          u = fminf(fmaxf(u, -p.glu_limit), p.glu_limit);
          v = g / (1.f + expf(-p.glu_slope * g)) * (u + 1.f);
        } else {
          v = g / (1.f + expf(-g)) * u;
        }
      } else {
        v = act_apply(acc[0][i][j] * p.alpha, p.epi) * gmul;
      }
      out[static_cast<size_t>(r) * p.ldo + n] = from_f<OT>(v);
    }
  }
}

// The batched form on the tensor cores (bf16 in and out, K a multiple of 16, N a multiple of 8): CTA = 64 rows x 64
// columns of one group, 4 warps x 16 rows, mma.sync m16n8k16 with fp32 accumulators over K chunks of 32 staged in shared
// memory with 16-byte loads.  Every output is one accumulator fed in k order: a row's result does not depend on the rows
// that share the launch.
constexpr int BM_M = 64, BM_N = 64, BM_K = 32, BM_LD = BM_K + 8;

__global__ void __launch_bounds__(128) linear_batched_mma_kernel(LinearParams p) {
  __shared__ __align__(16) __nv_bfloat16 As[BM_M * BM_LD];
  __shared__ __align__(16) __nv_bfloat16 Bs[BM_N * BM_LD];
  pdl_sync();
  const int z = blockIdx.z, m0 = blockIdx.x * BM_M, n0 = blockIdx.y * BM_N;
  const __nv_bfloat16* X = static_cast<const __nv_bfloat16*>(p.x) + static_cast<size_t>(z) * p.x_group_stride;
  const __nv_bfloat16* Wm = static_cast<const __nv_bfloat16*>(p.w) + static_cast<size_t>(z) * p.w_group_stride;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  float acc[BM_N / 8][4];
#pragma unroll
  for (int n = 0; n < BM_N / 8; ++n) acc[n][0] = acc[n][1] = acc[n][2] = acc[n][3] = 0.f;
  for (int k0 = 0; k0 < p.K; k0 += BM_K) {
    // 64 rows x 4 pieces of 8 elements for each operand; pieces past K (K % 32 == 16) and rows past the edge are zero
#pragma unroll
    for (int i = tid; i < BM_M * 4; i += 128) {
      const int r = i >> 2, c = (i & 3) * 8;
      uint4 a = make_uint4(0u, 0u, 0u, 0u), b = a;
      if (k0 + c < p.K) {
        if (m0 + r < p.T) a = *reinterpret_cast<const uint4*>(X + static_cast<size_t>(m0 + r) * p.ldx + k0 + c);
        if (n0 + r < p.N) b = *reinterpret_cast<const uint4*>(Wm + static_cast<size_t>(n0 + r) * p.K + k0 + c);
      }
      *reinterpret_cast<uint4*>(As + r * BM_LD + c) = a;
      *reinterpret_cast<uint4*>(Bs + r * BM_LD + c) = b;
    }
    __syncthreads();
#pragma unroll
    for (int kb = 0; kb < BM_K / 16; ++kb) {
      uint32_t af[4];
      ldmatrix_x4(af, smem_u32(As + (warp * 16 + (lane & 15)) * BM_LD + kb * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int np = 0; np < BM_N / 16; ++np) {
        uint32_t bf[4];
        ldmatrix_x4(bf, smem_u32(Bs + (np * 16 + (lane >> 4) * 8 + (lane & 7)) * BM_LD + kb * 16 + ((lane >> 3) & 1) * 8));
        mma_bf16_16816(acc[2 * np], af, bf[0], bf[1]);
        mma_bf16_16816(acc[2 * np + 1], af, bf[2], bf[3]);
      }
    }
    __syncthreads();
  }
  __nv_bfloat16* out = static_cast<__nv_bfloat16*>(p.out) + static_cast<size_t>(z) * p.o_group_stride;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    const int r = m0 + warp * 16 + (lane >> 2) + 8 * half;
    if (r >= p.T) continue;
    float gmul = p.alpha;
    if (p.gate && !p.gate_values) gmul *= 1.f / (1.f + expf(-p.gate[static_cast<size_t>(r) * p.ld_gate + z]));
#pragma unroll
    for (int n = 0; n < BM_N / 8; ++n) {
      const int c = n0 + n * 8 + (lane & 3) * 2;
      if (c >= p.N) continue;
      float g0 = gmul, g1 = gmul;
      if (p.gate && p.gate_values) {
        const float* gv = p.gate + static_cast<size_t>(r) * p.ld_gate + static_cast<size_t>(z) * p.gate_values + c;
        g0 *= 1.f / (1.f + expf(-gv[0]));
        g1 *= 1.f / (1.f + expf(-gv[1]));
      }
      *reinterpret_cast<uint32_t*>(out + static_cast<size_t>(r) * p.ldo + c) =
          pack_bf16(acc[n][2 * half] * g0, acc[n][2 * half + 1] * g1);
    }
  }
}

template <typename XT, typename WT, typename OT>
static int launch_linear(const LinearParams& p, int groups, int max_rows, cudaStream_t stream) {
  dim3 grid((max_rows + LB_M - 1) / LB_M, (p.N + LB_N - 1) / LB_N, groups);
  if (p.epi == 1) VB_LAUNCH_PDL((linear_kernel<XT, WT, OT, 1>), grid, 256, 0, stream, p);
  else VB_LAUNCH_PDL((linear_kernel<XT, WT, OT, 0>), grid, 256, 0, stream, p);
  return 0;
}

__global__ void cast_f32_bf16_kernel(__nv_bfloat16* __restrict__ out, const float* __restrict__ in, long long n) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i < n) out[i] = __float2bfloat16_rn(in[i]);
}

// out[i] = sum over planes of partials[plane][i] in plane order (the reduction of a split-K projection)
__global__ void sum_planes_kernel(float* __restrict__ out, const float* __restrict__ partials, int planes, long long n) {
  pdl_sync();
  const long long i = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  if (i + 3 < n) {
    float4 a = *reinterpret_cast<const float4*>(partials + i);
    for (int s = 1; s < planes; ++s) {
      const float4 b = *reinterpret_cast<const float4*>(partials + s * n + i);
      a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
    }
    *reinterpret_cast<float4*>(out + i) = a;
  } else {
    for (long long j = i; j < n; ++j) {
      float a = partials[j];
      for (int s = 1; s < planes; ++s) a += partials[s * n + j];
      out[j] = a;
    }
  }
}

}  // namespace vb

using namespace vb;
using bf16 = __nv_bfloat16;

extern "C" {

int vb_embed_rows_f32(float* d_out, const void* d_table, const int32_t* d_ids, int T, int width, int vocab, int dtype,
                      const void* d_pos_table, const int32_t* d_pos, int n_pos, float scale, float* d_out2, void* stream) {
  VB_CHECK_ARG(d_out && d_table && d_ids && width > 0 && vocab > 0, "vb_embed_rows_f32: bad arguments");
  VB_CHECK_ARG(!d_pos_table || (d_pos && n_pos > 0), "vb_embed_rows_f32: a position table needs positions");
  if (T <= 0) return 0;
  if (dtype == 1) VB_LAUNCH_PDL(embed_rows_kernel<float>, T, 128, 0, stream, d_out, static_cast<const float*>(d_table), d_ids, width, vocab, static_cast<const float*>(d_pos_table), d_pos, n_pos, scale, d_out2);
  else VB_LAUNCH_PDL(embed_rows_kernel<bf16>, T, 128, 0, stream, d_out, static_cast<const bf16*>(d_table), d_ids, width, vocab, static_cast<const bf16*>(d_pos_table), d_pos, n_pos, scale, d_out2);
  return 0;
}

int vb_gated_residual_norm_f32(float* d_x, const float* d_y, const float* d_r, int ld_r, const float* d_bias,
                               const float* d_add, void* d_out, const float* d_w, int T, int width, float eps, int out_dtype,
                               void* stream) {
  VB_CHECK_ARG(d_x && d_y && width > 0 && (!d_out || d_w) && (!d_r || ld_r >= width), "vb_gated_residual_norm_f32: bad arguments");
  if (T <= 0) return 0;
  const size_t smem = (static_cast<size_t>(width) + 64) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_gated_residual_norm_f32: width %d too large", width);
  auto al16 = [](const void* q) { return q == nullptr || reinterpret_cast<uintptr_t>(q) % 16 == 0; };
  const int vec = width % 4 == 0 && (!d_r || ld_r % 4 == 0) && al16(d_x) && al16(d_y) && al16(d_r) && al16(d_bias) && al16(d_add) &&
                  al16(d_w) && (!d_out || reinterpret_cast<uintptr_t>(d_out) % 8 == 0);
  if (out_dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(gated_residual_norm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(gated_residual_norm_kernel<float>, T, 256, smem, stream, d_x, d_y, d_r, ld_r, d_bias, d_add, static_cast<float*>(d_out), d_w, width, eps, vec);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(gated_residual_norm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(gated_residual_norm_kernel<bf16>, T, 256, smem, stream, d_x, d_y, d_r, ld_r, d_bias, d_add, static_cast<bf16*>(d_out), d_w, width, eps, vec);
  }
  return 0;
}

int vb_rmsnorm2_f32(void* d_out1, void* d_out2, const float* d_x, const float* d_w1, const float* d_w2,
                    const int32_t* d_rows, int T, int width, float eps, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out1 && d_x && d_w1 && width > 0 && (!d_out2 || d_w2), "vb_rmsnorm2_f32: bad arguments");
  if (T <= 0) return 0;
  const size_t smem = (static_cast<size_t>(width) + 64) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_rmsnorm2_f32: width %d too large", width);
  if (out_dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(rmsnorm2_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(rmsnorm2_kernel<float>, T, 256, smem, stream, static_cast<float*>(d_out1), static_cast<float*>(d_out2), d_x, d_w1, d_w2, width, eps, d_rows);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(rmsnorm2_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(rmsnorm2_kernel<bf16>, T, 256, smem, stream, static_cast<bf16*>(d_out1), static_cast<bf16*>(d_out2), d_x, d_w1, d_w2, width, eps, d_rows);
  }
  return 0;
}

}  // extern "C"

template <typename WT, typename OT, int ROWS>
static int launch_residual_side_rows(const ResidualSideParams& p, int T, int threads, cudaStream_t stream) {
  const size_t smem = ROWS * (2 * static_cast<size_t>(p.W) + p.side_dim) * sizeof(float) + 64 * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_residual_side_f32: width %d too large", p.W);
  if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(residual_side_kernel<WT, OT, ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
  VB_LAUNCH_PDL((residual_side_kernel<WT, OT, ROWS>), (T + ROWS - 1) / ROWS, threads, smem, stream, p);
  return 0;
}

template <typename WT, typename OT>
static int launch_residual_side(const ResidualSideParams& p, int T, cudaStream_t stream) {
  // long steps: four rows per CTA share one pass over the side matrices (measured at 1024 rows of width 2048: 38 us against
  // 49 us with two rows and 44 us with one; more warps per CTA were slower).  Short steps: one row per CTA of 16 warps, so
  // that more of the row's weight streams are in flight.
  const size_t four = 4 * (2 * static_cast<size_t>(p.W) + p.side_dim) * sizeof(float) + 256;
  if (p.side_gate && T >= 256 && four <= static_cast<size_t>(VB_MAX_DYN_SMEM)) return launch_residual_side_rows<WT, OT, 4>(p, T, 256, stream);
  return launch_residual_side_rows<WT, OT, 1>(p, T, 512, stream);
}

extern "C" {

int vb_residual_side_f32(float* d_x, const float* d_y1, const float* d_y2, float mult, const void* d_side_gate,
                         const void* d_side_proj, const float* d_side_norm, const void* d_side_embed, const int32_t* d_ids,
                         int side_dim, int ld_e, int e_off, int vocab, int w_dtype, void* d_out1, const float* d_w1,
                         void* d_out2, const float* d_w2, int T, int width, float eps, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_x && d_y1 && width > 0, "vb_residual_side_f32: bad arguments");
  VB_CHECK_ARG(!d_side_gate || (d_side_proj && d_side_norm && d_side_embed && d_ids && side_dim > 0 && vocab > 0 &&
                                e_off >= 0 && e_off + side_dim <= ld_e),
               "vb_residual_side_f32: the side input needs its matrices, norm weight, table and token ids");
  VB_CHECK_ARG((!d_out1 || d_w1) && (!d_out2 || (d_out1 && d_w2)), "vb_residual_side_f32: norms need weights");
  if (T <= 0) return 0;
  const int sd = d_side_gate ? side_dim : 0;
  ResidualSideParams p{d_x, d_y1, d_y2, d_side_gate, d_side_proj, d_side_norm, d_side_embed, d_ids, d_out1, d_out2, d_w1, d_w2,
                       width, sd, ld_e, e_off, vocab, T, mult, eps};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (w_dtype == 1) return out_dtype == 1 ? launch_residual_side<float, float>(p, T, s) : launch_residual_side<float, bf16>(p, T, s);
  return out_dtype == 1 ? launch_residual_side<bf16, float>(p, T, s) : launch_residual_side<bf16, bf16>(p, T, s);
}

int vb_rms_postnorm_residual_f32(float* d_x, const float* d_y, const float* d_w, void* d_out, int T, int width, float eps,
                                 int out_dtype, void* stream) {
  VB_CHECK_ARG(d_x && d_y && d_w && width > 0, "vb_rms_postnorm_residual_f32: bad arguments");
  if (T <= 0) return 0;
  const size_t smem = (static_cast<size_t>(width) + 64) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_rms_postnorm_residual_f32: width %d too large", width);
  if (out_dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(rms_postnorm_residual_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(rms_postnorm_residual_kernel<float>, T, 256, smem, stream, d_x, d_y, d_w, static_cast<float*>(d_out), width, eps);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(rms_postnorm_residual_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(rms_postnorm_residual_kernel<bf16>, T, 256, smem, stream, d_x, d_y, d_w, static_cast<bf16*>(d_out), width, eps);
  }
  return 0;
}

int vb_softcap_f32(float* d_x, long long n, float cap, void* stream) {
  VB_CHECK_ARG(d_x && cap > 0.f, "vb_softcap_f32: bad arguments");
  if (n <= 0) return 0;
  VB_LAUNCH_PDL(softcap_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, stream, d_x, n, cap);
  return 0;
}

int vb_linear_batched(void* d_out, const void* d_x, const void* d_w, int T, int N, int K, int ldx, int ldo,
                      long long x_group_stride, long long o_group_stride, long long w_group_stride, int groups, int in_dtype,
                      int out_dtype, int epilogue, float alpha, const float* d_gate, int ld_gate, void* stream) {
  return vb_linear_batched_gated(d_out, d_x, d_w, T, N, K, ldx, ldo, x_group_stride, o_group_stride, w_group_stride, groups,
                                 in_dtype, out_dtype, epilogue, alpha, d_gate, ld_gate, 0, stream);
}

int vb_linear_batched_gated(void* d_out, const void* d_x, const void* d_w, int T, int N, int K, int ldx, int ldo,
                            long long x_group_stride, long long o_group_stride, long long w_group_stride, int groups,
                            int in_dtype, int out_dtype, int epilogue, float alpha, const float* d_gate, int ld_gate,
                            int gate_per_value, void* stream) {
  VB_CHECK_ARG(d_out && d_x && d_w && N > 0 && K > 0 && groups >= 1, "vb_linear_batched: bad arguments");
  VB_CHECK_ARG(epilogue == 0 || (epilogue >= 2 && epilogue <= 4), "vb_linear_batched: epilogue %d", epilogue);
  VB_CHECK_ARG(!d_gate || ld_gate >= groups * (gate_per_value ? N : 1), "vb_linear_batched: gate rows hold one value per group (or per output value)");
  if (T <= 0) return 0;
  LinearParams p{d_out, d_x, d_w, nullptr, nullptr, T, N, K, ldx, ldo, epilogue, w_group_stride, alpha, x_group_stride,
                 o_group_stride, d_gate, ld_gate, (d_gate && gate_per_value) ? N : 0};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  const bool aligned = ldx % 8 == 0 && x_group_stride % 8 == 0 && w_group_stride % 8 == 0 && ldo % 2 == 0 && o_group_stride % 2 == 0 &&
                       reinterpret_cast<uintptr_t>(d_x) % 16 == 0 && reinterpret_cast<uintptr_t>(d_w) % 16 == 0 &&
                       reinterpret_cast<uintptr_t>(d_out) % 4 == 0;
  if (in_dtype == 0 && out_dtype == 0 && epilogue == 0 && K % 16 == 0 && N % 8 == 0 && aligned) {
    dim3 grid((T + BM_M - 1) / BM_M, (N + BM_N - 1) / BM_N, groups);
    VB_LAUNCH_PDL(linear_batched_mma_kernel, grid, 128, 0, stream, p);
    return 0;
  }
  if (in_dtype == 1) return out_dtype == 1 ? launch_linear<float, float, float>(p, groups, T, s) : launch_linear<float, float, bf16>(p, groups, T, s);
  return out_dtype == 1 ? launch_linear<bf16, bf16, float>(p, groups, T, s) : launch_linear<bf16, bf16, bf16>(p, groups, T, s);
}

int vb_layernorm_f32(void* d_out, const float* d_x, const float* d_w, const float* d_b, const int32_t* d_rows, int T,
                     int width, float eps, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_x && d_w && d_b && width > 0, "vb_layernorm_f32: bad arguments");
  if (T <= 0) return 0;
  const size_t smem = (static_cast<size_t>(width) + 64) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_layernorm_f32: width %d too large", width);
  if (out_dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(layernorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(layernorm_kernel<float>, T, 256, smem, stream, static_cast<float*>(d_out), d_x, d_w, d_b, width, eps, d_rows);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(layernorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(layernorm_kernel<bf16>, T, 256, smem, stream, static_cast<bf16*>(d_out), d_x, d_w, d_b, width, eps, d_rows);
  }
  return 0;
}

int vb_postnorm_residual_f32(float* d_x, const float* d_y, int y_planes, const float* d_w1, const float* d_b1, void* d_out2,
                             const float* d_w2, const float* d_b2, int T, int width, float eps, int out_dtype,
                             void* stream) {
  VB_CHECK_ARG(y_planes >= 1, "vb_postnorm_residual_f32: planes");
  const long long plane_stride = static_cast<long long>(T) * width;
  VB_CHECK_ARG(d_x && d_y && d_w1 && d_b1 && width > 0, "vb_postnorm_residual_f32: bad arguments");
  VB_CHECK_ARG(!d_out2 || (d_w2 && d_b2), "vb_postnorm_residual_f32: the second norm needs weight and bias");
  if (T <= 0) return 0;
  const size_t smem = (static_cast<size_t>(width) + 64) * sizeof(float);
  VB_CHECK_ARG(smem <= static_cast<size_t>(VB_MAX_DYN_SMEM), "vb_postnorm_residual_f32: width %d too large", width);
  if (out_dtype == 1) {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(postnorm_residual_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(postnorm_residual_kernel<float>, T, 256, smem, stream, d_x, d_y, d_w1, d_b1, static_cast<float*>(d_out2), d_w2, d_b2, width, eps, y_planes, plane_stride);
  } else {
    if (smem > 48 * 1024) VB_CHECK_CUDA(cudaFuncSetAttribute(postnorm_residual_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, VB_MAX_DYN_SMEM));
    VB_LAUNCH_PDL(postnorm_residual_kernel<bf16>, T, 256, smem, stream, d_x, d_y, d_w1, d_b1, static_cast<bf16*>(d_out2), d_w2, d_b2, width, eps, y_planes, plane_stride);
  }
  return 0;
}

int vb_linear(void* d_out, const void* d_x, const void* d_w, int T, int N, int K, int ldx, int ldo, int in_dtype,
              int out_dtype, int epilogue, float alpha, const int32_t* d_row_off, const int32_t* d_gather, int groups,
              long long w_group_stride, float glu_limit, float glu_slope, void* stream) {
  VB_CHECK_ARG(d_out && d_x && d_w && N > 0 && K > 0 && ldx >= K && ldo >= N, "vb_linear: bad arguments");
  VB_CHECK_ARG(epilogue >= 0 && epilogue <= 4, "vb_linear: epilogue %d", epilogue);
  VB_CHECK_ARG(groups >= 1 && (groups == 1 || d_row_off), "vb_linear: grouped launches need row offsets");
  if (T <= 0) return 0;
  LinearParams p{d_out, d_x, d_w, d_row_off, d_gather, T, N, K, ldx, ldo, epilogue, w_group_stride, alpha, 0, 0, nullptr, 0, 0,
                 glu_limit, glu_slope};
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  // in_dtype: 0 = bf16 activations and weights, 1 = fp32 both; out_dtype likewise
  if (in_dtype == 1) return out_dtype == 1 ? launch_linear<float, float, float>(p, groups, T, s) : launch_linear<float, float, bf16>(p, groups, T, s);
  return out_dtype == 1 ? launch_linear<bf16, bf16, float>(p, groups, T, s) : launch_linear<bf16, bf16, bf16>(p, groups, T, s);
}

int vb_sum_planes_f32(float* d_out, const float* d_partials, int planes, long long n, void* stream) {
  VB_CHECK_ARG(d_out && d_partials && planes >= 1 && n % 4 == 0, "vb_sum_planes_f32: bad arguments (n a multiple of 4)");
  if (n <= 0) return 0;
  VB_LAUNCH_PDL(sum_planes_kernel, static_cast<unsigned>((n / 4 + 255) / 256), 256, 0, stream, d_out, d_partials, planes, n);
  return 0;
}

int vb_cast_f32_bf16(void* d_out, const float* d_in, long long n, void* stream) {
  VB_CHECK_ARG(d_out && d_in, "vb_cast_f32_bf16: null pointer");
  if (n <= 0) return 0;
  VB_LAUNCH_PDL(cast_f32_bf16_kernel, static_cast<unsigned>((n + 255) / 256), 256, 0, stream, static_cast<bf16*>(d_out), d_in, n);
  return 0;
}

}  // extern "C"
