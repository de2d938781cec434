// Mixture-of-experts routing for the hybrid decoder stacks (the expert matrices themselves run through the grouped mode
// of vb_linear):
//   vb_moe_route    router logits z = W_r h + b in fp32 (h bf16 or fp32), the `top` largest per token (ties: the lower
//                   expert index), weights = softmax over the chosen logits only
//   vb_moe_route_sigmoid  scores s = sigmoid(W_r h) in fp32; experts are CHOSEN by s + correction (a per-expert constant),
//                   optionally only among the experts of the `keep` best of n_groups equal groups of neighbours (a group
//                   ranks by the sum of its two largest corrected scores; experts outside count as -inf), and WEIGHTED
//                   by their uncorrected s divided by the chosen experts' sum (+ 1e-20).  Also the shared expert's
//                   per-token gate sigmoid(w_sg . h) when asked
//   vb_moe_group    counting sort (shared-memory counters, one CTA) of the (token, choice) pairs by expert: row_off[E + 1], the token of every sorted row and
//                   the sorted row of every (token, choice)
//   vb_moe_scale_dense  the dense form for tensor-core projections: every expert runs on every token as ONE stacked
//                   gate/up projection [E * ff (+ shared ff)] and ONE stacked down projection over that whole axis; in
//                   between, the activation columns of expert e are multiplied by the token's routing weight for e, or
//                   set to zero when e was not chosen (the shared expert's columns pass).  Weight-bound steps (decode)
//                   read every expert's matrices once either way; compute-bound steps pay experts / top times the FLOPs
//                   of the grouped form, on tensor cores instead of fp32 FMAs.
//   vb_moe_combine  y[t] = sum_c weight[t][c] * expert_out[sorted row of (t, c)] (+ shared[t]), summed in choice order so
//                   that a token's result does not depend on what else is in the batch
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 4
#include "common.cuh"

namespace vb {

template <typename XT>
__global__ void __launch_bounds__(256) moe_route_kernel(int32_t* __restrict__ idx, float* __restrict__ wts,
                                                        const XT* __restrict__ h, const float* __restrict__ wr,
                                                        const float* __restrict__ br, int W, int E, int top) {
  extern __shared__ float z[];      // [E] logits, then the row as fp32 [W]
  float* xs = z + E;
  pdl_sync();
  const size_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const XT* x = h + t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    if constexpr (sizeof(XT) == 4) xs[i] = x[i];
    else xs[i] = __bfloat162float(x[i]);
  }
  __syncthreads();
  for (int e = warp; e < E; e += nw) {
    const float* w = wr + static_cast<size_t>(e) * W;
    float s = 0.f;
    if ((W & 3) == 0) {
      for (int i = lane * 4; i < W; i += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(w + i);
        s = fmaf(xs[i], wv.x, s); s = fmaf(xs[i + 1], wv.y, s); s = fmaf(xs[i + 2], wv.z, s); s = fmaf(xs[i + 3], wv.w, s);
      }
    } else {
      for (int i = lane; i < W; i += 32) s = fmaf(xs[i], w[i], s);
    }
    s = warp_sum(s);
    if (lane == 0) z[e] = s + (br ? br[e] : 0.f);
  }
  __syncthreads();
  if (warp != 0) return;
  // `top` rounds of arg-max over the experts (lane-strided, then across the warp)
  float chosen_max = 0.f, denom = 0.f, my_val = 0.f;
  for (int c = 0; c < top; ++c) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32) {
      const float v = z[e];
      if (v > best || (v == best && e < bi)) { best = v; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ov = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
    }
    if (c == 0) chosen_max = best;
    const float ex = expf(best - chosen_max);
    denom += ex;
    if (lane == c % 32) my_val = ex;           // (top <= 32)
    if (lane == 0) {
      idx[t * top + c] = bi;
      z[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane < top) wts[t * top + lane] = my_val / denom;
}

// warp-wide arg-max over v[0 .. n) (ties: the lower index); every lane gets the result
__device__ __forceinline__ void warp_argmax(const float* v, int n, int lane, float& best, int& bi) {
  best = -INFINITY;
  bi = 0x7fffffff;
  for (int e = lane; e < n; e += 32) {
    const float x = v[e];
    if (x > best || (x == best && e < bi)) { best = x; bi = e; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) { best = ov; bi = oi; }
  }
}

template <typename XT>
__global__ void __launch_bounds__(256) moe_route_sigmoid_kernel(int32_t* __restrict__ idx, float* __restrict__ wts,
                                                                float* __restrict__ shared_gate, const XT* __restrict__ h,
                                                                const float* __restrict__ wr, const float* __restrict__ corr,
                                                                const float* __restrict__ wsg, int W, int E, int top,
                                                                int n_groups, int keep, int softmax_scores, int rank_by_max,
                                                                int normalize) {
  extern __shared__ float sm[];
  float* sc = sm;               // [E] sigmoid scores
  float* ch = sm + E;           // [E] choice scores (score + correction; -inf once taken or outside the kept groups)
  float* gs = ch + E;           // [n_groups] group scores
  float* xs = gs + n_groups;    // [W] the row as fp32
  pdl_sync();
  const size_t t = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
  const XT* x = h + t * W;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    if constexpr (sizeof(XT) == 4) xs[i] = x[i];
    else xs[i] = __bfloat162float(x[i]);
  }
  __syncthreads();
  const int rows = E + (wsg ? 1 : 0);
  for (int e = warp; e < rows; e += nw) {
    const float* w = e < E ? wr + static_cast<size_t>(e) * W : wsg;
    float s = 0.f;
    if ((W & 3) == 0) {
      for (int i = lane * 4; i < W; i += 128) {
        const float4 wv = *reinterpret_cast<const float4*>(w + i);
        s = fmaf(xs[i], wv.x, s); s = fmaf(xs[i + 1], wv.y, s); s = fmaf(xs[i + 2], wv.z, s); s = fmaf(xs[i + 3], wv.w, s);
      }
    } else {
      for (int i = lane; i < W; i += 32) s = fmaf(xs[i], w[i], s);
    }
    s = warp_sum(s);
    if (lane == 0) {
      const float sg = 1.f / (1.f + expf(-s));
      if (e < E) {
        sc[e] = softmax_scores ? s : sg;
        ch[e] = sg + (corr ? corr[e] : 0.f);
      } else {
        shared_gate[t] = sg;
      }
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (softmax_scores) {
    // scores = softmax of the logits over ALL experts (fp32); they also rank the experts
    float mx = -INFINITY;
    for (int e = lane; e < E; e += 32) mx = fmaxf(mx, sc[e]);
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(sc[e] - mx);
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) {
      const float v = expf(sc[e] - mx) / sum;
      sc[e] = v;
      ch[e] = v + (corr ? corr[e] : 0.f);
    }
    __syncwarp();
  }
  if (n_groups > 1 && keep < n_groups) {
    const int size = E / n_groups;
    for (int g = lane; g < n_groups; g += 32) {
      float a = -INFINITY, b = -INFINITY;           // the two largest choice scores of the group
      for (int e = g * size; e < (g + 1) * size; ++e) {
        const float v = ch[e];
        if (v > a) { b = a; a = v; }
        else if (v > b) b = v;
      }
      gs[g] = (size > 1 && !rank_by_max) ? a + b : a;
    }
    __syncwarp();
    // `keep` rounds of arg-max mark the kept groups with -inf; the experts of all other groups leave the choice
    for (int c = 0; c < keep; ++c) {
      float best;
      int bi;
      warp_argmax(gs, n_groups, lane, best, bi);
      if (lane == 0) gs[bi] = -INFINITY;
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / size] != -INFINITY) ch[e] = -INFINITY;
    __syncwarp();
  }
  float denom = 0.f, my_val = 0.f;
  for (int c = 0; c < top; ++c) {
    float best;
    int bi;
    warp_argmax(ch, E, lane, best, bi);
    const float s = sc[bi];
    denom += s;
    if (lane == c % 32) my_val = s;           // (top <= 32)
    __syncwarp();
    if (lane == 0) {
      idx[t * top + c] = bi;
      ch[bi] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane < top) wts[t * top + lane] = normalize ? my_val / (denom + 1e-20f) : my_val;
}

// single CTA: E <= 1024 experts, any number of pairs
__global__ void __launch_bounds__(1024) moe_group_kernel(int32_t* __restrict__ row_off, int32_t* __restrict__ sorted_token,
                                                         int32_t* __restrict__ pair_row, const int32_t* __restrict__ idx,
                                                         int T, int E, int top, int tile_rows,
                                                         int32_t* __restrict__ tile_group, int n_tiles) {
  __shared__ int cnt[1024];
  __shared__ int base[1025];
  pdl_sync();
  const int tid = threadIdx.x, n = T * top;
  for (int e = tid; e < E; e += 1024) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) atomicAdd(&cnt[idx[i]], 1);
  __syncthreads();
  if (tid == 0) {
    int s = 0;
    for (int e = 0; e < E; ++e) {
      base[e] = s;
      s += tile_rows > 0 ? (cnt[e] + tile_rows - 1) / tile_rows * tile_rows : cnt[e];
    }
    base[E] = s;
  }
  __syncthreads();
  for (int e = tid; e <= E; e += 1024) row_off[e] = base[e];
  if (tile_rows > 0) {
    // padded layout: rows that hold no pair read as token -1; every row tile belongs to one expert
    for (int r = tid; r < n_tiles * tile_rows; r += 1024) sorted_token[r] = -1;
    for (int i = tid; i < n_tiles; i += 1024) {
      int g = 0;
      for (int e = 0; e < E; ++e)
        if (i * tile_rows >= base[e] && i * tile_rows < base[e + 1]) g = e;
      tile_group[i] = g;
    }
    __syncthreads();
  }
  // placement: a pair takes the next free row of its expert.  The order of an expert's rows varies from run to run; every
  // row is computed on its own and found again through pair_row, so results do not depend on it.
  __syncthreads();
  for (int e = tid; e < E; e += 1024) cnt[e] = 0;
  __syncthreads();
  for (int i = tid; i < n; i += 1024) {
    const int e = idx[i];
    const int r = base[e] + atomicAdd(&cnt[e], 1);
    sorted_token[r] = i / top;
    pair_row[i] = r;
  }
}

__global__ void moe_combine_kernel(float* __restrict__ y, const float* __restrict__ expert_out,
                                   const float* __restrict__ shared_out, const float* __restrict__ wts,
                                   const int32_t* __restrict__ pair_row, int W, int top,
                                   const float* __restrict__ shared_scale) {
  pdl_sync();
  const size_t t = blockIdx.x;
  const float ss = shared_scale ? shared_scale[t] : 1.f;
  for (int i = threadIdx.x; i < W; i += blockDim.x) {
    float a = 0.f;
    for (int c = 0; c < top; ++c)
      a = fmaf(wts[t * top + c], expert_out[static_cast<size_t>(pair_row[t * top + c]) * W + i], a);
    if (shared_out) a = fmaf(ss, shared_out[t * W + i], a);
    y[t * W + i] = a;
  }
}

__global__ void moe_scale_dense_kernel(__nv_bfloat16* __restrict__ act, const int32_t* __restrict__ idx,
                                       const float* __restrict__ wts, int ld, int E, int ff, int top,
                                       const float* __restrict__ shared_gate, int shared_ff) {
  extern __shared__ float we[];     // [E] routing weight of every expert for this token (0: not chosen)
  pdl_sync();
  const size_t t = blockIdx.x;
  if (shared_gate) {                // the shared expert's columns (after the experts') times the token's gate
    const float gsh = shared_gate[t];
    __nv_bfloat16* sh = act + t * ld + static_cast<size_t>(E) * ff;
    if ((shared_ff & 7) == 0 && (ld & 7) == 0 && ((E * ff) & 7) == 0) {
      uint4* sh4 = reinterpret_cast<uint4*>(sh);
      for (int v = threadIdx.x; v < shared_ff / 8; v += blockDim.x) {
        uint4 x = sh4[v];
        x.x = pack_bf16(gsh * bf16_lo(x.x), gsh * bf16_hi(x.x));
        x.y = pack_bf16(gsh * bf16_lo(x.y), gsh * bf16_hi(x.y));
        x.z = pack_bf16(gsh * bf16_lo(x.z), gsh * bf16_hi(x.z));
        x.w = pack_bf16(gsh * bf16_lo(x.w), gsh * bf16_hi(x.w));
        sh4[v] = x;
      }
    } else {
      for (int c = threadIdx.x; c < shared_ff; c += blockDim.x) sh[c] = __float2bfloat16_rn(gsh * __bfloat162float(sh[c]));
    }
  }
  for (int e = threadIdx.x; e < E; e += blockDim.x) we[e] = 0.f;
  __syncthreads();
  if (threadIdx.x < top) we[idx[t * top + threadIdx.x]] = wts[t * top + threadIdx.x];
  __syncthreads();
  __nv_bfloat16* row = act + t * ld;
  const int n = E * ff;
  if ((ff & 7) == 0 && (ld & 7) == 0) {            // eight columns (16 bytes) of one expert at a time
    uint4* row4 = reinterpret_cast<uint4*>(row);
    for (int v = threadIdx.x; v < n / 8; v += blockDim.x) {
      const float w = we[v * 8 / ff];
      uint4 x = make_uint4(0u, 0u, 0u, 0u);
      if (w != 0.f) {
        x = row4[v];
        x.x = pack_bf16(w * bf16_lo(x.x), w * bf16_hi(x.x));
        x.y = pack_bf16(w * bf16_lo(x.y), w * bf16_hi(x.y));
        x.z = pack_bf16(w * bf16_lo(x.z), w * bf16_hi(x.z));
        x.w = pack_bf16(w * bf16_lo(x.w), w * bf16_hi(x.w));
      }
      row4[v] = x;
    }
    return;
  }
  for (int c = threadIdx.x; c < n; c += blockDim.x) {
    const float w = we[c / ff];
    row[c] = w == 0.f ? __float2bfloat16_rn(0.f) : __float2bfloat16_rn(w * __bfloat162float(row[c]));
  }
}

__global__ void moe_gather_rows_kernel(uint4* __restrict__ out, const uint4* __restrict__ x, const int32_t* __restrict__ token,
                                       int vecs) {
  pdl_sync();
  const size_t r = blockIdx.x;
  const int t = token[r];
  for (int i = threadIdx.x; i < vecs; i += blockDim.x)
    out[r * vecs + i] = t >= 0 ? x[static_cast<size_t>(t) * vecs + i] : make_uint4(0u, 0u, 0u, 0u);
}

}  // namespace vb

using namespace vb;

extern "C" {

int vb_moe_route(int32_t* d_idx, float* d_wts, const void* d_h, const float* d_router_w, const float* d_router_b, int T,
                 int width, int experts, int top, int h_dtype, void* stream) {
  VB_CHECK_ARG(d_idx && d_wts && d_h && d_router_w, "vb_moe_route: null pointer");
  VB_CHECK_ARG(experts >= 1 && experts <= 1024 && top >= 1 && top <= 32 && top <= experts,
               "vb_moe_route: experts %d (<= 1024), top %d (<= 32, <= experts)", experts, top);
  if (T <= 0) return 0;
  const size_t smem = (static_cast<size_t>(experts) + width) * sizeof(float);
  VB_CHECK_ARG(smem <= 48 * 1024, "vb_moe_route: width %d too large", width);
  if (h_dtype == 1) VB_LAUNCH_PDL(moe_route_kernel<float>, T, 256, smem, stream, d_idx, d_wts, static_cast<const float*>(d_h), d_router_w, d_router_b, width, experts, top);
  else VB_LAUNCH_PDL(moe_route_kernel<__nv_bfloat16>, T, 256, smem, stream, d_idx, d_wts, static_cast<const __nv_bfloat16*>(d_h), d_router_w, d_router_b, width, experts, top);
  return 0;
}

int vb_moe_route_sigmoid(int32_t* d_idx, float* d_wts, float* d_shared_gate, const void* d_h, const float* d_router_w,
                         const float* d_correction, const float* d_shared_gate_w, int T, int width, int experts, int top,
                         int n_groups, int keep, int h_dtype, void* stream) {
  return vb_moe_route_groups(d_idx, d_wts, d_shared_gate, d_h, d_router_w, d_correction, d_shared_gate_w, T, width, experts, top,
                             n_groups, keep, 0, 0, 1, h_dtype, stream);
}

int vb_moe_route_groups(int32_t* d_idx, float* d_wts, float* d_shared_gate, const void* d_h, const float* d_router_w,
                        const float* d_correction, const float* d_shared_gate_w, int T, int width, int experts, int top,
                        int n_groups, int keep, int softmax_scores, int rank_by_max, int normalize, int h_dtype, void* stream) {
  VB_CHECK_ARG(d_idx && d_wts && d_h && d_router_w, "vb_moe_route_sigmoid: null pointer");
  VB_CHECK_ARG(experts >= 1 && experts <= 1024 && top >= 1 && top <= 32 && top <= experts,
               "vb_moe_route_sigmoid: experts %d (<= 1024), top %d (<= 32, <= experts)", experts, top);
  VB_CHECK_ARG(n_groups <= 1 || (experts % n_groups == 0 && keep >= 1 && keep <= n_groups &&
                                 keep * (experts / n_groups) >= top),
               "vb_moe_route_sigmoid: %d groups (keep %d) do not fit %d experts, top %d", n_groups, keep, experts, top);
  VB_CHECK_ARG(!d_shared_gate_w || d_shared_gate, "vb_moe_route_sigmoid: the shared gate needs an output");
  if (T <= 0) return 0;
  const int ng = n_groups > 1 ? n_groups : 1;
  const size_t smem = (2 * static_cast<size_t>(experts) + ng + width) * sizeof(float);
  VB_CHECK_ARG(smem <= 48 * 1024, "vb_moe_route_sigmoid: width %d too large", width);
  if (h_dtype == 1) VB_LAUNCH_PDL(moe_route_sigmoid_kernel<float>, T, 256, smem, stream, d_idx, d_wts, d_shared_gate, static_cast<const float*>(d_h), d_router_w, d_correction, d_shared_gate_w, width, experts, top, ng, keep, softmax_scores, rank_by_max, normalize);
  else VB_LAUNCH_PDL(moe_route_sigmoid_kernel<__nv_bfloat16>, T, 256, smem, stream, d_idx, d_wts, d_shared_gate, static_cast<const __nv_bfloat16*>(d_h), d_router_w, d_correction, d_shared_gate_w, width, experts, top, ng, keep, softmax_scores, rank_by_max, normalize);
  return 0;
}

int vb_moe_group(int32_t* d_row_off, int32_t* d_sorted_token, int32_t* d_pair_row, const int32_t* d_idx, int T,
                 int experts, int top, int tile_rows, int32_t* d_tile_group, int n_tiles, void* stream) {
  VB_CHECK_ARG(d_row_off && d_sorted_token && d_pair_row && d_idx, "vb_moe_group: null pointer");
  VB_CHECK_ARG(experts >= 1 && experts <= 1024, "vb_moe_group: experts %d (<= 1024)", experts);
  VB_CHECK_ARG(tile_rows == 0 || (d_tile_group && n_tiles >= (T * top + tile_rows - 1) / tile_rows + experts),
               "vb_moe_group: the padded layout needs tile groups for ceil(pairs / tile_rows) + experts tiles");
  if (T <= 0) return 0;
  VB_LAUNCH_PDL(moe_group_kernel, 1, 1024, 0, stream, d_row_off, d_sorted_token, d_pair_row, d_idx, T, experts, top,
                tile_rows, d_tile_group, n_tiles);
  return 0;
}

int vb_moe_gather_rows(void* d_out, const void* d_x, const int32_t* d_token, int rows, int width, void* stream) {
  VB_CHECK_ARG(d_out && d_x && d_token && width % 8 == 0, "vb_moe_gather_rows: bad arguments (bf16 rows, width %% 8 == 0)");
  if (rows <= 0) return 0;
  VB_LAUNCH_PDL(moe_gather_rows_kernel, rows, 128, 0, stream, static_cast<uint4*>(d_out), static_cast<const uint4*>(d_x),
                d_token, width / 8);
  return 0;
}

int vb_moe_scale_dense(void* d_act, const int32_t* d_idx, const float* d_wts, int T, int ld, int experts, int ff, int top,
                       const float* d_shared_gate, int shared_ff, void* stream) {
  VB_CHECK_ARG(!d_shared_gate || (shared_ff > 0 && ld >= experts * ff + shared_ff), "vb_moe_scale_dense: shared columns");
  VB_CHECK_ARG(d_act && d_idx && d_wts, "vb_moe_scale_dense: null pointer");
  VB_CHECK_ARG(experts >= 1 && experts <= 1024 && top >= 1 && top <= 32 && ld >= experts * ff, "vb_moe_scale_dense: bad sizes");
  if (T <= 0) return 0;
  VB_LAUNCH_PDL(moe_scale_dense_kernel, T, 256, static_cast<size_t>(experts) * sizeof(float), stream,
                static_cast<__nv_bfloat16*>(d_act), d_idx, d_wts, ld, experts, ff, top, d_shared_gate,
                shared_ff);
  return 0;
}

int vb_moe_combine(float* d_y, const float* d_expert_out, const float* d_shared_out, const float* d_wts,
                   const int32_t* d_pair_row, int T, int width, int top, const float* d_shared_scale, void* stream) {
  VB_CHECK_ARG(d_y && d_expert_out && d_wts && d_pair_row, "vb_moe_combine: null pointer");
  if (T <= 0) return 0;
  VB_LAUNCH_PDL(moe_combine_kernel, T, 256, 0, stream, d_y, d_expert_out, d_shared_out, d_wts, d_pair_row, width, top,
                d_shared_scale);
  return 0;
}

}  // extern "C"
