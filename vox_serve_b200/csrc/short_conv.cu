// Short causal convolutions over time with a per-request state slot, and the row index of a hashed token-pair embedding.
//
//   y_t[c] = bias[c] + sum_j w[c][j] * u_(t - taps + 1 + j)[c]        (the last column weighs the current token; inputs before a
//                                                                       request's position 0 are zero)
//   out_t  = act(y_t) (+ u_t: the residual form h + conv(h))
//
// u is a column range of fp32 rows (the residual stream, or the rows of a fused projection), so several convolutions over
// neighbouring columns of one projection run as ONE call with their weights stacked.  A request's last taps - 1 inputs live
// in an fp32 slot [taps - 1][C]; rows whose taps reach before the step's first row read them from there.  A request that
// brings one row has its slot shifted by that row's own thread; the slots of the others are rewritten by a second kernel after
// the outputs (every thread owns one (request, channel) and reads all it needs before it writes).  A slot's content is ignored
// wherever a tap reaches before position 0, so slots are reused without clearing.
// Every output is one fp32 FMA chain over the taps in the same order, whatever the step's cut.
//
//   vb_pair_hash_rows   row[t] = (prev * mul_prev + id * mul_cur) mod buckets, `buckets` itself for a request's first token;
//                       the previous token of a step's first row comes from the request's slot, which then takes the step's
//                       last token
//   vb_short_conv       the convolution and the state update
//   vb_cast_rows        a column range of fp32 rows -> dense rows of the compute type (the operand of a following projection)
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 4
#include "common.cuh"

namespace vb {

constexpr int SC_MAX_TAPS = 16;

struct ShortConvParams {
  const float* in;        // [T][ld_in]
  int ld_in;
  const float* w;         // [C][taps]
  const float* bias;      // [C] or nullptr
  float* state;           // [slots][taps - 1][C]
  void* out;              // [T][ld_out] compute type, or nullptr
  int ld_out;
  float* out_f32;         // [T][ld_f32] or nullptr
  int ld_f32;
  const int32_t* qo_indptr;
  const int32_t* row_req;
  const int32_t* pos;
  const int32_t* slots;
  int T, B, C, taps, act, residual;
  int single_inline;      // requests that bring one row had their slot shifted by the convolution kernel itself
};

template <typename CT> __device__ __forceinline__ void sc_store(void* out, size_t i, float v);
template <> __device__ __forceinline__ void sc_store<float>(void* out, size_t i, float v) { static_cast<float*>(out)[i] = v; }
template <> __device__ __forceinline__ void sc_store<__nv_bfloat16>(void* out, size_t i, float v) {
  static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
}

template <typename CT>
__global__ void __launch_bounds__(256) short_conv_kernel(ShortConvParams p) {
  pdl_sync();
  const int c = blockIdx.x * 256 + threadIdx.x, t = blockIdx.y;
  if (c >= p.C) return;
  const int b = p.row_req[t], r = t - p.qo_indptr[b], ps = p.pos[t], K = p.taps - 1;
  const float* st = p.state + (static_cast<size_t>(p.slots[b]) * K) * p.C + c;
  const float* w = p.w + static_cast<size_t>(c) * p.taps;
  float acc = p.bias ? p.bias[c] : 0.f;
  for (int j = 0; j < p.taps; ++j) {
    const int back = K - j;
    if (ps - back < 0) continue;
    const float u = r - back >= 0 ? p.in[static_cast<size_t>(t - back) * p.ld_in + c] : st[static_cast<size_t>(r + j) * p.C];
    acc = fmaf(w[j], u, acc);
  }
  if (p.act == 1) acc = acc / (1.f + expf(-acc));
  const float cur = p.in[static_cast<size_t>(t) * p.ld_in + c];
  if (p.residual) acc += cur;
  if (p.out) sc_store<CT>(p.out, static_cast<size_t>(t) * p.ld_out + c, acc);
  if (p.out_f32) p.out_f32[static_cast<size_t>(t) * p.ld_f32 + c] = acc;
  // a request that brings exactly one row: this thread is the slot's only reader for the channel, so it also shifts the slot
  // (zeros for positions before 0) -- the second kernel leaves such requests alone, and steps made of them skip it
  if (K > 0 && p.qo_indptr[b + 1] - p.qo_indptr[b] == 1) {
    float* sw = p.state + (static_cast<size_t>(p.slots[b]) * K) * p.C + c;
    float keep[SC_MAX_TAPS];
#pragma unroll
    for (int i = 0; i < SC_MAX_TAPS; ++i) {
      if (i >= K) break;
      keep[i] = i + 1 < K ? ((ps - K + i + 1 >= 0) ? sw[static_cast<size_t>(i + 1) * p.C] : 0.f) : cur;
    }
#pragma unroll
    for (int i = 0; i < SC_MAX_TAPS; ++i) {
      if (i >= K) break;
      sw[static_cast<size_t>(i) * p.C] = keep[i];
    }
  }
}

// Long steps, 2 to 4 taps: a thread computes SC_RPT consecutive rows of its channel from one read of the rows' inputs (the
// taps of neighbouring rows overlap), with the same FMA chain per output as the kernel above.
constexpr int SC_RPT = 8;

template <typename CT, int TAPS>
__global__ void __launch_bounds__(256) short_conv_rows_kernel(ShortConvParams p) {
  pdl_sync();
  const int c = blockIdx.x * 256 + threadIdx.x, t0 = blockIdx.y * SC_RPT;
  if (c >= p.C) return;
  constexpr int K = TAPS - 1;
  float u[SC_RPT + K], w[TAPS];
#pragma unroll
  for (int i = 0; i < SC_RPT + K; ++i) {
    const int t = t0 - K + i;
    u[i] = (t >= 0 && t < p.T) ? p.in[static_cast<size_t>(t) * p.ld_in + c] : 0.f;
  }
#pragma unroll
  for (int j = 0; j < TAPS; ++j) w[j] = p.w[static_cast<size_t>(c) * TAPS + j];
  const float bias = p.bias ? p.bias[c] : 0.f;
#pragma unroll
  for (int rr = 0; rr < SC_RPT; ++rr) {
    const int t = t0 + rr;
    if (t < p.T) {
      const int b = p.row_req[t], r = t - p.qo_indptr[b], ps = p.pos[t];
      const float* st = p.state + (static_cast<size_t>(p.slots[b]) * K) * p.C + c;
      float acc = bias;
#pragma unroll
      for (int j = 0; j < TAPS; ++j) {
        const int back = K - j;
        if (ps - back >= 0) acc = fmaf(w[j], r - back >= 0 ? u[rr + j] : st[static_cast<size_t>(r + j) * p.C], acc);
      }
      if (p.act == 1) acc = acc / (1.f + expf(-acc));
      if (p.residual) acc += u[rr + K];
      if (p.out) sc_store<CT>(p.out, static_cast<size_t>(t) * p.ld_out + c, acc);
      if (p.out_f32) p.out_f32[static_cast<size_t>(t) * p.ld_f32 + c] = acc;
    }
  }
}

// the slot after the step: the last taps - 1 inputs of [old slot | the step's rows], zeros for positions before 0
__global__ void __launch_bounds__(256) short_conv_state_kernel(ShortConvParams p) {
  pdl_sync();
  const int c = blockIdx.x * 256 + threadIdx.x, b = blockIdx.y;
  if (c >= p.C) return;
  const int r0 = p.qo_indptr[b], n = p.qo_indptr[b + 1] - r0, K = p.taps - 1;
  if (n <= 0 || K <= 0) return;
  if (n == 1 && p.single_inline) return;        // (shifted by the row's own thread)
  const int p0 = p.pos[r0];
  float* st = p.state + (static_cast<size_t>(p.slots[b]) * K) * p.C + c;
  float keep[SC_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < SC_MAX_TAPS; ++i) {
    if (i >= K) break;
    const int src = n + i;                      // index into [old slot (K) | rows (n)]
    float v = 0.f;
    if (p0 - K + src >= 0) v = src < K ? st[static_cast<size_t>(src) * p.C] : p.in[static_cast<size_t>(r0 + src - K) * p.ld_in + c];
    keep[i] = v;
  }
#pragma unroll
  for (int i = 0; i < SC_MAX_TAPS; ++i) {
    if (i >= K) break;
    st[static_cast<size_t>(i) * p.C] = keep[i];
  }
}

__global__ void __launch_bounds__(128) pair_hash_rows_kernel(int32_t* __restrict__ rows, int32_t* __restrict__ prev_tok,
                                                             const int32_t* __restrict__ ids, const int32_t* __restrict__ qo,
                                                             const int32_t* __restrict__ row_req, const int32_t* __restrict__ pos,
                                                             const int32_t* __restrict__ slots, int T, int buckets,
                                                             long long mul_prev, long long mul_cur) {
  pdl_sync();
  const int t = blockIdx.x * 128 + threadIdx.x;
  if (t >= T) return;
  const int b = row_req[t];
  long long prev;
  if (t == qo[b]) {
    // the step's first row of the request: this thread alone reads the slot and then hands it the step's last token
    prev = pos[t] == 0 ? -1 : prev_tok[slots[b]];
    prev_tok[slots[b]] = ids[qo[b + 1] - 1];
  } else {
    prev = ids[t - 1];
  }
  if (prev < 0) {
    rows[t] = buckets;
  } else {
    long long m = (prev * mul_prev + static_cast<long long>(ids[t]) * mul_cur) % buckets;
    if (m < 0) m += buckets;
    rows[t] = static_cast<int32_t>(m);
  }
}

template <typename CT>
__global__ void cast_rows_kernel(CT* __restrict__ out, const float* __restrict__ in, int ld_in, int n, long long total) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const long long t = i / n;
  const int c = static_cast<int>(i - t * n);
  sc_store<CT>(out, static_cast<size_t>(i), in[t * ld_in + c]);
}

}  // namespace vb

using namespace vb;
using bf16 = __nv_bfloat16;

extern "C" {

int vb_pair_hash_rows(int32_t* d_rows, int32_t* d_prev_tok, const int32_t* d_ids, const int32_t* d_qo_indptr,
                      const int32_t* d_row_req, const int32_t* d_pos, const int32_t* d_slots, int T, int buckets,
                      long long mul_prev, long long mul_cur, void* stream) {
  VB_CHECK_ARG(d_rows && d_prev_tok && d_ids && d_qo_indptr && d_row_req && d_pos && d_slots && buckets > 0,
               "vb_pair_hash_rows: bad arguments");
  if (T <= 0) return 0;
  VB_LAUNCH_PDL(pair_hash_rows_kernel, (T + 127) / 128, 128, 0, stream, d_rows, d_prev_tok, d_ids, d_qo_indptr, d_row_req, d_pos,
                d_slots, T, buckets, mul_prev, mul_cur);
  return 0;
}

int vb_short_conv(void* d_out, int ld_out, float* d_out_f32, int ld_f32, const float* d_in, int ld_in, const float* d_w,
                  const float* d_bias, float* d_state, const int32_t* d_qo_indptr, const int32_t* d_row_req, const int32_t* d_pos,
                  const int32_t* d_slots, int T, int B, int channels, int taps, int act, int residual, int out_dtype,
                  void* stream) {
  VB_CHECK_ARG(d_in && d_w && d_state && d_qo_indptr && d_row_req && d_pos && d_slots && (d_out || d_out_f32),
               "vb_short_conv: null pointer");
  VB_CHECK_ARG(channels > 0 && taps >= 1 && taps <= SC_MAX_TAPS && (act == 0 || act == 1) && ld_in >= channels,
               "vb_short_conv: channels %d, taps %d (1..%d), act %d", channels, taps, SC_MAX_TAPS, act);
  if (T <= 0 || B <= 0) return 0;
  const bool rows_form = T >= 64 && taps >= 2 && taps <= 4;
  ShortConvParams p{d_in, ld_in, d_w, d_bias, d_state, d_out, ld_out, d_out_f32, ld_f32, d_qo_indptr, d_row_req, d_pos, d_slots,
                    T, B, channels, taps, act, residual, rows_form ? 0 : 1};
  const int cx = (channels + 255) / 256;
  const dim3 rows_grid(cx, (T + SC_RPT - 1) / SC_RPT);
  const bool f32 = out_dtype == 1;
  if (T >= 64 && taps == 2) {
    if (f32) VB_LAUNCH_PDL((short_conv_rows_kernel<float, 2>), rows_grid, 256, 0, stream, p);
    else VB_LAUNCH_PDL((short_conv_rows_kernel<bf16, 2>), rows_grid, 256, 0, stream, p);
  } else if (T >= 64 && taps == 3) {
    if (f32) VB_LAUNCH_PDL((short_conv_rows_kernel<float, 3>), rows_grid, 256, 0, stream, p);
    else VB_LAUNCH_PDL((short_conv_rows_kernel<bf16, 3>), rows_grid, 256, 0, stream, p);
  } else if (T >= 64 && taps == 4) {
    if (f32) VB_LAUNCH_PDL((short_conv_rows_kernel<float, 4>), rows_grid, 256, 0, stream, p);
    else VB_LAUNCH_PDL((short_conv_rows_kernel<bf16, 4>), rows_grid, 256, 0, stream, p);
  } else if (f32) {
    VB_LAUNCH_PDL(short_conv_kernel<float>, dim3(cx, T), 256, 0, stream, p);
  } else {
    VB_LAUNCH_PDL(short_conv_kernel<bf16>, dim3(cx, T), 256, 0, stream, p);
  }
  // (T == B: every request brings one row, and the convolution kernel has shifted every slot)
  if (taps > 1 && !(p.single_inline && T == B)) VB_LAUNCH_PDL(short_conv_state_kernel, dim3(cx, B), 256, 0, stream, p);
  return 0;
}

int vb_cast_rows(void* d_out, const float* d_in, int ld_in, int T, int n, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_in && n > 0 && ld_in >= n, "vb_cast_rows: bad arguments");
  if (T <= 0) return 0;
  const long long total = static_cast<long long>(T) * n;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  if (out_dtype == 1) VB_LAUNCH_PDL(cast_rows_kernel<float>, blocks, 256, 0, stream, static_cast<float*>(d_out), d_in, ld_in, n, total);
  else VB_LAUNCH_PDL(cast_rows_kernel<bf16>, blocks, 256, 0, stream, static_cast<bf16*>(d_out), d_in, ld_in, n, total);
  return 0;
}

}  // extern "C"
