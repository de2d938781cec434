// Selective state-space recurrence (Mamba form) over a per-request fp32 state slot [inner][N]:
//
//   dt_t[c]   = softplus(pdt_t[c] + dt_bias[c])
//   S_t[c][n] = exp(dt_t[c] * A[c][n]) * S_(t-1)[c][n] + dt_t[c] * x_t[c] * B_t[n]          S = 0 before position 0
//   y_t[c]    = sum_n S_t[c][n] * C_t[n] + D[c] * x_t[c]
//   out_t[c]  = out_scale * y_t[c] * silu(z_t[c])
//
// x (after its short convolution and activation), pdt (the step-size projection before its bias), B | C (columns of the
// low-rank projection) and z (the gate's pre-activation) are fp32 rows; A = -exp(A_log) is formed once at load time.
// Everything is fp32; only `out` takes the compute type (it feeds the output projection).  A slot's stored state is ignored
// when the request's first row of the step has position 0, so slots are handed out again without clearing.
//
// Up to 16 states per channel: a thread owns a channel and all its states; a CTA of 128 channels walks rows in blocks of 16 whose
// B | C it stages in shared memory once and whose dt / x / z every thread loads up front (all in flight before the dependent
// chain starts).  More states: eight lanes share a channel, each holding every eighth state in registers, with the next row's
// operands already loaded while the current row's chain runs.
//
//   vb_selective_scan        every request of the step, rows in order (single tokens and portions)
//   vb_selective_scan_tiled  prompt portions cut into pieces of rows: the recurrence composes as S_end = P * S_start + L with
//                            P[c][n] = exp(A[c][n] * sum dt[c]) and L the piece's end state from zero, so pieces are
//                            summarised in parallel, a short scan over a request's pieces carries the state in, and the
//                            pieces then produce their rows in parallel (twice the arithmetic, rows / piece times the
//                            parallelism)
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 1
#include "common.cuh"

namespace vb {

struct ScanParams {
  const float* x;  int ld_x;
  const float* dt; int ld_dt;
  const float* dt_bias;
  const float* bc; int ld_bc, b_off, c_off;
  const float* z;  int ld_z;
  const float* A;         // [inner][N]
  const float* Dv;        // [inner]
  float* state;           // [slots][inner][N]
  void* out;  int ld_out;
  const int32_t* qo_indptr;
  const int32_t* pos;
  const int32_t* slots;
  int B, inner, N;
  float out_scale;
  int single_rows, multi_rows;
  // tiled form
  const int32_t* tile_req;
  const int32_t* tile_row0;
  int n_tiles, tile_rows, piece_rows;
  float* scratch;         // [pieces][inner][N + 1]: a piece's end state from zero and its sum of dt; after the scan: its carry-in
};

constexpr int SS_LANES = 8;          // lanes per channel
constexpr int SS_CH = 16;            // channels per CTA of 128 threads

__device__ __forceinline__ float ss_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }
template <typename CT> __device__ __forceinline__ void ss_store(void* out, size_t i, float v);
template <> __device__ __forceinline__ void ss_store<float>(void* out, size_t i, float v) { static_cast<float*>(out)[i] = v; }
template <> __device__ __forceinline__ void ss_store<__nv_bfloat16>(void* out, size_t i, float v) {
  static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
}

// rows [r0, r1) of one request for one channel: S (NPL states of this lane) advances; with WRITE the rows' outputs are
// stored; sum_dt (optional) accumulates the step sizes
template <typename CT, int NPL, bool WRITE>
__device__ __forceinline__ void ss_walk(const ScanParams& p, int ch, bool valid, int l, int r0, int r1, float (&S)[NPL],
                                        const float (&A)[NPL], float* sum_dt) {
  const float bias = p.dt_bias ? p.dt_bias[ch] : 0.f;
  const float Dc = p.Dv ? p.Dv[ch] : 0.f;
  float dtn = 0.f, xn = 0.f, zn = 0.f, Bn[NPL], Cn[NPL];
  auto load = [&](int t) {
    dtn = p.dt[static_cast<size_t>(t) * p.ld_dt + ch];
    xn = p.x[static_cast<size_t>(t) * p.ld_x + ch];
    if (WRITE) zn = p.z[static_cast<size_t>(t) * p.ld_z + ch];
    const float* row = p.bc + static_cast<size_t>(t) * p.ld_bc;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int n = l + SS_LANES * i;
      Bn[i] = n < p.N ? row[p.b_off + n] : 0.f;
      if (WRITE) Cn[i] = n < p.N ? row[p.c_off + n] : 0.f;
    }
  };
  if (r0 < r1) load(r0);
  float sdt = 0.f;
  for (int t = r0; t < r1; ++t) {
    const float dtv = ss_softplus(dtn + bias), xv = xn, zv = zn;
    float Bv[NPL], Cv[NPL];
#pragma unroll
    for (int i = 0; i < NPL; ++i) { Bv[i] = Bn[i]; if (WRITE) Cv[i] = Cn[i]; }
    if (t + 1 < r1) load(t + 1);
    sdt += dtv;
    const float dx = dtv * xv;
    float y = 0.f;
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      S[i] = fmaf(expf(dtv * A[i]), S[i], dx * Bv[i]);
      if (WRITE) y = fmaf(S[i], Cv[i], y);
    }
    if (WRITE) {
      y += __shfl_xor_sync(0xffffffffu, y, 4);
      y += __shfl_xor_sync(0xffffffffu, y, 2);
      y += __shfl_xor_sync(0xffffffffu, y, 1);
      if (l == 0 && valid) {
        y = fmaf(Dc, xv, y);
        ss_store<CT>(p.out, static_cast<size_t>(t) * p.ld_out + ch, p.out_scale * y * (zv / (1.f + expf(-zv))));
      }
    }
  }
  if (sum_dt) *sum_dt = sdt;
}

template <int NPL>
__device__ __forceinline__ void ss_load_A(const ScanParams& p, int ch, int l, float (&A)[NPL]) {
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int n = l + SS_LANES * i;
    A[i] = n < p.N ? p.A[static_cast<size_t>(ch) * p.N + n] : 0.f;
  }
}

template <typename CT, int NPL>
__global__ void __launch_bounds__(128) selective_scan_kernel(ScanParams p) {
  pdl_sync();
  const int b = blockIdx.y, l = threadIdx.x % SS_LANES;
  int ch = blockIdx.x * SS_CH + threadIdx.x / SS_LANES;
  const bool valid = ch < p.inner;
  if (!valid) ch = p.inner - 1;
  const int r0 = p.qo_indptr[b], r1 = p.qo_indptr[b + 1];
  const int n = r1 - r0;
  if (n <= 0 || (n == 1 && !p.single_rows) || (n > 1 && !p.multi_rows)) return;
  float* st = p.state + (static_cast<size_t>(p.slots[b]) * p.inner + ch) * p.N;
  float S[NPL], A[NPL];
  ss_load_A<NPL>(p, ch, l, A);
  const bool fresh = p.pos[r0] == 0;
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int s = l + SS_LANES * i;
    S[i] = (!fresh && s < p.N) ? st[s] : 0.f;
  }
  ss_walk<CT, NPL, true>(p, ch, valid, l, r0, r1, S, A, nullptr);
  if (valid) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int s = l + SS_LANES * i;
      if (s < p.N) st[s] = S[i];
    }
  }
}

// ---- prompt portions in pieces ------------------------------------------------------------------------------------------
// piece j of tile i is summary slot i * (tile_rows / piece_rows) + j; its rows are tile_row0[i] + j * piece_rows ... (cut at
// the tile's and the request's end)
__device__ __forceinline__ bool ss_piece_rows(const ScanParams& p, int piece, int& b, int& r0, int& r1) {
  const int per = p.tile_rows / p.piece_rows, tile = piece / per, j = piece - tile * per;
  b = p.tile_req[tile];
  const int t0 = p.tile_row0[tile], end = min(p.qo_indptr[b + 1], t0 + p.tile_rows);
  r0 = t0 + j * p.piece_rows;
  r1 = min(r0 + p.piece_rows, end);
  return r0 < r1;
}

template <int NPL>
__global__ void __launch_bounds__(128) scan_piece_sum_kernel(ScanParams p) {
  pdl_sync();
  const int piece = blockIdx.y, l = threadIdx.x % SS_LANES;
  int ch = blockIdx.x * SS_CH + threadIdx.x / SS_LANES;
  const bool valid = ch < p.inner;
  if (!valid) ch = p.inner - 1;
  int b, r0, r1;
  if (!ss_piece_rows(p, piece, b, r0, r1)) return;
  float S[NPL], A[NPL], sdt;
  ss_load_A<NPL>(p, ch, l, A);
#pragma unroll
  for (int i = 0; i < NPL; ++i) S[i] = 0.f;
  ss_walk<float, NPL, false>(p, ch, valid, l, r0, r1, S, A, &sdt);
  if (!valid) return;
  float* sc = p.scratch + (static_cast<size_t>(piece) * p.inner + ch) * (p.N + 1);
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int s = l + SS_LANES * i;
    if (s < p.N) sc[s] = S[i];
  }
  if (l == 0) sc[p.N] = sdt;
}

// one thread per (request, channel, state): walks the request's pieces in order, leaving every piece its carry-in and the
// slot the request's end state.  The pieces of a request are consecutive summary slots (its tiles are consecutive).
__global__ void __launch_bounds__(128) scan_piece_carry_kernel(ScanParams p) {
  pdl_sync();
  const long long i = static_cast<long long>(blockIdx.x) * 128 + threadIdx.x;
  const int b = blockIdx.y;
  if (i >= static_cast<long long>(p.inner) * p.N) return;
  const int ch = static_cast<int>(i / p.N), s = static_cast<int>(i - static_cast<long long>(ch) * p.N);
  const int r0 = p.qo_indptr[b], r1 = p.qo_indptr[b + 1];
  if (r1 - r0 <= 1) return;
  // the request's first tile: tiles are listed request by request in row order
  int first = -1;
  for (int k = 0; k < p.n_tiles; ++k)
    if (p.tile_req[k] == b) { first = k; break; }
  if (first < 0) return;
  const int per = p.tile_rows / p.piece_rows;
  const int n_pieces = (r1 - r0 + p.piece_rows - 1) / p.piece_rows;     // over whole tiles: piece k of the request covers rows r0 + k * piece_rows
  float* st = p.state + (static_cast<size_t>(p.slots[b]) * p.inner + ch) * p.N + s;
  float S = p.pos[r0] == 0 ? 0.f : *st;
  const float A = p.A[static_cast<size_t>(ch) * p.N + s];
  // (a request's pieces are consecutive summary slots: its tiles are consecutive and whole but for the last)
  float* sc0 = p.scratch + ((static_cast<size_t>(first) * per) * p.inner + ch) * (p.N + 1);
  const size_t stride = static_cast<size_t>(p.inner) * (p.N + 1);
  for (int k0 = 0; k0 < n_pieces; k0 += 8) {
    float L[8], sd[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {                    // independent loads first, the dependent chain after
      if (k0 + j < n_pieces) {
        L[j] = sc0[(k0 + j) * stride + s];
        sd[j] = sc0[(k0 + j) * stride + p.N];
      }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (k0 + j < n_pieces) {
        sc0[(k0 + j) * stride + s] = S;
        S = fmaf(expf(A * sd[j]), S, L[j]);
      }
    }
  }
  *st = S;
}

template <typename CT, int NPL>
__global__ void __launch_bounds__(128) scan_piece_out_kernel(ScanParams p) {
  pdl_sync();
  const int piece = blockIdx.y, l = threadIdx.x % SS_LANES;
  int ch = blockIdx.x * SS_CH + threadIdx.x / SS_LANES;
  const bool valid = ch < p.inner;
  if (!valid) ch = p.inner - 1;
  int b, r0, r1;
  if (!ss_piece_rows(p, piece, b, r0, r1)) return;
  float S[NPL], A[NPL];
  ss_load_A<NPL>(p, ch, l, A);
  const float* sc = p.scratch + (static_cast<size_t>(piece) * p.inner + ch) * (p.N + 1);
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int s = l + SS_LANES * i;
    S[i] = s < p.N ? sc[s] : 0.f;
  }
  ss_walk<CT, NPL, true>(p, ch, valid, l, r0, r1, S, A, nullptr);
}

template <int NPL>
static int launch_scan(const ScanParams& p, int out_dtype, bool tiled, cudaStream_t stream) {
  const int cx = (p.inner + SS_CH - 1) / SS_CH;
  if (!tiled) {
    if (out_dtype == 1) VB_LAUNCH_PDL((selective_scan_kernel<float, NPL>), dim3(cx, p.B), 128, 0, stream, p);
    else VB_LAUNCH_PDL((selective_scan_kernel<__nv_bfloat16, NPL>), dim3(cx, p.B), 128, 0, stream, p);
    return 0;
  }
  const int pieces = p.n_tiles * (p.tile_rows / p.piece_rows);
  const long long states = static_cast<long long>(p.inner) * p.N;
  VB_LAUNCH_PDL(scan_piece_sum_kernel<NPL>, dim3(cx, pieces), 128, 0, stream, p);
  VB_LAUNCH_PDL(scan_piece_carry_kernel, dim3(static_cast<unsigned>((states + 127) / 128), p.B), 128, 0, stream, p);
  if (out_dtype == 1) VB_LAUNCH_PDL((scan_piece_out_kernel<float, NPL>), dim3(cx, pieces), 128, 0, stream, p);
  else VB_LAUNCH_PDL((scan_piece_out_kernel<__nv_bfloat16, NPL>), dim3(cx, pieces), 128, 0, stream, p);
  return 0;
}


// ---- a thread per channel (up to 16 states) ---------------------------------------------------------------------------------
constexpr int S1_ROWS = 16;          // rows walked per staged block
constexpr int S1_THREADS = 128;

template <typename CT, int NM, bool WRITE>
__device__ __forceinline__ void ss_walk1(const ScanParams& p, int ch, bool valid, int r0, int r1, float (&S)[NM],
                                         const float (&A)[NM], float* sum_dt, float* bc_sm) {
  const float bias = p.dt_bias ? p.dt_bias[ch] : 0.f;
  const float Dc = p.Dv ? p.Dv[ch] : 0.f;
  float sdt = 0.f;
  for (int rb = r0; rb < r1; rb += S1_ROWS) {
    const int nr = min(S1_ROWS, r1 - rb);
    __syncthreads();                                   // the block before is consumed
    for (int i = threadIdx.x; i < nr * 2 * NM; i += S1_THREADS) {
      const int r = i / (2 * NM), j = i - r * 2 * NM, n = j < NM ? j : j - NM;
      bc_sm[i] = n < p.N ? p.bc[static_cast<size_t>(rb + r) * p.ld_bc + (j < NM ? p.b_off : p.c_off) + n] : 0.f;
    }
    float dtr[S1_ROWS], xr[S1_ROWS], zr[S1_ROWS];
#pragma unroll
    for (int r = 0; r < S1_ROWS; ++r) {
      if (r < nr) {
        dtr[r] = p.dt[static_cast<size_t>(rb + r) * p.ld_dt + ch];
        xr[r] = p.x[static_cast<size_t>(rb + r) * p.ld_x + ch];
        if (WRITE) zr[r] = p.z[static_cast<size_t>(rb + r) * p.ld_z + ch];
      }
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < S1_ROWS; ++r) {
      if (r < nr) {
        const float dtv = ss_softplus(dtr[r] + bias), xv = xr[r];
        sdt += dtv;
        const float dx = dtv * xv;
        const float* row = bc_sm + r * 2 * NM;
        float y = 0.f;
#pragma unroll
        for (int n = 0; n < NM; ++n) {
          S[n] = fmaf(expf(dtv * A[n]), S[n], dx * row[n]);
          if (WRITE) y = fmaf(S[n], row[NM + n], y);
        }
        if (WRITE && valid) {
          const float zv = zr[r];
          y = fmaf(Dc, xv, y);
          ss_store<CT>(p.out, static_cast<size_t>(rb + r) * p.ld_out + ch, p.out_scale * y * (zv / (1.f + expf(-zv))));
        }
      }
    }
  }
  if (sum_dt) *sum_dt = sdt;
}

template <int NM>
__device__ __forceinline__ void ss_load_A1(const ScanParams& p, int ch, float (&A)[NM]) {
#pragma unroll
  for (int n = 0; n < NM; ++n) A[n] = n < p.N ? p.A[static_cast<size_t>(ch) * p.N + n] : 0.f;
}

template <typename CT, int NM>
__global__ void __launch_bounds__(S1_THREADS) selective_scan1_kernel(ScanParams p) {
  __shared__ float bc_sm[S1_ROWS * 2 * NM];
  pdl_sync();
  const int b = blockIdx.y;
  int ch = blockIdx.x * S1_THREADS + threadIdx.x;
  const bool valid = ch < p.inner;
  if (!valid) ch = p.inner - 1;
  const int r0 = p.qo_indptr[b], r1 = p.qo_indptr[b + 1];
  const int n = r1 - r0;
  if (n <= 0 || (n == 1 && !p.single_rows) || (n > 1 && !p.multi_rows)) return;
  float* st = p.state + (static_cast<size_t>(p.slots[b]) * p.inner + ch) * p.N;
  float S[NM], A[NM];
  ss_load_A1<NM>(p, ch, A);
  const bool fresh = p.pos[r0] == 0;
#pragma unroll
  for (int i = 0; i < NM; ++i) S[i] = (!fresh && i < p.N) ? st[i] : 0.f;
  ss_walk1<CT, NM, true>(p, ch, valid, r0, r1, S, A, nullptr, bc_sm);
  if (valid) {
#pragma unroll
    for (int i = 0; i < NM; ++i)
      if (i < p.N) st[i] = S[i];
  }
}

template <int NM>
__global__ void __launch_bounds__(S1_THREADS) scan1_piece_sum_kernel(ScanParams p) {
  __shared__ float bc_sm[S1_ROWS * 2 * NM];
  pdl_sync();
  const int piece = blockIdx.y;
  int ch = blockIdx.x * S1_THREADS + threadIdx.x;
  const bool valid = ch < p.inner;
  if (!valid) ch = p.inner - 1;
  int b, r0, r1;
  if (!ss_piece_rows(p, piece, b, r0, r1)) return;
  float S[NM], A[NM], sdt;
  ss_load_A1<NM>(p, ch, A);
#pragma unroll
  for (int i = 0; i < NM; ++i) S[i] = 0.f;
  ss_walk1<float, NM, false>(p, ch, valid, r0, r1, S, A, &sdt, bc_sm);
  if (!valid) return;
  float* sc = p.scratch + (static_cast<size_t>(piece) * p.inner + ch) * (p.N + 1);
#pragma unroll
  for (int i = 0; i < NM; ++i)
    if (i < p.N) sc[i] = S[i];
  sc[p.N] = sdt;
}

template <typename CT, int NM>
__global__ void __launch_bounds__(S1_THREADS) scan1_piece_out_kernel(ScanParams p) {
  __shared__ float bc_sm[S1_ROWS * 2 * NM];
  pdl_sync();
  const int piece = blockIdx.y;
  int ch = blockIdx.x * S1_THREADS + threadIdx.x;
  const bool valid = ch < p.inner;
  if (!valid) ch = p.inner - 1;
  int b, r0, r1;
  if (!ss_piece_rows(p, piece, b, r0, r1)) return;
  float S[NM], A[NM];
  ss_load_A1<NM>(p, ch, A);
  const float* sc = p.scratch + (static_cast<size_t>(piece) * p.inner + ch) * (p.N + 1);
#pragma unroll
  for (int i = 0; i < NM; ++i) S[i] = i < p.N ? sc[i] : 0.f;
  ss_walk1<CT, NM, true>(p, ch, valid, r0, r1, S, A, nullptr, bc_sm);
}

template <int NM>
static int launch_scan1(const ScanParams& p, int out_dtype, bool tiled, cudaStream_t stream) {
  const int cx = (p.inner + S1_THREADS - 1) / S1_THREADS;
  if (!tiled) {
    if (out_dtype == 1) VB_LAUNCH_PDL((selective_scan1_kernel<float, NM>), dim3(cx, p.B), S1_THREADS, 0, stream, p);
    else VB_LAUNCH_PDL((selective_scan1_kernel<__nv_bfloat16, NM>), dim3(cx, p.B), S1_THREADS, 0, stream, p);
    return 0;
  }
  const int pieces = p.n_tiles * (p.tile_rows / p.piece_rows);
  const long long states = static_cast<long long>(p.inner) * p.N;
  VB_LAUNCH_PDL(scan1_piece_sum_kernel<NM>, dim3(cx, pieces), S1_THREADS, 0, stream, p);
  VB_LAUNCH_PDL(scan_piece_carry_kernel, dim3(static_cast<unsigned>((states + 127) / 128), p.B), 128, 0, stream, p);
  if (out_dtype == 1) VB_LAUNCH_PDL((scan1_piece_out_kernel<float, NM>), dim3(cx, pieces), S1_THREADS, 0, stream, p);
  else VB_LAUNCH_PDL((scan1_piece_out_kernel<__nv_bfloat16, NM>), dim3(cx, pieces), S1_THREADS, 0, stream, p);
  return 0;
}

static int dispatch_scan(const ScanParams& p, int out_dtype, bool tiled, cudaStream_t stream) {
  if (p.N <= 4) return launch_scan1<4>(p, out_dtype, tiled, stream);
  if (p.N <= 8) return launch_scan1<8>(p, out_dtype, tiled, stream);
  if (p.N <= 16) return launch_scan1<16>(p, out_dtype, tiled, stream);
  const int npl = (p.N + SS_LANES - 1) / SS_LANES;
  if (npl <= 1) return launch_scan<1>(p, out_dtype, tiled, stream);
  if (npl <= 2) return launch_scan<2>(p, out_dtype, tiled, stream);
  if (npl <= 4) return launch_scan<4>(p, out_dtype, tiled, stream);
  if (npl <= 8) return launch_scan<8>(p, out_dtype, tiled, stream);
  if (npl <= 16) return launch_scan<16>(p, out_dtype, tiled, stream);
  return launch_scan<32>(p, out_dtype, tiled, stream);
}

}  // namespace vb

using namespace vb;

extern "C" {

int vb_selective_scan_piece_rows(void) { return 16; }

int vb_selective_scan_scratch_floats(int n_tiles, int tile_rows, int inner, int states) {
  return n_tiles * (tile_rows / vb_selective_scan_piece_rows()) * inner * (states + 1);
}

int vb_selective_scan(void* d_out, int ld_out, float* d_state, const float* d_x, int ld_x, const float* d_dt, int ld_dt,
                      const float* d_dt_bias, const float* d_bc, int ld_bc, int b_off, int c_off, const float* d_z, int ld_z,
                      const float* d_A, const float* d_D, const int32_t* d_qo_indptr, const int32_t* d_pos,
                      const int32_t* d_slots, int B, int inner, int states, float out_scale, int single_rows, int multi_rows,
                      int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_state && d_x && d_dt && d_bc && d_z && d_A && d_qo_indptr && d_pos && d_slots,
               "vb_selective_scan: null pointer");
  VB_CHECK_ARG(inner > 0 && states > 0 && states <= 32 * SS_LANES, "vb_selective_scan: inner %d, states %d (<= %d)", inner,
               states, 32 * SS_LANES);
  if (B <= 0) return 0;
  ScanParams p{d_x, ld_x, d_dt, ld_dt, d_dt_bias, d_bc, ld_bc, b_off, c_off, d_z, ld_z, d_A, d_D, d_state, d_out, ld_out,
               d_qo_indptr, d_pos, d_slots, B, inner, states, out_scale, single_rows, multi_rows, nullptr, nullptr, 0, 0, 0,
               nullptr};
  return dispatch_scan(p, out_dtype, false, static_cast<cudaStream_t>(stream));
}

int vb_selective_scan_tiled(void* d_out, int ld_out, float* d_state, float* d_scratch, const float* d_x, int ld_x,
                            const float* d_dt, int ld_dt, const float* d_dt_bias, const float* d_bc, int ld_bc, int b_off,
                            int c_off, const float* d_z, int ld_z, const float* d_A, const float* d_D,
                            const int32_t* d_qo_indptr, const int32_t* d_pos, const int32_t* d_slots,
                            const int32_t* d_tile_req, const int32_t* d_tile_row0, int n_tiles, int tile_rows, int B, int inner,
                            int states, float out_scale, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_state && d_scratch && d_x && d_dt && d_bc && d_z && d_A && d_qo_indptr && d_pos && d_slots &&
               d_tile_req && d_tile_row0, "vb_selective_scan_tiled: null pointer");
  const int piece = vb_selective_scan_piece_rows();
  VB_CHECK_ARG(inner > 0 && states > 0 && states <= 32 * SS_LANES && tile_rows > 0 && tile_rows % piece == 0,
               "vb_selective_scan_tiled: inner %d, states %d (<= %d), tile_rows %d (a multiple of %d)", inner, states,
               32 * SS_LANES, tile_rows, piece);
  if (B <= 0 || n_tiles <= 0) return 0;
  ScanParams p{d_x, ld_x, d_dt, ld_dt, d_dt_bias, d_bc, ld_bc, b_off, c_off, d_z, ld_z, d_A, d_D, d_state, d_out, ld_out,
               d_qo_indptr, d_pos, d_slots, B, inner, states, out_scale, 0, 1, d_tile_req, d_tile_row0, n_tiles, tile_rows, piece,
               d_scratch};
  return dispatch_scan(p, out_dtype, true, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
