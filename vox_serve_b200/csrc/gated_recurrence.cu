// Element-wise gated recurrences over a per-request fp32 state slot (minGRU: gates that read only the current token).
//
//   z_t = sigmoid(pz_t + bz)                       update gate
//   c_t = u + 1/2 (u >= 0), sigmoid(u) (u < 0)     candidate, u = px_t + bx   (positive and continuous at 0)
//   S_t = (1 - z_t) S_(t-1) + z_t c_t              per channel, S = 0 before a request's position 0
//   out_t = S_t * silu(pg_t)
//
// pz | px | pg are columns of the fp32 rows of a fused projection.  Everything here is fp32; only `out` takes the compute
// type (it feeds the output projection).  A slot's stored state is ignored when the request's first row of the step has
// position 0, so slots are handed out again without clearing.
//
//   vb_mingru        one thread per (request, channel) walks the request's rows in order: single-token rows and short portions
//   vb_mingru_tiled  prompt portions cut into tiles of rows: the recurrence S_t = a_t S_(t-1) + b_t composes as
//                    (A, B) = (prod a, local end state from zero), so tiles are summarised in parallel, a short scan over a
//                    request's tiles carries the state in, and the tiles then produce their rows in parallel.
#include "../../include/vb_api.h"
#define VB_PDL_FAMILY 1
#include "common.cuh"

namespace vb {

struct MinGruParams {
  const float* proj;      // [T][ldp]
  int ldp, z_off, x_off, g_off;
  const float* bz;        // [width] or nullptr
  const float* bx;
  float* state;           // [slots][width]
  void* out;              // [T][width]
  const int32_t* qo_indptr;
  const int32_t* pos;
  const int32_t* slots;
  int B, width;
  int single_rows, multi_rows;      // which requests this launch serves: those bringing one row / several rows
  // tiled form
  const int32_t* tile_req;
  const int32_t* tile_row0;
  int n_tiles, tile_rows;
  float* scratch;         // [n_tiles][2][width]: A, B of every tile; after the scan [..][0] holds the tile's carry-in
};

__device__ __forceinline__ float mg_sigmoid(float v) { return 1.f / (1.f + expf(-v)); }
__device__ __forceinline__ void mg_gates(const float* __restrict__ row, const MinGruParams& p, int ch, float bz, float bx,
                                         float& z, float& c) {
  z = mg_sigmoid(row[p.z_off + ch] + bz);
  const float u = row[p.x_off + ch] + bx;
  c = u >= 0.f ? u + 0.5f : mg_sigmoid(u);
}
template <typename CT> __device__ __forceinline__ void mg_store(void* out, size_t i, float v);
template <> __device__ __forceinline__ void mg_store<float>(void* out, size_t i, float v) { static_cast<float*>(out)[i] = v; }
template <> __device__ __forceinline__ void mg_store<__nv_bfloat16>(void* out, size_t i, float v) {
  static_cast<__nv_bfloat16*>(out)[i] = __float2bfloat16_rn(v);
}

template <typename CT>
__global__ void __launch_bounds__(128) mingru_seq_kernel(MinGruParams p) {
  pdl_sync();
  const int ch = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
  if (ch >= p.width) return;
  const int r0 = p.qo_indptr[b], r1 = p.qo_indptr[b + 1];
  const int n = r1 - r0;
  if (n <= 0 || (n == 1 && !p.single_rows) || (n > 1 && !p.multi_rows)) return;
  float* st = p.state + static_cast<size_t>(p.slots[b]) * p.width + ch;
  float S = p.pos[r0] == 0 ? 0.f : *st;
  const float bz = p.bz ? p.bz[ch] : 0.f, bx = p.bx ? p.bx[ch] : 0.f;
  for (int t = r0; t < r1; ++t) {
    const float* row = p.proj + static_cast<size_t>(t) * p.ldp;
    float z, c;
    mg_gates(row, p, ch, bz, bx, z, c);
    S = (1.f - z) * S + z * c;
    const float g = row[p.g_off + ch];
    mg_store<CT>(p.out, static_cast<size_t>(t) * p.width + ch, S * (g * mg_sigmoid(g)));
  }
  *st = S;
}

// tile summaries: A = prod (1 - z_t), B = the tile's end state from a zero start
__global__ void __launch_bounds__(128) mingru_tile_sum_kernel(MinGruParams p) {
  pdl_sync();
  const int ch = blockIdx.x * 128 + threadIdx.x, tile = blockIdx.y;
  if (ch >= p.width) return;
  const int b = p.tile_req[tile], r0 = p.tile_row0[tile], r1 = min(r0 + p.tile_rows, p.qo_indptr[b + 1]);
  const float bz = p.bz ? p.bz[ch] : 0.f, bx = p.bx ? p.bx[ch] : 0.f;
  float A = 1.f, Bv = 0.f;
  for (int t = r0; t < r1; ++t) {
    float z, c;
    mg_gates(p.proj + static_cast<size_t>(t) * p.ldp, p, ch, bz, bx, z, c);
    A *= 1.f - z;
    Bv = (1.f - z) * Bv + z * c;
  }
  float* s = p.scratch + static_cast<size_t>(tile) * 2 * p.width;
  s[ch] = A;
  s[p.width + ch] = Bv;
}

// per (request, channel): walk the request's tiles in order, leave every tile's carry-in in scratch[tile][0] and the
// request's end state in its slot
__global__ void __launch_bounds__(128) mingru_tile_scan_kernel(MinGruParams p) {
  pdl_sync();
  const int ch = blockIdx.x * 128 + threadIdx.x, b = blockIdx.y;
  if (ch >= p.width) return;
  const int r0 = p.qo_indptr[b], r1 = p.qo_indptr[b + 1];
  if (r1 - r0 <= 1) return;
  // the request's tiles are consecutive and in order; find the first (tiles are sorted by request)
  int lo = 0, hi = p.n_tiles;
  while (lo < hi) {
    const int mid = (lo + hi) >> 1;
    if (p.tile_req[mid] < b) lo = mid + 1; else hi = mid;
  }
  float* st = p.state + static_cast<size_t>(p.slots[b]) * p.width + ch;
  float S = p.pos[r0] == 0 ? 0.f : *st;
  for (int tile = lo; tile < p.n_tiles && p.tile_req[tile] == b; ++tile) {
    float* s = p.scratch + static_cast<size_t>(tile) * 2 * p.width;
    const float A = s[ch], Bv = s[p.width + ch];
    s[ch] = S;
    S = A * S + Bv;
  }
  *st = S;
}

template <typename CT>
__global__ void __launch_bounds__(128) mingru_tile_out_kernel(MinGruParams p) {
  pdl_sync();
  const int ch = blockIdx.x * 128 + threadIdx.x, tile = blockIdx.y;
  if (ch >= p.width) return;
  const int b = p.tile_req[tile], r0 = p.tile_row0[tile], r1 = min(r0 + p.tile_rows, p.qo_indptr[b + 1]);
  const float bz = p.bz ? p.bz[ch] : 0.f, bx = p.bx ? p.bx[ch] : 0.f;
  float S = p.scratch[static_cast<size_t>(tile) * 2 * p.width + ch];
  for (int t = r0; t < r1; ++t) {
    const float* row = p.proj + static_cast<size_t>(t) * p.ldp;
    float z, c;
    mg_gates(row, p, ch, bz, bx, z, c);
    S = (1.f - z) * S + z * c;
    const float g = row[p.g_off + ch];
    mg_store<CT>(p.out, static_cast<size_t>(t) * p.width + ch, S * (g * mg_sigmoid(g)));
  }
}

}  // namespace vb

using namespace vb;
using bf16 = __nv_bfloat16;

extern "C" {

int vb_mingru(void* d_out, float* d_state, const float* d_proj, int ldp, int z_off, int x_off, int g_off, const float* d_bz,
              const float* d_bx, const int32_t* d_qo_indptr, const int32_t* d_pos, const int32_t* d_slots, int B, int width,
              int single_rows, int multi_rows, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_state && d_proj && d_qo_indptr && d_pos && d_slots && width > 0, "vb_mingru: bad arguments");
  if (B <= 0) return 0;
  MinGruParams p{d_proj, ldp, z_off, x_off, g_off, d_bz, d_bx, d_state, d_out, d_qo_indptr, d_pos, d_slots, B, width,
                 single_rows, multi_rows, nullptr, nullptr, 0, 0, nullptr};
  dim3 grid((width + 127) / 128, B);
  if (out_dtype == 1) VB_LAUNCH_PDL(mingru_seq_kernel<float>, grid, 128, 0, stream, p);
  else VB_LAUNCH_PDL(mingru_seq_kernel<bf16>, grid, 128, 0, stream, p);
  return 0;
}

int vb_mingru_tiled(void* d_out, float* d_state, float* d_scratch, const float* d_proj, int ldp, int z_off, int x_off,
                    int g_off, const float* d_bz, const float* d_bx, const int32_t* d_qo_indptr, const int32_t* d_pos,
                    const int32_t* d_slots, const int32_t* d_tile_req, const int32_t* d_tile_row0, int n_tiles, int tile_rows,
                    int B, int width, int out_dtype, void* stream) {
  VB_CHECK_ARG(d_out && d_state && d_scratch && d_proj && d_qo_indptr && d_pos && d_slots && d_tile_req && d_tile_row0 &&
               width > 0 && tile_rows > 0, "vb_mingru_tiled: bad arguments");
  if (B <= 0 || n_tiles <= 0) return 0;
  MinGruParams p{d_proj, ldp, z_off, x_off, g_off, d_bz, d_bx, d_state, d_out, d_qo_indptr, d_pos, d_slots, B, width,
                 0, 1, d_tile_req, d_tile_row0, n_tiles, tile_rows, d_scratch};
  const int cx = (width + 127) / 128;
  VB_LAUNCH_PDL(mingru_tile_sum_kernel, dim3(cx, n_tiles), 128, 0, stream, p);
  VB_LAUNCH_PDL(mingru_tile_scan_kernel, dim3(cx, B), 128, 0, stream, p);
  if (out_dtype == 1) VB_LAUNCH_PDL(mingru_tile_out_kernel<float>, dim3(cx, n_tiles), 128, 0, stream, p);
  else VB_LAUNCH_PDL(mingru_tile_out_kernel<bf16>, dim3(cx, n_tiles), 128, 0, stream, p);
  return 0;
}

}  // extern "C"
