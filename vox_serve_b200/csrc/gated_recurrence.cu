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
//   vb_mingru_tiled  prompt portions cut into pieces of rows: the recurrence S_t = a_t S_(t-1) + b_t composes as
//                    (A, B) = (prod a, local end state from zero), so pieces are summarised in parallel, a short scan over a
//                    request's pieces carries the state in, and the pieces then produce their rows in parallel.
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
  float* scratch;         // [n_tiles * pieces per tile][2][width]: A, B of every piece; after the scan [..][0] is its carry-in
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

// Prompt portions.  A tile (tile_rows rows of one request, as the attention kernels use them) is cut into pieces of MG_ROWS
// rows; piece j of tile i is summary slot i * pieces_per_tile + j.  A thread owns one channel of one piece and first loads
// all of the piece's gate inputs (independent loads, all in flight), then runs the short dependent chain over them.
constexpr int MG_ROWS = 16;

// piece summaries: A = prod (1 - z_t), B = the piece's end state from a zero start
__global__ void __launch_bounds__(128) mingru_tile_sum_kernel(MinGruParams p) {
  pdl_sync();
  const int ch = blockIdx.x * 128 + threadIdx.x, ppt = p.tile_rows / MG_ROWS;
  const int tile = blockIdx.y / ppt, piece = blockIdx.y - tile * ppt;
  if (ch >= p.width) return;
  const int b = p.tile_req[tile], r0 = p.tile_row0[tile] + piece * MG_ROWS;
  const int n = min(min(r0 + MG_ROWS, p.tile_row0[tile] + p.tile_rows), p.qo_indptr[b + 1]) - r0;
  float* s = p.scratch + static_cast<size_t>(blockIdx.y) * 2 * p.width;
  if (n <= 0) { s[ch] = 1.f; s[p.width + ch] = 0.f; return; }
  const float bz = p.bz ? p.bz[ch] : 0.f, bx = p.bx ? p.bx[ch] : 0.f;
  float pz[MG_ROWS], px[MG_ROWS];
#pragma unroll
  for (int i = 0; i < MG_ROWS; ++i) {
    const float* row = p.proj + static_cast<size_t>(r0 + min(i, n - 1)) * p.ldp;
    pz[i] = row[p.z_off + ch];
    px[i] = row[p.x_off + ch];
  }
  float A = 1.f, Bv = 0.f;
#pragma unroll
  for (int i = 0; i < MG_ROWS; ++i) {
    if (i < n) {
      const float z = mg_sigmoid(pz[i] + bz), u = px[i] + bx;
      const float c = u >= 0.f ? u + 0.5f : mg_sigmoid(u);
      A *= 1.f - z;
      Bv = (1.f - z) * Bv + z * c;
    }
  }
  s[ch] = A;
  s[p.width + ch] = Bv;
}

// per (request, channel): walk the request's pieces in order, leave every piece's carry-in in its summary slot [0] and the
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
  int last = lo;
  while (last < p.n_tiles && p.tile_req[last] == b) ++last;
  const int ppt = p.tile_rows / MG_ROWS;
  float* st = p.state + static_cast<size_t>(p.slots[b]) * p.width + ch;
  float S = p.pos[r0] == 0 ? 0.f : *st;
  float* s = p.scratch + static_cast<size_t>(lo) * ppt * 2 * p.width + ch;
  const int n = (last - lo) * ppt;
  // (the summaries do not depend on S: eight pieces' loads are issued before their chain runs)
  for (int i0 = 0; i0 < n; i0 += 8) {
    float A[8], Bv[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const bool ok = i0 + i < n;
      A[i] = ok ? s[static_cast<size_t>(i0 + i) * 2 * p.width] : 1.f;
      Bv[i] = ok ? s[static_cast<size_t>(i0 + i) * 2 * p.width + p.width] : 0.f;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      if (i0 + i < n) {
        s[static_cast<size_t>(i0 + i) * 2 * p.width] = S;
        S = A[i] * S + Bv[i];
      }
    }
  }
  *st = S;
}

template <typename CT>
__global__ void __launch_bounds__(128) mingru_tile_out_kernel(MinGruParams p) {
  pdl_sync();
  const int ch = blockIdx.x * 128 + threadIdx.x, ppt = p.tile_rows / MG_ROWS;
  const int tile = blockIdx.y / ppt, piece = blockIdx.y - tile * ppt;
  if (ch >= p.width) return;
  const int b = p.tile_req[tile], r0 = p.tile_row0[tile] + piece * MG_ROWS;
  const int n = min(min(r0 + MG_ROWS, p.tile_row0[tile] + p.tile_rows), p.qo_indptr[b + 1]) - r0;
  if (n <= 0) return;
  const float bz = p.bz ? p.bz[ch] : 0.f, bx = p.bx ? p.bx[ch] : 0.f;
  float pz[MG_ROWS], px[MG_ROWS], pg[MG_ROWS];
#pragma unroll
  for (int i = 0; i < MG_ROWS; ++i) {
    const float* row = p.proj + static_cast<size_t>(r0 + min(i, n - 1)) * p.ldp;
    pz[i] = row[p.z_off + ch];
    px[i] = row[p.x_off + ch];
    pg[i] = row[p.g_off + ch];
  }
  float S = p.scratch[static_cast<size_t>(blockIdx.y) * 2 * p.width + ch];
#pragma unroll
  for (int i = 0; i < MG_ROWS; ++i) {
    if (i < n) {
      const float z = mg_sigmoid(pz[i] + bz), u = px[i] + bx;
      const float c = u >= 0.f ? u + 0.5f : mg_sigmoid(u);
      S = (1.f - z) * S + z * c;
      mg_store<CT>(p.out, static_cast<size_t>(r0 + i) * p.width + ch, S * (pg[i] * mg_sigmoid(pg[i])));
    }
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
               width > 0 && tile_rows > 0 && tile_rows % MG_ROWS == 0, "vb_mingru_tiled: bad arguments (tile_rows a multiple of %d)",
               MG_ROWS);
  if (B <= 0 || n_tiles <= 0) return 0;
  MinGruParams p{d_proj, ldp, z_off, x_off, g_off, d_bz, d_bx, d_state, d_out, d_qo_indptr, d_pos, d_slots, B, width,
                 0, 1, d_tile_req, d_tile_row0, n_tiles, tile_rows, d_scratch};
  const int cx = (width + 127) / 128, pieces = n_tiles * (tile_rows / MG_ROWS);
  VB_LAUNCH_PDL(mingru_tile_sum_kernel, dim3(cx, pieces), 128, 0, stream, p);
  VB_LAUNCH_PDL(mingru_tile_scan_kernel, dim3(cx, B), 128, 0, stream, p);
  if (out_dtype == 1) VB_LAUNCH_PDL(mingru_tile_out_kernel<float>, dim3(cx, pieces), 128, 0, stream, p);
  else VB_LAUNCH_PDL(mingru_tile_out_kernel<bf16>, dim3(cx, pieces), 128, 0, stream, p);
  return 0;
}

int vb_mingru_scratch_floats(int n_tiles, int tile_rows, int width) {
  return n_tiles * (tile_rows / MG_ROWS) * 2 * width;
}

}  // extern "C"
