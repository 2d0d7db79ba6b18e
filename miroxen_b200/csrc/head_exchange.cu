// Head exchange of the sequence-parallel attention path: the gather on the way back and the peer
// buffers both directions use (reference: src/models/minimax_h3/dit_sp.cpp:96-112 sends each card's
// q / k / v heads to the card that attends over them, :137-149 fetches the attention output of this
// card's rows back from the card that computed those heads).  The outbound side is
// mxk_qkv_norm_rope_scatter in head_norm_rope.cu: the norm + rope kernel stores each head group
// straight into its owner's buffer.
#include <cstring>

#include "common.cuh"
#include "tuning.h"

namespace mxk {
namespace {

struct GatherArgs {
  const uint4* src[MXK_MAX_HEAD_GROUPS];  // [*, group_vecs] 16-byte vectors per row
  int groups;
  int group_vecs;  // heads_per_group * D / 8
  int64_t src_row0, rows;
  uint4* out;  // [rows, groups * group_vecs]
};

// One 16-byte vector per thread per trip: out[r][g * group_vecs + v] = src[g][(src_row0 + r) * group_vecs + v].
// Consecutive threads walk one destination row, so both sides are contiguous per warp; sources may be
// peer mappings (plain loads over NVLink).
__global__ void __launch_bounds__(256) gather_head_groups_kernel(const GatherArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int64_t row_vecs = int64_t(a.groups) * a.group_vecs;
  const int64_t total = a.rows * row_vecs;
  const int64_t stride = int64_t(gridDim.x) * blockDim.x;
  for (int64_t i0 = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += 4 * stride) {
    uint4 v[4];
    bool on[4];
#pragma unroll
    for (int u = 0; u < 4; u++) {
      const int64_t i = i0 + u * stride;
      on[u] = i < total;
      if (on[u]) {
        const int64_t r = i / row_vecs;
        const int c = int(i - r * row_vecs);
        const int g = c / a.group_vecs;
        v[u] = a.src[g][(a.src_row0 + r) * a.group_vecs + (c - g * a.group_vecs)];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; u++)
      if (on[u]) a.out[i0 + u * stride] = v[u];
  }
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_gather_head_groups(const mxk_bf16* const* srcs_host, int groups, int64_t src_row0, int64_t rows,
                           int heads_per_group, int D, mxk_bf16* out, mxk_stream_t stream) {
  if (rows <= 0) return MXK_OK;
  if (!srcs_host || !out || groups < 1 || groups > MXK_MAX_HEAD_GROUPS || heads_per_group <= 0 || D <= 0 || D % 8 != 0 || src_row0 < 0)
    return fail(MXK_ERR_INVALID_ARG, "gather_head_groups: groups=%d (1..%d) heads_per_group=%d D=%d (multiple of 8) src_row0=%lld",
                groups, MXK_MAX_HEAD_GROUPS, heads_per_group, D, (long long)src_row0);
  GatherArgs a{};
  for (int g = 0; g < groups; g++) {
    if (!srcs_host[g] || !aligned(srcs_host[g], 16)) return fail(MXK_ERR_INVALID_ARG, "gather_head_groups: source %d is null or not 16-byte aligned", g);
    a.src[g] = reinterpret_cast<const uint4*>(srcs_host[g]);
  }
  if (!aligned(out, 16)) return fail(MXK_ERR_INVALID_ARG, "gather_head_groups: out is not 16-byte aligned");
  a.groups = groups, a.group_vecs = heads_per_group * D / 8, a.src_row0 = src_row0, a.rows = rows;
  a.out = reinterpret_cast<uint4*>(out);
  const int64_t total = rows * int64_t(groups) * a.group_vecs;
  int64_t grid = ceil_div(total, 256 * 4);
  // one tile of 4 x 256 vectors per CTA and as many CTAs as that takes unless ew_ctas_per_sm caps the grid
  const int64_t cap = int64_t(sm_count()) * tune(TUNE_EW_CTAS_PER_SM, 1 << 20);
  if (grid > cap) grid = cap;
  if (grid > (int64_t(1) << 31) - 1) grid = (int64_t(1) << 31) - 1;
  launch_pdl(gather_head_groups_kernel, dim3(unsigned(grid)), dim3(256), 0, as_stream(stream), a);
  return after_launch("gather_head_groups");
}

int mxk_peer_buffer_alloc(int64_t bytes, void** ptr, unsigned char* handle64) {
  if (!ptr || !handle64 || bytes <= 0) return fail(MXK_ERR_INVALID_ARG, "peer_buffer_alloc: bytes=%lld or a null argument", (long long)bytes);
  static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is passed around as 64 opaque bytes");
  *ptr = nullptr;
  cudaError_t e = cudaMalloc(ptr, size_t(bytes));
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "peer_buffer_alloc: cudaMalloc(%lld): %s", (long long)bytes, cudaGetErrorString(e));
  cudaIpcMemHandle_t h;
  e = cudaIpcGetMemHandle(&h, *ptr);
  if (e != cudaSuccess) {
    cudaFree(*ptr);
    *ptr = nullptr;
    return fail(MXK_ERR_CUDA, "peer_buffer_alloc: cudaIpcGetMemHandle: %s", cudaGetErrorString(e));
  }
  memcpy(handle64, &h, 64);
  return MXK_OK;
}

int mxk_peer_buffer_open(const unsigned char* handle64, void** ptr) {
  if (!ptr || !handle64) return fail(MXK_ERR_INVALID_ARG, "peer_buffer_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  *ptr = nullptr;
  cudaError_t e = cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "peer_buffer_open: cudaIpcOpenMemHandle: %s", cudaGetErrorString(e));
  return MXK_OK;
}

int mxk_peer_buffer_close(void* ptr) {
  if (!ptr) return MXK_OK;
  cudaError_t e = cudaIpcCloseMemHandle(ptr);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "peer_buffer_close: %s", cudaGetErrorString(e));
  return MXK_OK;
}

int mxk_peer_buffer_free(void* ptr) {
  if (!ptr) return MXK_OK;
  cudaError_t e = cudaFree(ptr);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "peer_buffer_free: %s", cudaGetErrorString(e));
  return MXK_OK;
}

}  // extern "C"
