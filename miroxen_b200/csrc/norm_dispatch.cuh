// Host-side plan and template dispatch for the row-norm kernels.
#pragma once

#include "norm_mod.cuh"
#include "tuning.h"

namespace mxk {

// Picks threads per CTA and 4-element vectors per thread so that threads * vpt covers dim / 4
// with the least padding; among equal paddings the CTA size nearest the preferred one wins.
inline bool plan_norm(int nvec, int64_t rows, NormPlan& p) {
  const int want = tune(TUNE_NORM_THREADS, 256);
  int best_waste = 1 << 30, best_dist = 1 << 30;
  p.threads = 0;
  for (int vpt = 1; vpt <= kNormMaxVpt; vpt++) {
    int threads = int(ceil_div(ceil_div(nvec, vpt), 32) * 32);
    if (threads > norm_max_threads(vpt)) continue;
    int waste = threads * vpt - nvec;
    int dist = threads > want ? threads - want : want - threads;
    if (waste < best_waste || (waste == best_waste && dist < best_dist)) {
      best_waste = waste, best_dist = dist;
      p.threads = threads, p.vpt = vpt;
    }
  }
  if (!p.threads) return false;
  p.exact = p.threads * p.vpt == nvec;
  const int per_sm = tune(TUNE_NORM_CTAS_PER_SM, p.threads <= 128 ? 8 : p.threads <= 256 ? 4 : 2);
  int64_t ctas = int64_t(sm_count()) * per_sm;
  if (ctas > rows) ctas = rows;
  p.rows_per_cta = int(ceil_div(rows, ctas));
  p.grid = unsigned(ceil_div(rows, p.rows_per_cta));
  return true;
}

template <int MODE, class TIN, int VPT, bool HAS_W, bool FUSE_RES>
inline void launch_norm_vpt(const NormPlan& p, const NormArgs& a, cudaStream_t s) {
  if (p.exact)
    norm_rows_kernel<MODE, TIN, VPT, HAS_W, FUSE_RES, true><<<p.grid, p.threads, 0, s>>>(a);
  else
    norm_rows_kernel<MODE, TIN, VPT, HAS_W, FUSE_RES, false><<<p.grid, p.threads, 0, s>>>(a);
}

template <int MODE, class TIN, bool HAS_W, bool FUSE_RES>
inline void launch_norm(const NormPlan& p, const NormArgs& a, cudaStream_t s) {
  switch (p.vpt) {
    case 1: launch_norm_vpt<MODE, TIN, 1, HAS_W, FUSE_RES>(p, a, s); break;
    case 2: launch_norm_vpt<MODE, TIN, 2, HAS_W, FUSE_RES>(p, a, s); break;
    case 3: launch_norm_vpt<MODE, TIN, 3, HAS_W, FUSE_RES>(p, a, s); break;
    case 4: launch_norm_vpt<MODE, TIN, 4, HAS_W, FUSE_RES>(p, a, s); break;
    case 5: launch_norm_vpt<MODE, TIN, 5, HAS_W, FUSE_RES>(p, a, s); break;
    case 6: launch_norm_vpt<MODE, TIN, 6, HAS_W, FUSE_RES>(p, a, s); break;
    case 7: launch_norm_vpt<MODE, TIN, 7, HAS_W, FUSE_RES>(p, a, s); break;
    default: launch_norm_vpt<MODE, TIN, 8, HAS_W, FUSE_RES>(p, a, s); break;
  }
}

// True when every pointer the vector kernel dereferences with 8/16-byte accesses is aligned.
template <class TIN>
inline bool norm_vector_ok(const NormArgs& a) {
  if (a.dim % 4) return false;
  auto ok = [](const void* p, size_t b) { return !p || (reinterpret_cast<uintptr_t>(p) & (b - 1)) == 0; };
  return ok(a.x, sizeof(TIN) * 4) && ok(a.out, 8) && ok(a.w, 16) && ok(a.scale.target, 16) &&
         ok(a.scale.prefix, 16) && ok(a.shift.target, 16) && ok(a.shift.prefix, 16) && ok(a.y, 8) &&
         ok(a.gate.target, 16) && ok(a.gate.prefix, 16);
}

// Runs one norm launch (vector kernel when shapes and alignment allow, generic otherwise).
template <int MODE, class TIN, bool FUSE_RES>
inline int run_norm(const char* name, NormArgs a, cudaStream_t s) {
  NormPlan p;
  // LayerNorm with an affine weight has no caller in the reference; it takes the generic kernel.
  if (!(MODE == 0 && a.w) && norm_vector_ok<TIN>(a) && plan_norm(a.nvec, a.rows, p)) {
    a.rows_per_cta = p.rows_per_cta;
    if constexpr (MODE == 1) {
      if (a.w) launch_norm<MODE, TIN, true, FUSE_RES>(p, a, s);
      else launch_norm<MODE, TIN, false, FUSE_RES>(p, a, s);
    } else {
      launch_norm<MODE, TIN, false, FUSE_RES>(p, a, s);
    }
    return after_launch(name);
  }
  // One CTA per row; the x-dimension of a grid holds 2^31 - 1 blocks.
  for (int64_t r0 = 0; r0 < a.rows; r0 += 0x7fffffff) {
    NormArgs b = a;
    int64_t n = a.rows - r0 < 0x7fffffff ? a.rows - r0 : 0x7fffffff;
    b.rows = n;
    b.x = static_cast<const TIN*>(a.x) + r0 * a.dim;
    b.out = a.out + r0 * a.dim;
    if (FUSE_RES) b.xw = a.xw + r0 * a.dim, b.y = a.y + r0 * a.dim;
    b.scale.prefix_len -= r0, b.shift.prefix_len -= r0, b.gate.prefix_len -= r0;
    norm_rows_generic_kernel<MODE, TIN, FUSE_RES><<<unsigned(n), 256, 0, s>>>(b);
    int rc = after_launch(name);
    if (rc) return rc;
  }
  return MXK_OK;
}

inline int check_norm_common(const char* name, const void* x, int64_t rows, int64_t dim,
                             const void* out, const MxkRowMod& scale, const MxkRowMod& shift) {
  if (dim <= 0 || dim > (int64_t(1) << 30)) return fail(MXK_ERR_INVALID_ARG, "%s: dim=%lld out of range", name, (long long)dim);
  if (!x || !out) return fail(MXK_ERR_INVALID_ARG, "%s: null x or out with rows=%lld", name, (long long)rows);
  if ((scale.target && !scale.prefix && scale.prefix_len > 0) ||
      (shift.target && !shift.prefix && shift.prefix_len > 0))
    return fail(MXK_ERR_INVALID_ARG, "%s: prefix_len > 0 with a null prefix vector", name);
  return MXK_OK;
}

}  // namespace mxk
