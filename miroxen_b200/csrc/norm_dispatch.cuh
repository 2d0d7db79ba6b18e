// Host-side plan and template dispatch for the row-norm kernels.
#pragma once

#include "norm_mod.cuh"
#include "tuning.h"

namespace mxk {

// Picks threads per CTA and 4-element vectors per thread so that threads * vpt covers dim / 4
// with the least padding; among equal paddings the CTA size nearest the preferred one wins.
inline bool plan_norm(int nvec, int64_t rows, NormPlan& p, int want_default = 128) {
  const int want = tune(TUNE_NORM_THREADS, want_default);  // 128 measured best for the norms on B200
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
  return true;
}

// Rows are split evenly over exactly one resident wave of CTAs (or fewer when rows are few).
inline unsigned norm_grid(NormArgs& a, int per_sm) {
  int64_t ctas = int64_t(sm_count()) * (per_sm > 0 ? per_sm : 1);
  if (ctas > a.rows) ctas = a.rows;
  a.rows_per_cta = int(ceil_div(a.rows, ctas));
  return unsigned(ceil_div(a.rows, a.rows_per_cta));
}

constexpr int kNormMaxStages = 8;

template <int MODE, class TIN, int VPT, bool HAS_W, bool FUSE_RES, bool EXACT, bool QUANT = false, bool YBIAS = false>
inline void launch_norm_inst(const NormPlan& p, NormArgs a, bool tma, cudaStream_t s) {
  if (tma) {
    a.err = device_error_word();
    auto k = norm_rows_tma_kernel<MODE, TIN, VPT, HAS_W, FUSE_RES, EXACT, QUANT, YBIAS>;
    const int xb = (a.dim * int(sizeof(TIN)) + 127) & ~127;
    const int stage_bytes = xb + (FUSE_RES ? ((a.dim * 2 + 127) & ~127) : 0);
    int stages = tune(TUNE_NORM_STAGES, 0);
    // Two stages per CTA measured best on B200: small stages leave room for more resident CTAs,
    // and the CTAs of one SM together keep enough rows in flight.
    // The residual-only mode (MODE 2) does better still as ONE ROW PER CTA, more CTAs than are resident, each with a
    // single stage: the hardware hands a new row to an SM the moment one finishes, there is no ramp or tail of a
    // persistent loop, and nothing is reduced over the row that would want the next row's copy under way
    // (8704 x 3072: 41.9 us against 46.5 us; 33272 x 5120: 242 us against 272 us).  The normalising modes lose
    // with that grid (their per-CTA set-up - modulation vectors into registers - is paid per row then).
    // (the form that also adds a bias reads a second per-column vector per CTA: one row per CTA paid for that at
    // d = 5120 - 298 us against 269 us - so it keeps the resident wave)
    const bool row_per_cta = MODE == 2 && !QUANT && !YBIAS && tune(TUNE_NORM_CTAS_PER_SM, 0) == 0;
    if (stages <= 0) stages = row_per_cta ? 1 : 2;
    if (stages < 2 && !row_per_cta) stages = 2;
    if (stages > kNormMaxStages) stages = kNormMaxStages;
    // the quantising form keeps the bf16 row in shared memory behind the stages
    const size_t smem = size_t(stages) * stage_bytes + (QUANT ? size_t(a.dim) * 2 : 0);
    // static shared memory (reduction scratch, barriers) counts against the 48 KB default too
    if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
    const unsigned grid = norm_grid(a, row_per_cta ? (1 << 20) : tune(TUNE_NORM_CTAS_PER_SM, resident_ctas(k, p.threads, smem)));
    a.row_step = tune(TUNE_NORM_INTERLEAVE, 1) == 1 ? int64_t(grid) : 1;
    launch_pdl(k, dim3(grid), dim3(p.threads), smem, s, a, stages, stage_bytes);
  } else if constexpr (!QUANT && !YBIAS) {  // the quantising and bias forms exist for the bulk-copy kernel only
    auto k = norm_rows_kernel<MODE, TIN, VPT, HAS_W, FUSE_RES, EXACT>;
    const unsigned grid = norm_grid(a, tune(TUNE_NORM_CTAS_PER_SM, resident_ctas(k, p.threads)));
    launch_pdl(k, dim3(grid), dim3(p.threads), 0, s, a);
  }
}

template <int MODE, class TIN, int VPT, bool HAS_W, bool FUSE_RES, bool QUANT = false, bool YBIAS = false>
inline void launch_norm_vpt(const NormPlan& p, const NormArgs& a, bool tma, cudaStream_t s) {
  if (p.exact) launch_norm_inst<MODE, TIN, VPT, HAS_W, FUSE_RES, true, QUANT, YBIAS>(p, a, tma, s);
  else launch_norm_inst<MODE, TIN, VPT, HAS_W, FUSE_RES, false, QUANT, YBIAS>(p, a, tma, s);
}

template <int MODE, class TIN, bool HAS_W, bool FUSE_RES, bool QUANT = false, bool YBIAS = false>
inline void launch_norm(const NormPlan& p, const NormArgs& a, bool tma, cudaStream_t s) {
  switch (p.vpt) {
    case 1: launch_norm_vpt<MODE, TIN, 1, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    case 2: launch_norm_vpt<MODE, TIN, 2, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    case 3: launch_norm_vpt<MODE, TIN, 3, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    case 4: launch_norm_vpt<MODE, TIN, 4, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    case 5: launch_norm_vpt<MODE, TIN, 5, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    case 6: launch_norm_vpt<MODE, TIN, 6, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    case 7: launch_norm_vpt<MODE, TIN, 7, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
    default: launch_norm_vpt<MODE, TIN, 8, HAS_W, FUSE_RES, QUANT, YBIAS>(p, a, tma, s); break;
  }
}

// True when every pointer the register row kernel dereferences with 8/16-byte accesses is aligned.
template <class TIN>
inline bool norm_vector_ok(const NormArgs& a) {
  if (a.dim % 4) return false;
  auto ok = [](const void* p, size_t b) { return !p || (reinterpret_cast<uintptr_t>(p) & (b - 1)) == 0; };
  return ok(a.x, sizeof(TIN) * 4) && ok(a.out, 8) && ok(a.w, 16) && ok(a.scale.target, 16) &&
         ok(a.scale.prefix, 16) && ok(a.shift.target, 16) && ok(a.shift.prefix, 16) && ok(a.y, 8) &&
         ok(a.gate.target, 16) && ok(a.gate.prefix, 16);
}

// What the bulk-copy row kernel needs on top of norm_vector_ok(): every row it copies with
// cp.async.bulk must start on a 16-byte boundary and be a multiple of 16 bytes long.  Callers pass
// offset pointers (a view that starts a few elements into a buffer), so the base address is checked
// as well as the row pitch: a bf16 x or y that is only 8-byte aligned takes the register kernel.
template <class TIN>
inline bool norm_bulk_ok(const NormArgs& a, bool fuse_res) {
  auto ok16 = [](const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; };
  if ((int64_t(a.dim) * int64_t(sizeof(TIN))) % 16 != 0 || !ok16(a.x)) return false;
  if (fuse_res && (a.dim % 8 != 0 || !ok16(a.y) || !ok16(a.xw))) return false;
  return a.rows >= 2;
}

// Kernel family a norm launch takes.  Pure host arithmetic on pointer values and sizes (nothing is
// dereferenced), so the choice can be checked without a GPU (mxk_norm_path_probe).
enum NormPath { kNormPathGeneric = 0, kNormPathVector = 1, kNormPathBulk = 2 };

template <int MODE, class TIN, bool FUSE_RES>
inline NormPath choose_norm_path(const NormArgs& a, NormPlan& p) {
  // LayerNorm with an affine weight has no caller in the reference; it takes the generic kernel.
  if ((MODE == 0 && a.w) || !norm_vector_ok<TIN>(a) || !plan_norm(a.nvec, a.rows, p)) return kNormPathGeneric;
  if (tune(TUNE_NORM_PATH, 1) == 1 && norm_bulk_ok<TIN>(a, FUSE_RES)) return kNormPathBulk;
  return kNormPathVector;
}

// Runs one norm launch (bulk-copy or register row kernel when shapes and alignment allow, generic otherwise).
template <int MODE, class TIN, bool FUSE_RES>
inline int run_norm(const char* name, NormArgs a, cudaStream_t s) {
  NormPlan p;
  const NormPath path = choose_norm_path<MODE, TIN, FUSE_RES>(a, p);
  if (path != kNormPathGeneric) {
    const bool tma = path == kNormPathBulk;
    if constexpr (MODE == 1) {
      if (a.w) launch_norm<MODE, TIN, true, FUSE_RES>(p, a, tma, s);
      else launch_norm<MODE, TIN, false, FUSE_RES>(p, a, tma, s);
    } else {
      launch_norm<MODE, TIN, false, FUSE_RES>(p, a, tma, s);
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

// The norm + MXFP8 one-pass forms run on the bulk-copy row kernel only; true when this call can take it.
template <bool FUSE_RES>
inline bool norm_quant_ok(const NormArgs& a, NormPlan& p) {
  NormArgs b = a;
  b.rows = a.rows < 2 ? 2 : a.rows;  // a single row runs through the same kernel
  return norm_vector_ok<float>(a) && norm_bulk_ok<float>(b, FUSE_RES) && plan_norm(a.nvec, a.rows, p);
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
