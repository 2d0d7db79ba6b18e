// TEST INFRASTRUCTURE ONLY.  Runs the REFERENCE's own statements for the host-side table and
// embedding builders: the bodies below are `#include`d line ranges of
// src/models/qwen_image/dit.cpp (prepare: run layout + MSRoPE table; time_mod: timestep embedding)
// and src/models/minimax_h3/dit.cpp (time_basis; prepare: cos / sin from positions), cut out at
// build time by oracle/extract_ref_builders.py into oracle/_ref/*.inc.  This file only declares the
// names those statements read (method arguments and class members) and copies their results out.
// Types come from the reference's own headers.
#include <algorithm>
#include <cmath>
#include <cstring>
#include <vector>

#include <cuda_bf16.h>

#include "core/common.h"
#include "models/qwen_image/dit.h"

namespace {
#include "qwen_round_bf16.inc"
}  // namespace

extern "C" {

// QwenImageDit::prepare up to the point where the tables are uploaded.  conds: n_conds x
// {slot0, H, W}.  cos / sin (fp32 [S, 64]) may be null to query S.  Returns S, -1 on a throw.
int64_t ref_qwen_rope_table(int64_t T, int64_t H, int64_t W, const int64_t* cond_slot_h_w, int n_conds, float* cos_out,
                            float* sin_out) {
  try {
    std::vector<mx::QwenImageCond> conds(n_conds);
    for (int i = 0; i < n_conds; i++)
      conds[i].slot0 = cond_slot_h_w[3 * i], conds[i].H = cond_slot_h_w[3 * i + 1], conds[i].W = cond_slot_h_w[3 * i + 2];
    mx::QwenImageSeq seq;
    seq.H = H, seq.W = W;
    mx::QwenImageDitConfig cfg_;
#include "qwen_rope.inc"
    (void)dim;
    if (cos_out) memcpy(cos_out, hc.data(), hc.size() * sizeof(float));
    if (sin_out) memcpy(sin_out, hs.data(), hs.size() * sizeof(float));
    return S;
  } catch (const std::exception&) {
    return -1;
  }
}

// QwenImageDit::time_mod's embedding: emb fp32 [2, 256] (row 0 = t, row 1 = 0).
void ref_qwen_timestep_embedding(float t, float* emb_out) {
#include "qwen_time_embed.inc"
  memcpy(emb_out, emb.data(), emb.size() * sizeof(float));
}

// H3Dit::time_basis: table fp32 [grid, basis] -> out fp32 [n, basis].
void ref_h3_time_basis(const float* ts_in, int64_t n, const float* table_in, int64_t grid_, int64_t basis_, float* out) {
  const std::vector<float> ts(ts_in, ts_in + n);
  const std::vector<float> table_(table_in, table_in + grid_ * basis_);
#include "h3_time_basis.inc"
  memcpy(out, h.data(), h.size() * sizeof(float));
}

// H3Dit::prepare's tables: positions fp32 [S, 3], inv_freq fp32 [nf] -> cos / sin fp32 [S, rot / 2].
void ref_h3_rope_table(const float* positions_in, int64_t S, const float* inv_freq_in, int64_t n_freq, int rot_, float* cos_out,
                       float* sin_out) {
  const std::vector<float> positions(positions_in, positions_in + S * 3);
  const std::vector<float> inv_freq_(inv_freq_in, inv_freq_in + n_freq);
#include "h3_rope.inc"
  memcpy(cos_out, hc.data(), hc.size() * sizeof(float));
  memcpy(sin_out, hs.data(), hs.size() * sizeof(float));
}

}  // extern "C"
