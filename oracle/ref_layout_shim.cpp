// TEST INFRASTRUCTURE ONLY.  extern "C" doorway to the REFERENCE's own host code for the
// MiniMax-H3 rotary positions (mx::h3_build_layout and mx::h3_build_ref2va_layout,
// src/models/minimax_h3/layout.cpp:68-188),
// compiled from the reference tree next to this file (oracle/Makefile, target _ref).  It runs on
// the CPU, so the oracle's restatement of the positions is checked against it directly.
#include <cstring>
#include <string>
#include <vector>

#include "models/minimax_h3/pipeline.h"

extern "C" {

// anchors[i]: 0 = "first", 1 = "last".  positions (fp32 [S, 3]) may be null to query S.
// Returns S, or -1 when the reference throws.
int64_t ref_h3_positions(int64_t T, int64_t F_lat, int64_t H, int64_t W, int64_t A, const int32_t* anchors,
                         int n_anchors, float* positions) {
  try {
    std::vector<std::string> names;
    for (int i = 0; i < n_anchors; i++) names.push_back(anchors[i] == 0 ? "first" : "last");
    mx::H3Layout L = mx::h3_build_layout(T, F_lat, H, W, A, names);
    if (positions) memcpy(positions, L.positions.data(), L.positions.size() * sizeof(float));
    return L.seq.S;
  } catch (const std::exception&) {
    return -1;
  }
}

// mx::h3_build_ref2va_layout (src/models/minimax_h3/layout.cpp:121-188).  kind[i]: 0 image, 1 video,
// 2 audio.  positions may be null to query S.  Returns S, or -1 when the reference throws.
int64_t ref_h3_ref2va_positions(int64_t T, int n_refs, const int32_t* kind, const int64_t* frames, const int64_t* rh,
                                const int64_t* rw, const int64_t* audio, int64_t F_lat, int64_t H, int64_t W, int64_t A,
                                float* positions) {
  try {
    std::vector<mx::H3RefGeom> refs(n_refs);
    for (int i = 0; i < n_refs; i++) {
      refs[i].kind = kind[i] == 0 ? mx::H3RefGeom::IMAGE : kind[i] == 1 ? mx::H3RefGeom::VIDEO : mx::H3RefGeom::AUDIO;
      refs[i].frames = frames[i], refs[i].h = rh[i], refs[i].w = rw[i], refs[i].audio = audio[i];
    }
    mx::H3Layout L = mx::h3_build_ref2va_layout(T, {}, refs, F_lat, H, W, A);
    if (positions) memcpy(positions, L.positions.data(), L.positions.size() * sizeof(float));
    return L.seq.S;
  } catch (const std::exception&) {
    return -1;
  }
}

}  // extern "C"
