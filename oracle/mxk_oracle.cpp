// CPU ORACLE - TEST INFRASTRUCTURE ONLY.  Nothing in the product (miroxen_b200/, include/) may
// call, link or import this file; it exists so that the tests, the smoke check and the CPU-baseline
// leg of the benchmark have an independent statement of what the reference computes.
//
// It restates, in plain fp32 C++ (no FMA contraction, libm for every transcendental), the
// algorithm of the reference's fused layer ops (src/kernels/ops.cu) and of its host-side table
// builders (src/models/qwen_image/dit.cpp, src/models/minimax_h3/dit.cpp, layout.cpp); each
// function cites the lines it follows.  Where the reference reduces over a CUDA block, the same
// association order is used: per-thread strided partial sums, an xor-butterfly inside each warp,
// then a butterfly over the per-warp totals (src/kernels/ops.cu:8-30).
//
// Pinning: the reference holds no unit test, golden vector or CPU implementation for these ops
// (its only checks are whole-model comparisons that need checkpoints).  The ops are pinned
// against outputs of the reference's own kernels - src/kernels/ops.cu compiled unmodified for
// sm_100a (oracle/Makefile, target _ref) and run on a B200 - stored in
// tests/golden/ref_ops_sm100a.npz, and the H3 rotary positions against the reference's own host
// code (tests/golden/h3_positions.npz).  The Qwen table builder and the timestep embedding have
// no runnable counterpart outside the reference's model classes: for those two parity is
// unpinned beyond the closed-form spot checks against libm in the tests.
// The block-scale quantiser at the end of this file (src/kernels/blockscale.cu) is pinned the same
// way as the ops: byte outputs of the reference's kernel on a B200 (tests/golden/
// ref_blockscale_sm100a.npz), plus the error bounds of the reference's own test
// (tests/blockscale_test.cpp:83-105) on the decoded values.
#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstring>
#include <thread>
#include <vector>

namespace {

int g_threads = 1;

inline float bf2f(uint16_t b) {
  uint32_t u = uint32_t(b) << 16;
  float f;
  memcpy(&f, &u, 4);
  return f;
}
// round-to-nearest-even, as __float2bfloat16
inline uint16_t f2bf(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  if ((u & 0x7fffffffu) > 0x7f800000u) return 0x7fff;
  u += 0x7fffu + ((u >> 16) & 1u);
  return uint16_t(u >> 16);
}
inline float round_bf16(float v) { return bf2f(f2bf(v)); }

template <class F>
void parallel_rows(int64_t rows, F f) {
  int nt = int(std::min<int64_t>(g_threads, rows));
  if (nt <= 1) {
    f(0, rows);
    return;
  }
  std::vector<std::thread> th;
  int64_t per = (rows + nt - 1) / nt;
  for (int t = 0; t < nt; t++) {
    int64_t a = t * per, b = std::min(rows, a + per);
    if (a < b) th.emplace_back([=] { f(a, b); });
  }
  for (auto& t : th) t.join();
}

// block_sum of src/kernels/ops.cu:14-30 for a block of `threads` threads (multiple of 32).
float block_sum(const float* partial, int threads) {
  const int nw = threads / 32;
  float tot[32];
  for (int w = 0; w < 32; w++) tot[w] = 0.f;
  for (int w = 0; w < nw; w++) {
    float v[32], n[32];
    for (int l = 0; l < 32; l++) v[l] = partial[w * 32 + l];
    for (int o = 16; o > 0; o >>= 1) {
      for (int l = 0; l < 32; l++) n[l] = v[l] + v[l ^ o];
      memcpy(v, n, sizeof(v));
    }
    tot[w] = v[0];
  }
  float v[32], n[32];
  memcpy(v, tot, sizeof(v));
  for (int o = 16; o > 0; o >>= 1) {
    for (int l = 0; l < 32; l++) n[l] = v[l] + v[l ^ o];
    memcpy(v, n, sizeof(v));
  }
  return v[0];
}

struct RowMod {
  const float* target;
  const float* prefix;
  int64_t prefix_len;
};
inline const float* pick(const RowMod& m, int64_t row) { return row < m.prefix_len ? m.prefix : m.target; }

// norm_mod_kernel, src/kernels/ops.cu:43-71.  MODE 0 LayerNorm, 1 RMSNorm; 256 threads.
template <int MODE, bool BF16_IN>
void norm_mod(const void* xin, int64_t rows, int64_t dim, float eps, const float* w, RowMod scale, RowMod shift,
              uint16_t* out) {
  parallel_rows(rows, [=](int64_t a, int64_t b) {
    std::vector<float> xr(dim);
    for (int64_t row = a; row < b; row++) {
      if (BF16_IN) {
        const uint16_t* p = static_cast<const uint16_t*>(xin) + row * dim;
        for (int64_t i = 0; i < dim; i++) xr[i] = bf2f(p[i]);
      } else {
        memcpy(xr.data(), static_cast<const float*>(xin) + row * dim, dim * 4);
      }
      float part[256];
      float mean = 0.f;
      if (MODE == 0) {
        for (int t = 0; t < 256; t++) part[t] = 0.f;
        for (int64_t i = 0; i < dim; i++) part[i & 255] += xr[i];
        mean = block_sum(part, 256) / float(dim);
      }
      for (int t = 0; t < 256; t++) part[t] = 0.f;
      for (int64_t i = 0; i < dim; i++) {
        float d = xr[i] - mean;
        part[i & 255] += d * d;
      }
      const float rstd = 1.0f / std::sqrt(block_sum(part, 256) / float(dim) + eps);
      const float* sc = scale.target ? pick(scale, row) : nullptr;
      const float* sh = shift.target ? pick(shift, row) : nullptr;
      uint16_t* orow = out + row * dim;
      for (int64_t i = 0; i < dim; i++) {
        float v = (xr[i] - mean) * rstd;
        if (w) v *= w[i];
        if (sc) v *= 1.f + sc[i];
        if (sh) v += sh[i];
        orow[i] = f2bf(v);
      }
    }
  });
}

}  // namespace

extern "C" {

void or_set_threads(int n) { g_threads = n < 1 ? 1 : n; }
int or_get_threads() { return g_threads; }

// src/kernels/ops.cu:153-159
void or_layernorm_mod(const float* x, int64_t rows, int64_t dim, float eps, RowMod scale, RowMod shift, uint16_t* out) {
  if (rows <= 0) return;
  norm_mod<0, false>(x, rows, dim, eps, nullptr, scale, shift, out);
}
// src/kernels/ops.cu:161-167
void or_rmsnorm_mod(const float* x, int64_t rows, int64_t dim, float eps, const float* w, RowMod scale, RowMod shift,
                    uint16_t* out) {
  if (rows <= 0) return;
  norm_mod<1, false>(x, rows, dim, eps, w, scale, shift, out);
}
// src/kernels/ops.cu:169-175
void or_rmsnorm_bf16(const uint16_t* x, int64_t rows, int64_t dim, float eps, const float* w, uint16_t* out) {
  if (rows <= 0) return;
  norm_mod<1, true>(x, rows, dim, eps, w, RowMod{nullptr, nullptr, 0}, RowMod{nullptr, nullptr, 0}, out);
}

// gated_residual_kernel, src/kernels/ops.cu:73-84
void or_gated_residual(float* x, const uint16_t* y, int64_t rows, int64_t dim, RowMod gate, int gate_tanh) {
  parallel_rows(rows, [=](int64_t a, int64_t b) {
    for (int64_t row = a; row < b; row++)
      for (int64_t i = 0; i < dim; i++) {
        float v = bf2f(y[row * dim + i]);
        if (gate.target) {
          float g = pick(gate, row)[i];
          v *= gate_tanh ? std::tanh(g) : g;
        }
        x[row * dim + i] += v;
      }
  });
}

// src/kernels/ops.cu:191-195
void or_add_inplace_bf16(uint16_t* x, const uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) x[i] = f2bf(bf2f(x[i]) + bf2f(y[i]));
}

// head_norm_rope_kernel, src/kernels/ops.cu:87-119; mode 0 none, 1 interleaved, 2 half.
// Returns -1 for the shapes the launcher rejects (src/kernels/ops.cu:201).
int or_head_norm_rope(const uint16_t* in, int64_t S, int64_t in_stride, int64_t col0, int H, int D, const float* norm_w,
                      float eps, const float* cs, const float* sn, int rot, int mode, uint16_t* out) {
  if (S <= 0) return 0;
  if (!(D % 2 == 0 && D <= 256 && rot <= D && rot % 2 == 0)) return -1;
  const int threads = (D + 31) / 32 * 32;
  parallel_rows(S, [=](int64_t a, int64_t b) {
    float buf[256], part[256];
    for (int64_t s = a; s < b; s++)
      for (int h = 0; h < H; h++) {
        for (int d = 0; d < D; d++) buf[d] = bf2f(in[s * in_stride + col0 + int64_t(h) * D + d]);
        if (norm_w) {
          for (int d = 0; d < threads; d++) part[d] = d < D ? buf[d] * buf[d] : 0.f;
          const float ss = block_sum(part, threads);
          const float r = 1.0f / std::sqrt(ss / float(D) + eps);
          for (int d = 0; d < D; d++) buf[d] = buf[d] * r * norm_w[d];
        }
        uint16_t* o = out + (s * H + h) * D;
        for (int d = 0; d < D; d++) {
          float v = buf[d];
          if (d < rot && mode != 0) {
            const int half = rot / 2;
            int pair, idx;
            float other;
            if (mode == 1) {
              pair = d >> 1, idx = d & 1, other = buf[d ^ 1];
            } else {
              pair = d < half ? d : d - half;
              idx = d < half ? 0 : 1;
              other = buf[d < half ? d + half : d - half];
            }
            const float c = cs[s * half + pair], si = sn[s * half + pair];
            v = idx == 0 ? v * c - other * si : other * si + v * c;
          }
          o[d] = f2bf(v);
        }
      }
  });
  return 0;
}

// silu_mul_kernel, src/kernels/ops.cu:121-128
void or_silu_mul(const uint16_t* gu, int64_t rows, int64_t F, uint16_t* out) {
  parallel_rows(rows, [=](int64_t a, int64_t b) {
    for (int64_t row = a; row < b; row++)
      for (int64_t i = 0; i < F; i++) {
        const float g = bf2f(gu[row * 2 * F + i]);
        const float u = bf2f(gu[row * 2 * F + F + i]);
        out[row * F + i] = f2bf(g / (1.f + std::exp(-g)) * u);
      }
  });
}

// src/kernels/ops.cu:220-226
void or_gelu_tanh_inplace(uint16_t* x, int64_t n) {
  parallel_rows(n, [=](int64_t a, int64_t b) {
    for (int64_t i = a; i < b; i++) {
      const float v = bf2f(x[i]);
      const float t = std::tanh(0.7978845608f * (v + 0.044715f * v * v * v));
      x[i] = f2bf(0.5f * v * (1.f + t));
    }
  });
}

// src/kernels/ops.cu:228-233
void or_gelu_erf_inplace(uint16_t* x, int64_t n) {
  parallel_rows(n, [=](int64_t a, int64_t b) {
    for (int64_t i = a; i < b; i++) {
      const float v = bf2f(x[i]);
      x[i] = f2bf(0.5f * v * (1.f + std::erf(v * 0.7071067811865476f)));
    }
  });
}

// src/kernels/ops.cu:244-246
void or_silu_inplace_f32(float* x, int64_t n) {
  for (int64_t i = 0; i < n; i++) x[i] = x[i] / (1.f + std::exp(-x[i]));
}

// src/kernels/ops.cu:235-242
void or_scatter_rows(float* x, int64_t dim, const int32_t* rows, const uint16_t* src, int64_t n, int add) {
  for (int64_t i = 0; i < n * dim; i++) {
    const int64_t r = i / dim, d = i % dim;
    const float v = bf2f(src[i]);
    float* p = x + int64_t(rows[r]) * dim + d;
    *p = add ? *p + v : v;
  }
}

// src/kernels/ops.cu:249-270
void or_add_bias_bf16(uint16_t* y, const float* bias, int64_t rows, int64_t dim) {
  for (int64_t r = 0; r < rows; r++)
    for (int64_t j = 0; j < dim; j++) y[r * dim + j] = f2bf(bf2f(y[r * dim + j]) + bias[j]);
}
// src/kernels/ops.cu:272-274
void or_add_bias_f32(float* y, const float* bias, int64_t rows, int64_t dim) {
  for (int64_t i = 0; i < rows * dim; i++) y[i] += bias[i % dim];
}
// src/kernels/ops.cu:276-282
void or_f32_to_bf16(const float* x, uint16_t* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = f2bf(x[i]);
}
void or_bf16_to_f32(const uint16_t* x, float* y, int64_t n) {
  for (int64_t i = 0; i < n; i++) y[i] = bf2f(x[i]);
}
// src/kernels/ops.cu:284-290
void or_axpy_f32(float* x, const float* y, float a, int64_t n) {
  for (int64_t i = 0; i < n; i++) x[i] += a * y[i];
}
void or_axpby_f32(float* x, const float* y, float a, float b, int64_t n) {
  for (int64_t i = 0; i < n; i++) x[i] = a * x[i] + b * y[i];
}

// ---- table builders ------------------------------------------------------------------------

// A sequence segment of the Qwen-Image layout: a text run of `len` rows, or an image of ih x iw rows.
struct QwenSeg {
  int32_t is_text;
  int32_t pad;
  int64_t len, ih, iw;
};

// src/models/qwen_image/dit.cpp:151-185.  segs lists the prefix runs in order; the target image
// (H x W) comes last, as `image(H, W)` does at :181.  cos/sin: fp32 [S, sum(axes)/2].
// Returns the number of rows written.
int64_t or_qwen_rope_table(const QwenSeg* segs, int n_segs, const int32_t* axes, float theta, float* hc, float* hs) {
  std::vector<float> invf;
  for (int a = 0; a < 3; a++)
    for (int j = 0; j < axes[a] / 2; j++) invf.push_back(1.0f / std::pow(theta, float(2 * j) / float(axes[a])));
  const int pairs = int(invf.size());
  const int p0 = axes[0] / 2, p1 = p0 + axes[1] / 2;
  auto put = [&](int64_t s, int64_t f, int64_t h, int64_t w) {
    for (int p = 0; p < pairs; p++) {
      int64_t pos = p < p0 ? f : p < p1 ? h : w;
      float ang = float(pos) * invf[p];
      hc[s * pairs + p] = std::cos(ang);
      hs[s * pairs + p] = std::sin(ang);
    }
  };
  int64_t position = 0, row = 0;
  for (int i = 0; i < n_segs; i++) {
    if (segs[i].is_text) {
      for (int64_t k = 0; k < segs[i].len; k++, position++) put(row++, position, position, position);
    } else {
      const int64_t ih = segs[i].ih, iw = segs[i].iw;
      for (int64_t r = 0; r < ih; r++)
        for (int64_t col = 0; col < iw; col++) put(row++, position, r - (ih - ih / 2), col - (iw - iw / 2));
      position += std::max(ih, iw);
    }
  }
  return row;
}

// src/models/minimax_h3/layout.cpp:15-21
static std::vector<double> spatial_grid(int64_t dim, double sqrt_area) {
  double ratio = double(dim) / sqrt_area, left = (1.0 - ratio) / 2.0;
  int64_t n = dim / 2;
  std::vector<double> g(n);
  for (int64_t k = 0; k < n; k++) g[k] = (left + ratio * double(k) / double(n)) * 32.0;
  return g;
}

// Rotary positions of the first/last-frame layout, src/models/minimax_h3/layout.cpp:68-118:
// rows = T text | n_anchors condition frames | 2A audio | F_lat video frames, each frame
// (H/2) x (W/2) rows.  anchors[i]: 0 = "first", 1 = "last".  positions: fp32 [S, 3].
// Returns S.
int64_t or_h3_positions(int64_t T, int64_t F_lat, int64_t H, int64_t W, int64_t A, const int32_t* anchors, int n_anchors,
                        float* positions) {
  const int64_t rpf = (H / 2) * (W / 2);
  const int64_t cond = int64_t(n_anchors) * rpf, audio = 2 * A, video = F_lat * rpf;
  const int64_t S = T + cond + audio + video;
  auto set = [&](int64_t r, double t, double h, double w) {
    positions[r * 3] = float(t), positions[r * 3 + 1] = float(h), positions[r * 3 + 2] = float(w);
  };
  for (int64_t i = 0; i < T; i++) set(i, double(i), 0, 0);
  const double sa = std::sqrt(double(H * W));
  auto hg = spatial_grid(H, sa), wg = spatial_grid(W, sa);
  static const int per_latent[5] = {1, 4, 4, 4, 4};
  std::vector<double> ft(F_lat);
  double acc = double(T), total = 0;
  for (int64_t f = 0; f < F_lat; f++) {
    ft[f] = acc;
    double span = (5.0 / 3.0) * per_latent[f % 5];
    acc += span;
    total += span;
  }
  auto frame_rows = [&](int64_t r0, double t) {
    for (int64_t y = 0; y < H / 2; y++)
      for (int64_t x = 0; x < W / 2; x++) set(r0 + y * (W / 2) + x, t, hg[y], wg[x]);
  };
  for (int i = 0; i < n_anchors; i++) {
    double t = anchors[i] == 0 ? double(T) : double(T) + total - 5.0 / 3.0;
    frame_rows(T + int64_t(i) * rpf, t);
  }
  const int64_t audio_start = T + cond, video_start = T + cond + audio;
  for (int64_t c = 0; c < 2; c++)
    for (int64_t a = 0; a < A; a++) set(audio_start + c * A + a, double(T) + double(a), 0, c == 0 ? wg.front() : wg.back());
  for (int64_t f = 0; f < F_lat; f++) frame_rows(video_start + f * rpf, ft[f]);
  return S;
}

// src/models/minimax_h3/layout.cpp:121-188 (h3_build_ref2va_layout), positions only.
// rows = T text | reference blocks in request order | 2A target audio | F_lat target video frames.
// Reference i: kind[i] 0 image, 1 video, 2 audio; frames/h/w = latent geometry (image, video);
// audio[i] = audio latents per channel (audio reference, or a video's sound track, whose rows come
// before the video's rows and share its start time).  One shared clock starts at T; an image takes
// one unit, an audio reference its length, a video the longer of its track and its frame spans.
// positions may be null to query S.  Returns S.
int64_t or_h3_ref2va_positions(int64_t T, int n_refs, const int32_t* kind, const int64_t* frames, const int64_t* rh,
                               const int64_t* rw, const int64_t* audio, int64_t F_lat, int64_t H, int64_t W, int64_t A,
                               float* positions) {
  static const int per_latent[5] = {1, 4, 4, 4, 4};
  const double rescale = 5.0 / 3.0;
  std::vector<double> pos;  // t, h, w triples
  auto push = [&](double t, double h, double w) { pos.push_back(t), pos.push_back(h), pos.push_back(w); };
  for (int64_t i = 0; i < T; i++) push(double(i), 0, 0);
  struct Grid {
    std::vector<double> h, w;
  };
  auto grid = [&](int64_t gh, int64_t gw) {
    const double sa = std::sqrt(double(gh * gw));
    return Grid{spatial_grid(gh, sa), spatial_grid(gw, sa)};
  };
  auto video_rows = [&](const Grid& g, int64_t nf, double t0, bool image) {
    double t = t0;
    for (int64_t f = 0; f < nf; f++) {
      for (double h : g.h)
        for (double w : g.w) push(t, h, w);
      if (!image) t += rescale * per_latent[f % 5];
    }
  };
  auto audio_rows = [&](int64_t n, double t0, const Grid& g) {
    for (int c = 0; c < 2; c++)
      for (int64_t a = 0; a < n; a++) push(t0 + double(a), 0, c == 0 ? g.w.front() : g.w.back());
  };
  const Grid target = grid(H, W);
  double clock = double(T);
  for (int i = 0; i < n_refs; i++) {
    if (kind[i] == 2) {
      audio_rows(audio[i], clock, target);
      clock += double(audio[i]);
      continue;
    }
    const Grid g = grid(rh[i], rw[i]);
    if (kind[i] == 0) {
      video_rows(g, 1, clock, true);
      clock += 1.0;
      continue;
    }
    if (audio[i] > 0) audio_rows(audio[i], clock, g);
    video_rows(g, frames[i], clock, false);
    double span = 0;
    for (int64_t f = 0; f < frames[i]; f++) span += rescale * per_latent[f % 5];
    clock += std::max(double(audio[i]), span);
  }
  audio_rows(A, clock, target);
  video_rows(target, F_lat, clock, false);
  const int64_t S = int64_t(pos.size() / 3);
  if (positions)
    for (size_t i = 0; i < pos.size(); i++) positions[i] = float(pos[i]);
  return S;
}

// src/models/minimax_h3/dit.cpp:254-262: entry [s, a*nf + j] = cosf/sinf(positions[s, a] * inv_freq[j]).
void or_h3_rope_table(const float* positions, int64_t S, const float* inv_freq, int nf, float* hc, float* hs) {
  const int64_t half = 3 * int64_t(nf);
  for (int64_t s = 0; s < S; s++)
    for (int a = 0; a < 3; a++)
      for (int j = 0; j < nf; j++) {
        float ang = positions[s * 3 + a] * inv_freq[j];
        hc[s * half + a * nf + j] = std::cos(ang);
        hs[s * half + a * nf + j] = std::sin(ang);
      }
}

// src/models/qwen_image/dit.cpp:219-230; out fp32 [2, 256]
void or_qwen_timestep_embedding(float t, float* emb) {
  const int half = 128;
  float ts[2] = {round_bf16(t) * 1000.f, 0.f};
  for (int r = 0; r < 2; r++)
    for (int i = 0; i < half; i++) {
      float f = std::exp(-std::log(10000.f) * float(i) / float(half));
      float arg = ts[r] * f;
      emb[r * 256 + i] = round_bf16(std::cos(arg));
      emb[r * 256 + half + i] = round_bf16(std::sin(arg));
    }
}

// src/models/minimax_h3/dit.cpp:166-179
void or_h3_time_basis(const float* ts, int64_t nt, const float* table, int64_t grid, int64_t basis, float* out) {
  for (int64_t i = 0; i < nt; i++) {
    float pos = std::clamp(ts[i], 0.f, 1.f) * float(grid - 1);
    int64_t lo = std::min<int64_t>(int64_t(std::floor(pos)), grid - 2);
    float fr = pos - float(lo);
    for (int64_t j = 0; j < basis; j++) {
      float a = table[lo * basis + j], b = table[(lo + 1) * basis + j];
      out[i * basis + j] = a + (b - a) * fr;
    }
  }
}

}  // extern "C"

// ---- activation block-scale quantiser (src/kernels/blockscale.cu:39-129) ----------------------
//
// e4m3 (4 exponent bits, bias 7, 3 mantissa bits, no infinity, 0x7f = NaN, largest finite 448):
// round to nearest even, saturate to +-448 - what __nv_cvt_float_to_fp8(x, __NV_SATFINITE, __NV_E4M3)
// of cuda_fp8.h returns, which the reference calls at blockscale.cu:100 and :122.
static uint8_t f32_to_e4m3_satfinite(float f) {
  uint32_t u;
  memcpy(&u, &f, 4);
  const uint8_t sign = uint8_t((u >> 24) & 0x80u);
  const double a = std::fabs(double(f));
  if (a != a) return 0x7f;
  if (a >= 464.0) return sign | 0x7e;  // the midpoint 464 ties to the even 480, which saturates
  if (a < 0.015625) {                  // below 2^-6: multiples of 2^-9; 8 of them is the first normal
    return sign | uint8_t(std::nearbyint(a * 512.0));
  }
  int ex;
  const double m = std::frexp(a, &ex);  // a = m 2^ex, m in [0.5, 1)
  int E = ex - 1;
  int mant = int(std::nearbyint((2.0 * m - 1.0) * 8.0));
  if (mant == 8) mant = 0, E++;
  const int code = ((E + 7) << 3) | mant;
  return sign | uint8_t(code > 0x7e ? 0x7e : code);
}

static float e4m3_to_f32(uint8_t b) {
  const int E = (b >> 3) & 15, m = b & 7;
  if (E == 15 && m == 7) return NAN;
  const float mag = E == 0 ? std::ldexp(float(m), -9) : std::ldexp(1.f + float(m) / 8.f, E - 7);
  return (b & 0x80) ? -mag : mag;
}

// src/kernels/blockscale.cu:39-43
static uint32_t e2m1_code(float x) {
  const float a = std::fabs(x);
  const uint32_t c = (a > 0.25f) + (a >= 0.75f) + (a > 1.25f) + (a >= 1.75f) + (a > 2.5f) + (a >= 3.5f) + (a > 5.f);
  return c | (x < 0.f ? 8u : 0u);
}

static inline int64_t pad_to(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Offset of the scale of (row r, scale block kb) in the 128 x 4 interleaved layout
// (src/kernels/blockscale.cu:83 and :127).
static inline int64_t sf_offset(int64_t r, int64_t kb, int64_t nkb_pad) {
  return (r / 128) * nkb_pad * 128 + (r % 32) * 16 + (r % 128) / 32 * 4 + (kb / 4) * 512 + kb % 4;
}

extern "C" {

uint8_t or_f32_to_e4m3(float f) { return f32_to_e4m3_satfinite(f); }
float or_e4m3_to_f32(uint8_t b) { return e4m3_to_f32(b); }
int64_t or_qscale_bytes(int mode, int64_t rows, int64_t K) { return pad_to(rows, 128) * pad_to(K / (mode == 2 ? 16 : 32), 4); }
int64_t or_sf_offset(int64_t r, int64_t kb, int64_t nkb_pad) { return sf_offset(r, kb, nkb_pad); }

// mode 1 MXFP8, 2 NVFP4.  x: bf16 bits [rows, ldx]; q, sf as the reference's QMat; amax: one float
// (NVFP4 only).  The scale buffer is cleared first, padding included (blockscale.cu:154).
void or_quantize_blockscaled(int mode, const uint16_t* x, int64_t ldx, int64_t rows, int64_t K, uint8_t* q, uint8_t* sf,
                             float* amax) {
  const int V = mode == 2 ? 16 : 32;
  const int64_t nb = K / V, nkb_pad = pad_to(nb, 4);
  memset(sf, 0, size_t(or_qscale_bytes(mode, rows, K)));
  float g = 1.f, inv6g = 1.f;
  if (mode == 2) {
    float am = 0.f;  // blockscale.cu:47-70
    for (int64_t r = 0; r < rows; r++)
      for (int64_t k = 0; k < K; k++) am = std::fmax(am, std::fabs(bf2f(x[r * ldx + k])));
    *amax = am;
    g = am > 0.f ? am / (6.f * 448.f) : 1.f;  // blockscale.cu:79
    inv6g = 1.f / (6.f * g);
  }
  parallel_rows(rows, [=](int64_t r0, int64_t r1) {
    float v[32];
    for (int64_t r = r0; r < r1; r++)
      for (int64_t kb = 0; kb < nb; kb++) {
        float bmax = 0.f;
        for (int j = 0; j < V; j++) {
          v[j] = bf2f(x[r * ldx + kb * V + j]);
          bmax = std::fmax(bmax, std::fabs(v[j]));
        }
        uint8_t sbyte;
        if (mode == 2) {  // blockscale.cu:99-109
          const uint8_t se = f32_to_e4m3_satfinite(bmax * inv6g);
          const float sd = e4m3_to_f32(se) * g;
          const float inv = sd > 0.f ? 1.f / sd : 0.f;
          uint8_t* dst = q + (r * K + kb * V) / 2;
          for (int j = 0; j < 16; j += 2)
            dst[j / 2] = uint8_t(e2m1_code(v[j] * inv) | (e2m1_code(v[j + 1] * inv) << 4));
          sbyte = se;
        } else {  // blockscale.cu:111-125
          int e = -127;
          if (bmax > 0.f) {
            int ex;
            const float mant = std::frexp(bmax / 448.f, &ex);
            e = mant == 0.5f ? ex - 1 : ex;
            e = std::max(-127, std::min(127, e));
          }
          const float inv = std::ldexp(1.f, -e);
          for (int j = 0; j < 32; j++) q[r * K + kb * V + j] = f32_to_e4m3_satfinite(v[j] * inv);
          sbyte = uint8_t(e + 127);
        }
        sf[sf_offset(r, kb, nkb_pad)] = sbyte;
      }
  });
}

// Decodes a quantised matrix back to fp32 [rows, K] (what the block-scaled GEMM multiplies by):
// the test-side inverse, after the reference's own host decoder (tests/blockscale_test.cpp:25-52).
void or_dequantize_blockscaled(int mode, const uint8_t* q, const uint8_t* sf, float amax, int64_t rows, int64_t K, float* out) {
  static const float kE2m1[8] = {0.f, 0.5f, 1.f, 1.5f, 2.f, 3.f, 4.f, 6.f};
  const int V = mode == 2 ? 16 : 32;
  const int64_t nkb_pad = pad_to(K / V, 4);
  const float g = mode == 2 ? (amax > 0.f ? amax / (6.f * 448.f) : 1.f) : 1.f;
  for (int64_t r = 0; r < rows; r++)
    for (int64_t k = 0; k < K; k++) {
      const uint8_t sb = sf[sf_offset(r, k / V, nkb_pad)];
      if (mode == 2) {
        const uint8_t byte = q[(r * K + k) / 2];
        const uint32_t c = (k & 1) ? byte >> 4 : byte & 15;
        const float mag = kE2m1[c & 7] * e4m3_to_f32(sb) * g;
        out[r * K + k] = (c & 8) ? -mag : mag;
      } else {
        out[r * K + k] = e4m3_to_f32(q[r * K + k]) * std::ldexp(1.f, int(sb) - 127);
      }
    }
}

}  // extern "C"

// ---- latent layout either side of the DiT -------------------------------------------------------
// The reference's tests hold the CPU formulas these restate: tests/qwen_latent_test.cpp:30-46 (every
// step rounded on its own: `volatile float delta = x - mean; expected = delta / scale`, and
// `product = x * scale; expected = product + mean`) and tests/h3_latent_test.cpp:25-36 (pure index
// maps).  This file is compiled with -ffp-contract=off, so the two-step forms below round twice.
extern "C" {

void or_qwen_latent_encode(const float* x, float* y, int64_t n, const float* mean, const float* sd) {
  for (int64_t p = 0; p < n; p++)
    for (int c = 0; c < 64; c++) {
      const float delta = x[int64_t(c) * n + p] - mean[c];
      y[p * 64 + c] = delta / sd[c];
    }
}

void or_qwen_latent_decode(const float* x, float* y, int64_t n, const float* mean, const float* sd) {
  for (int c = 0; c < 64; c++)
    for (int64_t p = 0; p < n; p++) {
      const float product = x[p * 64 + c] * sd[c];
      y[int64_t(c) * n + p] = product + mean[c];
    }
}

void or_h3_latent_video(const float* rows, float* z, int64_t F, int64_t H, int64_t W) {
  for (int64_t f = 0; f < F; f++)
    for (int64_t y = 0; y < H / 2; y++)
      for (int64_t x = 0; x < W / 2; x++)
        for (int ch = 0; ch < 24; ch++)
          for (int ph = 0; ph < 2; ph++)
            for (int pw = 0; pw < 2; pw++) {
              const int64_t row = (f * (H / 2) + y) * (W / 2) + x;
              z[((ch * F + f) * H + 2 * y + ph) * W + 2 * x + pw] = rows[row * 96 + ch * 4 + ph * 2 + pw];
            }
}

void or_h3_latent_audio(const float* rows, float* z, int64_t A) {
  for (int ch = 0; ch < 2; ch++)
    for (int64_t a = 0; a < A; a++)
      for (int k = 0; k < 32; k++) z[(ch * 32 + k) * A + a] = rows[(ch * A + a) * 32 + k];
}

}  // extern "C"

