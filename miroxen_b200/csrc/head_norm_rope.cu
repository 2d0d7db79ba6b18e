// head_norm_rope: per-head RMSNorm + rotary embedding + gather into [S, H, D]
// (reference: src/kernels/ops.cu:87-119 kernel, 197-210 launcher).
//
// For token s and head h:  v[d] = in[s*in_stride + col0 + h*D + d];  with norm_w:
// v = v * rsqrtf(mean_D(v^2) + eps) * norm_w[d];  for d < rot the value is rotated with its pair
// partner, (a, b) -> (a c - b s, a s + b c), pairs being (2i, 2i+1) in interleaved mode and
// (i, i + rot/2) in half mode, c/s = cos/sin[s*rot/2 + pair]; nothing is rounded between the
// norm and the rotation.
//
// Work layout of the fast kernel: a head is held by LPH = D/8 lanes, 8 consecutive channels
// (one 128-bit load) per lane.  A token is shared by `gpt` such lane groups; each group walks
// the heads gh, gh + gpt, ... of every tensor of the launch (q, k, v) with the token's cos/sin
// values in registers, so the table row is fetched once per token per group, not once per head.
#include "common.cuh"
#include "tuning.h"

namespace mxk {
namespace {

constexpr int kMaxTensors = 3;
constexpr int kHeadsInFlight = 4;  // independent 128-bit loads each lane issues per batch

struct RopeArgs {
  MxkHeadTensor t[kMaxTensors];
  int n_tensors;
  int64_t S;
  int H, D;
  float eps;
  const float* cos;
  const float* sin;
  int gpt;              // lane groups per token
  int tokens_per_pass;  // tokens a CTA holds at once
};

template <int LPH>
__global__ void __launch_bounds__(512) head_rope_kernel(const RopeArgs a) {
  constexpr int U = kHeadsInFlight;
  const int lane = threadIdx.x & 31;
  const int l = threadIdx.x % LPH;  // lane within the head: channels 8l .. 8l+7
  const int group = threadIdx.x / LPH;
  const int slot = group / a.gpt, gh = group % a.gpt;
  const bool slot_on = slot < a.tokens_per_pass;
  const int group_base = lane & ~(LPH - 1);
  const float inv_d = 1.f / float(a.D);
  (void)inv_d;

  for (int64_t s0 = int64_t(blockIdx.x) * a.tokens_per_pass; s0 < a.S;
       s0 += int64_t(gridDim.x) * a.tokens_per_pass) {
    const int64_t s = s0 + slot;
    const bool tok_on = slot_on && s < a.S;
    int cur_rot = -1, cur_mode = -1;
    float cs[8], sn[8];
    int partner = lane;
    bool rotates = false;
#pragma unroll 1
    for (int ti = 0; ti < a.n_tensors; ti++) {
      const MxkHeadTensor& t = a.t[ti];
      const int rot = t.mode == MXK_ROPE_NONE ? 0 : t.rot;
      if (rot != cur_rot || t.mode != cur_mode) {
        cur_rot = rot, cur_mode = t.mode;
        const int half = rot >> 1;
        rotates = 8 * l < rot;
        partner = lane;
        if (rotates && tok_on) {
          const float* cr = a.cos + s * half;
          const float* sr = a.sin + s * half;
          if (t.mode == MXK_ROPE_INTERLEAVED) {
            // channels 8l..8l+7 are pairs 4l..4l+3; even channels take -sin, odd ones +sin
            float4 c = *reinterpret_cast<const float4*>(cr + 4 * l);
            float4 q = *reinterpret_cast<const float4*>(sr + 4 * l);
            cs[0] = cs[1] = c.x, cs[2] = cs[3] = c.y, cs[4] = cs[5] = c.z, cs[6] = cs[7] = c.w;
            sn[0] = -q.x, sn[1] = q.x, sn[2] = -q.y, sn[3] = q.y;
            sn[4] = -q.z, sn[5] = q.z, sn[6] = -q.w, sn[7] = q.w;
          } else {
            const int hl = half >> 3;  // lanes per half
            const bool first = l < hl;
            const int lp = first ? l : l - hl;
            float4 c0 = *reinterpret_cast<const float4*>(cr + 8 * lp);
            float4 c1 = *reinterpret_cast<const float4*>(cr + 8 * lp + 4);
            float4 q0 = *reinterpret_cast<const float4*>(sr + 8 * lp);
            float4 q1 = *reinterpret_cast<const float4*>(sr + 8 * lp + 4);
            cs[0] = c0.x, cs[1] = c0.y, cs[2] = c0.z, cs[3] = c0.w;
            cs[4] = c1.x, cs[5] = c1.y, cs[6] = c1.z, cs[7] = c1.w;
            const float sg = first ? -1.f : 1.f;
            sn[0] = sg * q0.x, sn[1] = sg * q0.y, sn[2] = sg * q0.z, sn[3] = sg * q0.w;
            sn[4] = sg * q1.x, sn[5] = sg * q1.y, sn[6] = sg * q1.z, sn[7] = sg * q1.w;
          }
        }
        if (rotates && t.mode == MXK_ROPE_HALF) {
          const int hl = half >> 3;
          partner = group_base + (l < hl ? l + hl : l - hl);
        }
      }
      float w[8];
      if (t.norm_w) {
        float4 w0 = *reinterpret_cast<const float4*>(t.norm_w + 8 * l);
        float4 w1 = *reinterpret_cast<const float4*>(t.norm_w + 8 * l + 4);
        w[0] = w0.x, w[1] = w0.y, w[2] = w0.z, w[3] = w0.w;
        w[4] = w1.x, w[5] = w1.y, w[6] = w1.z, w[7] = w1.w;
      }
      const mxk_bf16* src = t.in + s * t.in_stride + t.col0 + 8 * l;
      mxk_bf16* dst = t.out + s * int64_t(a.H) * a.D + 8 * l;
      // Every lane of the CTA runs the same number of iterations (shuffles need whole warps).
      for (int h0 = 0; h0 < a.H; h0 += a.gpt * U) {
        uint4 raw[U];
        bool on[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
          const int h = h0 + gh + u * a.gpt;
          on[u] = tok_on && h < a.H;
          raw[u] = make_uint4(0u, 0u, 0u, 0u);
          if (on[u]) raw[u] = ld_stream(reinterpret_cast<const uint4*>(src + int64_t(h) * a.D));
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
          float v[8];
          unpack8(raw[u], v);
          if (t.norm_w) {
            float ss = 0.f;
#pragma unroll
            for (int i = 0; i < 8; i++) ss += v[i] * v[i];
            ss = group_sum<LPH>(ss);
            const float rstd = rsqrtf(ss / float(a.D) + a.eps);
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = v[i] * rstd * w[i];
          }
          if (cur_mode == MXK_ROPE_INTERLEAVED) {
            if (rotates) {
              float o[8];
#pragma unroll
              for (int i = 0; i < 8; i++) o[i] = v[i] * cs[i] + v[i ^ 1] * sn[i];
#pragma unroll
              for (int i = 0; i < 8; i++) v[i] = o[i];
            }
          } else if (cur_mode == MXK_ROPE_HALF && cur_rot > 0) {
#pragma unroll
            for (int i = 0; i < 8; i++) {
              const float other = __shfl_sync(0xffffffffu, v[i], partner);
              if (rotates) v[i] = v[i] * cs[i] + other * sn[i];
            }
          }
          if (on[u]) {
            const int h = h0 + gh + u * a.gpt;
            st_stream(reinterpret_cast<uint4*>(dst + int64_t(h) * a.D), pack8(v));
          }
        }
      }
    }
  }
}

// Any even D <= 256, any rot, any alignment: one warp per (token, head), the head's values pass
// through shared memory for the partner exchange.
__global__ void __launch_bounds__(256) head_rope_generic_kernel(const RopeArgs a) {
  __shared__ float buf[8][256];
  const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
  float* hv = buf[wid];
  const int64_t total = a.S * a.H;
  for (int64_t item = int64_t(blockIdx.x) * 8 + wid; item < total; item += int64_t(gridDim.x) * 8) {
    const int64_t s = item / a.H;
    const int h = int(item % a.H);
    for (int ti = 0; ti < a.n_tensors; ti++) {
      const MxkHeadTensor& t = a.t[ti];
      const bf16* src = reinterpret_cast<const bf16*>(t.in) + s * t.in_stride + t.col0 + int64_t(h) * a.D;
      bf16* dst = reinterpret_cast<bf16*>(t.out) + (s * a.H + h) * a.D;
      float ss = 0.f;
      for (int d = lane; d < a.D; d += 32) {
        float v = bf16_to_f(src[d]);
        hv[d] = v;
        ss += v * v;
      }
      if (t.norm_w) {
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / float(a.D) + a.eps);
        for (int d = lane; d < a.D; d += 32) hv[d] = hv[d] * rstd * t.norm_w[d];
      }
      __syncwarp();
      const int rot = t.mode == MXK_ROPE_NONE ? 0 : t.rot, half = rot >> 1;
      for (int d = lane; d < a.D; d += 32) {
        float v = hv[d];
        if (d < rot) {
          int pair, idx;
          float other;
          if (t.mode == MXK_ROPE_INTERLEAVED) {
            pair = d >> 1, idx = d & 1, other = hv[d ^ 1];
          } else {
            pair = d < half ? d : d - half, idx = d < half ? 0 : 1;
            other = hv[d < half ? d + half : d - half];
          }
          const float c = a.cos[s * half + pair], si = a.sin[s * half + pair];
          v = idx == 0 ? v * c - other * si : other * si + v * c;
        }
        dst[d] = __float2bfloat16(v);
      }
      __syncwarp();
    }
  }
}

bool fast_ok(const RopeArgs& a) {
  const int D = a.D;
  if (!(D == 32 || D == 64 || D == 128 || D == 256)) return false;
  bool any_rot = false;
  for (int i = 0; i < a.n_tensors; i++) {
    const MxkHeadTensor& t = a.t[i];
    if (!aligned(t.in, 16) || !aligned(t.out, 16) || t.in_stride % 8 || t.col0 % 8) return false;
    if (t.norm_w && !aligned(t.norm_w, 16)) return false;
    if (t.mode == MXK_ROPE_INTERLEAVED && t.rot % 8) return false;
    if (t.mode == MXK_ROPE_HALF && t.rot % 16) return false;
    if (t.mode != MXK_ROPE_NONE && t.rot > 0) any_rot = true;
  }
  if (any_rot && (!aligned(a.cos, 16) || !aligned(a.sin, 16))) return false;
  return true;
}

int run(const char* name, RopeArgs a, cudaStream_t stream) {
  if (fast_ok(a)) {
    const int lph = a.D / 8;
    a.gpt = int(ceil_div(a.H, kHeadsInFlight));
    const int per_token = lph * a.gpt;
    if (per_token <= 512) {
      const int want = tune(TUNE_ROPE_THREADS, 256);
      int tpp = want / per_token;
      if (tpp < 1) tpp = 1;
      int threads = int(ceil_div(int64_t(per_token) * tpp, 32) * 32);
      a.tokens_per_pass = tpp;
      const int per_sm = tune(TUNE_ROPE_CTAS_PER_SM, 2048 / threads > 6 ? 6 : 2048 / threads);
      int64_t grid = ceil_div(a.S, tpp);
      int64_t cap = int64_t(sm_count()) * (per_sm > 0 ? per_sm : 1);
      if (grid > cap) grid = cap;
      switch (lph) {
        case 4: head_rope_kernel<4><<<unsigned(grid), threads, 0, stream>>>(a); break;
        case 8: head_rope_kernel<8><<<unsigned(grid), threads, 0, stream>>>(a); break;
        case 16: head_rope_kernel<16><<<unsigned(grid), threads, 0, stream>>>(a); break;
        default: head_rope_kernel<32><<<unsigned(grid), threads, 0, stream>>>(a); break;
      }
      return after_launch(name);
    }
  }
  int64_t grid = ceil_div(a.S * a.H, 8);
  const int64_t cap = int64_t(sm_count()) * 32;
  if (grid > cap) grid = cap;
  head_rope_generic_kernel<<<unsigned(grid), 256, 0, stream>>>(a);
  return after_launch(name);
}

int check(const char* name, const MxkHeadTensor& t, int H, int D, const float* cos, const float* sin) {
  if (!t.in || !t.out) return fail(MXK_ERR_INVALID_ARG, "%s: null in or out", name);
  if (t.mode != MXK_ROPE_NONE && t.mode != MXK_ROPE_INTERLEAVED && t.mode != MXK_ROPE_HALF)
    return fail(MXK_ERR_INVALID_ARG, "%s: unknown rope mode %d", name, t.mode);
  // the reference's own argument check (src/kernels/ops.cu:201)
  if (!(D > 0 && D % 2 == 0 && D <= 256 && t.rot >= 0 && t.rot <= D && t.rot % 2 == 0))
    return fail(MXK_ERR_INVALID_ARG, "%s: D=%d rot=%d", name, D, t.rot);
  if (H <= 0) return fail(MXK_ERR_INVALID_ARG, "%s: H=%d", name, H);
  if (t.in_stride < 0 || t.col0 < 0) return fail(MXK_ERR_INVALID_ARG, "%s: negative in_stride or col0", name);
  if (t.mode != MXK_ROPE_NONE && t.rot > 0 && (!cos || !sin))
    return fail(MXK_ERR_INVALID_ARG, "%s: rotary mode %d needs cos and sin tables", name, t.mode);
  return MXK_OK;
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int mxk_head_norm_rope(const mxk_bf16* in, int64_t S, int64_t in_stride, int64_t col0, int H,
                       int D, const float* norm_w, float eps, const float* cos, const float* sin,
                       int rot, int mode, mxk_bf16* out, mxk_stream_t stream) {
  if (S <= 0) return MXK_OK;
  RopeArgs a{};
  a.t[0] = MxkHeadTensor{in, in_stride, col0, norm_w, out, rot, mode};
  a.n_tensors = 1;
  a.S = S, a.H = H, a.D = D, a.eps = eps, a.cos = cos, a.sin = sin;
  if (int rc = check("head_norm_rope", a.t[0], H, D, cos, sin)) return rc;
  return run("head_norm_rope", a, as_stream(stream));
}

int mxk_qkv_norm_rope(const MxkHeadTensor* tensors_host, int n_tensors, int64_t S, int H, int D,
                      float eps, const float* cos, const float* sin, mxk_stream_t stream) {
  if (S <= 0 || n_tensors == 0) return MXK_OK;
  if (!tensors_host || n_tensors < 0 || n_tensors > kMaxTensors)
    return fail(MXK_ERR_INVALID_ARG, "qkv_norm_rope: n_tensors=%d (1..%d)", n_tensors, kMaxTensors);
  RopeArgs a{};
  for (int i = 0; i < n_tensors; i++) {
    a.t[i] = tensors_host[i];
    if (int rc = check("qkv_norm_rope", a.t[i], H, D, cos, sin)) return rc;
  }
  a.n_tensors = n_tensors;
  a.S = S, a.H = H, a.D = D, a.eps = eps, a.cos = cos, a.sin = sin;
  return run("qkv_norm_rope", a, as_stream(stream));
}

}  // extern "C"
