// Latent layout kernels either side of the DiT (reference: src/kernels/qwen_latent.cu:7-57,
// src/kernels/h3_latent.cu:5-30): channel-first <-> token-row transposes, with the Qwen latent
// statistics applied in the reference's exact operation order (no contraction, IEEE division).
// A few megabytes per call, so these are about coalescing both sides through shared memory, not about
// pipelining: every global access of a warp is one contiguous segment.
#include "common.cuh"

namespace mxk {
namespace {

constexpr int kLatC = 64;    // Qwen latent channels after 2x2 packing (qwen_latent.h:6-8)
constexpr int kPosTile = 32;  // positions per CTA

// ENCODE: x [64, n] -> y [n, 64], (x - mean[c]) / std[c].  DECODE: x [n, 64] -> y [64, n], x * std[c] + mean[c].
template <bool ENCODE>
__global__ void __launch_bounds__(256) qwen_latent_kernel(const float* __restrict__ x, float* __restrict__ y, int64_t n,
                                                           const float* __restrict__ mean, const float* __restrict__ sd) {
  __shared__ float tile[kLatC][kPosTile + 1];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;  // 8 warps
  const int64_t p0 = int64_t(blockIdx.x) * kPosTile;
  if (ENCODE) {
    // load: a warp reads 32 consecutive positions of one channel; store: 64 consecutive channels of a position
    for (int c = warp; c < kLatC; c += 8) {
      const int64_t p = p0 + lane;
      if (p < n) tile[c][lane] = __fdiv_rn(__fsub_rn(x[int64_t(c) * n + p], mean[c]), sd[c]);
    }
    __syncthreads();
    for (int i = warp; i < kPosTile; i += 8) {
      const int64_t p = p0 + i;
      if (p < n) {
        y[p * kLatC + lane] = tile[lane][i];
        y[p * kLatC + 32 + lane] = tile[32 + lane][i];
      }
    }
  } else {
    for (int i = warp; i < kPosTile; i += 8) {
      const int64_t p = p0 + i;
      if (p < n) {
        tile[lane][i] = __fadd_rn(__fmul_rn(x[p * kLatC + lane], sd[lane]), mean[lane]);
        tile[32 + lane][i] = __fadd_rn(__fmul_rn(x[p * kLatC + 32 + lane], sd[32 + lane]), mean[32 + lane]);
      }
    }
    __syncthreads();
    for (int c = warp; c < kLatC; c += 8) {
      const int64_t p = p0 + lane;
      if (p < n) y[int64_t(c) * n + p] = tile[c][lane];
    }
  }
}

constexpr int kVidC = 24, kVidRow = 96;  // 24 channels x 2 x 2 patch per DiT row (h3_latent.cu:9-10)
constexpr int kVidChunk = 32;            // DiT rows (output column pairs) per pass

// One CTA per (frame t, patch line yh): the line's w/2 DiT rows are contiguous in `rows`; they pass
// through shared memory in chunks and leave as 48 contiguous output lines (24 channels x 2 patch rows).
__global__ void __launch_bounds__(256) h3_video_kernel(const float* __restrict__ rows, float* __restrict__ z, int64_t f,
                                                        int64_t h, int64_t w) {
  __shared__ float tile[kVidChunk][kVidRow + 1];
  const int64_t hw = w / 2, line = blockIdx.x;  // line = t * (h / 2) + yh
  const int64_t t = line / (h / 2), yh = line - t * (h / 2);
  const float* src = rows + line * hw * kVidRow;
  for (int64_t x0 = 0; x0 < hw; x0 += kVidChunk) {
    const int nrow = int(hw - x0 < kVidChunk ? hw - x0 : kVidChunk);
    for (int i = threadIdx.x; i < nrow * kVidRow; i += blockDim.x) tile[i / kVidRow][i % kVidRow] = src[x0 * kVidRow + i];
    __syncthreads();
    // output line (c, ph): 2 * nrow consecutive floats
    const int per_line = 2 * nrow;
    for (int i = threadIdx.x; i < kVidC * 2 * per_line; i += blockDim.x) {
      const int l = i / per_line, xo = i - l * per_line;  // l = c * 2 + ph
      const int c = l >> 1, ph = l & 1;
      z[((int64_t(c) * f + t) * h + 2 * yh + ph) * w + 2 * x0 + xo] = tile[xo >> 1][c * 4 + ph * 2 + (xo & 1)];
    }
    __syncthreads();
  }
}

// z [2, 32, a] <- rows [2 * a, 32]: a 32 x 32 tile transpose per CTA (h3_latent.cu:12-17).
__global__ void __launch_bounds__(256) h3_audio_kernel(const float* __restrict__ rows, float* __restrict__ z, int64_t a) {
  __shared__ float tile[32][33];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t t0 = int64_t(blockIdx.x) * 32, ch = blockIdx.y;
  for (int i = warp; i < 32; i += 8)
    if (t0 + i < a) tile[i][lane] = rows[(ch * a + t0 + i) * 32 + lane];
  __syncthreads();
  for (int c = warp; c < 32; c += 8)
    if (t0 + lane < a) z[(ch * 32 + c) * a + t0 + lane] = tile[lane][c];
}

}  // namespace
}  // namespace mxk

using namespace mxk;

namespace {
int qwen_latent(const char* name, bool encode, const float* x, float* y, int64_t n, const float* mean, const float* sd,
                mxk_stream_t stream) {
  // the reference's own check (src/kernels/qwen_latent.cu:43)
  if (!x || !y || !mean || !sd || n <= 0) return fail(MXK_ERR_INVALID_ARG, "%s: null pointer or n <= 0", name);
  const int64_t grid = ceil_div(n, kPosTile);
  if (grid > 0x7fffffff) return fail(MXK_ERR_TOO_LARGE, "%s: n=%lld too large", name, (long long)n);
  if (encode) qwen_latent_kernel<true><<<unsigned(grid), 256, 0, as_stream(stream)>>>(x, y, n, mean, sd);
  else qwen_latent_kernel<false><<<unsigned(grid), 256, 0, as_stream(stream)>>>(x, y, n, mean, sd);
  return after_launch(name);
}
}  // namespace

extern "C" {

int mxk_qwen_latent_encode(const float* x, float* y, int64_t n, const float* mean, const float* std, mxk_stream_t stream) {
  return qwen_latent("qwen_latent_encode", true, x, y, n, mean, std, stream);
}

int mxk_qwen_latent_decode(const float* x, float* y, int64_t n, const float* mean, const float* std, mxk_stream_t stream) {
  return qwen_latent("qwen_latent_decode", false, x, y, n, mean, std, stream);
}

int mxk_h3_latent_video(const float* rows, float* z, int64_t frames, int64_t h, int64_t w, mxk_stream_t stream) {
  // the reference's own check (src/kernels/h3_latent.cu:21-22)
  if (!rows || !z || frames <= 0 || h <= 0 || w <= 0 || h % 2 || w % 2)
    return fail(MXK_ERR_INVALID_ARG, "h3_latent_video: null pointer, non-positive or odd extent");
  const int64_t lines = frames * (h / 2);
  if (lines > 0x7fffffff) return fail(MXK_ERR_TOO_LARGE, "h3_latent_video: %lld lines", (long long)lines);
  h3_video_kernel<<<unsigned(lines), 256, 0, as_stream(stream)>>>(rows, z, frames, h, w);
  return after_launch("h3_latent_video");
}

int mxk_h3_latent_audio(const float* rows, float* z, int64_t samples, mxk_stream_t stream) {
  if (!rows || !z || samples <= 0) return fail(MXK_ERR_INVALID_ARG, "h3_latent_audio: null pointer or samples <= 0");
  const int64_t gx = ceil_div(samples, 32);
  if (gx > 0x7fffffff) return fail(MXK_ERR_TOO_LARGE, "h3_latent_audio: %lld samples", (long long)samples);
  h3_audio_kernel<<<dim3(unsigned(gx), 2), 256, 0, as_stream(stream)>>>(rows, z, samples);
  return after_launch("h3_latent_audio");
}

}  // extern "C"
