// mx_latent.h - drop-in for the reference's src/kernels/qwen_latent.h and src/kernels/h3_latent.h: the same
// `namespace mx::qwen_latent` / `mx::h3_latent` signatures (qwen_latent.h:7-8, h3_latent.h:6-7), implemented by
// calls into libmxk's C ABI.  A non-zero status becomes std::runtime_error carrying mxk_last_error(), which is
// what the reference's MX_CHECK throws for the same bad arguments (qwen_latent.cu:43, h3_latent.cu:21-22,26).
// Header-only; link with -lmxk.
#pragma once

#include <cstdint>
#include <stdexcept>

#include <cuda_runtime.h>

#include "mxk.h"

namespace mx {
namespace latent_detail {
inline void ok(int status) {
  if (status != MXK_OK) throw std::runtime_error(mxk_last_error());
}
}  // namespace latent_detail

namespace qwen_latent {
// encode: [64, N] -> [N, 64], (x - mean) / std.  decode: [N, 64] -> [64, N], x * std + mean.
inline void encode(const float* x, float* y, int64_t n, const float* mean, const float* std, cudaStream_t stream) {
  latent_detail::ok(mxk_qwen_latent_encode(x, y, n, mean, std, stream));
}
inline void decode(const float* x, float* y, int64_t n, const float* mean, const float* std, cudaStream_t stream) {
  latent_detail::ok(mxk_qwen_latent_decode(x, y, n, mean, std, stream));
}
}  // namespace qwen_latent

namespace h3_latent {
inline void video(const float* rows, float* z, int64_t frames, int64_t h, int64_t w, cudaStream_t stream) {
  latent_detail::ok(mxk_h3_latent_video(rows, z, frames, h, w, stream));
}
inline void audio(const float* rows, float* z, int64_t samples, cudaStream_t stream) {
  latent_detail::ok(mxk_h3_latent_audio(rows, z, samples, stream));
}
}  // namespace h3_latent
}  // namespace mx
