// C entry points over the REFERENCE's latent layout kernels (src/kernels/qwen_latent.cu,
// src/kernels/h3_latent.cu, compiled from the reference tree by oracle/Makefile).  Test infrastructure only.
#include <cstdint>
#include <exception>

#include "kernels/h3_latent.h"
#include "kernels/qwen_latent.h"

#define GUARD(call)                  \
  try {                              \
    call;                            \
    return 0;                        \
  } catch (const std::exception&) {  \
    return -1;                       \
  }

extern "C" {
int ref_qwen_latent_encode(const float* x, float* y, int64_t n, const float* mean, const float* sd, void* s) {
  GUARD(mx::qwen_latent::encode(x, y, n, mean, sd, static_cast<cudaStream_t>(s)))
}
int ref_qwen_latent_decode(const float* x, float* y, int64_t n, const float* mean, const float* sd, void* s) {
  GUARD(mx::qwen_latent::decode(x, y, n, mean, sd, static_cast<cudaStream_t>(s)))
}
int ref_h3_latent_video(const float* rows, float* z, int64_t f, int64_t h, int64_t w, void* s) {
  GUARD(mx::h3_latent::video(rows, z, f, h, w, static_cast<cudaStream_t>(s)))
}
int ref_h3_latent_audio(const float* rows, float* z, int64_t a, void* s) {
  GUARD(mx::h3_latent::audio(rows, z, a, static_cast<cudaStream_t>(s)))
}
}
