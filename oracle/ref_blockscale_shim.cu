// C entry point over the REFERENCE's activation quantiser, so that tests can call the reference's
// own kernel (src/kernels/blockscale.cu, compiled from the reference tree by oracle/Makefile).
// Test infrastructure only.
#include <cstdint>
#include <exception>
#include <string>

#include "kernels/blockscale.h"

static thread_local std::string g_err;

extern "C" {

const char* ref_bs_last_error() { return g_err.c_str(); }

int64_t ref_qscale_bytes(int mode, int64_t rows, int64_t K) {
  return mx::qscale_bytes(mode == 2 ? mx::QMode::NVFP4 : mx::QMode::MXFP8, rows, K);
}

int ref_quantize_blockscaled(int mode, const void* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf,
                             float* amax, void* stream) {
  try {
    mx::QMat out{q, sf, amax};
    mx::quantize_blockscaled(mode == 2 ? mx::QMode::NVFP4 : mx::QMode::MXFP8, static_cast<const mx::bf16*>(x), ldx, rows,
                             K, out, static_cast<cudaStream_t>(stream));
    return 0;
  } catch (const std::exception& e) {
    g_err = e.what();
    return -1;
  }
}

}  // extern "C"
