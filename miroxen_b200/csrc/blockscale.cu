// Activation block-scale quantiser: bf16 [rows, K] -> MXFP8 (e4m3 + one ue8m0 scale per 32) or
// NVFP4 (e2m1 + one e4m3 scale per 16 + a per-tensor fp32 scale), scales in cuBLASLt's 128 x 4
// interleaved layout (reference: src/kernels/blockscale.cu:47-129 kernels, 147-164 launcher;
// declared in src/kernels/blockscale.h:30-43).  It is the step the reference runs on every
// activation right after the norm / activation ops of this library when its fp8 / fp4 path is on
// (src/core/weights.cpp:189-195).
//
// Bit-exactness with the reference's quantiser is the bar (byte outputs), so every float step is the
// reference's: bmax / 448 through an IEEE division and frexpf, exact power-of-two scaling, the
// e4m3 conversion of cuda_fp8.h with saturation, __frcp_rn for the NVFP4 block reciprocal, and
// the same threshold ladder for e2m1.
//
// Work layout: 4 lanes share a 32-element block (2 lanes a 16-element one), one 128-bit vector per
// lane, block maximum by 2 (1) shuffle steps, 64-bit (32-bit) packed stores, so a warp's accesses are
// contiguous segments.  Default path: the bulk-copy streaming pipeline (stream_pipe.cuh) - a producer
// warp lands row pieces of up to 8 KB in shared memory, consumer warps quantise from there; NVFP4's
// tensor maximum is a first pass through the same pipeline.  quant_path = 2 selects plain register
// kernels (also taken when a row piece cannot be cut on a block boundary).
//
// Three steps are computed differently from the reference but give the same bits:
//  - the ue8m0 exponent comes from the bits of the block maximum instead of frexpf(bmax / 448): with
//    bmax = 1.m * 2^E a bf16 value, RN(bmax / 448) = RN(1.m / 1.75) * 2^(E-8); 1.m / 1.75 is within
//    [0.5715, 1.139], equals 1 only for 1.m = 1.75 and is otherwise more than 2^-8 away from 1, so the
//    reference's e is E - 8 when 1.m <= 1.75 and E - 7 above, clamped to [-127, 127];
//  - 2^-e is assembled from its exponent field (exp2f of an integer is exact);
//  - e2m1 codes come from cvt.rn.satfinite.e2m1x2.f32, which rounds to nearest even on the grid
//    {0, .5, 1, 1.5, 2, 3, 4, 6} exactly like the reference's comparison ladder (ties .25 -> 0,
//    .75 -> 1, 1.25 -> 1, 1.75 -> 2, 2.5 -> 2, 3.5 -> 4, 5 -> 4); adding +0 first turns -0 into +0,
//    the one input where the ladder (no sign for -0) and the instruction (sign kept) differ.
#include <cuda_fp8.h>

#include "common.cuh"
#include "stream_pipe.cuh"
#include "tuning.h"

namespace mxk {
namespace {

constexpr float kFp4Range = 6.f * 448.f;  // src/kernels/blockscale.cu:33
constexpr int kRowsInFlight = 4;

__device__ __forceinline__ void st_stream32(unsigned int* p, unsigned int v) { __stcs(p, v); }

__host__ __device__ inline int64_t pad_to(int64_t v, int64_t m) { return (v + m - 1) / m * m; }

// Two floats -> two e4m3 bytes (x in the low byte), round to nearest even, saturating.
__device__ __forceinline__ uint32_t e4m3x2(float x, float y) {
  return __nv_cvt_float2_to_fp8x2(make_float2(x, y), __NV_SATFINITE, __NV_E4M3);
}

// Eight floats -> eight e2m1 codes, element 0 in the lowest nibble.
__device__ __forceinline__ uint32_t e2m1x8(const float (&v)[8]) {
  uint32_t w;
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3}; }"
      : "=r"(w)
      : "f"(v[0] + 0.f), "f"(v[1] + 0.f), "f"(v[2] + 0.f), "f"(v[3] + 0.f), "f"(v[4] + 0.f), "f"(v[5] + 0.f),
        "f"(v[6] + 0.f), "f"(v[7] + 0.f));
  return w;
}

// The per-tensor constants of NVFP4 (src/kernels/blockscale.cu:79).
struct Fp4Scale {
  float g, inv6g;
};
__device__ __forceinline__ Fp4Scale fp4_scale(const float* amax) {
  // Written by the launch before this one, which may still be running when this grid is scheduled: the
  // load must stay behind the dependency wait, so it is a volatile asm statement on a pointer that
  // carries no no-alias promise the compiler could use to hoist it.
  float am;
  asm volatile("ld.global.cg.f32 %0, [%1];" : "=f"(am) : "l"(amax) : "memory");
  Fp4Scale s;
  s.g = am > 0.f ? __fdiv_rn(am, kFp4Range) : 1.f;
  s.inv6g = __fdiv_rn(1.f, __fmul_rn(6.f, s.g));
  return s;
}

// Quantises the 8 elements of one lane given the maximum of its scale block; returns the scale byte.
// MXFP8: codes in (lo, hi); NVFP4: codes in lo.
template <int MODE>
__device__ __forceinline__ uint8_t quant8(const float (&v)[8], float bmax, const Fp4Scale& fs, uint32_t& lo, uint32_t& hi) {
  if (MODE == 2) {
    // src/kernels/blockscale.cu:100-109
    const __nv_fp8_storage_t se = __nv_cvt_float_to_fp8(__fmul_rn(bmax, fs.inv6g), __NV_SATFINITE, __NV_E4M3);
    __nv_fp8_e4m3 sq;
    sq.__x = se;
    const float sd = __fmul_rn(float(sq), fs.g);
    const float inv = sd > 0.f ? __frcp_rn(sd) : 0.f;
    float t[8];
#pragma unroll
    for (int i = 0; i < 8; i++) t[i] = __fmul_rn(v[i], inv);
    lo = e2m1x8(t);
    hi = 0;
    return se;
  }
  // ue8m0: the smallest 2^e with bmax / 2^e <= 448 (src/kernels/blockscale.cu:111-119), from the bits
  // of bmax (see the head of this file); bmax is a bf16 value, so its low 16 bits are zero.
  const uint32_t b = __float_as_uint(bmax);
  const int E = int(b >> 23);  // biased exponent; 0 for zero and subnormals, whose e clamps to -127
  int e = E - 127 - 8 + ((b & 0x007fffffu) > 0x00600000u ? 1 : 0);
  e = E == 0 ? -127 : max(-127, e);
  // 2^-e: e is in [-127, 120], so -e + 127 is in [7, 254]
  const float inv = __uint_as_float(uint32_t(127 - e) << 23);
  lo = e4m3x2(__fmul_rn(v[0], inv), __fmul_rn(v[1], inv)) | e4m3x2(__fmul_rn(v[2], inv), __fmul_rn(v[3], inv)) << 16;
  hi = e4m3x2(__fmul_rn(v[4], inv), __fmul_rn(v[5], inv)) | e4m3x2(__fmul_rn(v[6], inv), __fmul_rn(v[7], inv)) << 16;
  return uint8_t(e + 127);
}

template <int LPB>
__device__ __forceinline__ float block_max(const float (&v)[8]) {
  float m = 0.f;
#pragma unroll
  for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(v[i]));
#pragma unroll
  for (int o = LPB / 2; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  return m;
}

// Address of the scale of (row r, scale block kb): 128 x 4 tiles of 512 bytes
// (src/kernels/blockscale.cu:83 and :127).
__device__ __forceinline__ int64_t sf_row_offset(int64_t r, int nkb_pad) {
  return (r / 128) * int64_t(nkb_pad) * 128 + (r % 32) * 16 + (r % 128) / 32 * 4;
}
__device__ __forceinline__ int sf_col_offset(int kb) { return (kb >> 2) * 512 + (kb & 3); }

__device__ __forceinline__ void amax_commit(float m, float* out) {
#pragma unroll
  for (int o = 16; o; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  // non-negative floats order like their bit patterns (src/kernels/blockscale.cu:68)
  if ((threadIdx.x & 31) == 0 && m > 0.f) atomicMax(reinterpret_cast<int*>(out), __float_as_int(m));
}

// ---- bulk-copy pipeline ops: chunk = one piece (pieces_per_row of them) of one row ----

struct RowPieces {
  const unsigned char* x;
  int64_t ldx_bytes;
  int K, pieces_per_row, piece_elems;
  __device__ void where(int64_t chunk, int64_t& row, int& k0, int& n) const {
    row = chunk / pieces_per_row;
    k0 = int(chunk - row * pieces_per_row) * piece_elems;
    n = K - k0 < piece_elems ? K - k0 : piece_elems;
  }
  __device__ void locate(int64_t chunk, Chunk& c) const {
    int64_t row;
    int k0, n;
    where(chunk, row, k0, n);
    c.src0 = x + row * ldx_bytes + int64_t(k0) * 2, c.src1 = nullptr, c.dst = nullptr;
    c.bytes = unsigned(n) * 2;
  }
};

struct AmaxPipeOp : RowPieces {
  static constexpr int NSRC = 1;
  float* out;
  struct State {
    float m;
  };
  __device__ State init() const { return State{0.f}; }
  __device__ void consume(State& st, int64_t chunk, const unsigned char* stage, int tid, int n_cons) const {
    int64_t row;
    int k0, n;
    where(chunk, row, k0, n);
    const uint4* s = reinterpret_cast<const uint4*>(stage);
    const int nvec = n >> 3;
    float m = st.m;
    for (int i = tid; i < nvec; i += n_cons) {
      float v[8];
      unpack8(s[i], v);
#pragma unroll
      for (int j = 0; j < 8; j++) m = fmaxf(m, fabsf(v[j]));
    }
    st.m = m;
  }
  __device__ void finish(State& st, int) const { amax_commit(st.m, out); }
};

template <int MODE>
struct QuantPipeOp : RowPieces {
  static constexpr int NSRC = 1;
  static constexpr int V = MODE == 2 ? 16 : 32, LPB = V / 8;
  uint8_t* q;
  uint8_t* sf;
  const float* amax;
  int nkb_pad;
  using State = Fp4Scale;
  __device__ State init() const { return MODE == 2 ? fp4_scale(amax) : Fp4Scale{1.f, 1.f}; }
  __device__ void consume(State& fs, int64_t chunk, const unsigned char* stage, int tid, int n_cons) const {
    constexpr int U = 2;
    int64_t row;
    int k0, n;
    where(chunk, row, k0, n);
    const uint4* s = reinterpret_cast<const uint4*>(stage);
    const int nvec = n >> 3, lane = tid & 31;
    uint8_t* sfr = sf + sf_row_offset(row, nkb_pad);
    uint8_t* qrow = q + (row * K + k0) / (MODE == 2 ? 2 : 1);
    // every lane of a warp runs the same trips (the block maximum is a warp shuffle); a piece holds
    // whole scale blocks, so the lanes of one block are on or off together
    for (int i0 = tid - lane; i0 < nvec; i0 += U * n_cons) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int i = i0 + u * n_cons + lane;
        raw[u] = i < nvec ? s[i] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int i = i0 + u * n_cons + lane;
        float v[8];
        unpack8(raw[u], v);
        const float bmax = block_max<LPB>(v);
        uint32_t lo, hi;
        const uint8_t sbyte = quant8<MODE>(v, bmax, fs, lo, hi);
        if (i < nvec) {
          if (MODE == 2) st_stream32(reinterpret_cast<unsigned int*>(qrow) + i, lo);
          else st_stream(reinterpret_cast<uint2*>(qrow) + i, make_uint2(lo, hi));
          if ((lane & (LPB - 1)) == 0) sfr[sf_col_offset((k0 + i * 8) / V)] = sbyte;
        }
      }
    }
  }
  __device__ void finish(State&, int) const {}
};

// ---- register kernels ----

// Whole-tensor absolute maximum (src/kernels/blockscale.cu:47-70), four rows in flight per thread.
__global__ void __launch_bounds__(256) amax_kernel(const bf16* __restrict__ x, int64_t ldx, int64_t rows, int nvec,
                                                    float* out) {
  constexpr int U = kRowsInFlight;
  pdl_launch_dependents();
  pdl_wait();
  float m = 0.f;
  for (int64_t r = int64_t(blockIdx.x) * U; r < rows; r += int64_t(gridDim.x) * U) {
    for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; u++)
        raw[u] = r + u < rows ? ld_stream(reinterpret_cast<const uint4*>(x + (r + u) * ldx) + j) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < U; u++) {
        float f[8];
        unpack8(raw[u], f);
#pragma unroll
        for (int i = 0; i < 8; i++) m = fmaxf(m, fabsf(f[i]));
      }
    }
  }
  amax_commit(m, out);
}

// MODE 1 = MXFP8, 2 = NVFP4.  Thread t of CTA column blockIdx.y owns the 8 elements starting at
// column 8 * (blockIdx.y * blockDim.x + t) of every row it visits.
template <int MODE>
__global__ void __launch_bounds__(256) quant_kernel(const bf16* __restrict__ x, int64_t ldx, int64_t rows, int K,
                                                     uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const float* amax,
                                                     int rows_per_chunk) {
  constexpr int V = MODE == 2 ? 16 : 32;   // elements per scale block
  constexpr int LPB = V / 8;               // lanes per scale block
  constexpr int U = kRowsInFlight;
  pdl_launch_dependents();
  pdl_wait();
  const int vec = blockIdx.y * blockDim.x + threadIdx.x;  // 8-element vector index inside the row
  const bool col_on = vec * 8 < K;
  const int nkb_pad = int(pad_to(K / V, 4));
  const bool leader = (threadIdx.x & (LPB - 1)) == 0;
  const int sf_col = sf_col_offset((vec * 8) / V);
  const Fp4Scale fs = MODE == 2 ? fp4_scale(amax) : Fp4Scale{1.f, 1.f};
  const int64_t nchunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int64_t r0 = c * rows_per_chunk;
    const int64_t r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    for (int64_t rb = r0; rb < r1; rb += U) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; u++) {
        raw[u] = make_uint4(0u, 0u, 0u, 0u);
        if (col_on && rb + u < r1) raw[u] = ld_stream(reinterpret_cast<const uint4*>(x + (rb + u) * ldx) + vec);
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int64_t r = rb + u;
        float v[8];
        unpack8(raw[u], v);
        const float bmax = block_max<LPB>(v);
        uint32_t lo, hi;
        const uint8_t sbyte = quant8<MODE>(v, bmax, fs, lo, hi);
        if (col_on && r < r1) {
          if (MODE == 2) st_stream32(reinterpret_cast<unsigned int*>(q + (r * K + int64_t(vec) * 8) / 2), lo);
          else st_stream(reinterpret_cast<uint2*>(q + r * K + int64_t(vec) * 8), make_uint2(lo, hi));
          if (leader) sf[sf_row_offset(r, nkb_pad) + sf_col] = sbyte;
        }
      }
    }
  }
}

}  // namespace
}  // namespace mxk

using namespace mxk;

extern "C" {

int64_t mxk_qdata_bytes(int mode, int64_t rows, int64_t K) { return rows * K / (mode == MXK_Q_NVFP4 ? 2 : 1); }

int64_t mxk_qscale_bytes(int mode, int64_t rows, int64_t K) {
  return pad_to(rows, 128) * pad_to(K / (mode == MXK_Q_NVFP4 ? 16 : 32), 4);
}

int mxk_quantize_blockscaled(int mode, const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf,
                             float* amax, mxk_stream_t stream) {
  if (mode != MXK_Q_MXFP8 && mode != MXK_Q_NVFP4)
    return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: mode %d is not a quantised mode (1 MXFP8, 2 NVFP4)", mode);
  // the reference's own check (src/kernels/blockscale.cu:151)
  if (K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldx < K || !aligned(x, 16) || K > (int64_t(1) << 30))
    return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: need K %% 32 == 0, ldx %% 8 == 0, ldx >= K, 16-byte aligned input");
  if (rows == 0) return MXK_OK;
  if (rows < 0 || !x || !q || !sf || (mode == MXK_Q_NVFP4 && !amax))
    return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: null buffer or negative rows");
  if (!aligned(q, 8)) return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: q must be 8-byte aligned");
  cudaStream_t s = as_stream(stream);
  const bf16* xb = reinterpret_cast<const bf16*>(x);
  // padded scale rows / columns are read by the GEMM (0xff is NaN in ue8m0): clear everything first
  cudaError_t e = cudaMemsetAsync(sf, 0, size_t(mxk_qscale_bytes(mode, rows, K)), s);
  if (e == cudaSuccess && mode == MXK_Q_NVFP4) e = cudaMemsetAsync(amax, 0, sizeof(float), s);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "quantize_blockscaled: cudaMemsetAsync: %s", cudaGetErrorString(e));
  const int nvec = int(K / 8);
  const int V = mode == MXK_Q_NVFP4 ? 16 : 32;
  // bulk-copy pipeline: rows cut into equal pieces of whole scale blocks, at most one chunk each
  int chunk_bytes = tune(TUNE_STREAM_CHUNK_KB, 8) * 1024;
  if (chunk_bytes > 32 * 1024) chunk_bytes = 32 * 1024;
  const int pieces = int(ceil_div(K * 2, chunk_bytes));
  const int piece_elems = int(ceil_div(ceil_div(K, pieces), 128) * 128);
  if (tune(TUNE_QUANT_PATH, 1) == 1 && piece_elems * 2 <= chunk_bytes) {
    const int ppr = int(ceil_div(K, piece_elems));
    RowPieces rp{reinterpret_cast<const unsigned char*>(x), ldx * 2, int(K), ppr, piece_elems};
    if (mode == MXK_Q_NVFP4) {
      AmaxPipeOp op;
      static_cast<RowPieces&>(op) = rp;
      op.out = amax;
      if (int rc = run_stream_pipe("quantize_blockscaled (amax)", op, rows * ppr, piece_elems * 2, s, 4, 3)) return rc;
      QuantPipeOp<2> qo;
      static_cast<RowPieces&>(qo) = rp;
      qo.q = static_cast<uint8_t*>(q), qo.sf = sf, qo.amax = amax, qo.nkb_pad = int(pad_to(K / V, 4));
      return run_stream_pipe("quantize_blockscaled", qo, rows * ppr, piece_elems * 2, s, 8, 3);
    }
    QuantPipeOp<1> qo;
    static_cast<RowPieces&>(qo) = rp;
    qo.q = static_cast<uint8_t*>(q), qo.sf = sf, qo.amax = nullptr, qo.nkb_pad = int(pad_to(K / V, 4));
    return run_stream_pipe("quantize_blockscaled", qo, rows * ppr, piece_elems * 2, s, 8, 3);
  }
  if (mode == MXK_Q_NVFP4) {
    int64_t grid = int64_t(sm_count()) * resident_ctas(amax_kernel, 256);
    if (grid > ceil_div(rows, kRowsInFlight)) grid = ceil_div(rows, kRowsInFlight);
    launch_pdl(amax_kernel, dim3(unsigned(grid)), dim3(256), 0, s, xb, ldx, rows, nvec, amax);
    if (int rc = after_launch("quantize_blockscaled")) return rc;
  }
  const int threads = nvec >= 256 ? 256 : int(ceil_div(nvec, 32) * 32);
  const unsigned gy = unsigned(ceil_div(nvec, threads));
  const int rpc = tune(TUNE_QUANT_ROWS_PER_CTA, 8);
  const int64_t nchunks = ceil_div(rows, rpc);
  auto go = [&](auto kern) {
    int64_t gx = ceil_div(int64_t(sm_count()) * resident_ctas(kern, threads), gy);
    if (gx > nchunks) gx = nchunks;
    if (gx < 1) gx = 1;
    launch_pdl(kern, dim3(unsigned(gx), gy), dim3(threads), 0, s, xb, ldx, rows, int(K), static_cast<uint8_t*>(q), sf,
               static_cast<const float*>(amax), rpc);
  };
  if (mode == MXK_Q_NVFP4) go(quant_kernel<2>);
  else go(quant_kernel<1>);
  return after_launch("quantize_blockscaled");
}

}  // extern "C"
