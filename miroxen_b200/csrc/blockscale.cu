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
// Work layout: a thread owns 16 consecutive elements (two 128-bit vectors): a whole NVFP4 block, half
// an MXFP8 block (one shuffle joins the two halves' maxima).  It stores 128 (64) bits of codes, so a
// warp's stores are one contiguous segment.  The arithmetic is packed where the result is the same
// bits: |.|-maxima on bf16 pairs (max.xorsign.abs.bf16x2; a maximum picks one of its inputs), scaling
// on fp32 pairs (mul.rn.f32x2), conversion two elements per instruction.  That layout serves the bulk-copy
// streaming pipeline (stream_pipe.cuh; NVFP4's default, quant_path = 1) - a producer warp lands row pieces of up
// to 32 KB in shared memory, consumer warps quantise from there; NVFP4's tensor maximum is a first pass through
// the same pipeline - and the register kernels on one resident wave (quant_path = 2, also taken when a row piece
// cannot be cut on a block boundary).  MXFP8's default is quant_mxfp8_block_kernel: a thread owns a whole
// 32-element block, a CTA one row, and the grid is as many CTAs as rows.
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

#include "act_math.cuh"
#include "blockscale_math.cuh"
#include "common.cuh"
#include "stream_pipe.cuh"
#include "tuning.h"

namespace mxk {
namespace {

constexpr float kFp4Range = 6.f * 448.f;  // src/kernels/blockscale.cu:33
constexpr int kRowsInFlight = 4;
constexpr int64_t kMaxQuantK = int64_t(1) << 24;  // keeps the register kernels' grid.y (K / 4096) inside 65535

// Four float pairs -> eight e2m1 codes, element 0 in the lowest nibble.
__device__ __forceinline__ uint32_t e2m1x8(float2 a, float2 b, float2 c, float2 d) {
  uint32_t w;
  asm("{ .reg .b8 b0, b1, b2, b3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b0, %2, %1;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b1, %4, %3;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b2, %6, %5;\n"
      "cvt.rn.satfinite.e2m1x2.f32 b3, %8, %7;\n"
      "mov.b32 %0, {b0, b1, b2, b3}; }"
      : "=r"(w)
      : "f"(a.x), "f"(a.y), "f"(b.x), "f"(b.y), "f"(c.x), "f"(c.y), "f"(d.x), "f"(d.y));
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

// Quantises the 16 elements of one thread: raw = two vectors of 8 bf16.  MODE 1: bmax_bits is the
// packed maximum over the thread's half block; out = 16 e4m3 bytes.  MODE 2: out.x, out.y = 16 e2m1
// codes.  Returns the scale byte.
template <int MODE>
__device__ __forceinline__ uint8_t quant16(const uint4 (&raw)[2], uint32_t packed_max, const Fp4Scale& fs, uint4& out) {
  const uint32_t w[8] = {raw[0].x, raw[0].y, raw[0].z, raw[0].w, raw[1].x, raw[1].y, raw[1].z, raw[1].w};
  if (MODE == 2) {
    // src/kernels/blockscale.cu:100-109
    const float bmax = bf16x2_max_to_float(packed_max);
    const __nv_fp8_storage_t se = __nv_cvt_float_to_fp8(__fmul_rn(bmax, fs.inv6g), __NV_SATFINITE, __NV_E4M3);
    __nv_fp8_e4m3 sq;
    sq.__x = se;
    const float sd = __fmul_rn(float(sq), fs.g);
    const float inv = sd > 0.f ? __frcp_rn(sd) : 0.f;
    const float2 inv2 = make_float2(inv, inv), zero2 = make_float2(0.f, 0.f);
    float2 t[8];
#pragma unroll
    for (int i = 0; i < 8; i++) t[i] = __fadd2_rn(__fmul2_rn(bf16x2_to_float2(w[i]), inv2), zero2);  // -0 -> +0
    out.x = e2m1x8(t[0], t[1], t[2], t[3]);
    out.y = e2m1x8(t[4], t[5], t[6], t[7]);
    out.z = out.w = 0;
    return se;
  }
  // ue8m0 scale and e4m3 codes (src/kernels/blockscale.cu:111-125), see blockscale_math.cuh
  return mxfp8_quant16(raw, packed_max, out);
}

// Packed |.|-maximum of a thread's 16 elements, joined with the other half of the block for MXFP8.
template <int MODE>
__device__ __forceinline__ uint32_t block_absmax(const uint4 (&raw)[2]) {
  if (MODE == 1) return mxfp8_block_absmax(raw);
  return absmax_bf16x2(absmax_bf16x2(raw[0]), absmax_bf16x2(raw[1]));
}


// A consumer thread of the activation + MXFP8 pipeline takes 16 elements per trip, so a piece of n16 = elements / 16
// keeps n16 / (32 * warps * trips) of the consumer threads busy.  Among the cuts of a row of K elements into
// min_pieces .. min_pieces + 4 pieces (whole 128-element groups each), takes the one that wastes the fewest, with
// 4 .. 16 consumer warps.  Measured on silu_mul + MXFP8 of 33272 x 13824: 378 us with the fitted cut (seven pieces
// of 2048 on four warps) against 415 - 435 us with four pieces of 3456 on eight warps.  The plain quantiser does NOT
// use it: there twelve warps measured best for every cut that fits them (5120 columns: 86 us on twelve warps, 93 us
// on the "fitting" ten; 13824 columns as three pieces on nine warps: no faster than two pieces on twelve).
inline void fit_row_pieces(int64_t K, int64_t rows, int min_pieces, int& elems, int& warps) {
  double best = 0.0;
  for (int p = min_pieces; p <= min_pieces + 4 && rows * p < (int64_t(1) << 31); p++) {
    const int e = int(ceil_div(ceil_div(K, p), 128) * 128);
    const int n16 = e / 16;
    int wv = int(ceil_div(n16, 32));
    wv = wv < 4 ? 4 : wv > 16 ? 16 : wv;
    const double eff = double(n16) / double(32 * wv * ceil_div(n16, 32 * wv));
    if (eff > best + 0.02) best = eff, elems = e, warps = wv;
  }
}

// ---- bulk-copy pipeline ops: chunk = one piece (pieces_per_row of them) of one row ----

struct AmaxPipeOp : RowPieces {
  static constexpr int NSRC = 1;
  float* out;
  struct State {
    uint32_t m;  // two running bf16 maxima
  };
  __device__ State init() const { return State{0u}; }
  __device__ void consume(State& st, int64_t chunk, const unsigned char* stage, int tid, int n_cons) const {
    unsigned row;
    int k0, n;
    where(chunk, row, k0, n);
    const uint4* s = reinterpret_cast<const uint4*>(stage);
    const int nvec = n >> 3;
    uint32_t m = st.m;
    for (int i = tid; i < nvec; i += n_cons) m = absmax_bf16x2(m, absmax_bf16x2(s[i]));
    st.m = m;
  }
  __device__ void finish(State& st, int) const { amax_commit(bf16x2_max_to_float(st.m), out); }
};

// ACT < 0: quantise the source as it is; otherwise apply the activation (act_math.cuh) to the source
// first, round to bf16 as the stand-alone activation kernel does, and quantise that.
template <int MODE, int ACT = -1>
struct QuantPipeOp : RowPieces {
  static constexpr int NSRC = ACT == ACT_SILU_MUL ? 2 : 1;
  uint8_t* q;
  uint8_t* sf;
  const float* amax;
  int nkb_pad;
  const float* bias = nullptr;  // ACT >= 0: fp32 [K] (or [2K], gate then up) added and rounded to bf16 first
  using State = Fp4Scale;
  __device__ State init() const { return MODE == 2 ? fp4_scale(amax) : Fp4Scale{1.f, 1.f}; }
  __device__ void consume(State& fs, int64_t chunk, const unsigned char* stage, int tid, int n_cons) const {
    unsigned row;
    int k0, n;
    where(chunk, row, k0, n);
    const uint4* s = reinterpret_cast<const uint4*>(stage);
    const int n16 = n >> 4, lane = tid & 31;  // n is a multiple of 32: the two halves of a block are both in range
    uint8_t* sfr = sf + sf_row_offset(row, nkb_pad);
    uint8_t* qrow = q + (int64_t(row) * K + k0) / (MODE == 2 ? 2 : 1);
    // every lane of a warp runs the same trips (the block maximum is a warp shuffle)
    for (int i0 = tid - lane; i0 < n16; i0 += n_cons) {
      const int i = i0 + lane, ic = i < n16 ? i : n16 - 1;  // lanes past the end compute on a copy, store nothing
      uint4 raw[2] = {s[2 * ic], s[2 * ic + 1]};
      if (ACT >= 0) {
        const uint4* s2 = reinterpret_cast<const uint4*>(stage + stage_off);
        uint4 up[2] = {raw[0], raw[1]};
        if (NSRC == 2) up[0] = s2[2 * ic], up[1] = s2[2 * ic + 1];
        if (bias) {
          const float* bp = bias + k0 + 16 * ic;
          raw[0] = add_bias8(raw[0], bp), raw[1] = add_bias8(raw[1], bp + 8);
          if (NSRC == 2) up[0] = add_bias8(up[0], bp + K), up[1] = add_bias8(up[1], bp + K + 8);
        }
        raw[0] = act8<ACT>(raw[0], up[0]);
        raw[1] = act8<ACT>(raw[1], up[1]);
      }
      uint4 out;
      const uint8_t sbyte = quant16<MODE>(raw, block_absmax<MODE>(raw), fs, out);
      if (i < n16) {
        if (MODE == 2) {
          st_stream(reinterpret_cast<uint2*>(qrow) + i, make_uint2(out.x, out.y));
          sfr[sf_col_offset((k0 >> 4) + i)] = sbyte;
        } else {
          st_stream(reinterpret_cast<uint4*>(qrow) + i, out);
          if ((lane & 1) == 0) sfr[sf_col_offset((k0 >> 5) + (i >> 1))] = sbyte;
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
  uint32_t m = 0u;
  for (int64_t r = int64_t(blockIdx.x) * U; r < rows; r += int64_t(gridDim.x) * U) {
    for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; u++)
        raw[u] = r + u < rows ? ld_stream(reinterpret_cast<const uint4*>(x + (r + u) * ldx) + j) : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < U; u++) m = absmax_bf16x2(m, absmax_bf16x2(raw[u]));
    }
  }
  amax_commit(bf16x2_max_to_float(m), out);
}

// MODE 1 = MXFP8, 2 = NVFP4.  Thread t of CTA column blockIdx.y owns the 16 elements starting at
// column 16 * (blockIdx.y * blockDim.x + t) of every row it visits.
template <int MODE>
__global__ void __launch_bounds__(256) quant_kernel(const bf16* __restrict__ x, int64_t ldx, int64_t rows, int K,
                                                     uint8_t* __restrict__ q, uint8_t* __restrict__ sf, const float* amax,
                                                     int rows_per_chunk) {
  constexpr int V = MODE == 2 ? 16 : 32;  // elements per scale block
  constexpr int U = kRowsInFlight;
  pdl_launch_dependents();
  pdl_wait();
  const int col = blockIdx.y * blockDim.x + threadIdx.x;  // 16-element column index inside the row
  const bool col_on = col * 16 < K;                        // K is a multiple of 32: pairs are on or off together
  const int nkb_pad = int(pad_to(K / V, 4));
  const bool leader = MODE == 2 || (threadIdx.x & 1) == 0;
  const int sf_col = sf_col_offset(col * 16 / V);
  const Fp4Scale fs = MODE == 2 ? fp4_scale(amax) : Fp4Scale{1.f, 1.f};
  const int64_t nchunks = (rows + rows_per_chunk - 1) / rows_per_chunk;
  for (int64_t c = blockIdx.x; c < nchunks; c += gridDim.x) {
    const int64_t r0 = c * rows_per_chunk;
    const int64_t r1 = r0 + rows_per_chunk < rows ? r0 + rows_per_chunk : rows;
    for (int64_t rb = r0; rb < r1; rb += U) {
      uint4 raw[U][2];
#pragma unroll
      for (int u = 0; u < U; u++) {
        raw[u][0] = raw[u][1] = make_uint4(0u, 0u, 0u, 0u);
        if (col_on && rb + u < r1) {
          const uint4* src = reinterpret_cast<const uint4*>(x + (rb + u) * ldx) + 2 * col;
          raw[u][0] = ld_stream(src), raw[u][1] = ld_stream(src + 1);
        }
      }
#pragma unroll
      for (int u = 0; u < U; u++) {
        const int64_t r = rb + u;
        uint4 out;
        const uint8_t sbyte = quant16<MODE>(raw[u], block_absmax<MODE>(raw[u]), fs, out);
        if (col_on && r < r1) {
          if (MODE == 2) st_stream(reinterpret_cast<uint2*>(q + (r * K) / 2) + col, make_uint2(out.x, out.y));
          else st_stream(reinterpret_cast<uint4*>(q + r * K) + col, out);
          if (leader) sf[sf_row_offset(uint64_t(r), nkb_pad) + sf_col] = sbyte;
        }
      }
    }
  }
}

// MXFP8 with one thread per 32-element scale block (quant_path = 3, the default): four independent 128-bit loads per
// thread and no exchange between lanes; launched with one CTA per row (the row loop only matters for a smaller grid),
// threads walk the blocks of the row.  Plain cached accesses measured a little ahead of the streaming hints here
// (207 against 218 us on 33272 x 13824).
__global__ void __launch_bounds__(256) quant_mxfp8_block_kernel(const bf16* __restrict__ x, int64_t ldx, int64_t rows, int K,
                                                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf) {
  pdl_launch_dependents();
  pdl_wait();
  const int nb = K / 32, nkb_pad = int(pad_to(nb, 4));
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(x + r * ldx);
    uint4* qrow = reinterpret_cast<uint4*>(q + r * K);
    uint8_t* sfr = sf + sf_row_offset(uint64_t(r), nkb_pad);
    for (int kb = threadIdx.x; kb < nb; kb += blockDim.x) {
      const uint4 lo[2] = {row[4 * kb], row[4 * kb + 1]};
      const uint4 hi[2] = {row[4 * kb + 2], row[4 * kb + 3]};
      const uint32_t m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(lo[0]), absmax_bf16x2(lo[1])),
                                       absmax_bf16x2(absmax_bf16x2(hi[0]), absmax_bf16x2(hi[1])));
      uint4 o0, o1;
      const uint8_t sbyte = mxfp8_quant16(lo, m, o0);
      mxfp8_quant16(hi, m, o1);
      qrow[2 * kb] = o0, qrow[2 * kb + 1] = o1;
      sfr[sf_col_offset(kb)] = sbyte;
    }
  }
}

// NVFP4 in the same form (quant_path = 3): a thread owns two 16-element blocks (four 128-bit loads, one 128-bit store of
// codes, the two scale bytes as one 16-bit store: block pairs sit next to each other in the interleaved scale layout).
__global__ void __launch_bounds__(256) quant_nvfp4_block_kernel(const bf16* __restrict__ x, int64_t ldx, int64_t rows, int K,
                                                                 uint8_t* __restrict__ q, uint8_t* __restrict__ sf,
                                                                 const float* amax) {
  pdl_launch_dependents();
  pdl_wait();
  const Fp4Scale fs = fp4_scale(amax);
  const int np = K / 32, nkb_pad = int(pad_to(K / 16, 4));
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(x + r * ldx);
    uint4* qrow = reinterpret_cast<uint4*>(q + r * (K / 2));
    uint8_t* sfr = sf + sf_row_offset(uint64_t(r), nkb_pad);
    for (int p = threadIdx.x; p < np; p += blockDim.x) {
      const uint4 lo[2] = {row[4 * p], row[4 * p + 1]};
      const uint4 hi[2] = {row[4 * p + 2], row[4 * p + 3]};
      uint4 o0, o1;
      const uint8_t s0 = quant16<2>(lo, block_absmax<2>(lo), fs, o0);
      const uint8_t s1 = quant16<2>(hi, block_absmax<2>(hi), fs, o1);
      qrow[p] = make_uint4(o0.x, o0.y, o1.x, o1.y);
      *reinterpret_cast<uint16_t*>(sfr + sf_col_offset(2 * p)) = uint16_t(s0) | uint16_t(uint16_t(s1) << 8);
    }
  }
}

// The tensor maximum in the same spirit: four rows per CTA, as many CTAs as that takes, ONE atomic per CTA.
__global__ void __launch_bounds__(256) amax_rows_kernel(const bf16* __restrict__ x, int64_t ldx, int64_t rows, int nvec, float* out) {
  constexpr int U = kRowsInFlight;
  __shared__ float part[8];
  pdl_launch_dependents();
  pdl_wait();
  uint32_t m = 0u;
  for (int64_t r = int64_t(blockIdx.x) * U; r < rows; r += int64_t(gridDim.x) * U) {
    for (int j = threadIdx.x; j < nvec; j += blockDim.x) {
      uint4 raw[U];
#pragma unroll
      for (int u = 0; u < U; u++)
        raw[u] = r + u < rows ? reinterpret_cast<const uint4*>(x + (r + u) * ldx)[j] : make_uint4(0u, 0u, 0u, 0u);
#pragma unroll
      for (int u = 0; u < U; u++) m = absmax_bf16x2(m, absmax_bf16x2(raw[u]));
    }
  }
  float v = bf16x2_max_to_float(m);
#pragma unroll
  for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = v;
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < int(blockDim.x >> 5); w++) v = fmaxf(v, part[w]);
    // non-negative floats order like their bit patterns (src/kernels/blockscale.cu:68)
    if (v > 0.f) atomicMax(reinterpret_cast<int*>(out), __float_as_int(v));
  }
}

// Activation + MXFP8 in the same form (thread per scale block, row per CTA): the 32 activation inputs of a block (and
// the 32 of the up half for silu_mul) are loaded, an optional bias is added and rounded to bf16 as add_bias_bf16 leaves
// it, the activation is applied and rounded to bf16 exactly as the stand-alone kernel rounds it, and the block is
// quantised from those bits.
template <int ACT>
__global__ void __launch_bounds__(256) act_quant_mxfp8_block_kernel(const bf16* __restrict__ in, const float* __restrict__ bias,
                                                                     int64_t rows, int F, uint8_t* __restrict__ q,
                                                                     uint8_t* __restrict__ sf) {
  constexpr bool TWO = ACT == ACT_SILU_MUL;
  pdl_launch_dependents();
  pdl_wait();
  const int nb = F / 32, nkb_pad = int(pad_to(nb, 4));
  for (int64_t r = blockIdx.x; r < rows; r += gridDim.x) {
    const uint4* row = reinterpret_cast<const uint4*>(in + r * int64_t(F) * (TWO ? 2 : 1));
    const uint4* up_row = row + F / 8;  // silu_mul: the up half of the row
    uint4* qrow = reinterpret_cast<uint4*>(q + r * F);
    uint8_t* sfr = sf + sf_row_offset(uint64_t(r), nkb_pad);
    for (int kb = threadIdx.x; kb < nb; kb += blockDim.x) {
      uint4 g[4], u[4];
#pragma unroll
      for (int j = 0; j < 4; j++) {
        g[j] = row[4 * kb + j];
        u[j] = TWO ? up_row[4 * kb + j] : g[j];
      }
      if (bias) {
        const float* bp = bias + 32 * kb;
#pragma unroll
        for (int j = 0; j < 4; j++) {
          g[j] = add_bias8(g[j], bp + 8 * j);
          if (TWO) u[j] = add_bias8(u[j], bp + F + 8 * j);
        }
      }
      uint4 a[4];
#pragma unroll
      for (int j = 0; j < 4; j++) a[j] = act8<ACT>(g[j], u[j]);
      const uint4 lo[2] = {a[0], a[1]}, hi[2] = {a[2], a[3]};
      const uint32_t m = absmax_bf16x2(absmax_bf16x2(absmax_bf16x2(a[0]), absmax_bf16x2(a[1])),
                                       absmax_bf16x2(absmax_bf16x2(a[2]), absmax_bf16x2(a[3])));
      uint4 o0, o1;
      const uint8_t sbyte = mxfp8_quant16(lo, m, o0);
      mxfp8_quant16(hi, m, o1);
      qrow[2 * kb] = o0, qrow[2 * kb + 1] = o1;
      sfr[sf_col_offset(kb)] = sbyte;
    }
  }
}

}  // namespace
}  // namespace mxk

// Padded scale rows / columns are read by the GEMM (0xff is NaN in ue8m0) and the reference clears
// the whole buffer first (src/kernels/blockscale.cu:154).  Every byte of a real (row, block) is
// written by the kernels, so clearing what is padding gives the same bytes: nothing when rows fill
// their 128-row tiles and blocks their groups of 4, the last row tile when only rows are ragged, and
// everything when the column padding is interleaved through all tiles.
static int clear_scale_padding(int mode, int64_t rows, int64_t K, uint8_t* sf, cudaStream_t s) {
  const int64_t nkb = K / (mode == MXK_Q_NVFP4 ? 16 : 32);
  cudaError_t e = cudaSuccess;
  if (nkb % 4 != 0) {
    e = cudaMemsetAsync(sf, 0, size_t(mxk::pad_to(rows, 128) * mxk::pad_to(nkb, 4)), s);
  } else if (rows % 128 != 0) {
    const int64_t tile = nkb * 128;
    e = cudaMemsetAsync(sf + rows / 128 * tile, 0, size_t(tile), s);
  }
  if (e != cudaSuccess) return mxk::fail(MXK_ERR_CUDA, "cudaMemsetAsync (scale padding): %s", cudaGetErrorString(e));
  return MXK_OK;
}

using namespace mxk;

template <int ACT>
static int run_act_quant(const mxk_bf16* in, const float* bias, int64_t rows, int64_t F, void* q, uint8_t* sf, cudaStream_t s) {
  const bool two = ACT == ACT_SILU_MUL;
  // Default for the one-source activations: thread per scale block, row per CTA, as many CTAs as rows (as the plain
  // MXFP8 quantiser): GELU + MXFP8 of 8704 x 12288 61.3 us against 82.0 us through the pipeline below.  silu_mul, with
  // two sources per block, measured 388 us in that form against 378 us through the fitted pipeline on 33272 x 13824,
  // so it keeps the pipeline unless quant_path = 3 is set.
  const int path = tune(TUNE_QUANT_PATH, two ? 1 : 3);
  if (path == 3 && rows < (int64_t(1) << 31)) {
    const int nb = int(F / 32);
    int threads = 128, best = 1 << 30;
    for (int t = 128; t <= 256; t += 32) {
      const int waste = int(ceil_div(nb, t)) * t - nb;
      if (waste < best) best = waste, threads = t;
    }
    if (nb < 128) threads = int(ceil_div(nb, 32) * 32);
    launch_pdl(act_quant_mxfp8_block_kernel<ACT>, dim3(unsigned(rows)), dim3(threads), 0, s, reinterpret_cast<const bf16*>(in), bias,
               rows, int(F), static_cast<uint8_t*>(q), sf);
    return after_launch("act_quantize_mxfp8");
  }
  // two sources share a stage: half the chunk each
  int chunk_bytes = tune(TUNE_STREAM_CHUNK_KB, 16) * 1024 / (two ? 2 : 1);
  if (chunk_bytes > 32 * 1024) chunk_bytes = 32 * 1024;
  const int pieces = int(ceil_div(F * 2, chunk_bytes));
  const int piece_elems = int(ceil_div(ceil_div(F, pieces), 128) * 128);
  if (piece_elems * 2 > chunk_bytes || rows * pieces >= (int64_t(1) << 31))
    return fail(MXK_ERR_TOO_LARGE, "act_quantize_mxfp8: %lld rows of %lld do not fit the pipeline's chunking", (long long)rows, (long long)F);
  int elems = piece_elems, warps = two ? 8 : 12;
  fit_row_pieces(F, rows, pieces, elems, warps);
  QuantPipeOp<1, ACT> qo;
  qo.x = reinterpret_cast<const unsigned char*>(in), qo.ldx_bytes = F * (two ? 4 : 2), qo.K = int(F);
  qo.set_pieces(int(ceil_div(F, elems)), elems);
  qo.src1_off = two ? F * 2 : 0, qo.stage_off = (elems * 2 + 127) & ~127;
  qo.q = static_cast<uint8_t*>(q), qo.sf = sf, qo.amax = nullptr, qo.nkb_pad = int(pad_to(F / 32, 4)), qo.bias = bias;
  return run_stream_pipe("act_quantize_mxfp8", qo, rows * qo.pieces_per_row, elems * 2, s, warps, 3);
}

extern "C" {

int64_t mxk_qdata_bytes(int mode, int64_t rows, int64_t K) { return rows * K / (mode == MXK_Q_NVFP4 ? 2 : 1); }

int64_t mxk_qscale_bytes(int mode, int64_t rows, int64_t K) {
  return pad_to(rows, 128) * pad_to(K / (mode == MXK_Q_NVFP4 ? 16 : 32), 4);
}

static int quantize_impl(int mode, const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf, float* amax,
                         bool amax_known, mxk_stream_t stream);

int mxk_quantize_blockscaled(int mode, const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf,
                             float* amax, mxk_stream_t stream) {
  return quantize_impl(mode, x, ldx, rows, K, q, sf, amax, false, stream);
}

int mxk_quantize_nvfp4_known_amax(const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf,
                                  const float* amax, mxk_stream_t stream) {
  return quantize_impl(MXK_Q_NVFP4, x, ldx, rows, K, q, sf, const_cast<float*>(amax), true, stream);
}

static int quantize_impl(int mode, const mxk_bf16* x, int64_t ldx, int64_t rows, int64_t K, void* q, uint8_t* sf, float* amax,
                         bool amax_known, mxk_stream_t stream) {
  if (mode != MXK_Q_MXFP8 && mode != MXK_Q_NVFP4)
    return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: mode %d is not a quantised mode (1 MXFP8, 2 NVFP4)", mode);
  // the reference's own check (src/kernels/blockscale.cu:151)
  if (K <= 0 || K % 32 != 0 || ldx % 8 != 0 || ldx < K || !aligned(x, 16))
    return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: need K %% 32 == 0, ldx %% 8 == 0, ldx >= K, 16-byte aligned input");
  if (K > kMaxQuantK) return fail(MXK_ERR_TOO_LARGE, "quantize_blockscaled: K=%lld beyond %lld", (long long)K, (long long)kMaxQuantK);
  if (rows == 0) return MXK_OK;
  if (rows < 0 || !x || !q || !sf || (mode == MXK_Q_NVFP4 && !amax))
    return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: null buffer or negative rows");
  if (!aligned(q, 16)) return fail(MXK_ERR_INVALID_ARG, "quantize_blockscaled: q must be 16-byte aligned");
  cudaStream_t s = as_stream(stream);
  const bf16* xb = reinterpret_cast<const bf16*>(x);
  if (int rc = clear_scale_padding(mode, rows, K, sf, s)) return rc;
  cudaError_t e = cudaSuccess;
  if (mode == MXK_Q_NVFP4 && !amax_known) e = cudaMemsetAsync(amax, 0, sizeof(float), s);
  if (e != cudaSuccess) return fail(MXK_ERR_CUDA, "quantize_blockscaled: cudaMemsetAsync: %s", cudaGetErrorString(e));
  const int nvec = int(K / 8);
  const int V = mode == MXK_Q_NVFP4 ? 16 : 32;
  // Bulk-copy pipeline: rows cut into equal pieces of whole scale blocks, at most one chunk each.
  // Measured on B200 (8704 x 12288, 8704 x 3072, 33272 x 5120, 33272 x 13824 bf16): MXFP8 runs best
  // with 12 consumer warps on 16 KB chunks, 3 stages; NVFP4, with more arithmetic per element, with 4
  // warps on 32 KB chunks, 2 stages.  An MXFP8 input that fits in L2 with its output goes to the register kernel, whose fixed
  // cost is a few microseconds lower.
  const bool fp4 = mode == MXK_Q_NVFP4;
  if (!fp4 && tune(TUNE_QUANT_PATH, 3) == 3 && rows < (int64_t(1) << 31)) {
    // MXFP8 default: one thread per scale block, ONE ROW PER CTA and as many CTAs as rows.  Against the two persistent
    // forms below (one resident wave of CTAs): 33272 x 13824: 207 us against 230 (pipeline) and 248 (register kernel);
    // 8704 x 3072: 12.7 us against 15.6 and 14.9 - the same kernel walking the rows grid-stride from one resident
    // wave took 271 / 15.3 us.  Threads: the blocks of a row in whole trips if 128 .. 256 threads allow it.
    const int nb = int(K / 32);
    int threads = 128, best = 1 << 30;
    for (int t = 128; t <= 256; t += 32) {
      const int waste = int(ceil_div(nb, t)) * t - nb;
      if (waste < best) best = waste, threads = t;
    }
    if (nb < 128) threads = int(ceil_div(nb, 32) * 32);
    launch_pdl(quant_mxfp8_block_kernel, dim3(unsigned(rows)), dim3(threads), 0, s, xb, ldx, rows, int(K), static_cast<uint8_t*>(q), sf);
    return after_launch("quantize_blockscaled");
  }
  if (fp4 && tune(TUNE_QUANT_PATH, 1) == 3 && rows < (int64_t(1) << 31)) {
    // NVFP4 with a thread per pair of scale blocks and a row per CTA; the maximum pass with four rows per CTA.  Opt-in:
    // within a few per cent of the pipeline either way (8704 x 12288: 83.7 against 85.6 us; 33272 x 5120: 137.7 against
    // 134.1 us) - the two passes over the input bound this mode, not the form of either kernel.
    if (!amax_known) {
      launch_pdl(amax_rows_kernel, dim3(unsigned(ceil_div(rows, kRowsInFlight))), dim3(256), 0, s, xb, ldx, rows, nvec, amax);
      if (int rc = after_launch("quantize_blockscaled (amax)")) return rc;
    }
    const int np = int(K / 32);
    int threads = 128, best = 1 << 30;
    for (int t = 128; t <= 256; t += 32) {
      const int waste = int(ceil_div(np, t)) * t - np;
      if (waste < best) best = waste, threads = t;
    }
    if (np < 128) threads = int(ceil_div(np, 32) * 32);
    launch_pdl(quant_nvfp4_block_kernel, dim3(unsigned(rows)), dim3(threads), 0, s, xb, ldx, rows, int(K), static_cast<uint8_t*>(q), sf,
               static_cast<const float*>(amax));
    return after_launch("quantize_blockscaled");
  }
  int chunk_bytes = tune(TUNE_STREAM_CHUNK_KB, fp4 ? 32 : 16) * 1024;
  if (chunk_bytes > 32 * 1024) chunk_bytes = 32 * 1024;
  const int pieces = int(ceil_div(K * 2, chunk_bytes));
  const int piece_elems = int(ceil_div(ceil_div(K, pieces), 128) * 128);
  const bool small = !fp4 && rows * K * 2 < (int64_t(96) << 20);
  if (tune(TUNE_QUANT_PATH, small ? 2 : 1) == 1 && piece_elems * 2 <= chunk_bytes && rows * pieces < (int64_t(1) << 31)) {
    const int ppr = int(ceil_div(K, piece_elems));
    RowPieces rp;
    rp.x = reinterpret_cast<const unsigned char*>(x), rp.ldx_bytes = ldx * 2, rp.K = int(K);
    rp.set_pieces(ppr, piece_elems);
    if (fp4) {
      if (!amax_known) {
        AmaxPipeOp op;
        static_cast<RowPieces&>(op) = rp;
        op.out = amax;
        if (int rc = run_stream_pipe("quantize_blockscaled (amax)", op, rows * ppr, piece_elems * 2, s, 4, 2)) return rc;
      }
      QuantPipeOp<2> qo;
      static_cast<RowPieces&>(qo) = rp;
      qo.q = static_cast<uint8_t*>(q), qo.sf = sf, qo.amax = amax, qo.nkb_pad = int(pad_to(K / V, 4));
      return run_stream_pipe("quantize_blockscaled", qo, rows * ppr, piece_elems * 2, s, 4, 2);
    }
    QuantPipeOp<1> qo;
    static_cast<RowPieces&>(qo) = rp;
    qo.q = static_cast<uint8_t*>(q), qo.sf = sf, qo.amax = nullptr, qo.nkb_pad = int(pad_to(K / V, 4));
    // twelve consumer warps (384 threads, 16 elements each per trip); a piece of 385 .. 512 threads' work would need a
    // second, nearly empty trip, so it gets sixteen warps (33272 x 13824: 230 us against 258 us; 33272 x 14336: 237 / 275)
    const int n16 = piece_elems / 16;
    return run_stream_pipe("quantize_blockscaled", qo, rows * ppr, piece_elems * 2, s, n16 > 384 && n16 <= 512 ? 16 : 12, 3);
  }
  if (mode == MXK_Q_NVFP4 && !amax_known) {
    int64_t grid = int64_t(sm_count()) * resident_ctas(amax_kernel, 256);
    if (grid > ceil_div(rows, kRowsInFlight)) grid = ceil_div(rows, kRowsInFlight);
    launch_pdl(amax_kernel, dim3(unsigned(grid)), dim3(256), 0, s, xb, ldx, rows, nvec, amax);
    if (int rc = after_launch("quantize_blockscaled")) return rc;
  }
  const int ncol = int(K / 16);
  const int threads = ncol >= 256 ? 256 : int(ceil_div(ncol, 32) * 32);
  const unsigned gy = unsigned(ceil_div(ncol, threads));
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

int mxk_act_quantize_mxfp8(int act_mode, const mxk_bf16* in, const float* bias, int64_t rows, int64_t F, void* q, uint8_t* sf,
                           mxk_stream_t stream) {
  if (act_mode < 0 || act_mode > 2) return fail(MXK_ERR_INVALID_ARG, "act_quantize_mxfp8: act_mode %d (0 gelu tanh, 1 silu_mul, 2 gelu erf)", act_mode);
  if (F <= 0 || F % 32 != 0 || !aligned(in, 16) || !aligned(bias, 16))
    return fail(MXK_ERR_INVALID_ARG, "act_quantize_mxfp8: need F %% 32 == 0 and 16-byte aligned input and bias");
  if (F > kMaxQuantK) return fail(MXK_ERR_TOO_LARGE, "act_quantize_mxfp8: F=%lld beyond %lld", (long long)F, (long long)kMaxQuantK);
  if (rows == 0) return MXK_OK;
  if (rows < 0 || !in || !q || !sf) return fail(MXK_ERR_INVALID_ARG, "act_quantize_mxfp8: null buffer or negative rows");
  if (!aligned(q, 16)) return fail(MXK_ERR_INVALID_ARG, "act_quantize_mxfp8: q must be 16-byte aligned");
  cudaStream_t s = as_stream(stream);
  if (int rc = clear_scale_padding(MXK_Q_MXFP8, rows, F, sf, s)) return rc;
  if (act_mode == 1) return run_act_quant<ACT_SILU_MUL>(in, bias, rows, F, q, sf, s);
  if (act_mode == 2) return run_act_quant<ACT_GELU_ERF>(in, bias, rows, F, q, sf, s);
  return run_act_quant<ACT_GELU_TANH>(in, bias, rows, F, q, sf, s);
}

}  // extern "C"
