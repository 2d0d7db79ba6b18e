// Row-normalisation kernels: LayerNorm / RMSNorm + modulation + bf16 cast, optionally preceded
// by the gated residual update of the same row.
//
// Behaviour follows the reference's norm_mod_kernel (src/kernels/ops.cu:43-71) and
// gated_residual_kernel (src/kernels/ops.cu:73-84): mean, then sum of squared deviations (two
// passes over the row's values), rstd = rsqrtf(sum / dim + eps), then in this order
// normalise -> * w -> * (1 + scale) -> + shift -> round to bf16.
//
// Layout of the work: one CTA walks a contiguous range of rows.  Thread t of a T-thread CTA owns
// the 4-element column groups t, t + T, ... (VPT of them), the same for every row, so the
// modulation values of those columns live in registers for the whole range and the row itself
// is read from HBM exactly once into registers; mean and variance come from those registers.
#pragma once

#include "blockscale_math.cuh"
#include "bulk_copy.cuh"
#include "common.cuh"

namespace mxk {

constexpr int kNormMaxVpt = 8;

struct NormArgs {
  const void* x;   // fp32 or bf16 [rows, dim]
  float* xw;       // fused residual: updated x is written here (== x)
  const bf16* y;   // fused residual: bf16 [rows, dim]
  MxkRowMod gate;  // fused residual
  int gate_tanh;
  int64_t rows;
  int dim;
  int nvec;  // dim / 4
  float eps;
  const float* w;
  MxkRowMod scale, shift;
  bf16* out;
  int rows_per_cta;
  int64_t row_step;  // bulk-copy kernel: 1 = contiguous row range per CTA, gridDim.x = interleaved rows
  const float* ybias;  // YBIAS kernels: fp32 [dim] added to y (and rounded to bf16) before the residual update
  int* err;  // device error word (bounded waits report here)
  // MXFP8 output instead of bf16 (QUANT kernels): e4m3 codes [rows, dim], interleaved ue8m0 scales
  uint8_t* q;
  uint8_t* sf;
  int nkb_pad;
  // optional: max |out| over the launch, folded into *amax with atomicMax (the caller clears it first); what the
  // NVFP4 quantiser needs before it can scale any block (src/kernels/blockscale.cu:47-70 is a pass of its own)
  float* amax;
};

// Sum over the CTA; `red` is a 16-float scratch that must not be reused before the next
// __syncthreads() of the caller's control flow (callers alternate two scratch arrays).
__device__ __forceinline__ float cta_sum(float v, float* red, int nwarps) {
  v = warp_sum(v);
  if (nwarps == 1) return v;
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = red[0];
  for (int i = 1; i < nwarps; i++) t += red[i];
  return t;
}

// Raw 4-element vector as it sits in memory.
template <class TIN> struct Raw4;
template <> struct Raw4<float> { using type = float4; };
template <> struct Raw4<bf16> { using type = uint2; };
__device__ __forceinline__ float4 widen(const float4& v) { return v; }
__device__ __forceinline__ float4 widen(const uint2& v) {
  return make_float4(bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y));
}

// CTA sizes the vector kernel may be launched with, by vectors per thread: the wide variants
// need more than 128 registers per thread, which a 512-thread CTA cannot have.
__host__ __device__ constexpr int norm_max_threads(int vpt) { return vpt <= 4 ? 512 : 256; }

// MODE 0 = LayerNorm, 1 = RMSNorm.  EXACT: blockDim.x * VPT == nvec (no column predicate).
// The loads of row r + 1 are issued before the reductions of row r, so that each CTA keeps two
// rows in flight.
template <int MODE, class TIN, int VPT, bool HAS_W, bool FUSE_RES, bool EXACT>
__global__ void __launch_bounds__(norm_max_threads(VPT))
    norm_rows_kernel(const NormArgs a) {
  using raw_t = typename Raw4<TIN>::type;
  __shared__ float red[2][16];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x, T = blockDim.x, nwarps = T >> 5;
  const int64_t r0 = int64_t(blockIdx.x) * a.rows_per_cta;
  const int64_t r1 = r0 + a.rows_per_cta < a.rows ? r0 + a.rows_per_cta : a.rows;
  const TIN* x = static_cast<const TIN*>(a.x);
  const float fdim = float(a.dim);

  bool on[VPT];
#pragma unroll
  for (int k = 0; k < VPT; k++) on[k] = EXACT || (k * T + tid < a.nvec);

  // Modulation of this thread's columns: A = 1 + scale, B = shift, W = w, G = act(gate).
  float4 A[VPT], B[VPT], W[HAS_W ? VPT : 1], G[FUSE_RES ? VPT : 1];
  int cur_set = -1;
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    if (HAS_W) W[k] = on[k] ? *reinterpret_cast<const float4*>(a.w + 4 * (k * T + tid))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  raw_t xn[VPT];
  uint2 yn[FUSE_RES ? VPT : 1];
  auto fetch = [&](int64_t row) {
    const TIN* xr = x + row * a.dim;
#pragma unroll
    for (int k = 0; k < VPT; k++)
      if (on[k]) xn[k] = ld_stream(reinterpret_cast<const raw_t*>(xr + 4 * (k * T + tid)));
    if (FUSE_RES) {
      const bf16* yr = a.y + row * a.dim;
#pragma unroll
      for (int k = 0; k < VPT; k++)
        if (on[k]) yn[k] = ld_stream(reinterpret_cast<const uint2*>(yr + 4 * (k * T + tid)));
    }
  };
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    if constexpr (sizeof(TIN) == 4) xn[k] = make_float4(0.f, 0.f, 0.f, 0.f);
    else xn[k] = make_uint2(0u, 0u);
    if (FUSE_RES) yn[k] = make_uint2(0u, 0u);
  }
  if (r0 < r1) fetch(r0);

  int parity = 0;
  uint32_t run_max = 0u;  // two running bf16 maxima of this thread's outputs
  for (int64_t row = r0; row < r1; row++) {
    const int set = (row < a.scale.prefix_len ? 1 : 0) | (row < a.shift.prefix_len ? 2 : 0) |
                    (FUSE_RES && row < a.gate.prefix_len ? 4 : 0);
    if (set != cur_set) {
      cur_set = set;
      const float* sc = a.scale.target ? pick(a.scale, row) : nullptr;
      const float* sh = a.shift.target ? pick(a.shift, row) : nullptr;
      const float* gt = FUSE_RES && a.gate.target ? pick(a.gate, row) : nullptr;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        const int c = 4 * (k * T + tid);
        // An absent scale multiplies by 1; an absent shift adds -0, which leaves every value,
        // signed zeros included, as it was.
        A[k] = make_float4(1.f, 1.f, 1.f, 1.f);
        B[k] = make_float4(-0.f, -0.f, -0.f, -0.f);
        if (on[k]) {
          if (sc) {
            float4 v = *reinterpret_cast<const float4*>(sc + c);
            A[k] = make_float4(1.f + v.x, 1.f + v.y, 1.f + v.z, 1.f + v.w);
          }
          if (sh) B[k] = *reinterpret_cast<const float4*>(sh + c);
        }
        if (FUSE_RES) {
          G[k] = make_float4(1.f, 1.f, 1.f, 1.f);
          if (gt && on[k]) {
            float4 g = *reinterpret_cast<const float4*>(gt + c);
            G[k] = a.gate_tanh ? make_float4(tanhf(g.x), tanhf(g.y), tanhf(g.z), tanhf(g.w)) : g;
          }
        }
      }
    }

    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) v[k] = widen(xn[k]);
    if (FUSE_RES) {
      float* xo = a.xw + row * a.dim;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        float4 yv = widen(yn[k]);
        v[k].x = fmaf(yv.x, G[k].x, v[k].x);
        v[k].y = fmaf(yv.y, G[k].y, v[k].y);
        v[k].z = fmaf(yv.z, G[k].z, v[k].z);
        v[k].w = fmaf(yv.w, G[k].w, v[k].w);
        if (on[k]) st_stream(reinterpret_cast<float4*>(xo + 4 * (k * T + tid)), v[k]);
      }
    }
    if (row + 1 < r1) fetch(row + 1);

    float mean = 0.f;
    if (MODE == 0) {
      float s = 0.f;
#pragma unroll
      for (int k = 0; k < VPT; k++) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
      mean = cta_sum(s, red[0], nwarps) / fdim;
    }
    float ss = 0.f;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
      // Padding lanes hold zeros; in LayerNorm mode their deviation would be -mean, so they
      // are masked out of the sum of squares.
      float dx = v[k].x - mean, dy = v[k].y - mean, dz = v[k].z - mean, dw = v[k].w - mean;
      float q = (dx * dx + dy * dy) + (dz * dz + dw * dw);
      ss += (EXACT || MODE == 1 || on[k]) ? q : 0.f;
    }
    const float rstd = rsqrtf(cta_sum(ss, red[MODE == 0 ? 1 : parity], nwarps) / fdim + a.eps);
    parity ^= 1;

    bf16* orow = a.out + row * a.dim;
#pragma unroll
    for (int k = 0; k < VPT; k++) {
      float o[4] = {(v[k].x - mean) * rstd, (v[k].y - mean) * rstd, (v[k].z - mean) * rstd,
                    (v[k].w - mean) * rstd};
      if (HAS_W) o[0] *= W[k].x, o[1] *= W[k].y, o[2] *= W[k].z, o[3] *= W[k].w;
      o[0] = o[0] * A[k].x + B[k].x;
      o[1] = o[1] * A[k].y + B[k].y;
      o[2] = o[2] * A[k].z + B[k].z;
      o[3] = o[3] * A[k].w + B[k].w;
      if (on[k]) {
        const uint2 pk = pack4(o);
        st_stream(reinterpret_cast<uint2*>(orow + 4 * (k * T + tid)), pk);
        if (a.amax) run_max = absmax_bf16x2(run_max, absmax_bf16x2(pk.x, pk.y));
      }
    }
  }
  if (a.amax) amax_commit(bf16x2_max_to_float(run_max), a.amax);
}

// ---- bulk-copy (TMA) pipelined variant ----------------------------------------------------------
//
// Same arithmetic and the same thread-to-column mapping as norm_rows_kernel (MODE 2 = the gated
// residual update alone, no norm and no bf16 output), but the rows arrive
// through a ring of shared-memory stages filled by cp.async.bulk (one elected thread issues a
// whole-row copy that completes on an mbarrier), so `stages` rows per CTA are in flight no matter
// how many registers the math needs.  A stage is refilled right after the CTA-wide barrier of the
// row's first reduction, by which point every thread has moved its part of the row to registers.
//
// Every wait on an mbarrier is bounded: when the limit is hit the CTA agrees on it through the
// barrier vote, records kErrBulkTimeout in the device's error word, drains the copies it still has in
// flight (bounded again) and returns.

template <int MODE, class TIN, int VPT, bool HAS_W, bool FUSE_RES, bool EXACT, bool QUANT = false, bool YBIAS = false>
__global__ void __launch_bounds__(norm_max_threads(VPT))
    norm_rows_tma_kernel(const NormArgs a, const int stages, const int stage_bytes) {
  using raw_t = typename Raw4<TIN>::type;
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ float red[2][16];
  __shared__ __align__(8) unsigned long long bars[8];
  const int tid = threadIdx.x, T = blockDim.x, nwarps = T >> 5;
  // Rows of this CTA: a contiguous range (row_step 1) or every gridDim.x-th row (row_step =
  // gridDim.x), in which case the CTAs of the grid sweep one compact window of rows together.
  const int64_t step = a.row_step;
  const int64_t r0 = step == 1 ? int64_t(blockIdx.x) * a.rows_per_cta : int64_t(blockIdx.x);
  const int64_t r1 = step == 1 ? (r0 + a.rows_per_cta < a.rows ? r0 + a.rows_per_cta : a.rows) : a.rows;
  const TIN* x = static_cast<const TIN*>(a.x);
  const float fdim = float(a.dim);
  const unsigned xbytes = unsigned(a.dim) * sizeof(TIN);
  const unsigned ybytes = FUSE_RES ? unsigned(a.dim) * 2u : 0u;
  const unsigned yoff = (xbytes + 127u) & ~127u;  // y row sits after the x row inside a stage

  pdl_launch_dependents();
  if (tid == 0) {
    for (int i = 0; i < stages; i++) mbar_init(smem_u32(&bars[i]), 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  pdl_wait();  // nothing above touches global memory

  auto issue = [&](int64_t row, int st) {  // thread 0 only
    const unsigned bar = smem_u32(&bars[st]);
    const unsigned dst = smem_u32(dyn + size_t(st) * stage_bytes);
    mbar_expect_tx(bar, xbytes + ybytes);
    bulk_g2s(dst, x + row * a.dim, xbytes, bar);
    if (FUSE_RES) bulk_g2s(dst + yoff, a.y + row * a.dim, ybytes, bar);
  };
  if (tid == 0)
    for (int i = 0; i < stages && r0 + i * step < r1; i++) issue(r0 + i * step, i);

  bool on[VPT];
#pragma unroll
  for (int k = 0; k < VPT; k++) on[k] = EXACT || (k * T + tid < a.nvec);

  float4 A[VPT], B[VPT], W[HAS_W ? VPT : 1], G[FUSE_RES ? VPT : 1], YB[YBIAS ? VPT : 1];
  int cur_set = -1;
#pragma unroll
  for (int k = 0; k < VPT; k++) {
    if (HAS_W) W[k] = on[k] ? *reinterpret_cast<const float4*>(a.w + 4 * (k * T + tid))
                            : make_float4(0.f, 0.f, 0.f, 0.f);
    if (YBIAS) YB[k] = on[k] ? *reinterpret_cast<const float4*>(a.ybias + 4 * (k * T + tid))
                             : make_float4(0.f, 0.f, 0.f, 0.f);
  }

  int st = 0;
  unsigned phase = 0;
  int parity = 0;
  bool failed = false;
  uint32_t run_max = 0u;  // two running bf16 maxima of this thread's outputs
  int64_t row = r0;
  for (; row < r1; row += step) {
    const int set = (row < a.scale.prefix_len ? 1 : 0) | (row < a.shift.prefix_len ? 2 : 0) |
                    (FUSE_RES && row < a.gate.prefix_len ? 4 : 0);
    if (set != cur_set) {
      cur_set = set;
      const float* sc = a.scale.target ? pick(a.scale, row) : nullptr;
      const float* sh = a.shift.target ? pick(a.shift, row) : nullptr;
      const float* gt = FUSE_RES && a.gate.target ? pick(a.gate, row) : nullptr;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        const int c = 4 * (k * T + tid);
        A[k] = make_float4(1.f, 1.f, 1.f, 1.f);
        B[k] = make_float4(-0.f, -0.f, -0.f, -0.f);
        if (on[k]) {
          if (sc) {
            float4 v = *reinterpret_cast<const float4*>(sc + c);
            A[k] = make_float4(1.f + v.x, 1.f + v.y, 1.f + v.z, 1.f + v.w);
          }
          if (sh) B[k] = *reinterpret_cast<const float4*>(sh + c);
        }
        if (FUSE_RES) {
          G[k] = make_float4(1.f, 1.f, 1.f, 1.f);
          if (gt && on[k]) {
            float4 g = *reinterpret_cast<const float4*>(gt + c);
            G[k] = a.gate_tanh ? make_float4(tanhf(g.x), tanhf(g.y), tanhf(g.z), tanhf(g.w)) : g;
          }
        }
      }
    }

    const bool arrived = mbar_wait(smem_u32(&bars[st]), phase);
    const unsigned char* sx = dyn + size_t(st) * stage_bytes;
    float4 v[VPT];
#pragma unroll
    for (int k = 0; k < VPT; k++) {
      v[k] = make_float4(0.f, 0.f, 0.f, 0.f);
      if (on[k] && arrived) v[k] = widen(reinterpret_cast<const raw_t*>(sx)[k * T + tid]);
    }
    if (FUSE_RES) {
      float* xo = a.xw + row * a.dim;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        float4 yv = make_float4(0.f, 0.f, 0.f, 0.f);
        if (on[k] && arrived) yv = widen(reinterpret_cast<const uint2*>(sx + yoff)[k * T + tid]);
        if (YBIAS) {
          // y + bias rounded to bf16, as add_bias_bf16 leaves it (src/kernels/ops.cu:249-262)
          const float t[4] = {yv.x + YB[k].x, yv.y + YB[k].y, yv.z + YB[k].z, yv.w + YB[k].w};
          yv = widen(pack4(t));
        }
        v[k].x = fmaf(yv.x, G[k].x, v[k].x);
        v[k].y = fmaf(yv.y, G[k].y, v[k].y);
        v[k].z = fmaf(yv.z, G[k].z, v[k].z);
        v[k].w = fmaf(yv.w, G[k].w, v[k].w);
        if (on[k] && arrived) st_stream(reinterpret_cast<float4*>(xo + 4 * (k * T + tid)), v[k]);
      }
    }

    if constexpr (MODE == 2) {
      // residual update only: nothing to reduce, the barrier is just the stage hand-over + vote
      const bool all_ok = nwarps == 1 ? bool(__all_sync(0xffffffffu, arrived)) : __syncthreads_and(arrived) != 0;
      if (!all_ok) {
        failed = true;
        break;
      }
      if (tid == 0 && row + stages * step < r1) issue(row + stages * step, st);
      if (++st == stages) st = 0, phase ^= 1u;
    } else {
      // first reduction: its barrier also tells every thread whether all of them saw the row arrive
      bool all_ok;
      float mean = 0.f, ss = 0.f;
      if (MODE == 0) {
        float s = 0.f;
#pragma unroll
        for (int k = 0; k < VPT; k++) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
        mean = cta_sum_vote(s, red[0], nwarps, arrived, all_ok) / fdim;
      }
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        float dx = v[k].x - mean, dy = v[k].y - mean, dz = v[k].z - mean, dw = v[k].w - mean;
        float q = (dx * dx + dy * dy) + (dz * dz + dw * dw);
        ss += (EXACT || MODE == 1 || on[k]) ? q : 0.f;
        v[k] = make_float4(dx, dy, dz, dw);  // the centred row is what the epilogue scales
      }
      float total;
      if (MODE == 0) {
        total = cta_sum(ss, red[1], nwarps);
      } else {
        total = cta_sum_vote(ss, red[parity], nwarps, arrived, all_ok);
        parity ^= 1;
      }
      if (!all_ok) {
        failed = true;
        break;
      }
      // every thread has its part of the row in registers: the stage can take row + stages
      if (tid == 0 && row + stages * step < r1) issue(row + stages * step, st);
      if (++st == stages) st = 0, phase ^= 1u;

      const float rstd = rsqrtf(total / fdim + a.eps);
      bf16* orow = a.out + row * a.dim;
#pragma unroll
      for (int k = 0; k < VPT; k++) {
        float o[4] = {v[k].x * rstd, v[k].y * rstd, v[k].z * rstd, v[k].w * rstd};
        if (HAS_W) o[0] *= W[k].x, o[1] *= W[k].y, o[2] *= W[k].z, o[3] *= W[k].w;
        o[0] = o[0] * A[k].x + B[k].x;
        o[1] = o[1] * A[k].y + B[k].y;
        o[2] = o[2] * A[k].z + B[k].z;
        o[3] = o[3] * A[k].w + B[k].w;
        const uint2 pk = pack4(o);
        if constexpr (QUANT) {
          // the bf16 row goes to shared memory instead of global memory
          if (on[k]) reinterpret_cast<uint2*>(dyn + size_t(stages) * stage_bytes)[k * T + tid] = pk;
        } else {
          if (on[k]) st_stream(reinterpret_cast<uint2*>(orow + 4 * (k * T + tid)), pk);
          if (a.amax && on[k]) run_max = absmax_bf16x2(run_max, absmax_bf16x2(pk.x, pk.y));
        }
      }
      if constexpr (QUANT) {
        // Quantise the row as blockscale.cu quantises a bf16 row, 16 elements per thread (the two
        // halves of a 32-element block in neighbouring lanes; dim is a multiple of 32).  The next
        // row's writes to the buffer come after that row's reduction barrier, which every thread
        // reaches only when it is done reading here.
        __syncthreads();
        const uint4* orow16 = reinterpret_cast<const uint4*>(dyn + size_t(stages) * stage_bytes);
        const int n16 = a.dim >> 4, lane = tid & 31;
        uint8_t* qrow = a.q + row * a.dim;
        uint8_t* sfr = a.sf + sf_row_offset(uint64_t(row), a.nkb_pad);
        for (int i0 = tid - lane; i0 < n16; i0 += T) {
          const int i = i0 + lane, ic = i < n16 ? i : n16 - 1;
          const uint4 raw[2] = {orow16[2 * ic], orow16[2 * ic + 1]};
          uint4 codes;
          const uint8_t sbyte = mxfp8_quant16(raw, mxfp8_block_absmax(raw), codes);
          if (i < n16) {
            st_stream(reinterpret_cast<uint4*>(qrow) + i, codes);
            if ((lane & 1) == 0) sfr[sf_col_offset(i >> 1)] = sbyte;
          }
        }
        if (nwarps == 1) __syncwarp();
      }
    }
  }

  if constexpr (MODE != 2 && !QUANT) {
    if (a.amax) amax_commit(bf16x2_max_to_float(run_max), a.amax);  // every thread of the CTA gets here
  }
  if (failed && tid == 0) {
    if (a.err) atomicExch(a.err, kErrBulkTimeout);
    // Copies issued for rows [row, min(r1, row + stages)) may still be in flight into this CTA's
    // shared memory: give each a bounded chance to land before the CTA goes away.
    int s2 = st;
    unsigned ph = phase;
    for (int64_t r = row; r < r1 && r < row + stages * step; r += step) {
      mbar_wait(smem_u32(&bars[s2]), ph);
      if (++s2 == stages) s2 = 0, ph ^= 1u;
    }
  }
}

// Any dim, any alignment: one CTA per row, three sweeps over the row (the later sweeps hit L1/L2).
template <int MODE, class TIN, bool FUSE_RES>
__global__ void __launch_bounds__(256) norm_rows_generic_kernel(const NormArgs a) {
  __shared__ float red[2][16];
  const int tid = threadIdx.x, T = blockDim.x, nwarps = T >> 5;
  const int64_t row = blockIdx.x;
  const TIN* xr = static_cast<const TIN*>(a.x) + row * a.dim;
  const float fdim = float(a.dim);
  auto ldx = [&](int i) -> float {
    if constexpr (sizeof(TIN) == 4) return xr[i];
    else return bf16_to_f(xr[i]);
  };
  if (FUSE_RES) {
    const float* gt = a.gate.target ? pick(a.gate, row) : nullptr;
    const bf16* yr = a.y + row * a.dim;
    float* xo = a.xw + row * a.dim;
    for (int i = tid; i < a.dim; i += T) {
      const float g = gt ? (a.gate_tanh ? tanhf(gt[i]) : gt[i]) : 1.f;
      xo[i] = fmaf(bf16_to_f(yr[i]), g, ldx(i));  // the same thread re-reads this element in the sweeps below
    }
  }
  float mean = 0.f;
  if (MODE == 0) {
    float s = 0.f;
    for (int i = tid; i < a.dim; i += T) s += ldx(i);
    mean = cta_sum(s, red[0], nwarps) / fdim;
  }
  float ss = 0.f;
  for (int i = tid; i < a.dim; i += T) {
    float d = ldx(i) - mean;
    ss += d * d;
  }
  const float rstd = rsqrtf(cta_sum(ss, red[1], nwarps) / fdim + a.eps);
  const float* sc = a.scale.target ? pick(a.scale, row) : nullptr;
  const float* sh = a.shift.target ? pick(a.shift, row) : nullptr;
  bf16* orow = a.out + row * a.dim;
  float run_max = 0.f;
  for (int i = tid; i < a.dim; i += T) {
    float v = (ldx(i) - mean) * rstd;
    if (a.w) v *= a.w[i];
    if (sc) v *= 1.f + sc[i];
    if (sh) v += sh[i];
    const bf16 o = __float2bfloat16(v);
    orow[i] = o;
    run_max = fmaxf(run_max, fabsf(bf16_to_f(o)));
  }
  if (a.amax) amax_commit(run_max, a.amax);
}

// Launch plan shared by every instantiation: threads per CTA and vectors per thread.
struct NormPlan {
  int threads, vpt;
  bool exact;
};

}  // namespace mxk
