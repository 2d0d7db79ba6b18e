// Bulk-copy (TMA) pipeline for the 16-bytes-in / 16-bytes-out streaming ops (GELU in place,
// SiLU-gated multiply).  The work is a list of contiguous chunks; the CTA's last warp is a
// producer that cp.async.bulk-copies each chunk's source bytes (one or two sources) into a
// shared-memory stage completing on the stage's `full` mbarrier; the other warps read 128-bit
// vectors from the stage, apply the op and store 128 bits to global memory, then arrive on the
// stage's `empty` mbarrier.  No CTA-wide barrier in the loop; all waits are bounded
// (bulk_copy.cuh), with the same wind-down as the head pipeline.
//
// An op provides
//   static constexpr int NSRC;                                   1 or 2 source streams
//   __device__ void locate(int64_t chunk, Chunk& c) const;        fills sources, destination, bytes
//   __device__ uint4 apply(const uint4& a, const uint4& b) const; 8 bf16 (+8) in, 8 bf16 out
//
// An op whose output is not 16 bytes per 16 bytes (the block-scale quantiser, a reduction) defines a
// per-thread `State` type instead of apply() and consumes a landed chunk itself:
//   __device__ State init() const;                                 once per consumer thread, after the
//                                                                  dependency wait
//   __device__ void consume(State&, int64_t chunk, const unsigned char* stage, int tid, int n_cons) const;
//   __device__ void finish(State&, int lane) const;                after the thread's last chunk
#pragma once

#include <type_traits>

#include "bulk_copy.cuh"
#include "common.cuh"
#include "tuning.h"

namespace mxk {

struct Chunk {
  const unsigned char* src0;
  const unsigned char* src1;
  unsigned char* dst;
  unsigned bytes;  // per source and of the destination; multiple of 16
};

// Chunking of a [rows, K] bf16 matrix for ops that need to know the column of what they process: a
// chunk is one piece (pieces_per_row of them, whole multiples of 128 elements) of one row.
struct RowPieces {
  const unsigned char* x;
  int64_t ldx_bytes;
  int K, pieces_per_row, piece_elems;
  int64_t src1_off = 0;  // bytes from a piece to its second source (silu_mul's `up` half), 0 = none
  int stage_off = 0;     // where the second source sits inside a stage
  // chunk / pieces_per_row for chunk < 2^31 as a multiply-high and a shift (set_pieces)
  unsigned div_mul = 0, div_shift = 0;
  // m = ceil(2^(31 + s) / d) with s = ceil(log2 d) fits 32 bits and gives floor(n / d) exactly for
  // every n < 2^31 (the error term m d - 2^(31 + s) is below d <= 2^s).
  void set_pieces(int ppr, int elems) {
    pieces_per_row = ppr, piece_elems = elems;
    if (ppr > 1) {
      unsigned s = 0;
      while ((1u << s) < unsigned(ppr)) s++;
      const unsigned long long p = 1ull << (31 + s);
      div_mul = unsigned((p + unsigned(ppr) - 1) / unsigned(ppr));
      div_shift = s - 1;
    }
  }
  // This runs once per chunk in every consumer thread, so: 32-bit arithmetic, no division.
  __device__ __forceinline__ void where(int64_t chunk, unsigned& row, int& k0, int& n) const {
    const unsigned c = unsigned(chunk);
    if (pieces_per_row == 1) {
      row = c, k0 = 0, n = K;
      return;
    }
    row = __umulhi(c, div_mul) >> div_shift;
    k0 = int(c - row * unsigned(pieces_per_row)) * piece_elems;
    n = K - k0 < piece_elems ? K - k0 : piece_elems;
  }
  __device__ void locate(int64_t chunk, Chunk& c) const {
    unsigned row;
    int k0, n;
    where(chunk, row, k0, n);
    c.src0 = x + row * ldx_bytes + int64_t(k0) * 2, c.src1 = c.src0 + src1_off, c.dst = nullptr;
    c.bytes = unsigned(n) * 2;
  }
};

template <class Op, class = void>
struct consumes_itself : std::false_type {};
template <class Op>
struct consumes_itself<Op, std::void_t<typename Op::State>> : std::true_type {};

__device__ __forceinline__ void mbar_arrive_one(unsigned bar) {
  asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

template <class Op>
__global__ void __launch_bounds__(544) stream_pipe_kernel(const Op op, const int64_t n_chunks, const int64_t chunks_per_cta,
                                                          const int stages, const int stage_bytes, const int src_bytes,
                                                          const int interleave, int* err) {
  extern __shared__ __align__(128) unsigned char dyn[];
  __shared__ __align__(8) unsigned long long full[8], empty[8];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int n_cons_warps = (blockDim.x >> 5) - 1, n_cons = n_cons_warps * 32;
  // This CTA's chunks: a contiguous range, or every gridDim.x-th chunk (the grid then sweeps one
  // compact window of memory together).
  const int64_t c_step = interleave ? int64_t(gridDim.x) : 1;
  const int64_t c_begin = interleave ? int64_t(blockIdx.x) : int64_t(blockIdx.x) * chunks_per_cta;
  const int64_t c_end = interleave ? n_chunks : (c_begin + chunks_per_cta < n_chunks ? c_begin + chunks_per_cta : n_chunks);
  const int mine = c_end > c_begin ? int((c_end - c_begin + c_step - 1) / c_step) : 0;

  if (tid == 0) {
    for (int i = 0; i < stages; i++) {
      mbar_init(smem_u32(&full[i]), 1);
      mbar_init(smem_u32(&empty[i]), unsigned(n_cons_warps));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  pdl_launch_dependents();
  __syncthreads();
  pdl_wait();  // nothing above touches global memory

  bool ok = true;
  int issued = 0;
  if (warp == n_cons_warps) {
    if (lane == 0) {
      int st = 0;
      unsigned ph = 0;  // the k-th refill of a stage (k >= 1) waits for phase k - 1 of `empty`
      for (int it = 0; it < mine; it++) {
        if (it >= stages && !mbar_wait(smem_u32(&empty[st]), ph)) {
          ok = false;
          break;
        }
        Chunk c;
        op.locate(c_begin + it * c_step, c);
        const unsigned bar = smem_u32(&full[st]);
        const unsigned dst = smem_u32(dyn + size_t(st) * stage_bytes);
        mbar_expect_tx(bar, c.bytes * Op::NSRC);
        bulk_g2s(dst, c.src0, c.bytes, bar);
        if (Op::NSRC == 2) bulk_g2s(dst + src_bytes, c.src1, c.bytes, bar);
        issued++;
        if (++st == stages) st = 0, ph ^= (it >= stages ? 1u : 0u);
      }
    }
  } else if constexpr (consumes_itself<Op>::value) {
    typename Op::State state = op.init();
    int st = 0;
    unsigned ph = 0;
    for (int it = 0; it < mine; it++) {
      if (!mbar_wait(smem_u32(&full[st]), ph)) {
        ok = false;
        break;
      }
      op.consume(state, c_begin + it * c_step, dyn + size_t(st) * stage_bytes, tid, n_cons);
      __syncwarp();
      if (lane == 0) mbar_arrive_one(smem_u32(&empty[st]));
      if (++st == stages) st = 0, ph ^= 1u;
    }
    op.finish(state, lane);
  } else {
    int st = 0;
    unsigned ph = 0;
    for (int it = 0; it < mine; it++) {
      if (!mbar_wait(smem_u32(&full[st]), ph)) {
        ok = false;
        break;
      }
      Chunk c;
      op.locate(c_begin + it * c_step, c);
      const uint4* s0 = reinterpret_cast<const uint4*>(dyn + size_t(st) * stage_bytes);
      const uint4* s1 = reinterpret_cast<const uint4*>(dyn + size_t(st) * stage_bytes + src_bytes);
      uint4* d = reinterpret_cast<uint4*>(c.dst);
      const int nvec = int(c.bytes >> 4);
      if (nvec == 2 * n_cons) {
        // a full chunk at the default shapes: two vectors per thread, no loop and no bounds checks
        const uint4 a0 = s0[tid], a1 = s0[tid + n_cons];
        const uint4 b0 = Op::NSRC == 2 ? s1[tid] : a0, b1 = Op::NSRC == 2 ? s1[tid + n_cons] : a1;
        st_stream(d + tid, op.apply(a0, b0));
        st_stream(d + tid + n_cons, op.apply(a1, b1));
      } else
      for (int v = tid; v < nvec; v += 4 * n_cons) {
        uint4 a[4], b[4];
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int i = v + u * n_cons;
          if (i < nvec) {
            a[u] = s0[i];
            if (Op::NSRC == 2) b[u] = s1[i];
          }
        }
#pragma unroll
        for (int u = 0; u < 4; u++) {
          const int i = v + u * n_cons;
          if (i < nvec) st_stream(d + i, op.apply(a[u], Op::NSRC == 2 ? b[u] : a[u]));
        }
      }
      __syncwarp();
      if (lane == 0) mbar_arrive_one(smem_u32(&empty[st]));
      if (++st == stages) st = 0, ph ^= 1u;
    }
  }

  if (!ok && err) atomicExch(err, kErrBulkTimeout);
  // All waits are bounded, so every warp arrives here; after a failure the producer gives the
  // copies of its last `stages` chunks a bounded chance to land before the CTA exits.
  const bool any_failed = __syncthreads_or(!ok) != 0;
  if (any_failed && warp == n_cons_warps && lane == 0) {
    for (int it = issued > stages ? issued - stages : 0; it < issued; it++)
      mbar_wait(smem_u32(&full[it % stages]), unsigned((it / stages) & 1));
  }
}

// Launches the pipeline over n_chunks chunks whose sources are at most src_bytes long.
template <class Op>
inline int run_stream_pipe(const char* name, const Op& op, int64_t n_chunks, int src_bytes, cudaStream_t s,
                           int default_warps, int default_stages) {
  auto k = stream_pipe_kernel<Op>;
  int warps = tune(TUNE_STREAM_WARPS, default_warps);
  if (warps < 1) warps = 1;
  if (warps > 16) warps = 16;
  const int threads = warps * 32 + 32;
  const int padded = (src_bytes + 127) & ~127;
  const int stage_bytes = padded * Op::NSRC;
  int stages = tune(TUNE_STREAM_STAGES, default_stages);
  if (stages < 2) stages = 2;
  if (stages > 8) stages = 8;
  const size_t smem = size_t(stages) * stage_bytes;
  if (smem > 40 * 1024) cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
  const int per_sm = tune(TUNE_STREAM_CTAS_PER_SM, resident_ctas(k, threads, smem));
  int64_t ctas = int64_t(sm_count()) * (per_sm > 0 ? per_sm : 1);
  if (ctas > n_chunks) ctas = n_chunks;
  const int64_t per_cta = ceil_div(n_chunks, ctas);
  launch_pdl(k, dim3(unsigned(ceil_div(n_chunks, per_cta))), dim3(threads), smem, s, op, n_chunks, per_cta, stages,
             stage_bytes, padded, int(tune(TUNE_PIPE_INTERLEAVE, 1) == 1), device_error_word());
  return after_launch(name);
}

}  // namespace mxk
